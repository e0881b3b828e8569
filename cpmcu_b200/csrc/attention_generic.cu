// Attention over the paged cache, one warp per (query token, head), fp32 arithmetic
// throughout.  This is the kernel of the true 32-bit path and the plain twin the
// tensor-core kernels are checked against; it takes every head size, group size,
// window and block selection.
//
// A query at absolute position p of its sequence sees keys j <= p (the rule of
// the reference's causal mask, src/flash_attn/src/mask.h:185-211), further limited to
// j > p - window when a window is given, or to the key blocks listed for it when a
// block list is given (the reference's block mask, src/flash_attn/src/flash_blockmask.h:15-93).
// Scores are scaled by ``scale`` before the softmax (src/model/attn.cuh:218).
#include "common.cuh"
#include <math.h>

constexpr int kMaxDimsPerLane = 8;   // head_dim <= 256

template <typename T>
__global__ void attention_generic_kernel(
    const T* __restrict__ q,            // [tokens, heads, d]
    const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    T* __restrict__ out,                // [tokens, heads, d]
    const int* __restrict__ positions, const int* __restrict__ token_seq, const int* __restrict__ slots,
    const int* __restrict__ page_table, int max_pages,
    const int* __restrict__ block_list, // [tokens, kv_heads, list_cap] or nullptr
    int list_cap, int block_size, int window,
    int n_heads, int n_kv, int d, float scale) {
    extern __shared__ float q_smem[];   // [warps][d]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    if (h >= n_heads) return;
    const int group = n_heads / n_kv;
    const int kvh = h / group;
    const int p = positions[t];
    const int slot = slots[token_seq[t]];
    const int* pages = page_table + (int64_t)slot * max_pages;

    float* qs = q_smem + warp * d;
    const T* qrow = q + ((int64_t)t * n_heads + h) * d;
    for (int c = lane; c < d; c += 32) qs[c] = to_f32(qrow[c]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[kMaxDimsPerLane];
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] = 0.f;

    const int* list = block_list ? block_list + ((int64_t)t * n_kv + kvh) * list_cap : nullptr;
    const bool listed = list != nullptr && list[0] != -2;
    int seg_index = 0;
    while (true) {
        int seg_lo, seg_hi;                // keys [seg_lo, seg_hi)
        if (listed) {
            if (seg_index >= list_cap) break;
            const int b = list[seg_index];
            if (b < 0) break;
            seg_lo = b * block_size;
            seg_hi = min(seg_lo + block_size, p + 1);
        } else {
            if (seg_index > 0) break;
            seg_lo = window > 0 ? max(0, p - window + 1) : 0;
            seg_hi = p + 1;
        }
        ++seg_index;
        for (int j0 = seg_lo; j0 < seg_hi; j0 += 32) {
            const int j = j0 + lane;
            const bool valid = j < seg_hi;
            float s = -INFINITY;
            if (valid) {
                const int page = CPM_PAGE(pages, j / kPageTokens, max_pages);
                const T* krow = k_cache + page_row_offset(page, kvh, j % kPageTokens, n_kv, d);
                float dot = 0.f;
                for (int c = 0; c < d; ++c) dot = fmaf(qs[c], to_f32(krow[c]), dot);
                s = dot * scale;
            }
            const float m_new = fmaxf(m, warp_max(s));
            const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
            const float pr = valid ? expf(s - m_new) : 0.f;
            l = l * corr + warp_sum(pr);
#pragma unroll
            for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] *= corr;
            m = m_new;
            const int n_here = min(32, seg_hi - j0);
            for (int jj = 0; jj < n_here; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, pr, jj);
                const int key = j0 + jj;
                const int page = CPM_PAGE(pages, key / kPageTokens, max_pages);
                const T* vcol = v_cache + value_offset(page, kvh, 0, key % kPageTokens, n_kv, d);
#pragma unroll
                for (int i = 0; i < kMaxDimsPerLane; ++i) {
                    const int c = lane + 32 * i;
                    if (c < d) acc[i] = fmaf(pj, to_f32(vcol[(int64_t)c * kPageTokens]), acc[i]);
                }
            }
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* orow = out + ((int64_t)t * n_heads + h) * d;
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < d) orow[c] = from_f32<T>(acc[i] * inv);
    }
}

CPM_API int cpm_attention_generic(const void* q, const void* k_cache, const void* v_cache, void* out,
                                  const int* positions, const int* token_seq, const int* slots,
                                  const int* page_table, int max_pages, const int* block_list, int list_cap,
                                  int block_size, int window, int n_tokens, int n_heads, int n_kv, int d,
                                  float scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (d <= 0 || d > 32 * kMaxDimsPerLane || n_kv <= 0 || n_heads % n_kv != 0) return CPM_BAD_ARGUMENT;
    if (block_list && (block_size <= 0 || list_cap <= 0)) return CPM_BAD_ARGUMENT;
    const int warps = 4;
    dim3 grid(n_tokens, (n_heads + warps - 1) / warps);
    const size_t smem = (size_t)warps * d * sizeof(float);
    if (dtype == CPM_BF16)
        attention_generic_kernel<bf16><<<grid, warps * 32, smem, stream>>>((const bf16*)q, (const bf16*)k_cache,
            (const bf16*)v_cache, (bf16*)out, positions, token_seq, slots, page_table, max_pages, block_list,
            list_cap, block_size, window, n_heads, n_kv, d, scale);
    else
        attention_generic_kernel<float><<<grid, warps * 32, smem, stream>>>((const float*)q, (const float*)k_cache,
            (const float*)v_cache, (float*)out, positions, token_seq, slots, page_table, max_pages, block_list,
            list_cap, block_size, window, n_heads, n_kv, d, scale);
    return launch_status();
}

CPM_BOUNDS_TU(attention_generic)
