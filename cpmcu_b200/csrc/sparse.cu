// InfLLM-v2 block selection: mean-pooled ("compressed") keys kept beside the cache,
// and the choice of key blocks for each query.
//
// Reference pieces: mean pooling of 32 cached keys every 16
// (src/model/minicpm4/minicpm4_kvcache.cuh:6-30), stage-1 score = softmax of a query
// against the pooled keys summed over the heads of its group
// (src/flash_attn/src/flash_fwd_kernel.h:1770-2265, src/model/minicpm4/minicpm4_attn.cuh:119-141),
// block score = max over the pooled keys that overlap a block, leading blocks forced,
// the local window left out of the choice (minicpm4_kvcache.cuh:64-108), top-k with ties
// to the lower index (src/model/topk.cuh:17, 26), block mask (minicpm4_kvcache.cuh:110-142).
//
// Differences by design: window, stride and block size are parameters (the reference
// fixes 32/16/64 and a group of 16); everything is decided per query from the keys at or
// before it, so the result does not depend on how tokens are cut into steps (the
// reference's pooled keys and selection see earlier chunks only); the local window is
// always attended; scores, pooling and the choice are fp32, and pooled keys are stored
// in fp32 whatever the cache's type.
#include "common.cuh"

// One block per (token, kv head).  If the token at position pos completes a pooling
// window [first, first + kernel) with first = pos + 1 - kernel a multiple of stride,
// the mean of those cached keys is stored as pooled entry first / stride.
template <typename T>
__global__ void pool_keys_kernel(const T* __restrict__ k_cache, float* __restrict__ pooled,
                                 const int* __restrict__ positions, const int* __restrict__ token_seq,
                                 const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                 int n_kv, int d, int kernel, int stride) {
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int first = positions[t] + 1 - kernel;
    if (first < 0 || first % stride != 0) return;
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int per_page = kPageTokens / stride;
    const int64_t dst = (((int64_t)pages[first / kPageTokens] * n_kv + kvh) * per_page
                         + (first % kPageTokens) / stride) * d;
    const float inv = 1.0f / (float)kernel;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float s = 0.f;
        for (int r = 0; r < kernel; ++r) {
            const int j = first + r;
            s += to_f32(k_cache[page_row_offset(pages[j / kPageTokens], kvh, j % kPageTokens, n_kv, d) + c]);
        }
        pooled[dst + c] = s * inv;
    }
}

CPM_API int cpm_pool_keys(const void* k_cache, float* pooled, const int* positions, const int* token_seq,
                          const int* slots, const int* page_table, int max_pages, int n_tokens, int n_kv, int d,
                          int kernel, int stride, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (stride <= 0 || kernel <= 0 || kPageTokens % stride != 0 || n_kv > 65535) return CPM_BAD_ARGUMENT;
    dim3 grid(n_tokens, n_kv);
    const int threads = d >= 128 ? 128 : 64;
    if (dtype == CPM_BF16)
        pool_keys_kernel<bf16><<<grid, threads, 0, stream>>>((const bf16*)k_cache, pooled, positions, token_seq, slots,
                                                             page_table, max_pages, n_kv, d, kernel, stride);
    else
        pool_keys_kernel<float><<<grid, threads, 0, stream>>>((const float*)k_cache, pooled, positions, token_seq,
                                                              slots, page_table, max_pages, n_kv, d, kernel, stride);
    return launch_status();
}

// One block per (token, kv head): writes the ascending list of key blocks the query
// attends to, ended by -1; a first entry of -2 says "dense" (the query sees at most
// dense_len keys).
template <typename T>
__global__ void __launch_bounds__(256)
select_blocks_kernel(const T* __restrict__ q, const float* __restrict__ pooled, const int* __restrict__ positions,
                     const int* __restrict__ token_seq, const int* __restrict__ slots,
                     const int* __restrict__ page_table, int max_pages, int* __restrict__ lists, int list_cap,
                     int n_heads, int n_kv, int d, float scale, int kernel, int stride, int block_size,
                     int init_blocks, int topk, int local_blocks, int dense_len, int max_entries) {
    extern __shared__ float sm[];
    float* score = sm;                       // [max_entries]
    float* tmp = sm + max_entries;           // [max_entries]: logits of one head, then block scores
    float* qs = tmp + max_entries;           // [d]
    float* red = qs + d;                     // [33]
    ArgMax* am = (ArgMax*)(red + 34);        // [33]
    const int t = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x;
    int* list = lists + ((int64_t)t * n_kv + kvh) * list_cap;
    const int p = positions[t];
    if (p + 1 <= dense_len) {
        if (tid == 0) list[0] = -2;
        return;
    }
    const int group = n_heads / n_kv;
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int per_page = kPageTokens / stride;
    int n_vis = p + 1 >= kernel ? (p + 1 - kernel) / stride + 1 : 0;
    n_vis = min(n_vis, max_entries);

    for (int i = tid; i < n_vis; i += blockDim.x) score[i] = 0.f;
    for (int g = 0; g < group; ++g) {
        const T* qrow = q + ((int64_t)t * n_heads + kvh * group + g) * d;
        __syncthreads();
        for (int c = tid; c < d; c += blockDim.x) qs[c] = to_f32(qrow[c]);
        __syncthreads();
        float mx = -INFINITY;
        for (int i = tid; i < n_vis; i += blockDim.x) {
            const int tok = i * stride;
            const float* row = pooled + (((int64_t)pages[tok / kPageTokens] * n_kv + kvh) * per_page
                                         + (tok % kPageTokens) / stride) * d;
            float dot = 0.f;
            for (int c = 0; c < d; ++c) dot = fmaf(qs[c], row[c], dot);
            dot *= scale;
            tmp[i] = dot;
            mx = fmaxf(mx, dot);
        }
        // block max through the argmax reduction (only the value is used)
        mx = block_argmax(ArgMax{mx, 0}, am).v;
        float part = 0.f;
        for (int i = tid; i < n_vis; i += blockDim.x) part += expf(tmp[i] - mx);
        const float total = block_sum(part, red);
        const float inv = total > 0.f ? 1.f / total : 0.f;
        for (int i = tid; i < n_vis; i += blockDim.x) score[i] += expf(tmp[i] - mx) * inv;
    }
    __syncthreads();

    // block scores of the blocks that can be chosen: init_blocks <= k <= last_choice
    const int qb = p / block_size;
    const int last_choice = qb - local_blocks;
    const int per_block = block_size / stride;
    const int reach_back = kernel / stride - 1;
    const int n_cand = max(0, last_choice + 1 - init_blocks);
    for (int i = tid; i < n_cand; i += blockDim.x) {
        const int k = init_blocks + i;
        const int lo = max(0, k * per_block - reach_back), hi = min(n_vis, (k + 1) * per_block);
        float b = -INFINITY;
        for (int e = lo; e < hi; ++e) b = fmaxf(b, score[e]);
        tmp[i] = b;
    }
    __syncthreads();
    // repeated arg-max: the chosen candidates are marked with NaN
    const int room = min(max(0, topk - init_blocks), n_cand);
    for (int r = 0; r < room; ++r) {
        ArgMax best{-INFINITY, 0x7fffffff};
        for (int i = tid; i < n_cand; i += blockDim.x) {
            const float v = tmp[i];
            if (v == v) best = better(best, ArgMax{v, i});
        }
        best = block_argmax(best, am);
        if (best.i == 0x7fffffff || best.v == -INFINITY) break;     // nothing left with a visible pooled key
        if (tid == 0) tmp[best.i] = __int_as_float(0x7fc00000);
        __syncthreads();
    }
    __syncthreads();
    if (tid == 0) {
        int n = 0;
        const int n_init = min(init_blocks, qb + 1);
        for (int k = 0; k < n_init && n < list_cap - 1; ++k) list[n++] = k;
        for (int i = 0; i < n_cand && n < list_cap - 1; ++i)
            if (tmp[i] != tmp[i]) list[n++] = init_blocks + i;
        for (int k = max(n_init, last_choice + 1); k <= qb && n < list_cap - 1; ++k) list[n++] = k;
        list[n] = -1;
    }
}

CPM_API int cpm_select_blocks(const void* q, const float* pooled, const int* positions, const int* token_seq,
                              const int* slots, const int* page_table, int max_pages, int* lists, int list_cap,
                              int n_tokens, int n_heads, int n_kv, int d, float scale, int kernel, int stride,
                              int block_size, int init_blocks, int topk, int local_blocks, int dense_len,
                              int max_entries, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (stride <= 0 || kernel % stride || block_size % stride || kPageTokens % stride || n_kv > 65535 ||
        n_heads % n_kv || list_cap < topk + local_blocks + 1 || max_entries < 1)
        return CPM_BAD_ARGUMENT;
    const size_t smem = ((size_t)2 * max_entries + d + 34) * sizeof(float) + 33 * sizeof(ArgMax);
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    dim3 grid(n_tokens, n_kv);
    cudaError_t e = cudaSuccess;
    if (dtype == CPM_BF16) {
        auto kern = select_blocks_kernel<bf16>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, 256, smem, stream>>>((const bf16*)q, pooled, positions, token_seq, slots, page_table, max_pages,
            lists, list_cap, n_heads, n_kv, d, scale, kernel, stride, block_size, init_blocks, topk, local_blocks,
            dense_len, max_entries);
    } else {
        auto kern = select_blocks_kernel<float>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, 256, smem, stream>>>((const float*)q, pooled, positions, token_seq, slots, page_table, max_pages,
            lists, list_cap, n_heads, n_kv, d, scale, kernel, stride, block_size, init_blocks, topk, local_blocks,
            dense_len, max_entries);
    }
    return launch_status();
}
