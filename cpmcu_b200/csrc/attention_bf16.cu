// bf16 attention over the paged cache on the tensor cores, for decode (one query token
// per sequence, split over the keys) and for prefill (many query tokens per sequence).
//
// One warp owns a tile of 16 query rows and walks over key pages.  Keys are read
// straight from global memory into mma fragments with 16-byte loads along head_dim, and
// values likewise along the token axis of the transposed value pages, so there is no
// shared-memory staging and no barrier: the sums over head_dim and over keys do not
// care about order, which lets a thread's 8 consecutive elements stand for the k-slots
// of two m16n8k16 instructions as long as both operands use the same assignment.
//
// Decode: the 16 rows are the query heads that share one key-value head (grouped-query
// attention), every warp takes a share of the sequence's pages and writes an unnormalised
// partial result; a second kernel combines the shares.  The reference runs its flash
// kernel with 16 fixed splits and a combine kernel (src/flash_attn/flash_api.hpp:385-391,
// src/flash_attn/src/flash_fwd_kernel.h:2320-2501).  Prefill: the 16 rows are consecutive
// tokens of one head; the causal rule is per row (src/flash_attn/src/mask.h:185-211).
// Softmax statistics, scores and output accumulators are fp32; probabilities are rounded
// to bf16 for the second product, as in the reference (src/flash_attn/src/flash_fwd_kernel.h:1560-1616).
#include "common.cuh"

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Keys and values are read once by one warp: keep them out of L1.
__device__ __forceinline__ uint4 ldg16(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// State of a 16-row tile in one warp: thread (g = lane / 4, j = lane % 4) holds rows g and
// g + 8; o[nt] are output dims 8*nt + 2j, 2j+1 of both rows.
template <int D>
struct TileState {
    float o[D / 8][4];
    float m[2];      // running maximum of the scaled scores (log2 domain)
    float l[2];      // this thread's share of the running sum
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
    }
};

// One page of 64 keys.  q[r][w]: 8 consecutive dims 32w + 8j .. of row g (r = 0) and g + 8
// (r = 1).  Keys with index > limit[r] (index inside the sequence) are masked for row r.
// Column n = 2j' + e of score tile t in the 32-key half u stands for key
// 32u + 8j' + 2t + e, so that thread j ends up with the probabilities of 8 consecutive
// keys, which is what the 16-byte value loads along the token axis need.
template <int D>
__device__ __forceinline__ void attend_page(TileState<D>& st, const uint4 (&q)[2][D / 32], const bf16* __restrict__ kpage,
                                            const bf16* __restrict__ vpage, int key0, int limit0, int limit1,
                                            float scale_log2, int lane) {
    const int j = lane & 3, n = lane >> 2;
    float s[2][4][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            s[u][t][0] = s[u][t][1] = s[u][t][2] = s[u][t][3] = 0.f;
            const int krow = 32 * u + 8 * (n >> 1) + 2 * t + (n & 1);
            const bf16* kp = kpage + krow * D + 8 * j;
#pragma unroll
            for (int w = 0; w < D / 32; ++w) {
                const uint4 kv = ldg16(kp + 32 * w);
                mma_16816(s[u][t], q[0][w].x, q[1][w].x, q[0][w].y, q[1][w].y, kv.x, kv.y);
                mma_16816(s[u][t], q[0][w].z, q[1][w].z, q[0][w].w, q[1][w].w, kv.z, kv.w);
            }
        }
    }
    // scale, mask, row maxima
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + 32 * u + 8 * j + 2 * t + e;
                const float a = key <= limit0 ? s[u][t][e] * scale_log2 : -INFINITY;
                const float b = key <= limit1 ? s[u][t][2 + e] * scale_log2 : -INFINITY;
                s[u][t][e] = a;
                s[u][t][2 + e] = b;
                mx0 = fmaxf(mx0, a);
                mx1 = fmaxf(mx1, b);
            }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
    const float use0 = mn0 == -INFINITY ? 0.f : mn0, use1 = mn1 == -INFINITY ? 0.f : mn1;
    const float corr0 = exp2f(st.m[0] - use0), corr1 = exp2f(st.m[1] - use1);
    st.m[0] = mn0;
    st.m[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float a = exp2f(s[u][t][e] - use0), b = exp2f(s[u][t][2 + e] - use1);
                s[u][t][e] = a;
                s[u][t][2 + e] = b;
                sum0 += a;
                sum1 += b;
            }
    st.l[0] = st.l[0] * corr0 + sum0;
    st.l[1] = st.l[1] * corr1 + sum1;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        st.o[nt][0] *= corr0;
        st.o[nt][1] *= corr0;
        st.o[nt][2] *= corr1;
        st.o[nt][3] *= corr1;
    }
    // weighted sum of values
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t a0 = pack_bf16(s[u][0][0], s[u][0][1]), a1 = pack_bf16(s[u][0][2], s[u][0][3]);
        const uint32_t a2 = pack_bf16(s[u][1][0], s[u][1][1]), a3 = pack_bf16(s[u][1][2], s[u][1][3]);
        const uint32_t c0 = pack_bf16(s[u][2][0], s[u][2][1]), c1 = pack_bf16(s[u][2][2], s[u][2][3]);
        const uint32_t c2 = pack_bf16(s[u][3][0], s[u][3][1]), c3 = pack_bf16(s[u][3][2], s[u][3][3]);
        const bf16* vp = vpage + n * kPageTokens + 32 * u + 8 * j;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            const uint4 vv = ldg16(vp + nt * 8 * kPageTokens);
            mma_16816(st.o[nt], a0, a1, a2, a3, vv.x, vv.y);
            mma_16816(st.o[nt], c0, c1, c2, c3, vv.z, vv.w);
        }
    }
}

// ---------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------
// Asynchronous copies (cp.async, 16 bytes per thread) bring a warp's next pages into its own
// shared-memory buffers while it works on the current one, so the bytes in flight do not
// depend on how the compiler orders loads.  The 16-byte chunks of odd rows are stored
// shifted by four chunks where rows are a multiple of 128 bytes apart, which keeps the
// fragment reads free of bank conflicts.
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(smem_addr), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds16(uint32_t smem_addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr));
    return v;
}

constexpr int kDecodeStages = 2;

template <int D>
struct DecodeSmem {
    static constexpr int kChunksPerKeyRow = D / 8;                         // 16-byte chunks in a key row
    static constexpr bool kSwizzleKeys = (kChunksPerKeyRow % 8) == 0;
    static constexpr int kKeyBytes = kPageTokens * D * 2;
    static constexpr int kStageBytes = 2 * kKeyBytes;                      // a key page and a value page
    // Warps of a block, each with its own two stages: three fill an SM's shared memory at head size 128 (196 KB);
    // smaller heads have smaller pages, and more warps keep as many bytes in flight per SM (six at head size 64:
    // the 0.5B sizes' decode step at batch 64 went from 2.29 to 1.93 ms).
    static constexpr int kWarps = D >= 128 ? 3 : D >= 96 ? 4 : D >= 64 ? 6 : 8;
    static constexpr int kTotal = kWarps * kDecodeStages * kStageBytes;
};

// Copies one key page and one value page (both contiguous in global memory) into a stage.
template <int D, int kThreads = 32>
__device__ __forceinline__ void copy_page_async(uint32_t stage, const bf16* __restrict__ kpage,
                                                const bf16* __restrict__ vpage, int lane) {
    using S = DecodeSmem<D>;
    constexpr int kChunks = S::kKeyBytes / 16;
#pragma unroll 4
    for (int c = lane; c < kChunks; c += kThreads) {
        const int row = c / S::kChunksPerKeyRow, col = c % S::kChunksPerKeyRow;
        const int pcol = S::kSwizzleKeys ? (col ^ ((row & 1) << 2)) : col;
        cp_async16(stage + (row * S::kChunksPerKeyRow + pcol) * 16, kpage + c * 8);
    }
#pragma unroll 4
    for (int c = lane; c < kChunks; c += kThreads) {
        const int row = c >> 3, col = c & 7;                               // value rows hold 64 tokens = 8 chunks
        cp_async16(stage + S::kKeyBytes + (row * 8 + (col ^ ((row & 1) << 2))) * 16, vpage + c * 8);
    }
}

// attend_page with both pages in shared memory (same fragment assignment).
template <int D>
__device__ __forceinline__ void attend_page_smem(TileState<D>& st, const uint4 (&q)[2][D / 32], uint32_t stage, int key0,
                                                 int limit0, int limit1, float scale_log2, int lane) {
    using S = DecodeSmem<D>;
    const int j = lane & 3, n = lane >> 2;
    float s[2][4][4];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int t = 0; t < 4; ++t) s[u][t][0] = s[u][t][1] = s[u][t][2] = s[u][t][3] = 0.f;
    // the eight score tiles are independent accumulator chains: walk head_dim in the outer loop
#pragma unroll
    for (int w = 0; w < D / 32; ++w) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int krow = 32 * u + 8 * (n >> 1) + 2 * t + (n & 1);
                const int swz = S::kSwizzleKeys ? ((krow & 1) << 2) : 0;
                const uint4 kv = lds16(stage + (krow * S::kChunksPerKeyRow + ((4 * w + j) ^ swz)) * 16);
                mma_16816(s[u][t], q[0][w].x, q[1][w].x, q[0][w].y, q[1][w].y, kv.x, kv.y);
                mma_16816(s[u][t], q[0][w].z, q[1][w].z, q[0][w].w, q[1][w].w, kv.z, kv.w);
            }
        }
    }
    // Row maxima of the raw scores; a page that lies wholly at or before both rows' limits (all pages but a
    // sequence's last) needs no mask.  The scale goes into the exponent's multiply-add: exp2(s * scale - m).
    float mx0 = -INFINITY, mx1 = -INFINITY;
    if (key0 + kPageTokens - 1 > min(limit0, limit1)) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int t = 0; t < 4; ++t)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = key0 + 32 * u + 8 * j + 2 * t + e;
                    if (key > limit0) s[u][t][e] = -INFINITY;
                    if (key > limit1) s[u][t][2 + e] = -INFINITY;
                }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            mx0 = fmaxf(mx0, fmaxf(s[u][t][0], s[u][t][1]));
            mx1 = fmaxf(mx1, fmaxf(s[u][t][2], s[u][t][3]));
        }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(st.m[0], mx0 * scale_log2), mn1 = fmaxf(st.m[1], mx1 * scale_log2);
    const float use0 = mn0 == -INFINITY ? 0.f : mn0, use1 = mn1 == -INFINITY ? 0.f : mn1;
    const float corr0 = exp2f(st.m[0] - use0), corr1 = exp2f(st.m[1] - use1);
    st.m[0] = mn0;
    st.m[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float a = exp2f(fmaf(s[u][t][e], scale_log2, -use0)), b = exp2f(fmaf(s[u][t][2 + e], scale_log2, -use1));
                s[u][t][e] = a;
                s[u][t][2 + e] = b;
                sum0 += a;
                sum1 += b;
            }
    st.l[0] = st.l[0] * corr0 + sum0;
    st.l[1] = st.l[1] * corr1 + sum1;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        st.o[nt][0] *= corr0;
        st.o[nt][1] *= corr0;
        st.o[nt][2] *= corr1;
        st.o[nt][3] *= corr1;
    }
    // Four output tiles at a time: their four value loads, then the four products of the keys' first half and the
    // four of the second, so that the two products into one accumulator do not follow each other directly.
    const uint32_t vbase = stage + S::kKeyBytes;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t a0 = pack_bf16(s[u][0][0], s[u][0][1]), a1 = pack_bf16(s[u][0][2], s[u][0][3]);
        const uint32_t a2 = pack_bf16(s[u][1][0], s[u][1][1]), a3 = pack_bf16(s[u][1][2], s[u][1][3]);
        const uint32_t c0 = pack_bf16(s[u][2][0], s[u][2][1]), c1 = pack_bf16(s[u][2][2], s[u][2][3]);
        const uint32_t c2 = pack_bf16(s[u][3][0], s[u][3][1]), c3 = pack_bf16(s[u][3][2], s[u][3][3]);
#pragma unroll
        for (int nt0 = 0; nt0 < D / 8; nt0 += 4) {
            uint4 vv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = 8 * (nt0 + i) + n;
                vv[i] = lds16(vbase + (row * 8 + ((4 * u + j) ^ ((row & 1) << 2))) * 16);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) mma_16816(st.o[nt0 + i], a0, a1, a2, a3, vv[i].x, vv[i].y);
#pragma unroll
            for (int i = 0; i < 4; ++i) mma_16816(st.o[nt0 + i], c0, c1, c2, c3, vv[i].z, vv[i].w);
        }
    }
}

// The decode step's rotation of q and k and the store of the new key and value, done by the attention
// kernel itself instead of a kernel before it (head sizes 64 and 128, where the two members of a
// rotary pair lie in one thread's fragments).  qkv: the step's product [seqs, (heads + 2 kv) * D],
// null = q is given rotated and the cache holds the step's token already.  inv_freq null = no
// rotation.  write_cache 0: the cache holds the step's token already (a run that shares another
// run's lane), only q is taken from qkv.
struct DecodeRope {
    const bf16* qkv;
    const float* inv_freq;
    float magnitude;
    int write_cache;
    bf16* k_out;
    bf16* v_out;
    int early;            // ask for the first pages before waiting for the kernel ahead (cpm_set_decode_early)
};

static int g_decode_early = 1;
CPM_API void cpm_set_decode_early(int on) { g_decode_early = on ? 1 : 0; }

// x' = x cos - y sin, y' = x sin + y cos on the 8 bf16 pairs (x from ``lo``, y from ``hi``), cos and sin
// of the 8 dimensions in cs[], sn[]; rounded to bf16 as the stand-alone rotary kernel does.
__device__ __forceinline__ void rotate8(uint4& lo, uint4& hi, const float (&cs)[8], const float (&sn)[8]) {
    uint32_t a[4] = {lo.x, lo.y, lo.z, lo.w}, b[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a[i]));
        const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b[i]));
        a[i] = pack_bf16(x.x * cs[2 * i] - y.x * sn[2 * i], x.y * cs[2 * i + 1] - y.y * sn[2 * i + 1]);
        b[i] = pack_bf16(x.x * sn[2 * i] + y.x * cs[2 * i], x.y * sn[2 * i + 1] + y.y * cs[2 * i + 1]);
    }
    lo = make_uint4(a[0], a[1], a[2], a[3]);
    hi = make_uint4(b[0], b[1], b[2], b[3]);
}

// The new token's key (rotated) and value into the stage that holds its page (so that this block attends to
// it) and, if ``to_cache``, into the cache pages for later steps.  One warp; row = the token's place in its page.
template <int D>
__device__ __forceinline__ void put_new_token(unsigned char* stage, const bf16* __restrict__ k_raw,
                                              const bf16* __restrict__ v_raw, const float* __restrict__ inv_freq,
                                              float magnitude, int pos, int row, bf16* __restrict__ k_page,
                                              bf16* __restrict__ v_page, bool to_cache, int lane) {
    using S = DecodeSmem<D>;
    constexpr int kHalf = D / 2;
    const int swz = S::kSwizzleKeys ? ((row & 1) << 2) : 0;
    bf16* k_row = reinterpret_cast<bf16*>(stage);
    for (int c = lane; c < kHalf; c += 32) {
        float cs = 1.f, sn = 0.f;
        if (inv_freq) {
            sincosf((float)pos * inv_freq[c], &sn, &cs);
            cs *= magnitude;
            sn *= magnitude;
        }
        const float x = __bfloat162float(k_raw[c]), y = __bfloat162float(k_raw[c + kHalf]);
        const bf16 xr = __float2bfloat16_rn(x * cs - y * sn), yr = __float2bfloat16_rn(x * sn + y * cs);
        const int c2 = c + kHalf;
        k_row[(row * S::kChunksPerKeyRow + ((c >> 3) ^ swz)) * 8 + (c & 7)] = xr;
        k_row[(row * S::kChunksPerKeyRow + ((c2 >> 3) ^ swz)) * 8 + (c2 & 7)] = yr;
        if (to_cache) {
            k_page[row * D + c] = xr;
            k_page[row * D + c2] = yr;
        }
    }
    bf16* v_rows = reinterpret_cast<bf16*>(stage + S::kKeyBytes);
    for (int dd = lane; dd < D; dd += 32) {
        const bf16 v = v_raw[dd];
        v_rows[(dd * 8 + ((row >> 3) ^ ((dd & 1) << 2))) * 8 + (row & 7)] = v;
        if (to_cache) v_page[dd * kPageTokens + row] = v;
    }
}

template <int D>
__global__ void __launch_bounds__(DecodeSmem<D>::kWarps * 32, 1)
decode_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        const int* __restrict__ kv_len, const int* __restrict__ slots,
                        const int* __restrict__ page_table, int max_pages, float* __restrict__ part_o,
                        float* __restrict__ part_ml, bf16* __restrict__ out, int n_heads, int n_kv, int m_tiles,
                        int n_splits, float scale_log2, DecodeRope rope) {
    // A block takes one share of a sequence's pages; its warps take every third page of the
    // share and merge their results in shared memory before anything is written.  With one share
    // per sequence the block writes the final result to ``out`` itself and no combine kernel follows.
    using S = DecodeSmem<D>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float sm_m[DecodeSmem<D>::kWarps][16], sm_l[DecodeSmem<D>::kWarps][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x;
    const int kvh = blockIdx.y / m_tiles, mt = blockIdx.y % m_tiles, b = blockIdx.z;
    const int group = n_heads / n_kv;
    const int j = lane & 3, g = lane >> 2;
    pdl_launch_dependents();
    // Lengths, slots, page numbers and every page but the sequence's last were written by earlier steps (or by the
    // host before this one): they are read, and the first pages asked for, before this kernel waits for the
    // one ahead of it, which writes only the step's own token (into the last page) and q.
    const int len = kv_len[b];
    const int n_pages = (len + kPageTokens - 1) / kPageTokens;
    const int per = (n_pages + n_splits - 1) / n_splits;
    const int p0 = split * per, p1 = min(n_pages, p0 + per);
    const int* pages = page_table + (int64_t)slots[b] * max_pages;
    const uint32_t my_stages = (uint32_t)__cvta_generic_to_shared(smem_raw) + warp * kDecodeStages * S::kStageBytes;
    const int64_t page_elems = (int64_t)n_kv * kPageTokens * D;

    auto issue = [&](int k) {           // the warp's k-th page into stage k % kDecodeStages
        const int p = p0 + warp + k * DecodeSmem<D>::kWarps;
        if (p < p1) {
            const int64_t base = (int64_t)CPM_PAGE(pages, p, max_pages) * page_elems + (int64_t)kvh * kPageTokens * D;
            copy_page_async<D>(my_stages + (k % kDecodeStages) * S::kStageBytes, k_cache + base, v_cache + base, lane);
        }
        cp_async_commit();
    };
    // the warp whose first two pages include the last page waits first (its copies must stay in order)
    const bool early = rope.early && p0 + warp != n_pages - 1 && p0 + warp + DecodeSmem<D>::kWarps != n_pages - 1;
    if (early) {
        issue(0);
        issue(1);
    }
    pdl_wait();
    if (!early) {
        issue(0);
        issue(1);
    }

    TileState<D> st;
    st.init();
    uint4 qf[2][D / 32];
    const int64_t q_row_stride = rope.qkv ? (int64_t)(n_heads + 2 * n_kv) * D : (int64_t)n_heads * D;
    const bf16* q_rows = rope.qkv ? rope.qkv : q;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int local = min(mt * 16 + g + 8 * r, group - 1);      // rows beyond the group repeat a valid head; never stored
        const bf16* qrow = q_rows + (int64_t)b * q_row_stride + (int64_t)(kvh * group + local) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) qf[r][w] = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
    }
    if constexpr (D == 64 || D == 128) {
        if (rope.qkv && rope.inv_freq) {
            // this thread's dims 32w + 8j .. + 7 of the first half pair with the same dims of fragment w + D/64
#pragma unroll
            for (int w = 0; w < D / 64; ++w) {
                float cs[8], sn[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    sincosf((float)(len - 1) * rope.inv_freq[32 * w + 8 * j + e], &sn[e], &cs[e]);
                    cs[e] *= rope.magnitude;
                    sn[e] *= rope.magnitude;
                }
                rotate8(qf[0][w], qf[0][w + D / 64], cs, sn);
                rotate8(qf[1][w], qf[1][w + D / 64], cs, sn);
            }
        }
    }
    for (int k = 0; p0 + warp + k * DecodeSmem<D>::kWarps < p1; ++k) {
        cp_async_wait<kDecodeStages - 1>();
        __syncwarp();
        const int p = p0 + warp + k * DecodeSmem<D>::kWarps;
        if constexpr (D == 64 || D == 128) {
            if (rope.qkv && rope.write_cache && p == n_pages - 1) {
                // the step's own token is not in the cache yet: this warp holds its page and puts it there
                const bf16* raw = rope.qkv + (int64_t)b * q_row_stride + (int64_t)(n_heads + kvh) * D;
                const int64_t base = (int64_t)CPM_PAGE(pages, p, max_pages) * page_elems + (int64_t)kvh * kPageTokens * D;
                put_new_token<D>(smem_raw + (warp * kDecodeStages + (k % kDecodeStages)) * S::kStageBytes, raw,
                                 raw + (int64_t)n_kv * D, rope.inv_freq, rope.magnitude, len - 1, (len - 1) % kPageTokens,
                                 rope.k_out + base, rope.v_out + base, mt == 0, lane);
                __syncwarp();
            }
        }
        attend_page_smem<D>(st, qf, my_stages + (k % kDecodeStages) * S::kStageBytes, p * kPageTokens, len - 1, len - 1,
                            scale_log2, lane);
        __syncwarp();
        issue(k + kDecodeStages);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
    __syncthreads();                                       // every warp is done with its stages: reuse them
    float* sm_o = reinterpret_cast<float*>(smem_raw);      // [warps][16][D + 4]
    constexpr int kLd = D + 4;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g) * kLd + 8 * nt + 2 * j]) = make_float2(st.o[nt][0], st.o[nt][1]);
        *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g + 8) * kLd + 8 * nt + 2 * j]) = make_float2(st.o[nt][2], st.o[nt][3]);
    }
    if (j == 0) {
        sm_m[warp][g] = st.m[0];
        sm_l[warp][g] = st.l[0];
        sm_m[warp][g + 8] = st.m[1];
        sm_l[warp][g + 8] = st.l[1];
    }
    __syncthreads();
    const int64_t unit = (((int64_t)b * n_kv + kvh) * m_tiles + mt) * n_splits + split;
    float* po = part_o + unit * 16 * D;
    for (int i = threadIdx.x; i < 16 * D; i += DecodeSmem<D>::kWarps * 32) {
        const int row = i / D, c = i - row * D;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < DecodeSmem<D>::kWarps; ++w) mx = fmaxf(mx, sm_m[w][row]);
        const float use = mx == -INFINITY ? 0.f : mx;
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < DecodeSmem<D>::kWarps; ++w) {
            const float f = exp2f(sm_m[w][row] - use);
            o += sm_o[(w * 16 + row) * kLd + c] * f;
            l += sm_l[w][row] * f;
        }
        if (n_splits == 1) {
            const int local = mt * 16 + row;
            if (local < group)
                out[((int64_t)b * n_heads + kvh * group + local) * D + c] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
            continue;
        }
        po[i] = o;
        if (c == 0) {
            part_ml[unit * 32 + 2 * row] = mx;
            part_ml[unit * 32 + 2 * row + 1] = l;
        }
    }
}

// out[b, h, :] = sum_s o_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
__global__ void combine_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      bf16* __restrict__ out, int n_heads, int n_kv, int m_tiles, int n_splits,
                                      int D) {
    pdl_launch_dependents();
    pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const int group = n_heads / n_kv;
    const int kvh = h / group, local = h % group;
    const int mt = local / 16, row = local % 16;
    const int64_t unit0 = (((int64_t)b * n_kv + kvh) * m_tiles + mt) * n_splits;
    float mx = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, part_ml[(unit0 + s) * 32 + 2 * row]);
    float denom = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float m = part_ml[(unit0 + s) * 32 + 2 * row];
        if (m != -INFINITY) denom += part_ml[(unit0 + s) * 32 + 2 * row + 1] * exp2f(m - mx);
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float m = part_ml[(unit0 + s) * 32 + 2 * row];
            if (m != -INFINITY) acc += part_o[((unit0 + s) * 16 + row) * D + c] * exp2f(m - mx);
        }
        out[((int64_t)b * n_heads + h) * D + c] = __float2bfloat16_rn(acc * inv);
    }
}

// Floats of scratch the decode kernels need for these sizes.
CPM_API int64_t cpm_decode_attention_scratch_floats(int n_seqs, int n_heads, int n_kv, int d, int n_splits) {
    const int m_tiles = (n_heads / n_kv + 15) / 16;
    return (int64_t)n_seqs * n_kv * m_tiles * n_splits * (16 * d + 32);
}

template <int D>
static int launch_decode(const void* q, const void* k_cache, const void* v_cache, void* out, const int* kv_len,
                         const int* slots, const int* page_table, int max_pages, float* scratch, int n_seqs,
                         int n_heads, int n_kv, int n_splits, float scale, cudaStream_t stream,
                         DecodeRope rope = DecodeRope{nullptr, nullptr, 1.f, 0, nullptr, nullptr, 0}) {
    const int m_tiles = (n_heads / n_kv + 15) / 16;
    float* part_o = scratch;
    float* part_ml = scratch + (int64_t)n_seqs * n_kv * m_tiles * n_splits * 16 * D;
    dim3 grid(n_splits, n_kv * m_tiles, n_seqs);
    auto kern = decode_attention_kernel<D>;
    rope.early = g_decode_early;
    constexpr int smem = DecodeSmem<D>::kTotal;
    static bool configured[kMaxDevices] = {};            // per kernel and per device
    if (int st = ensure_dynamic_smem(kern, smem, configured)) return st;
    cpm_launch(kLaunchAttention, kern, grid, DecodeSmem<D>::kWarps * 32, smem, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
               kv_len, slots, page_table, max_pages, part_o, part_ml, (bf16*)out, n_heads, n_kv, m_tiles, n_splits,
               scale * 1.4426950408889634f, rope);
    if (n_splits > 1)
        cpm_launch(kLaunchCombine, combine_splits_kernel, dim3(n_heads, n_seqs), D >= 128 ? 128 : 64, 0, stream, (const float*)part_o,
                   (const float*)part_ml, (bf16*)out, n_heads, n_kv, m_tiles, n_splits, (int)D);
    return launch_status();
}

// q [n_seqs, heads, d] bf16, one token per sequence; out [n_seqs, heads, d] bf16.
CPM_API int cpm_decode_attention_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int* kv_len, const int* slots, const int* page_table, int max_pages,
                                      float* scratch, int n_seqs, int n_heads, int n_kv, int d, int n_splits,
                                      float scale, cudaStream_t stream) {
    if (n_seqs <= 0) return CPM_OK;
    if (n_kv <= 0 || n_heads % n_kv || n_splits < 1 || n_seqs > 65535 || !scratch) return CPM_BAD_ARGUMENT;
    switch (d) {
        case 32: return launch_decode<32>(q, k_cache, v_cache, out, kv_len, slots, page_table, max_pages, scratch, n_seqs, n_heads, n_kv, n_splits, scale, stream);
        case 64: return launch_decode<64>(q, k_cache, v_cache, out, kv_len, slots, page_table, max_pages, scratch, n_seqs, n_heads, n_kv, n_splits, scale, stream);
        case 96: return launch_decode<96>(q, k_cache, v_cache, out, kv_len, slots, page_table, max_pages, scratch, n_seqs, n_heads, n_kv, n_splits, scale, stream);
        case 128: return launch_decode<128>(q, k_cache, v_cache, out, kv_len, slots, page_table, max_pages, scratch, n_seqs, n_heads, n_kv, n_splits, scale, stream);
        default: return CPM_BAD_ARGUMENT;
    }
}

// The same with the step's rotation and cache store done inside (see DecodeRope): qkv [n_seqs, (heads + 2 kv) * d]
// is the step's fused product, positions are kv_len - 1, the cache pages of the step's tokens are written here.
// Head sizes 64 and 128 only.
CPM_API int cpm_decode_attention_rope_bf16(const void* qkv, void* k_cache, void* v_cache, void* out,
                                           const int* kv_len, const int* slots, const int* page_table, int max_pages,
                                           float* scratch, int n_seqs, int n_heads, int n_kv, int d, int n_splits,
                                           float scale, const float* inv_freq, float magnitude, int write_cache,
                                           cudaStream_t stream) {
    if (n_seqs <= 0) return CPM_OK;
    if (n_kv <= 0 || n_heads % n_kv || n_splits < 1 || n_seqs > 65535 || !scratch || !qkv) return CPM_BAD_ARGUMENT;
    const DecodeRope rope{(const bf16*)qkv, inv_freq, magnitude, write_cache, (bf16*)k_cache, (bf16*)v_cache, 0};
    switch (d) {
        case 64: return launch_decode<64>(nullptr, k_cache, v_cache, out, kv_len, slots, page_table, max_pages, scratch, n_seqs, n_heads, n_kv, n_splits, scale, stream, rope);
        case 128: return launch_decode<128>(nullptr, k_cache, v_cache, out, kv_len, slots, page_table, max_pages, scratch, n_seqs, n_heads, n_kv, n_splits, scale, stream, rope);
        default: return CPM_BAD_ARGUMENT;
    }
}

// ---------------------------------------------------------------------------
// attention over listed key blocks (block-sparse), one block of warps per (token, kv head)
// ---------------------------------------------------------------------------
// The 16 rows are the query heads of the token that share the kv head, as in decode; the key
// pages are those the token's block list names (selected by cpm_select_blocks), or all pages up
// to the token when the list says "dense" (first entry -2).  Serves block-sparse prefill and
// decode when the sparse block is a page (64 tokens).  The reference's counterpart is its
// block-mask flash kernel with 16-head tiles (src/flash_attn/src/flash_fwd_kernel.h:580-1170,
// src/flash_attn/src/flash_blockmask.h:5-109).
template <int D>
__global__ void __launch_bounds__(DecodeSmem<D>::kWarps * 32, 1)
listed_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        bf16* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ token_seq,
                        const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                        const int* __restrict__ block_list, int list_cap, int n_heads, int n_kv, int m_tiles,
                        float scale_log2, float* __restrict__ part_o, float* __restrict__ part_ml, int n_splits) {
    // With n_splits > 1 (few tokens: decode) the listed blocks of a token are shared out over
    // gridDim.z blocks of threads, which write unnormalised partial results for combine_splits_kernel.
    using S = DecodeSmem<D>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float sm_m[DecodeSmem<D>::kWarps][16], sm_l[DecodeSmem<D>::kWarps][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int kvh = blockIdx.y / m_tiles, mt = blockIdx.y % m_tiles;
    const int group = n_heads / n_kv;
    const int j = lane & 3, g = lane >> 2;
    pdl_launch_dependents();
    pdl_wait();
    const int p = positions[t];
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int* list = block_list + ((int64_t)t * n_kv + kvh) * list_cap;
    const bool dense = list[0] == -2;
    int n_items = 0;
    if (dense) n_items = p / kPageTokens + 1;
    else while (n_items < list_cap && list[n_items] >= 0) ++n_items;
    const int per_split = (n_items + n_splits - 1) / n_splits;
    const int item0 = blockIdx.z * per_split;
    n_items = min(n_items, item0 + per_split);
    const uint32_t my_stages = (uint32_t)__cvta_generic_to_shared(smem_raw) + warp * kDecodeStages * S::kStageBytes;
    const int64_t page_elems = (int64_t)n_kv * kPageTokens * D;

    auto block_of = [&](int k) { const int i = item0 + warp + k * DecodeSmem<D>::kWarps; return dense ? i : list[i]; };
    auto issue = [&](int k) {
        if (item0 + warp + k * DecodeSmem<D>::kWarps < n_items) {
            const int64_t base = (int64_t)CPM_PAGE(pages, block_of(k), max_pages) * page_elems + (int64_t)kvh * kPageTokens * D;
            copy_page_async<D>(my_stages + (k % kDecodeStages) * S::kStageBytes, k_cache + base, v_cache + base, lane);
        }
        cp_async_commit();
    };
    issue(0);
    issue(1);

    TileState<D> st;
    st.init();
    uint4 qf[2][D / 32];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int local = min(mt * 16 + g + 8 * r, group - 1);
        const bf16* qrow = q + ((int64_t)t * n_heads + kvh * group + local) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) qf[r][w] = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
    }
    for (int k = 0; item0 + warp + k * DecodeSmem<D>::kWarps < n_items; ++k) {
        cp_async_wait<kDecodeStages - 1>();
        __syncwarp();
        attend_page_smem<D>(st, qf, my_stages + (k % kDecodeStages) * S::kStageBytes, block_of(k) * kPageTokens, p, p,
                            scale_log2, lane);
        __syncwarp();
        issue(k + kDecodeStages);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
    __syncthreads();
    float* sm_o = reinterpret_cast<float*>(smem_raw);
    constexpr int kLd = D + 4;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
        *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g) * kLd + 8 * nt + 2 * j]) = make_float2(st.o[nt][0], st.o[nt][1]);
        *reinterpret_cast<float2*>(&sm_o[(warp * 16 + g + 8) * kLd + 8 * nt + 2 * j]) = make_float2(st.o[nt][2], st.o[nt][3]);
    }
    if (j == 0) {
        sm_m[warp][g] = st.m[0];
        sm_l[warp][g] = st.l[0];
        sm_m[warp][g + 8] = st.m[1];
        sm_l[warp][g + 8] = st.l[1];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * D; i += DecodeSmem<D>::kWarps * 32) {
        const int row = i / D, c = i - row * D;
        const int local = mt * 16 + row;
        if (local >= group) continue;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < DecodeSmem<D>::kWarps; ++w) mx = fmaxf(mx, sm_m[w][row]);
        const float use = mx == -INFINITY ? 0.f : mx;
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < DecodeSmem<D>::kWarps; ++w) {
            const float f = exp2f(sm_m[w][row] - use);
            o += sm_o[(w * 16 + row) * kLd + c] * f;
            l += sm_l[w][row] * f;
        }
        if (n_splits == 1) {
            out[((int64_t)t * n_heads + kvh * group + local) * D + c] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
        } else {
            const int64_t unit = (((int64_t)t * n_kv + kvh) * m_tiles + mt) * n_splits + blockIdx.z;
            part_o[(unit * 16 + row) * D + c] = o;
            if (c == 0) {
                part_ml[unit * 32 + 2 * row] = mx;
                part_ml[unit * 32 + 2 * row + 1] = l;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// attention over listed key blocks for the many tokens of a prompt chunk: a block of threads takes seven
// consecutive tokens, one per warp, and an eighth warp brings the key blocks
// ---------------------------------------------------------------------------
// The kernel above has every token bring its own 96 blocks from L2: 12.9 GB per layer and 2,048-token chunk
// of the 8B sizes, which is what bounds it.  Consecutive tokens of a prompt share the local window and the
// leading blocks and part of the rest, so here the tokens of a tile share what is brought: every warp marks
// its token's blocks in a bit mask, the union of the masks is walked in rising order, the producer warp
// copies each of its blocks once into a ring of shared-memory stages, and a token's warp attends to the
// blocks its token listed and passes over the others.  The warps meet only through the ring's barriers
// (full: the copies of a stage have landed; empty: all seven warps are done with it), so a warp that has
// nothing to do with a block runs ahead by up to the ring's length instead of waiting for the others at
// every block (with one barrier of all warps per block the warps idled 45 % of the steps on random data,
// where the union of seven lists is 175 blocks).  A tile whose tokens belong to several sequences (packed
// prompts) is done in passes, one per sequence.  Rows, masking and arithmetic are those of the kernel above.
// Every wait is bounded; a wait that runs out raises the block's abort flag, which ends the others' waits.
constexpr int kTileTokens = 7;
constexpr int kTileWarps = kTileTokens + 1;
constexpr int kTileStages = 6;
constexpr uint32_t kTileSpinLimit = 1u << 22;

__device__ int g_listed_tile_error = 0;

struct BlockCursor {            // walks the set bits of a mask in rising order
    int word;
    unsigned bits;
};
__device__ __forceinline__ int next_block(BlockCursor& c, const unsigned* __restrict__ mask, int words) {
    while (c.bits == 0u) {
        if (++c.word >= words) return -1;
        c.bits = mask[c.word];
    }
    const int b = __ffs(c.bits) - 1;
    c.bits &= c.bits - 1u;
    return c.word * 32 + b;
}

__device__ __forceinline__ void tile_bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tile_bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
// The barrier gets this thread's arrival when all its earlier cp.async copies have landed.
__device__ __forceinline__ void tile_bar_arrive_after_copies(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" :: "r"(bar) : "memory");
}
// Waits for the phase of this parity; false when the tries ran out or another warp gave up.
__device__ __forceinline__ bool tile_bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kTileSpinLimit; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}

template <int D>
__global__ void __launch_bounds__(kTileWarps * 32, 1)
listed_tile_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                   bf16* __restrict__ out, const int* __restrict__ positions, const int* __restrict__ token_seq,
                   const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                   const int* __restrict__ block_list, int list_cap, int n_tokens, int n_heads, int n_kv, int m_tiles,
                   float scale_log2, int words) {
    using S = DecodeSmem<D>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kTileStages], empty_bar[kTileStages];
    __shared__ int abort_flag;
    unsigned* all = reinterpret_cast<unsigned*>(smem_raw + kTileStages * S::kStageBytes);      // [words] the union
    unsigned* mine = all + words;                                                               // [tokens][words]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool producer = warp == kTileTokens;
    const int t0 = blockIdx.x * kTileTokens, t = t0 + warp;
    const int kvh = blockIdx.y / m_tiles, mt = blockIdx.y % m_tiles;
    const int group = n_heads / n_kv;
    const int j = lane & 3, g = lane >> 2;
    const uint32_t stages = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const int64_t page_elems = (int64_t)n_kv * kPageTokens * D;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTileStages; ++s) {
            tile_bar_init((uint32_t)__cvta_generic_to_shared(&full_bar[s]), 32);            // the producer's lanes
            tile_bar_init((uint32_t)__cvta_generic_to_shared(&empty_bar[s]), kTileTokens);  // one arrival per token's warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    pdl_launch_dependents();
    pdl_wait();
    const bool live = !producer && t < n_tokens;
    const int p = live ? positions[t] : 0;
    const int* list = block_list + ((int64_t)(live ? t : 0) * n_kv + kvh) * list_cap;

    TileState<D> st;
    st.init();
    uint4 qf[2][D / 32];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int local = min(mt * 16 + g + 8 * r, group - 1);
        const bf16* qrow = q + ((int64_t)(live ? t : 0) * n_heads + kvh * group + local) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) qf[r][w] = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
    }

    const int tile_tokens = min(kTileTokens, n_tokens - t0);
    uint32_t it = 0;                                            // blocks that have gone through the ring, all passes
    bool ok = true;
    for (int first = 0; first < tile_tokens;) {                // one pass per sequence in the tile
        const int seq = token_seq[t0 + first];
        int end = first + 1;
        while (end < tile_tokens && token_seq[t0 + end] == seq) ++end;
        const bool member = !producer && warp >= first && warp < end;
        const int* pages = page_table + (int64_t)slots[seq] * max_pages;
        // ---- the tokens' masks and their union ----
        for (int i = threadIdx.x; i < (kTileTokens + 1) * words; i += kTileWarps * 32) all[i] = 0u;
        __syncthreads();
        if (member) {
            unsigned* m = mine + warp * words;
            if (list[0] == -2) {                                // "dense": every block up to the token's own
                const int last = p / kPageTokens;
                for (int w = lane; w <= (last >> 5) && w < words; w += 32)
                    m[w] = w < (last >> 5) ? 0xffffffffu : (0xffffffffu >> (31 - (last & 31)));
            } else {
                for (int base = 0; base < list_cap; base += 32) {      // the list ends at its first negative entry;
                    const int i = base + lane;                          // what lies behind it is not the list's
                    const int b = i < list_cap ? list[i] : -1;
                    const unsigned ended = __ballot_sync(0xffffffffu, b < 0);
                    const int n_valid = ended ? __ffs(ended) - 1 : 32;
                    if (lane < n_valid && (b >> 5) < words) atomicOr(&m[b >> 5], 1u << (b & 31));
                    if (ended) break;
                }
            }
        }
        __syncthreads();
        for (int w = threadIdx.x; w < words; w += kTileWarps * 32) {
            unsigned u = 0u;
            for (int k = first; k < end; ++k) u |= mine[k * words + w];
            all[w] = u;
        }
        __syncthreads();
        // ---- the union's blocks through the ring ----
        ok = ok && !*(volatile int*)&abort_flag;
        BlockCursor cursor{-1, 0u};
        if (producer) {
            for (int b = ok ? next_block(cursor, all, words) : -1; b >= 0; b = next_block(cursor, all, words), ++it) {
                const uint32_t s = it % kTileStages, use = it / kTileStages;
                if (use > 0 && !tile_bar_wait((uint32_t)__cvta_generic_to_shared(&empty_bar[s]), (use - 1) & 1u, &abort_flag)) {
                    ok = false;
                    break;
                }
                const int64_t base = (int64_t)CPM_PAGE(pages, b, max_pages) * page_elems + (int64_t)kvh * kPageTokens * D;
                copy_page_async<D, 32>(stages + s * S::kStageBytes, k_cache + base, v_cache + base, lane);
                tile_bar_arrive_after_copies((uint32_t)__cvta_generic_to_shared(&full_bar[s]));
            }
        } else {
            const unsigned* my_mask = mine + warp * words;
            for (int b = ok ? next_block(cursor, all, words) : -1; b >= 0; b = next_block(cursor, all, words), ++it) {
                const uint32_t s = it % kTileStages, use = it / kTileStages;
                if (!tile_bar_wait((uint32_t)__cvta_generic_to_shared(&full_bar[s]), use & 1u, &abort_flag)) {
                    ok = false;
                    break;
                }
                if (member && ((my_mask[b >> 5] >> (b & 31)) & 1u))
                    attend_page_smem<D>(st, qf, stages + s * S::kStageBytes, b * kPageTokens, p, p, scale_log2, lane);
                __syncwarp();
                if (lane == 0) tile_bar_arrive((uint32_t)__cvta_generic_to_shared(&empty_bar[s]));
            }
        }
        if (!ok) {                                              // a wait ran out: say so, and end the others' waits
            atomicExch(&abort_flag, 1);
            atomicCAS(&g_listed_tile_error, 0, 1);
        }
        asm volatile("cp.async.wait_all;\n" ::: "memory");     // the producer's copies, before its stages are given up or reused
        __syncthreads();                                        // the masks are free for the next pass
        if (*(volatile int*)&abort_flag) return;
        // both kinds of warp have counted the same blocks; a warp that broke off has left through the line above
        first = end;
    }
    if (!live) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int local = mt * 16 + g + 8 * r;
        if (local >= group) continue;
        const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
        bf16* orow = out + ((int64_t)t * n_heads + kvh * group + local) * D + 2 * j;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt)
            *reinterpret_cast<__nv_bfloat162*>(orow + 8 * nt) =
                __floats2bfloat162_rn(st.o[nt][2 * r] * inv, st.o[nt][2 * r + 1] * inv);
    }
}

// 1 when a wait inside listed_tile_kernel ran out since the last call (and reset).  Synchronises the device.
CPM_API int cpm_listed_tile_error() {
    int code = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&code, g_listed_tile_error, sizeof(int)) != cudaSuccess) return -1;
    if (code) cudaMemcpyToSymbol(g_listed_tile_error, &zero, sizeof(int));
    return code;
}

template <int D>
static int launch_listed(const void* q, const void* k_cache, const void* v_cache, void* out, const int* positions,
                         const int* token_seq, const int* slots, const int* page_table, int max_pages,
                         const int* block_list, int list_cap, int n_tokens, int n_heads, int n_kv, float scale,
                         float* scratch, int n_splits, bool tiles, cudaStream_t stream) {
    const int m_tiles = (n_heads / n_kv + 15) / 16;
    // (a page table too wide for the masks to fit beside the ring: the kernel of one token per block)
    if (tiles && kTileStages * DecodeSmem<D>::kStageBytes + (kTileTokens + 1) * ((max_pages + 31) / 32) * 4 <= 227 * 1024 - 256) {
        const int words = (max_pages + 31) / 32;
        const int smem = kTileStages * DecodeSmem<D>::kStageBytes + (kTileTokens + 1) * words * 4;
        auto kern = listed_tile_kernel<D>;
        static bool configured[kMaxDevices] = {};
        if (int st = ensure_dynamic_smem(kern, 227 * 1024 - 256, configured)) return st;       // less the kernel's static part
        cpm_launch(kLaunchAttention, kern, dim3((n_tokens + kTileTokens - 1) / kTileTokens, n_kv * m_tiles), kTileWarps * 32,
                   (size_t)smem, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions,
                   token_seq, slots, page_table, max_pages, block_list, list_cap, n_tokens, n_heads, n_kv, m_tiles,
                   scale * 1.4426950408889634f, words);
        return launch_status();
    }
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (int64_t)n_tokens * n_kv * m_tiles * n_splits * 16 * D : nullptr;
    auto kern = listed_attention_kernel<D>;
    constexpr int smem = DecodeSmem<D>::kTotal;
    static bool configured[kMaxDevices] = {};            // per kernel and per device
    if (int st = ensure_dynamic_smem(kern, smem, configured)) return st;
    cpm_launch(kLaunchAttention, kern, dim3(n_tokens, n_kv * m_tiles, n_splits), DecodeSmem<D>::kWarps * 32, smem, stream, (const bf16*)q,
               (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, positions, token_seq, slots, page_table, max_pages,
               block_list, list_cap, n_heads, n_kv, m_tiles, scale * 1.4426950408889634f, part_o, part_ml, n_splits);
    if (n_splits > 1)
        combine_splits_kernel<<<dim3(n_heads, n_tokens), D >= 128 ? 128 : 64, 0, stream>>>(part_o, part_ml, (bf16*)out, n_heads,
                                                                                    n_kv, m_tiles, n_splits, D);
    return launch_status();
}

// q, out [tokens, heads, d] bf16; block_list int32 [tokens, kv_heads, list_cap] of 64-token blocks.
// tiles != 0 (n_splits 1 only): the tokens are those of prompts, consecutive ones mostly of one sequence; seven of
// them share the blocks that are brought (listed_tile_kernel).
CPM_API int cpm_listed_attention_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      const int* positions, const int* token_seq, const int* slots,
                                      const int* page_table, int max_pages, const int* block_list, int list_cap,
                                      int n_tokens, int n_heads, int n_kv, int d, float scale, float* scratch,
                                      int n_splits, int tiles, cudaStream_t stream) {
    // scratch: cpm_decode_attention_scratch_floats(n_tokens, ...) floats when n_splits > 1, else unused
    if (n_tokens <= 0) return CPM_OK;
    if (n_kv <= 0 || n_heads % n_kv || !block_list || list_cap < 1 || n_kv * ((n_heads / n_kv + 15) / 16) > 65535 ||
        n_splits < 1 || n_splits > 65535 || (n_splits > 1 && (!scratch || n_tokens > 65535)) || (tiles && n_splits != 1))
        return CPM_BAD_ARGUMENT;
    const bool tl = tiles != 0;
    switch (d) {
        case 32: return launch_listed<32>(q, k_cache, v_cache, out, positions, token_seq, slots, page_table, max_pages, block_list, list_cap, n_tokens, n_heads, n_kv, scale, scratch, n_splits, tl, stream);
        case 64: return launch_listed<64>(q, k_cache, v_cache, out, positions, token_seq, slots, page_table, max_pages, block_list, list_cap, n_tokens, n_heads, n_kv, scale, scratch, n_splits, tl, stream);
        case 96: return launch_listed<96>(q, k_cache, v_cache, out, positions, token_seq, slots, page_table, max_pages, block_list, list_cap, n_tokens, n_heads, n_kv, scale, scratch, n_splits, tl, stream);
        case 128: return launch_listed<128>(q, k_cache, v_cache, out, positions, token_seq, slots, page_table, max_pages, block_list, list_cap, n_tokens, n_heads, n_kv, scale, scratch, n_splits, tl, stream);
        default: return CPM_BAD_ARGUMENT;
    }
}

// ---------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------
// A block of 4 warps takes 64 consecutive query tokens of one sequence and one head, 16 per
// warp; tile_seq/tile_row name the sequence (index in the batch) and the first of the 64
// tokens (offset inside this step's tokens of the sequence) of every block.  The block walks
// over the key pages up to its last token; a page is brought into shared memory once
// (cp.async, two pages in flight) and read by all 4 warps.  Two blocks share an SM (measured
// faster than one block of 8 warps or three of 4).
constexpr int kPrefillWarps = 4;
constexpr int kPrefillRows = kPrefillWarps * 16;

template <int D>
__global__ void __launch_bounds__(kPrefillWarps * 32, 2)
prefill_attention_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                         bf16* __restrict__ out, const int* __restrict__ tile_seq, const int* __restrict__ tile_row,
                         const int* __restrict__ cu_q, const int* __restrict__ kv_len, const int* __restrict__ slots,
                         const int* __restrict__ page_table, int max_pages, int n_heads, int n_kv, float scale_log2) {
    using S = DecodeSmem<D>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t stages = (uint32_t)__cvta_generic_to_shared(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = lane & 3, g = lane >> 2;
    const int tile = gridDim.y - 1 - blockIdx.y;                 // later tiles of a sequence are longer: they go first
    const int seq = tile_seq[tile], h = blockIdx.x;
    const int kvh = h / (n_heads / n_kv);
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int tile_row0 = tile_row[tile];
    const int row0 = tile_row0 + 16 * warp;                      // first of this warp's 16 tokens
    const int history = kv_len[seq] - q_len;                     // keys cached before this step's tokens
    const int* pages = page_table + (int64_t)slots[seq] * max_pages;
    const int64_t page_elems = (int64_t)n_kv * kPageTokens * D;
    const int last_page = (history + min(tile_row0 + kPrefillRows, q_len) - 1) / kPageTokens;    // of the block
    const int my_last_page = row0 < q_len ? (history + min(row0 + 16, q_len) - 1) / kPageTokens : -1;

    auto issue = [&](int p) {
        if (p <= last_page) {
            const int64_t base = (int64_t)CPM_PAGE(pages, p, max_pages) * page_elems + (int64_t)kvh * kPageTokens * D;
            copy_page_async<D, kPrefillWarps * 32>(stages + (p & 1) * S::kStageBytes, k_cache + base, v_cache + base,
                                                   threadIdx.x);
        }
        cp_async_commit();
    };
    issue(0);
    issue(1);

    uint4 qf[2][D / 32];
    int limit[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + g + 8 * r;
        const bool valid = row < q_len;
        limit[r] = valid ? history + row : -1;
        const bf16* qrow = q + ((int64_t)(q_begin + (valid ? row : 0)) * n_heads + h) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) qf[r][w] = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
    }
    TileState<D> st;
    st.init();
    for (int p = 0; p <= last_page; ++p) {
        cp_async_wait<1>();
        __syncthreads();
        if (p <= my_last_page)
            attend_page_smem<D>(st, qf, stages + (p & 1) * S::kStageBytes, p * kPageTokens, limit[0], limit[1], scale_log2, lane);
        __syncthreads();
        issue(p + 2);
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 1);
        st.l[r] += __shfl_xor_sync(0xffffffffu, st.l[r], 2);
        const int row = row0 + g + 8 * r;
        if (row >= q_len) continue;
        const float inv = st.l[r] > 0.f ? 1.f / st.l[r] : 0.f;
        bf16* orow = out + ((int64_t)(q_begin + row) * n_heads + h) * D + 2 * j;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt)
            *reinterpret_cast<uint32_t*>(orow + 8 * nt) = pack_bf16(st.o[nt][2 * r] * inv, st.o[nt][2 * r + 1] * inv);
    }
}

// Query tokens per block of the prefill kernel (the tile lists are made for this size).
CPM_API int cpm_prefill_attention_tile_rows() { return kPrefillRows; }

template <int D>
static int launch_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq,
                          const int* tile_row, int n_tiles, const int* cu_q, const int* kv_len, const int* slots,
                          const int* page_table, int max_pages, int n_heads, int n_kv, float scale,
                          cudaStream_t stream) {
    auto kern = prefill_attention_kernel<D>;
    constexpr int smem = 2 * DecodeSmem<D>::kStageBytes;
    static bool configured[kMaxDevices] = {};            // per kernel and per device
    if (int st = ensure_dynamic_smem(kern, smem, configured)) return st;
    kern<<<dim3(n_heads, n_tiles), kPrefillWarps * 32, smem, stream>>>((const bf16*)q, (const bf16*)k_cache,
        (const bf16*)v_cache, (bf16*)out, tile_seq, tile_row, cu_q, kv_len, slots, page_table, max_pages, n_heads, n_kv,
        scale * 1.4426950408889634f);
    return launch_status();
}

// q, out [tokens, heads, d] bf16, tokens packed by sequence (cu_q); the cache already holds this step's keys.
CPM_API int cpm_prefill_attention_bf16(const void* q, const void* k_cache, const void* v_cache, void* out,
                                       const int* tile_seq, const int* tile_row, int n_tiles, const int* cu_q,
                                       const int* kv_len, const int* slots, const int* page_table, int max_pages,
                                       int n_heads, int n_kv, int d, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return CPM_OK;
    if (n_kv <= 0 || n_heads % n_kv || n_tiles > 65535) return CPM_BAD_ARGUMENT;
    switch (d) {
        case 32: return launch_prefill<32>(q, k_cache, v_cache, out, tile_seq, tile_row, n_tiles, cu_q, kv_len, slots, page_table, max_pages, n_heads, n_kv, scale, stream);
        case 64: return launch_prefill<64>(q, k_cache, v_cache, out, tile_seq, tile_row, n_tiles, cu_q, kv_len, slots, page_table, max_pages, n_heads, n_kv, scale, stream);
        case 96: return launch_prefill<96>(q, k_cache, v_cache, out, tile_seq, tile_row, n_tiles, cu_q, kv_len, slots, page_table, max_pages, n_heads, n_kv, scale, stream);
        case 128: return launch_prefill<128>(q, k_cache, v_cache, out, tile_seq, tile_row, n_tiles, cu_q, kv_len, slots, page_table, max_pages, n_heads, n_kv, scale, stream);
        default: return CPM_BAD_ARGUMENT;
    }
}

// ---------------------------------------------------------------------------
// The decode attention with scratch memory of its own (see cpm_no_alloc.h).
// ---------------------------------------------------------------------------
#include "cpm_no_alloc.h"
#include <mutex>
#include <stdio.h>

// Partial results of the split-key decode kernel.  In host code this name is only a
// stand-in for the symbol, never a device address: the address each device gives it is
// looked up below and that pointer is what the kernels get.
static __device__ __align__(256) float g_static_scratch[CPM_STATIC_SCRATCH_FLOATS];

static float* g_static_scratch_ptr[kMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mutex;

// Device address of g_static_scratch on the current device, looked up once per device.
static int static_scratch_for_current_device(float** out, char* error_text, int error_text_len) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        if (error_text && error_text_len > 0)
            snprintf(error_text, error_text_len, "cannot tell the current device (cudaGetDevice: %s, device %d)",
                     cudaGetErrorString(e), dev);
        return CPM_STATIC_SETUP_FAILED;
    }
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            if (error_text && error_text_len > 0)
                snprintf(error_text, error_text_len, "cudaGetSymbolAddress of the static scratch failed on device %d: %s",
                         dev, cudaGetErrorString(e));
            return CPM_STATIC_SETUP_FAILED;
        }
        g_static_scratch_ptr[dev] = p;
    }
    *out = g_static_scratch_ptr[dev];
    return CPM_OK;
}

int cpm_decode_attention_bf16_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int* kv_len, const int* slots, const int* page_table, int max_pages,
                                     int n_seqs, int n_heads, int n_kv, int d, int n_splits, float scale,
                                     cudaStream_t stream, char* error_text, int error_text_len) {
    if (error_text && error_text_len > 0) error_text[0] = 0;
    if (n_seqs <= 0) return CPM_OK;
    if (n_kv <= 0 || n_heads <= 0 || n_heads % n_kv || n_splits < 1 || (d != 32 && d != 64 && d != 96 && d != 128)) {
        if (error_text && error_text_len > 0)
            snprintf(error_text, error_text_len, "sizes not taken: heads %d, kv heads %d, head_dim %d (32/64/96/128), "
                     "splits %d", n_heads, n_kv, d, n_splits);
        return CPM_BAD_ARGUMENT;
    }
    const int64_t need = cpm_decode_attention_scratch_floats(n_seqs, n_heads, n_kv, d, n_splits);
    if (need > (int64_t)CPM_STATIC_SCRATCH_FLOATS) {
        if (error_text && error_text_len > 0)
            snprintf(error_text, error_text_len, "these sizes need %lld floats of scratch, the static scratch holds %d: "
                     "use fewer splits or sequences, or cpm_decode_attention_bf16 with scratch of your own",
                     (long long)need, (int)CPM_STATIC_SCRATCH_FLOATS);
        return CPM_STATIC_TOO_LARGE;
    }
    float* scratch = nullptr;
    const int status = static_scratch_for_current_device(&scratch, error_text, error_text_len);
    if (status != CPM_OK) return status;
    return cpm_decode_attention_bf16(q, k_cache, v_cache, out, kv_len, slots, page_table, max_pages, scratch, n_seqs,
                                     n_heads, n_kv, d, n_splits, scale, stream);
}

CPM_BOUNDS_TU(attention_bf16)
