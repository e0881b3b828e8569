// Causal attention of prompt tokens over the paged cache for head sizes 128 and 64, on the fifth-generation
// tensor cores: S = Q K^T and O += P V are tcgen05.mma with the accumulators in tensor memory (TMEM),
// Q, K and V tiles come by TMA straight from the query matrix and from the cache pages, and the softmax
// works on the rows of S that it reads from TMEM, one thread per row.
//
// A block takes 128 query tokens of two heads that share a key/value head, so that the tensor cores work
// on one head's products while the other head's rows are in the softmax ("ping-pong"), and both heads use
// the same K and V tiles in shared memory.  Keys come 128 at a time (two cache pages).  A key page
// [64 keys][128] is, as it lies in the cache, the K-major B operand of Q K^T; a value page is stored
// transposed, [head size][64 keys], which is the K-major B operand of P V.  P never goes through shared
// memory: the softmax threads write it as bf16 over the first 64 columns of the S they have just read,
// and the second product takes its A operand from TMEM.
//
// Warps 0-3 and 4-7 are the softmax of head 0 and head 1 (a warp reads TMEM lanes 32 * (warp % 4) ...),
// warp 8 allocates TMEM and issues every MMA from one thread, warp 9 is the TMA producer.  TMEM columns
// (head size 128): S0 0-127, S1 128-255, O0 256-383, O1 384-511.  The running maximum of a row is only raised when the new
// maximum exceeds it by more than 8 (in log2 units), in which case the thread rescales its row of O in
// TMEM; between the products of one head nothing else touches that head's O, because the barrier that
// announces S(j) is raised by a tcgen05.commit that also covers the earlier P V product.
//
// The reference uses its vendored flash-attention kernels (mma.sync) for this step
// (src/flash_attn/flash_api.hpp, src/model/attn.cuh:137-170).
//
// Every barrier wait is bounded; a block that runs out of patience records an error code, stops,
// waits (bounded) for its copies in flight, frees its TMEM and returns.
#include "tcgen05.cuh"

namespace fa5 {
using namespace tc5;

constexpr int kTileRows = 128;                   // query tokens of a block
constexpr int kBlockKeys = 128;                  // keys per step: two cache pages
constexpr int kHalfBytes = 128 * 64 * 2;         // 128 rows x 128 bytes, one swizzle atom wide: 16 KiB
constexpr int kKvStages = 2;
constexpr int kThreads = 320;
constexpr int kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;

// Sizes that depend on the head size D (64 or 128).  A Q tile and a K tile of 128 keys are D / 64 halves of
// [128 rows][64 elements]; a V tile of 128 keys is two pages of [D rows][64 keys].
template <int D>
struct Sizes {
    static constexpr int kHalves = D / 64;
    static constexpr int kTileBytes = kTileRows * D * 2;                  // Q, or 128 keys of K, or 128 keys of V
    static constexpr int kVPageBytes = D * 64 * 2;
    static constexpr int kSmemBytes = 2 * kTileBytes + 2 * kKvStages * kTileBytes + 1024;
    static constexpr uint32_t kIdescQK = instr_desc_bf16(128, 128);       // S = Q K^T: N = 128 keys
    static constexpr uint32_t kIdescPV = instr_desc_bf16(128, D);         // O += P V: N = D
    static constexpr int kOCol0 = 256;                                    // O of head i at column 256 + i * D
};

enum : int { ERR_NONE = 0, ERR_Q = 1, ERR_K_FULL = 2, ERR_V_FULL = 3, ERR_K_EMPTY = 4, ERR_V_EMPTY = 5, ERR_S_FULL = 6,
             ERR_P_FULL = 7, ERR_O_FULL = 8 };

__device__ int g_error = 0;

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// Two-wide fp32 arithmetic and the three-input maximum of sm_100: the softmax threads are short of issue
// slots, and these halve the instructions for scaling, summing and the row maximum.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    float2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long ra, rb, rd;
    float2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int kD>
__global__ void __launch_bounds__(kThreads, 1)
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                                 const int* __restrict__ tile_seq, const int* __restrict__ tile_row,
                                 const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                                 const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                 int n_pages, int n_heads, int n_kv, float scale_log2, float* __restrict__ part_o,
                                 float* __restrict__ part_ml, int n_splits, int n_tokens) {
    using Z = Sizes<kD>;
    constexpr int kTileBytes = Z::kTileBytes;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t q_full, k_full[kKvStages], v_full[kKvStages], k_empty[kKvStages], v_empty[kKvStages],
        s_full[2], p_full[2], o_full[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    // The tile lists are made of 64-token tiles; this kernel takes them in pairs.
    const int tile = gridDim.y - 1 - blockIdx.y;                 // later tiles of a sequence have more keys: they go first
    const int tile_row0 = tile_row[tile];
    if (tile_row0 % kTileRows != 0) return;
    const int seq = tile_seq[tile];
    const int h0 = 2 * blockIdx.x;                               // heads h0, h0 + 1
    const int kvh = h0 / (n_heads / n_kv);
    const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
    const int history = kv_len[seq] - q_len;                     // keys cached before this step's tokens
    const int n_keys = history + min(tile_row0 + kTileRows, q_len);
    const int last_page = (n_keys - 1) / kPageTokens;
    // With n_splits > 1 (few query tiles, many keys: a short chunk after a long history) the key steps of a tile
    // are shared out over gridDim.z blocks, which leave unnormalised partial results for a second kernel.
    const int all_blocks = (n_keys + kBlockKeys - 1) / kBlockKeys;
    const int per_split = (all_blocks + n_splits - 1) / n_splits;
    const int j_first = (int)blockIdx.z * per_split;
    const int n_blocks = max(0, min(all_blocks, j_first + per_split) - j_first);      // key steps of this block

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;          // swizzled tiles want 1 KiB alignment
    const uint32_t q_smem = base, k_smem = base + 2 * kTileBytes, v_smem = k_smem + kKvStages * kTileBytes;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        for (int s = 0; s < kKvStages; ++s) {
            mbar_init(smem_u32(&k_full[s]), 1);
            mbar_init(smem_u32(&v_full[s]), 1);
            mbar_init(smem_u32(&k_empty[s]), 1);
            mbar_init(smem_u32(&v_empty[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&s_full[i]), 1);
            mbar_init(smem_u32(&p_full[i]), 4);                  // the four softmax warps of a head
            mbar_init(smem_u32(&o_full[i]), 1);
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    auto fail = [&](int code) {
        atomicCAS(&g_error, 0, code);
        atomicExch(&abort_flag, 1);
    };
    auto aborted = [&]() { return *(volatile int*)&abort_flag != 0; };

    if (warp == 9) {
        // ---- TMA producer ----
        if (lane == 0) {
            const int* pages = page_table + (int64_t)slots[seq] * max_pages;
            if (n_blocks > 0) {
                mbar_expect_tx(smem_u32(&q_full), 2 * kTileBytes);
                for (int i = 0; i < 2; ++i)
                    for (int half = 0; half < Z::kHalves; ++half)
                        tma_load_2d(q_smem + i * kTileBytes + half * kHalfBytes, &map_q, smem_u32(&q_full),
                                    (h0 + i) * kD + half * 64, q_begin + tile_row0);
            }
            int issued = 0;
            for (int j = 0; j < n_blocks && !aborted(); ++j, ++issued) {
                const int s = j & 1, ph = (j >> 1) & 1;
                // the second page of the last step may lie beyond the keys: its scores are masked, any page will do
                const int pa = min(max(CPM_PAGE(pages, 2 * (j_first + j), max_pages), 0), n_pages - 1);
                const int pb = min(max(CPM_PAGE(pages, min(2 * (j_first + j) + 1, last_page), max_pages), 0), n_pages - 1);
                if (!mbar_wait_bounded(smem_u32(&k_empty[s]), ph ^ 1)) { fail(ERR_K_EMPTY); break; }
                mbar_expect_tx(smem_u32(&k_full[s]), kTileBytes);
                for (int half = 0; half < Z::kHalves; ++half) {
                    const uint32_t dst = k_smem + s * kTileBytes + half * kHalfBytes;
                    tma_load_2d(dst, &map_k, smem_u32(&k_full[s]), half * 64, (pa * n_kv + kvh) * kPageTokens);
                    tma_load_2d(dst + kHalfBytes / 2, &map_k, smem_u32(&k_full[s]), half * 64, (pb * n_kv + kvh) * kPageTokens);
                }
                if (!mbar_wait_bounded(smem_u32(&v_empty[s]), ph ^ 1)) { fail(ERR_V_EMPTY); break; }
                mbar_expect_tx(smem_u32(&v_full[s]), kTileBytes);
                tma_load_2d(v_smem + s * kTileBytes, &map_v, smem_u32(&v_full[s]), 0, (pa * n_kv + kvh) * kD);
                tma_load_2d(v_smem + s * kTileBytes + Z::kVPageBytes, &map_v, smem_u32(&v_full[s]), 0, (pb * n_kv + kvh) * kD);
            }
            if (aborted()) {
                // copies that nobody consumed: wait for them (bounded), so that none is in flight at the exit
                if (n_blocks > 0) mbar_wait_bounded(smem_u32(&q_full), 0);
                for (int j = max(0, issued - kKvStages); j < issued; ++j) {
                    mbar_wait_bounded(smem_u32(&k_full[j & 1]), (j >> 1) & 1);
                    mbar_wait_bounded(smem_u32(&v_full[j & 1]), (j >> 1) & 1);
                }
            }
        }
    } else if (warp == 8) {
        // ---- MMA issue ----
        if (lane == 0) {
            auto issue_qk = [&](int i, int s) {
#pragma unroll
                for (int half = 0; half < Z::kHalves; ++half) {
                    const uint64_t da = smem_desc_sw128(q_smem + i * kTileBytes + half * kHalfBytes);
                    const uint64_t db = smem_desc_sw128(k_smem + s * kTileBytes + half * kHalfBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tcgen05_mma_f16(tmem_base + i * 128, da + 2 * k, db + 2 * k, Z::kIdescQK, (half | k) != 0);
                }
            };
            auto issue_pv = [&](int i, int s, bool accumulate) {
#pragma unroll
                for (int page = 0; page < 2; ++page) {
                    const uint64_t db = smem_desc_sw128(v_smem + s * kTileBytes + page * Z::kVPageBytes);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tcgen05_mma_f16_ts(tmem_base + Z::kOCol0 + i * kD, tmem_base + i * 128 + page * 32 + k * 8, db + 2 * k,
                                           Z::kIdescPV, accumulate || (page | k) != 0);
                }
            };
            bool ok = n_blocks > 0;
            if (ok && !mbar_wait_bounded(smem_u32(&q_full), 0)) { fail(ERR_Q); ok = false; }
            if (ok && !mbar_wait_bounded(smem_u32(&k_full[0]), 0)) { fail(ERR_K_FULL); ok = false; }
            if (ok) {
                tcgen05_fence_after();
                issue_qk(0, 0);
                tcgen05_commit(smem_u32(&s_full[0]));
                issue_qk(1, 0);
                tcgen05_commit(smem_u32(&s_full[1]));
                tcgen05_commit(smem_u32(&k_empty[0]));
            }
            for (int j = 0; ok && j < n_blocks && !aborted(); ++j) {
                const int s = j & 1, ph = (j >> 1) & 1;
                const int s1 = (j + 1) & 1, ph1 = ((j + 1) >> 1) & 1;
                if (!mbar_wait_bounded(smem_u32(&v_full[s]), ph)) { fail(ERR_V_FULL); break; }
                for (int i = 0; i < 2; ++i) {
                    if (!mbar_wait_bounded(smem_u32(&p_full[i]), j & 1)) { fail(ERR_P_FULL); ok = false; break; }
                    tcgen05_fence_after();
                    issue_pv(i, s, j > 0);
                    if (i == 1) tcgen05_commit(smem_u32(&v_empty[s]));
                    if (j + 1 < n_blocks) {
                        if (i == 0 && !mbar_wait_bounded(smem_u32(&k_full[s1]), ph1)) { fail(ERR_K_FULL); ok = false; break; }
                        tcgen05_fence_after();
                        issue_qk(i, s1);
                        tcgen05_commit(smem_u32(&s_full[i]));
                        if (i == 1) tcgen05_commit(smem_u32(&k_empty[s1]));
                    } else {
                        tcgen05_commit(smem_u32(&o_full[i]));
                    }
                }
            }
        }
    } else {
        // ---- softmax and epilogue: head i, row of this thread ----
        const int i = warp >> 2, quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int row = tile_row0 + r;
        const int limit = row < q_len ? history + row : -1;      // last key this row may see
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_addr = lane_base + i * 128, o_addr = lane_base + Z::kOCol0 + i * kD;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blocks; ++j) {
            if (__any_sync(0xffffffffu, aborted())) { ok = false; break; }
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&s_full[i]), j & 1))) {
                if (lane == 0) fail(ERR_S_FULL);
                ok = false;
                break;
            }
            tcgen05_fence_after();
            uint32_t v[4][32];
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_load_32cols(s_addr + c * 32, v[c]);
            tmem_load_wait();
            const int key0 = (j_first + j) * kBlockKeys;
            if (key0 + kBlockKeys - 1 > history + tile_row0) {   // the diagonal, or the end of the keys
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        if (key0 + c * 32 + e > limit) v[c][e] = 0xff800000u;      // -inf
            }
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int e = 0; e < 32; e += 2) mx = max3(mx, __uint_as_float(v[c][e]), __uint_as_float(v[c][e + 1]));
            const float m_new = mx * scale_log2;
            const bool grow = m_new > m_ref + kRescaleThreshold || (m_ref == -INFINITY && m_new > -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? ex2(m_ref - m_new) : 1.f;     // 0 the first time
                l *= alpha;
                if (j > 0) {
#pragma unroll 1
                    for (int c = 0; c < kD / 32; ++c) {
                        uint32_t o[32];
                        tmem_load_32cols(o_addr + c * 32, o);
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                        tmem_store_32cols(o_addr + c * 32, o);
                    }
                }
                if (grow) m_ref = m_new;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            float2 sum2 = make_float2(0.f, 0.f);
            const float2 scale2 = make_float2(scale_log2, scale_log2), minus_m2 = make_float2(-m_use, -m_use);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t packed[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float2 x = fma2(make_float2(__uint_as_float(v[2 * c + (e >> 4)][(2 * e) & 31]),
                                                      __uint_as_float(v[2 * c + (e >> 4)][(2 * e + 1) & 31])), scale2, minus_m2);
                    const float2 pp = make_float2(ex2(x.x), ex2(x.y));
                    sum2 = add2(sum2, pp);
                    packed[e] = pack_bf16(pp.x, pp.y);
                }
                tmem_store_32cols(s_addr + c * 32, packed);
            }
            l += sum2.x + sum2.y;
            tmem_store_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[i]));
        }
        if (ok && n_blocks > 0) {
            if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&o_full[i]), 0))) {
                if (lane == 0) fail(ERR_O_FULL);
                ok = false;
            }
        }
        if (n_splits > 1) {
            // this block's share of the keys: the accumulator as it is, the maximum it refers to, and the sum
            const int64_t at = (((int64_t)blockIdx.z * n_tokens + q_begin + min(row, q_len - 1)) * n_heads + h0 + i);
            if (ok && n_blocks > 0) {
                tcgen05_fence_after();
#pragma unroll 1
                for (int c = 0; c < kD / 32; ++c) {
                    uint32_t o[32];
                    tmem_load_32cols(o_addr + c * 32, o);
                    tmem_load_wait();
                    if (row < q_len) {
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            *reinterpret_cast<uint4*>(part_o + at * kD + c * 32 + e) = make_uint4(o[e], o[e + 1], o[e + 2], o[e + 3]);
                    }
                }
            }
            if (row < q_len) {
                part_ml[2 * at] = n_blocks > 0 ? m_ref : -INFINITY;
                part_ml[2 * at + 1] = n_blocks > 0 ? l : 0.f;
            }
        } else if (ok && n_blocks > 0) {
            tcgen05_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* orow = out + ((int64_t)(q_begin + min(row, q_len - 1)) * n_heads + h0 + i) * kD;
#pragma unroll 1
            for (int c = 0; c < kD / 32; ++c) {
                uint32_t o[32];
                tmem_load_32cols(o_addr + c * 32, o);
                tmem_load_wait();
                if (row < q_len) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + e) = w;
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 8) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}


// ---------------------------------------------------------------------------
// Attention over listed key blocks (block-sparse) for the tokens of prompt chunks, head size 128, 16 query heads
// per key/value head: the 128 rows of the MMA tile are 8 consecutive tokens x the 16 heads of their group.
// ---------------------------------------------------------------------------
// Every token has its own list of 64-key blocks (the selection's choice, or "all" below the dense length).  The
// eight tokens of a block of threads share what is brought: each token's blocks are marked in a bit mask, the union
// of the masks is walked in rising order, two blocks of the union a step: their K pages side by side and their V
// pages by TMA, S = Q K^T (128 x 128) into tensor memory, the softmax threads (one per row) mask the rows whose
// token did not list a block and the keys behind the token's position, write P as bf16 over S, and O += P V takes P
// from tensor memory.  An odd union repeats its last block in the second place, masked for every row.  Keys and
// values have one buffer each: the next step's keys are brought while the rows are in the softmax, its values while
// the next S is computed.  One S and one O accumulator (256 TMEM columns) and 105 KB of shared memory let two blocks
// share an SM: one block's tensor-core work runs while the other's rows are in the softmax.  Rows of tokens that did
// not list a block cost the tensor cores their share all the same (on random data the union of eight lists of 96
// blocks holds about 185), but 64 keys are 0.15 us of tensor work against 2 us for a warp of the mma.sync kernel.
// Two blocks a step rather than one: half as many hand-offs between the roles per key.  A row's scores of the
// second block are read from tensor memory twice (for the maximum, then for the exponentials), which keeps the
// thread within the registers that two blocks an SM leave it.
// A tile whose tokens belong to several sequences (packed prompts) is done in passes, one per sequence.
// Waits are bounded as in the kernel above.
constexpr int kSparseTokens = 8;
constexpr int kSparseThreads = 192;                      // warps 0-3: softmax, one row a thread; 4: MMA issue; 5: TMA
constexpr int kSparseTmemCols = 256;                     // S at columns 0-127 (P over its first 64), O at 128-255
constexpr int kSparseQBytes = 128 * 128 * 2;             // 8 tokens x 16 heads x 128
constexpr int kSparseKBytes = 2 * 64 * 128 * 2;          // two key pages, as two halves of 64 dims x 128 rows
constexpr int kSparseVBytes = 2 * 64 * 128 * 2;          // two value pages
constexpr int kSparseTileBytes = kSparseQBytes + kSparseKBytes + kSparseVBytes;
constexpr uint32_t kSparseIdescQK = instr_desc_bf16(128, 128);
constexpr uint32_t kSparseIdescPV = instr_desc_bf16(128, 128);

struct UnionCursor {             // walks the set bits of a mask in rising order
    int word;
    unsigned bits;
};
__device__ __forceinline__ int next_listed(UnionCursor& c, const unsigned* __restrict__ mask, int words) {
    while (c.bits == 0u) {
        if (++c.word >= words) return -1;
        c.bits = mask[c.word];
    }
    const int b = __ffs(c.bits) - 1;
    c.bits &= c.bits - 1u;
    return c.word * 32 + b;
}

__global__ void __launch_bounds__(kSparseThreads, 2)
listed_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                                const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                                const int* __restrict__ positions, const int* __restrict__ token_seq,
                                const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                int n_pages, const int* __restrict__ block_list, int list_cap, int n_tokens, int n_heads,
                                int n_kv, float scale_log2, int words) {
    constexpr int kD = 128;
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t q_full, k_full, k_empty, v_full, v_empty, s_full, p_full, o_full;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * kSparseTokens, kvh = blockIdx.y;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_smem = base, k_smem = base + kSparseQBytes, v_smem = k_smem + kSparseKBytes;
    unsigned* all = reinterpret_cast<unsigned*>(smem_raw + (base - smem_u32(smem_raw)) + kSparseTileBytes);
    unsigned* mine = all + words;                                          // [tokens][words]

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        mbar_init(smem_u32(&k_full), 1);
        mbar_init(smem_u32(&k_empty), 1);
        mbar_init(smem_u32(&v_full), 1);
        mbar_init(smem_u32(&v_empty), 1);
        mbar_init(smem_u32(&s_full), 1);
        mbar_init(smem_u32(&p_full), 4);                                   // the four softmax warps
        mbar_init(smem_u32(&o_full), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)kSparseTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    pdl_launch_dependents();
    pdl_wait();

    auto fail = [&](int code) {
        atomicCAS(&g_error, 0, code);
        atomicExch(&abort_flag, 1);
    };
    auto aborted = [&]() { return *(volatile int*)&abort_flag != 0; };

    // the softmax thread's row: token r / 16 of the tile, head r % 16 of the group
    const int r = (warp & 3) * 32 + lane;
    const int my_token = r >> 4;
    const bool row_live = warp < 4 && t0 + my_token < n_tokens;
    const int my_pos = row_live ? positions[t0 + my_token] : -1;
    const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_base, o_addr = lane_base + 128;
    float m_ref = -INFINITY, l = 0.f;
    uint32_t k_loads = 0, v_loads = 0;                                     // the producer's, for the abort path

    if (warp == 5 && lane == 0) {                                          // the queries: two halves of 64 dims
        mbar_expect_tx(smem_u32(&q_full), kSparseQBytes);
        for (int half = 0; half < 2; ++half)
            tma_load_3d(q_smem + half * (kSparseQBytes / 2), &map_q, smem_u32(&q_full), half * 64, kvh * 16, t0);
    }

    const int tile_tokens = min(kSparseTokens, n_tokens - t0);
    uint32_t it = 0;                                                       // steps so far, all passes
    bool ok = true;
    for (int first = 0; first < tile_tokens;) {                           // one pass per sequence in the tile
        const int seq = token_seq[t0 + first];
        int end = first + 1;
        while (end < tile_tokens && token_seq[t0 + end] == seq) ++end;
        const int* pages = page_table + (int64_t)slots[seq] * max_pages;
        // ---- the tokens' masks and their union ----
        for (int i = threadIdx.x; i < (kSparseTokens + 1) * words; i += kSparseThreads) all[i] = 0u;
        __syncthreads();
        for (int tl = first + warp; tl < end; tl += kSparseThreads / 32) {
            unsigned* m = mine + tl * words;
            const int* list = block_list + ((int64_t)(t0 + tl) * n_kv + kvh) * list_cap;
            if (list[0] == -2) {                                          // "dense": every block up to the token's own
                const int last = positions[t0 + tl] / kPageTokens;
                for (int w = lane; w <= (last >> 5) && w < words; w += 32)
                    m[w] = w < (last >> 5) ? 0xffffffffu : (0xffffffffu >> (31 - (last & 31)));
            } else {
                for (int b0 = 0; b0 < list_cap; b0 += 32) {              // the list ends at its first negative entry
                    const int i = b0 + lane;
                    const int b = i < list_cap ? list[i] : -1;
                    const unsigned ended = __ballot_sync(0xffffffffu, b < 0);
                    const int n_valid = ended ? __ffs(ended) - 1 : 32;
                    if (lane < n_valid && (b >> 5) < words) atomicOr(&m[b >> 5], 1u << (b & 31));
                    if (ended) break;
                }
            }
        }
        __syncthreads();
        for (int w = threadIdx.x; w < words; w += kSparseThreads) {
            unsigned u = 0u;
            for (int k = first; k < end; ++k) u |= mine[k * words + w];
            all[w] = u;
        }
        __syncthreads();
        int n_blocks = 0;                                                  // the same number in every thread
        for (int w = 0; w < words; ++w) n_blocks += __popc(all[w]);
        int n_steps = (n_blocks + 1) / 2;
        ok = ok && !aborted();
        if (!ok) n_steps = 0;

        if (warp == 5) {
            // ---- TMA producer ----
            if (lane == 0) {
                UnionCursor cursor{-1, 0u};
                for (int j = 0; j < n_steps; ++j, ++it) {
                    const int b0 = next_listed(cursor, all, words);
                    const int b1 = 2 * j + 1 < n_blocks ? next_listed(cursor, all, words) : b0;
                    const int page0 = min(max(CPM_PAGE(pages, b0, max_pages), 0), n_pages - 1);
                    const int page1 = min(max(CPM_PAGE(pages, b1, max_pages), 0), n_pages - 1);
                    if (it > 0 && !mbar_wait_bounded(smem_u32(&k_empty), (it - 1) & 1u)) { fail(ERR_K_EMPTY); ok = false; break; }
                    if (aborted()) { ok = false; break; }
                    const uint32_t kbar = smem_u32(&k_full), vbar = smem_u32(&v_full);
                    mbar_expect_tx(kbar, kSparseKBytes);
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        tma_load_2d(k_smem + half * (kSparseKBytes / 2), &map_k, kbar, half * 64, (page0 * n_kv + kvh) * kPageTokens);
                        tma_load_2d(k_smem + half * (kSparseKBytes / 2) + kSparseKBytes / 4, &map_k, kbar, half * 64,
                                    (page1 * n_kv + kvh) * kPageTokens);
                    }
                    ++k_loads;
                    if (it > 0 && !mbar_wait_bounded(smem_u32(&v_empty), (it - 1) & 1u)) { fail(ERR_V_EMPTY); ok = false; break; }
                    mbar_expect_tx(vbar, kSparseVBytes);
                    tma_load_2d(v_smem, &map_v, vbar, 0, (page0 * n_kv + kvh) * kD);
                    tma_load_2d(v_smem + kSparseVBytes / 2, &map_v, vbar, 0, (page1 * n_kv + kvh) * kD);
                    ++v_loads;
                }
            }
        } else if (warp == 4) {
            // ---- MMA issue ----
            if (lane == 0 && n_steps > 0) {
                auto issue_qk = [&]() {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const uint64_t da = smem_desc_sw128(q_smem + half * (kSparseQBytes / 2));
                        const uint64_t db = smem_desc_sw128(k_smem + half * (kSparseKBytes / 2));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tcgen05_mma_f16(tmem_base, da + 2 * k, db + 2 * k, kSparseIdescQK, (half | k) != 0);
                    }
                };
                auto issue_pv = [&](bool accumulate) {
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const uint64_t db = smem_desc_sw128(v_smem + x * (kSparseVBytes / 2));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tcgen05_mma_f16_ts(tmem_base + 128, tmem_base + x * 32 + k * 8, db + 2 * k, kSparseIdescPV,
                                               accumulate || (x | k) != 0);
                    }
                };
                if (it == 0 && !mbar_wait_bounded(smem_u32(&q_full), 0)) { fail(ERR_Q); ok = false; }
                if (ok && !mbar_wait_bounded(smem_u32(&k_full), it & 1u)) { fail(ERR_K_FULL); ok = false; }
                if (ok) {
                    tcgen05_fence_after();
                    issue_qk();
                    tcgen05_commit(smem_u32(&s_full));
                    tcgen05_commit(smem_u32(&k_empty));
                }
                for (int j = 0; ok && j < n_steps; ++j, ++it) {
                    if (aborted()) { ok = false; break; }
                    if (!mbar_wait_bounded(smem_u32(&p_full), it & 1u)) { fail(ERR_P_FULL); ok = false; break; }
                    if (!mbar_wait_bounded(smem_u32(&v_full), it & 1u)) { fail(ERR_V_FULL); ok = false; break; }
                    tcgen05_fence_after();
                    issue_pv(it > 0);
                    tcgen05_commit(smem_u32(&v_empty));                    // the values are free when this product is done
                    if (j + 1 < n_steps) {
                        if (!mbar_wait_bounded(smem_u32(&k_full), (it + 1) & 1u)) { fail(ERR_K_FULL); ok = false; break; }
                        tcgen05_fence_after();
                        issue_qk();
                        tcgen05_commit(smem_u32(&s_full));                 // also covers the product into O before it
                        tcgen05_commit(smem_u32(&k_empty));
                    }
                }
            } else {
                it += n_steps;
            }
            it = __shfl_sync(0xffffffffu, it, 0);
        } else {
            // ---- softmax: one row a thread ----
            const bool member = row_live && my_token >= first && my_token < end;
            const unsigned* my_mask = mine + my_token * words;
            UnionCursor cursor{-1, 0u};
            for (int j = 0; j < n_steps; ++j, ++it) {
                const int b0 = next_listed(cursor, all, words);
                const int b1 = 2 * j + 1 < n_blocks ? next_listed(cursor, all, words) : -1;
                if (__any_sync(0xffffffffu, aborted())) { ok = false; break; }
                if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&s_full), it & 1u))) {
                    if (lane == 0) fail(ERR_S_FULL);
                    ok = false;
                    break;
                }
                tcgen05_fence_after();
                int visible[2];                                            // keys of each block this row sees
                visible[0] = member && ((my_mask[b0 >> 5] >> (b0 & 31)) & 1u) ? min(64, my_pos - b0 * kPageTokens + 1) : 0;
                visible[1] = b1 >= 0 && member && ((my_mask[b1 >> 5] >> (b1 & 31)) & 1u) ? min(64, my_pos - b1 * kPageTokens + 1) : 0;
                float mx = -INFINITY;
                uint32_t v[2][32];
#pragma unroll
                for (int x = 1; x >= 0; --x) {                             // the first block's scores stay in registers
                    tmem_load_32cols(s_addr + x * 64, v[0]);
                    tmem_load_32cols(s_addr + x * 64 + 32, v[1]);
                    tmem_load_wait();
                    if (visible[x] > 0) {
                        if (visible[x] < 64) {
#pragma unroll
                            for (int c = 0; c < 2; ++c)
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    if (c * 32 + e >= visible[x]) v[c][e] = 0xff800000u;          // -inf
                        }
#pragma unroll
                        for (int c = 0; c < 2; ++c)
#pragma unroll
                            for (int e = 0; e < 32; e += 2) mx = max3(mx, __uint_as_float(v[c][e]), __uint_as_float(v[c][e + 1]));
                    }
                }
                const float m_new = mx * scale_log2;
                const bool grow = m_new > m_ref + kRescaleThreshold || (m_ref == -INFINITY && m_new > -INFINITY);
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = grow ? ex2(m_ref - m_new) : 1.f;             // 0 the first time
                    l *= alpha;
                    if (it > 0) {
#pragma unroll 1
                        for (int c = 0; c < kD / 16; ++c) {
                            uint32_t o[16];
                            tmem_load_16cols(o_addr + c * 16, o);
                            tmem_load_wait();
#pragma unroll
                            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                            tmem_store_16cols(o_addr + c * 16, o);
                        }
                    }
                    if (grow) m_ref = m_new;
                }
                const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
                const float2 scale2 = make_float2(scale_log2, scale_log2), minus_m2 = make_float2(-m_use, -m_use);
                float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    if (x == 1) {                                          // the second block's scores again (the whole warp loads)
                        tmem_load_32cols(s_addr + 64, v[0]);
                        tmem_load_32cols(s_addr + 96, v[1]);
                        tmem_load_wait();
                        if (visible[1] > 0 && visible[1] < 64) {
#pragma unroll
                            for (int c = 0; c < 2; ++c)
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    if (c * 32 + e >= visible[1]) v[c][e] = 0xff800000u;
                        }
                    }
                    uint32_t packed[32];
                    if (visible[x] > 0) {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const float2 xx = fma2(make_float2(__uint_as_float(v[e >> 4][(2 * e) & 31]),
                                                               __uint_as_float(v[e >> 4][(2 * e + 1) & 31])), scale2, minus_m2);
                            const float2 pp = make_float2(ex2(xx.x), ex2(xx.y));
                            sum2 = add2(sum2, pp);
                            packed[e] = pack_bf16(pp.x, pp.y);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) packed[e] = 0u;
                    }
                    tmem_store_32cols(s_addr + x * 32, packed);
                }
                l += sum2.x + sum2.y;
                tmem_store_wait();
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&p_full));
            }
        }
        if (!ok) atomicExch(&abort_flag, 1);
        __syncthreads();                                                   // the masks are free for the next pass
        if (aborted()) break;
        // every role has counted the pass's steps
        if (warp == 5) it = __shfl_sync(0xffffffffu, it, 0);
        first = end;
    }

    if (warp == 4 && lane == 0 && !aborted() && it > 0) tcgen05_commit(smem_u32(&o_full));      // after the tile's last product
    if (warp < 4 && !aborted() && it > 0) {
        // ---- epilogue: the rows' results ----
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(smem_u32(&o_full), 0))) {
            if (lane == 0) fail(ERR_O_FULL);
        } else {
            tcgen05_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* orow = out + ((int64_t)min(t0 + my_token, n_tokens - 1) * n_heads + kvh * 16 + (r & 15)) * kD;
#pragma unroll 1
            for (int c = 0; c < kD / 32; ++c) {
                uint32_t o[32];
                tmem_load_32cols(o_addr + c * 32, o);
                tmem_load_wait();
                if (row_live) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + e) = w;
                    }
                }
            }
        }
    }
    if (warp == 5 && lane == 0 && aborted()) {
        // copies that nobody consumed: wait for them (bounded), so that none is in flight at the exit
        mbar_wait_bounded(smem_u32(&q_full), 0);
        if (k_loads > 0) mbar_wait_bounded(smem_u32(&k_full), (k_loads - 1) & 1u);
        if (v_loads > 0) mbar_wait_bounded(smem_u32(&v_full), (v_loads - 1) & 1u);
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 4) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)kSparseTmemCols) : "memory");
    }
}

}  // namespace fa5

namespace fa5 {
// out[t, h, :] = sum_s o_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M), M = max_s m_s, over the shares s of the keys.
__global__ void combine_key_shares_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          bf16* __restrict__ out, int n_tokens, int n_heads, int D, int n_splits) {
    const int64_t th = (int64_t)blockIdx.x * n_heads + blockIdx.y;
    const int64_t stride = (int64_t)n_tokens * n_heads;
    float mx = -INFINITY;
    for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, part_ml[2 * (s * stride + th)]);
    float denom = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float m = part_ml[2 * (s * stride + th)];
        if (m != -INFINITY) denom += part_ml[2 * (s * stride + th) + 1] * exp2f(m - mx);
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float m = part_ml[2 * (s * stride + th)];
            if (m != -INFINITY) acc += part_o[(s * stride + th) * D + c] * exp2f(m - mx);
        }
        out[th * D + c] = __float2bfloat16_rn(acc * inv);
    }
}

template <int D>
static int launch(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq, const int* tile_row,
                  int n_tiles, const int* cu_q, const int* kv_len, const int* slots, const int* page_table, int max_pages,
                  int n_tokens, int n_pages, int n_heads, int n_kv, float scale, float* scratch, int n_splits,
                  cudaStream_t stream) {
    CUtensorMap map_q, map_k, map_v;
    if (!tc5::make_map_2d_bf16(&map_q, q, (uint64_t)n_tokens, (uint64_t)n_heads * D, (uint64_t)n_heads * D * 2, 64, kTileRows) ||
        !tc5::make_map_2d_bf16(&map_k, k_cache, (uint64_t)n_pages * n_kv * kPageTokens, D, D * 2, 64, kPageTokens) ||
        !tc5::make_map_2d_bf16(&map_v, v_cache, (uint64_t)n_pages * n_kv * D, kPageTokens, kPageTokens * 2, 64, D))
        return CPM_BAD_ARGUMENT;
    auto kern = prefill_attention_tcgen05_kernel<D>;
    static bool configured[kMaxDevices] = {};            // per kernel and per device
    if (int st = ensure_dynamic_smem(kern, Sizes<D>::kSmemBytes, configured)) return st;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (int64_t)n_splits * n_tokens * n_heads * D : nullptr;
    kern<<<dim3(n_heads / 2, n_tiles, n_splits), kThreads, Sizes<D>::kSmemBytes, stream>>>(map_q, map_k, map_v, (bf16*)out,
        tile_seq, tile_row, cu_q, kv_len, slots, page_table, max_pages, n_pages, n_heads, n_kv, scale * 1.4426950408889634f,
        part_o, part_ml, n_splits, n_tokens);
    if (n_splits > 1)
        combine_key_shares_kernel<<<dim3(n_tokens, n_heads), D / 2, 0, stream>>>(part_o, part_ml, (bf16*)out, n_tokens, n_heads,
                                                                               D, n_splits);
    return launch_status();
}
}  // namespace fa5

// q, out [tokens, heads, d] bf16 with d = 128 or 64, tokens packed by sequence (cu_q); the cache (n_pages pages of 64
// tokens, K pages [n_kv][64][d], V pages [n_kv][d][64]) already holds this step's keys.  The tile lists are those of the
// 64-token prefill tiles.  Needs an even number of query heads per key/value head.  n_splits > 1: the keys of every
// tile are shared out over that many blocks (for few tiles and many keys) and scratch holds
// n_splits * n_tokens * n_heads * (d + 2) floats.
CPM_API int cpm_prefill_attention_tcgen05(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          const int* tile_seq, const int* tile_row, int n_tiles, const int* cu_q,
                                          const int* kv_len, const int* slots, const int* page_table, int max_pages,
                                          int n_tokens, int n_pages, int n_heads, int n_kv, int d, float scale,
                                          float* scratch, int n_splits, cudaStream_t stream) {
    if (n_tiles <= 0 || n_tokens <= 0) return CPM_OK;
    if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && !scratch) || n_tokens > 65535 * 1024) return CPM_BAD_ARGUMENT;
    if ((d != 128 && d != 64) || n_kv <= 0 || n_heads % n_kv || (n_heads / n_kv) % 2 || n_tiles > 65535 || n_pages <= 0 ||
        ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15))
        return CPM_BAD_ARGUMENT;
    if (d == 128)
        return fa5::launch<128>(q, k_cache, v_cache, out, tile_seq, tile_row, n_tiles, cu_q, kv_len, slots, page_table, max_pages,
                                n_tokens, n_pages, n_heads, n_kv, scale, scratch, n_splits, stream);
    return fa5::launch<64>(q, k_cache, v_cache, out, tile_seq, tile_row, n_tiles, cu_q, kv_len, slots, page_table, max_pages,
                           n_tokens, n_pages, n_heads, n_kv, scale, scratch, n_splits, stream);
}

// Block-list attention of prompt tokens on the tensor cores (see listed_attention_tcgen05_kernel): q, out [tokens, heads,
// 128] bf16, 16 query heads per key/value head, block_list int32 [tokens, kv_heads, list_cap] of 64-token blocks
// (first entry -2 = all blocks up to the token's own).  Other shapes, and page tables too wide for the masks to fit
// beside the tiles (more than cpm_listed_attention_tcgen05_max_pages() pages a sequence), are refused: the caller
// takes the mma.sync kernel for them.
CPM_API int cpm_listed_attention_tcgen05_max_pages() {
    return ((110 * 1024 - 1024 - fa5::kSparseTileBytes) / ((fa5::kSparseTokens + 1) * 4)) * 32;
}

CPM_API int cpm_listed_attention_tcgen05(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int* positions, const int* token_seq, const int* slots,
                                         const int* page_table, int max_pages, int n_pages, const int* block_list,
                                         int list_cap, int n_tokens, int n_heads, int n_kv, int d, float scale,
                                         cudaStream_t stream) {
    using namespace fa5;
    if (n_tokens <= 0) return CPM_OK;
    if (d != 128 || n_kv <= 0 || n_heads != 16 * n_kv || !block_list || list_cap < 1 || n_pages <= 0 || n_kv > 65535 ||
        ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)out & 15))
        return CPM_BAD_ARGUMENT;
    const int words = (max_pages + 31) / 32;
    const int smem = 1024 + kSparseTileBytes + (kSparseTokens + 1) * words * 4;
    if (smem > 110 * 1024) return CPM_BAD_ARGUMENT;                  // two blocks share an SM's shared memory
    CUtensorMap map_q, map_k, map_v;
    if (!tc5::make_map_3d_bf16(&map_q, q, 128, (uint64_t)n_heads, (uint64_t)n_tokens, 128 * 2, (uint64_t)n_heads * 128 * 2, 64, 16,
                               kSparseTokens) ||
        !tc5::make_map_2d_bf16(&map_k, k_cache, (uint64_t)n_pages * n_kv * kPageTokens, 128, 128 * 2, 64, kPageTokens) ||
        !tc5::make_map_2d_bf16(&map_v, v_cache, (uint64_t)n_pages * n_kv * 128, kPageTokens, kPageTokens * 2, 64, 128))
        return CPM_BAD_ARGUMENT;
    auto kern = listed_attention_tcgen05_kernel;
    static bool configured[kMaxDevices] = {};
    if (int st = ensure_dynamic_smem(kern, 110 * 1024, configured)) return st;
    cpm_launch(kLaunchAttention, kern, dim3((n_tokens + kSparseTokens - 1) / kSparseTokens, n_kv), dim3(kSparseThreads),
               (size_t)smem, stream, map_q, map_k, map_v, (bf16*)out, positions, token_seq, slots, page_table, max_pages, n_pages,
               block_list, list_cap, n_tokens, n_heads, n_kv, scale * 1.4426950408889634f, words);
    return launch_status();
}

// Error code recorded by the kernel since the last call (0 = none), and reset.  Synchronises the device.
CPM_API int cpm_attention_tcgen05_error() {
    int code = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&code, fa5::g_error, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(fa5::g_error, &zero, sizeof(int));
    return code;
}

CPM_BOUNDS_TU(attention_tcgen05)
