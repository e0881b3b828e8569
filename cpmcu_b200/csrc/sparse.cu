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
// always attended; scores, pooling and the choice are fp32; pooled keys are stored in fp32
// with an fp32 cache and as two bf16 terms (the mean to 16 bits) with a bf16 cache.
#include "common.cuh"

// One block per (token, kv head).  If the token at position pos completes a pooling
// window [first, first + kernel) with first = pos + 1 - kernel a multiple of stride,
// the mean of those cached keys is stored as pooled entry first / stride.
// How a pooled key lies in its d floats of storage.  With an fp32 cache: d floats.  With a bf16 cache: two bf16
// terms whose sum is the fp32 mean to 16 bits, d leading terms (the mean rounded to bf16) and then d residuals
// (the rest rounded to bf16); these are the two B operands that the tensor-core scores use, so the kernels that
// score load fragments straight from them (splitting the floats in registers, for every token and in both walks,
// was three quarters of the prefill selection kernel's instructions).
template <typename T>
__device__ __forceinline__ void store_pooled(float* __restrict__ pooled, int64_t entry, int d, int c, float mean) {
    pooled[entry + c] = mean;
}
template <>
__device__ __forceinline__ void store_pooled<bf16>(float* __restrict__ pooled, int64_t entry, int d, int c, float mean) {
    bf16* terms = reinterpret_cast<bf16*>(pooled + entry);
    const bf16 lead = __float2bfloat16_rn(mean);
    terms[c] = lead;
    terms[d + c] = __float2bfloat16_rn(mean - __bfloat162float(lead));
}
// Four consecutive dims of a pooled key as floats, from either form.
template <bool kTerms>
__device__ __forceinline__ float4 load_pooled4(const float* __restrict__ row, int d, int c) {
    if (!kTerms) return __ldg(reinterpret_cast<const float4*>(row + c));
    const bf16* terms = reinterpret_cast<const bf16*>(row);
    const uint2 lead = __ldg(reinterpret_cast<const uint2*>(terms + c)), rest = __ldg(reinterpret_cast<const uint2*>(terms + d + c));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lead.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lead.y));
    const float2 e = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rest.x));
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rest.y));
    return make_float4(a.x + e.x, a.y + e.y, b.x + f.x, b.y + f.y);
}

template <typename T>
__global__ void pool_keys_kernel(const T* __restrict__ k_cache, float* __restrict__ pooled,
                                 const int* __restrict__ positions, const int* __restrict__ token_seq,
                                 const int* __restrict__ slots, const int* __restrict__ page_table, int max_pages,
                                 int n_kv, int d, int kernel, int stride) {
    const int t = blockIdx.x, kvh = blockIdx.y;
    pdl_launch_dependents();
    pdl_wait();
    const int first = positions[t] + 1 - kernel;
    if (first < 0 || first % stride != 0) return;
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int per_page = kPageTokens / stride;
    const int64_t dst = (((int64_t)CPM_PAGE(pages, first / kPageTokens, max_pages) * n_kv + kvh) * per_page
                         + (first % kPageTokens) / stride) * d;
    const float inv = 1.0f / (float)kernel;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float s = 0.f;
        for (int r = 0; r < kernel; ++r) {
            const int j = first + r;
            s += to_f32(k_cache[page_row_offset(CPM_PAGE(pages, j / kPageTokens, max_pages), kvh, j % kPageTokens, n_kv, d) + c]);
        }
        store_pooled<T>(pooled, dst, d, c, s * inv);
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
        cpm_launch(kLaunchAttention, pool_keys_kernel<bf16>, grid, threads, 0, stream, (const bf16*)k_cache, pooled, positions,
                   token_seq, slots, page_table, max_pages, n_kv, d, kernel, stride);
    else
        pool_keys_kernel<float><<<grid, threads, 0, stream>>>((const float*)k_cache, pooled, positions, token_seq,
                                                              slots, page_table, max_pages, n_kv, d, kernel, stride);
    return launch_status();
}

// From the scores of the visible pooled keys to the list of blocks.  The block score is the
// maximum over the pooled keys that overlap the block; the leading blocks and the blocks of the
// local window are always taken; of the others the topk - init_blocks best are chosen (ties to
// the lower index).  Nothing here is sized by the number of pooled keys: every pooled key's score
// goes straight into the keys of the blocks it overlaps (note_score, an atomic maximum in
// shared memory), so the shared arrays grow with the number of candidate blocks only.
//
// A block's key is its score's bits made monotonic (an unsigned compare orders them like the
// floats); 0 is below every real key and stands for "no pooled key overlaps this block".  Among
// equal scores the lower block wins.
struct Selection {
    int qb;             // block of the query
    int last_choice;    // last block that can be chosen (those after it are the local window)
    int n_cand;         // candidates: blocks init_blocks .. last_choice
    int per_block;      // pooled keys that start inside one block
    int reach_back;     // pooled keys before a block's first that still overlap it
    int per_block_shift;   // log2(per_block) when it is a power of two (it is for every configuration seen), else -1
};

__device__ __forceinline__ Selection selection_of(int p, int kernel, int stride, int block_size, int init_blocks,
                                                  int local_blocks, int sort_cap) {
    Selection s;
    s.qb = p / block_size;
    s.last_choice = s.qb - local_blocks;
    s.per_block = block_size / stride;
    s.per_block_shift = (s.per_block & (s.per_block - 1)) == 0 ? __ffs(s.per_block) - 1 : -1;
    s.reach_back = kernel / stride - 1;
    s.n_cand = min(max(0, s.last_choice + 1 - init_blocks), sort_cap);
    return s;
}

// The selection's arrays in shared memory, sized by the launch for ``cap`` candidate blocks.
struct SelectionArrays {
    unsigned* keys;      // [cap] a candidate's best score, monotonic bits
    unsigned* chosen;    // [words] a bit per chosen candidate
    unsigned* equal;     // [words] a bit per candidate whose score equals the last one taken
};
__host__ __device__ constexpr int selection_words(int cap) { return (cap / 32 + 4) & ~3; }
__host__ __device__ constexpr size_t selection_bytes(int cap) { return (size_t)cap * 4 + 2 * (size_t)selection_words(cap) * 4; }
__device__ __forceinline__ SelectionArrays selection_arrays(unsigned char* base, int cap) {
    SelectionArrays a;
    a.keys = reinterpret_cast<unsigned*>(base);
    a.chosen = a.keys + cap;
    a.equal = a.chosen + selection_words(cap);
    return a;
}

// Clears the candidates' keys and the bit masks; all threads call it, a barrier must follow.
__device__ __forceinline__ void clear_selection(const Selection& s, const SelectionArrays& a) {
    for (int i = threadIdx.x; i < s.n_cand; i += blockDim.x) a.keys[i] = 0u;
    for (int i = threadIdx.x; i < (s.n_cand + 31) / 32; i += blockDim.x) a.chosen[i] = a.equal[i] = 0u;
}

// Pooled key ``entry`` has the score ``v`` (>= 0): raises the key of every candidate block it overlaps
// (a native 32-bit atomic maximum in shared memory).
__device__ __forceinline__ void note_score(const Selection& s, const SelectionArrays& a, int init_blocks, int entry, float v) {
    const unsigned bits = __float_as_uint(v);
    const unsigned mono = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    const bool shift = s.per_block_shift >= 0;              // a division costs the few lanes that come here some twenty instructions
    const int first = shift ? entry >> s.per_block_shift : entry / s.per_block;
    const int last = shift ? (entry + s.reach_back) >> s.per_block_shift : (entry + s.reach_back) / s.per_block;
    const int k_hi = min(last, init_blocks + s.n_cand - 1);
    for (int k = max(first, init_blocks); k <= k_hi; ++k) atomicMax(&a.keys[k - init_blocks], mono);
}

// The ``rank``-th largest (1 <= rank <= n) of keys[0..n), and in ``with_it`` how many keys of that value belong to
// the ``rank`` largest.  The value is built bit by bit from the top: a bit stays set if at least ``rank`` keys are
// not below the value so far with that bit.  One warp does it alone, its lanes holding the keys in registers (up
// to 16 each; more are read from shared memory at every step) and adding their counts with one warp reduction
// per bit, so a step waits for no other warp: 33 steps of about 60 cycles.  (A bitonic sort stood here first, 45
// block-wide barriers for 512 keys; then radix selections with shared counters, warp-matched adds or ballots, and
// this bisection with the block-wide counting barrier: 4.9 to 6.3 us inside the captured decode step for 440 keys,
// every block-wide barrier costing 150 ns and more.)  All threads call it and all get the values after one
// barrier; the keys stay as they are.
__device__ unsigned kth_largest(const unsigned* __restrict__ keys, int n, int rank, int* with_it) {
    __shared__ unsigned found[2];
    constexpr int kHeld = 16;
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        unsigned held[kHeld];
#pragma unroll
        for (int k = 0; k < kHeld; ++k) held[k] = lane + 32 * k < n ? keys[lane + 32 * k] : 0u;
        auto not_below = [&](unsigned value) {             // keys >= value (value > 0), the same number in every lane
            int count = 0;
#pragma unroll
            for (int k = 0; k < kHeld; ++k) count += held[k] >= value ? 1 : 0;
            for (int i = lane + 32 * kHeld; i < n; i += 32) count += keys[i] >= value ? 1 : 0;
            return __reduce_add_sync(0xffffffffu, count);
        };
        unsigned value = 0u;
#pragma unroll 1
        for (int bit = 31; bit >= 0; --bit) {
            const unsigned trial = value | (1u << bit);
            if (not_below(trial) >= rank) value = trial;
        }
        const int above = value == 0xffffffffu ? 0 : not_below(value + 1u);
        if (lane == 0) {
            found[0] = value;
            found[1] = (unsigned)(rank - above);
        }
    }
    __syncthreads();
    *with_it = (int)found[1];
    return found[0];
}

// keys: [n_cand] filled by note_score; chosen, equal: cleared.  All threads call this after a barrier that
// follows the last note_score.  Taken are the candidates above the room-th largest score, and of those equal to
// it the lowest blocks, as many as still fit.
__device__ void finish_selection(const Selection& s, const SelectionArrays& a, int* __restrict__ list, int list_cap,
                                 int init_blocks, int topk) {
    const int tid = threadIdx.x, n_threads = blockDim.x;
    const int n_cand = s.n_cand;
    const unsigned* keys = a.keys;
    unsigned* chosen = a.chosen;
    const int room = min(max(0, topk - init_blocks), n_cand);
    if (room >= n_cand) {                                 // room for every candidate that has a score
        for (int i = tid; i < n_cand; i += n_threads)
            if (keys[i] != 0u) atomicOr(&chosen[i >> 5], 1u << (i & 31));
    } else if (room > 0) {
        int with_it = 0;
        const unsigned least = kth_largest(keys, n_cand, room, &with_it);
        for (int i = tid; i < n_cand; i += n_threads) {
            const unsigned key = keys[i];
            if (key == 0u) continue;
            if (key > least) atomicOr(&chosen[i >> 5], 1u << (i & 31));
            else if (key == least) atomicOr(&a.equal[i >> 5], 1u << (i & 31));
        }
        __syncthreads();
        for (int i = tid; i < n_cand; i += n_threads) {
            const unsigned w = a.equal[i >> 5];
            if ((w >> (i & 31)) & 1u) {
                int before = __popc(w & ((1u << (i & 31)) - 1u));
                for (int j = 0; j < (i >> 5); ++j) before += __popc(a.equal[j]);
                if (before < with_it) atomicOr(&chosen[i >> 5], 1u << (i & 31));
            }
        }
    }
    __syncthreads();
    // the list in rising order: first blocks, the chosen ones, the local window; every entry's place follows
    // from the counts before it, so all threads write (a list that is too short keeps its first entries)
    const int n_init = min(init_blocks, s.qb + 1);
    const int last = list_cap - 1;
    for (int k = tid; k < n_init; k += n_threads)
        if (k < last) list[k] = k;
    for (int i = tid; i < n_cand; i += n_threads) {
        const unsigned w = chosen[i >> 5];
        if ((w >> (i & 31)) & 1u) {
            int at = n_init + __popc(w & ((1u << (i & 31)) - 1u));
            for (int j = 0; j < (i >> 5); ++j) at += __popc(chosen[j]);
            if (at < last) list[at] = init_blocks + i;
        }
    }
    int n_chosen = 0;
    for (int j = 0; j < (n_cand + 31) / 32; ++j) n_chosen += __popc(chosen[j]);
    const int first_local = max(n_init, s.last_choice + 1);
    const int base = n_init + n_chosen;
    for (int k = first_local + tid; k <= s.qb; k += n_threads)
        if (base + k - first_local < last) list[base + k - first_local] = k;
    if (tid == 0) list[min(base + max(0, s.qb - first_local + 1), last)] = -1;
}

// Set when a query had more candidate blocks than the launch made room for (the caller's bound on the
// longest sequence was too small); the lists of such a query are not valid.
__device__ int g_select_overflow = 0;

CPM_API int cpm_select_blocks_error() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_select_overflow, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_select_overflow, &zero, sizeof(int));
    return v;
}

// One block per (token, kv head): writes the ascending list of key blocks the query
// attends to, ended by -1; a first entry of -2 says "dense" (the query sees at most
// dense_len keys).
//
// Scores: a warp takes one pooled key at a time, its lanes spread over head_dim (coalesced
// 16-byte loads of the fp32 row), and forms the dot products with all query heads of the
// group; the softmax over the visible pooled keys needs each head's maximum and sum first,
// so the pooled keys are walked twice (statistics, then probabilities).
constexpr int kSelectThreads = 256;
constexpr int kSelectWarps = kSelectThreads / 32;
constexpr int kMaxGroup = 32;              // query heads per kv head this kernel takes

__device__ __forceinline__ const float* pooled_row(const float* __restrict__ pooled, const int* __restrict__ pages,
                                                   int entry, int stride, int per_page, int n_kv, int kvh, int d) {
    // the stride divides the page, so per_page is a power of two: entry / per_page is the page, the rest the place in it
    const int shift = __ffs(per_page) - 1;
    return pooled + (((int64_t)CPM_PAGE(pages, entry >> shift, 0x7fffffff) * n_kv + kvh) * per_page + (entry & (per_page - 1))) * d;
}

// Dot products of one pooled key with every head of the group; every lane returns all of them
// through ``dots`` (dots[h] valid for h < group).
template <bool kTerms>
__device__ __forceinline__ void group_dots(const float* __restrict__ row, const float* __restrict__ qs, int group, int d,
                                           int lane, float scale, float* dots /* [kMaxGroup] in registers */) {
#pragma unroll
    for (int h = 0; h < kMaxGroup; ++h) dots[h] = 0.f;
    for (int c0 = 0; c0 < d; c0 += 128) {
        const int c = c0 + 4 * lane;
        if (c < d) {
            const float4 kv = load_pooled4<kTerms>(row, d, c);
#pragma unroll
            for (int h = 0; h < kMaxGroup; ++h) {
                if (h < group) {
                    const float4 qv = *reinterpret_cast<const float4*>(qs + h * d + c);
                    dots[h] = fmaf(qv.x, kv.x, fmaf(qv.y, kv.y, fmaf(qv.z, kv.z, fmaf(qv.w, kv.w, dots[h]))));
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < kMaxGroup; ++h)
        if (h < group) dots[h] = warp_sum(dots[h]) * scale;
}

template <typename T>
__global__ void __launch_bounds__(kSelectThreads)
select_blocks_kernel(const T* __restrict__ q, const float* __restrict__ pooled, const int* __restrict__ positions,
                     const int* __restrict__ token_seq, const int* __restrict__ slots,
                     const int* __restrict__ page_table, int max_pages, int* __restrict__ lists, int list_cap,
                     int n_heads, int n_kv, int d, float scale, int kernel, int stride, int block_size,
                     int init_blocks, int topk, int local_blocks, int dense_len, int sort_cap) {
    extern __shared__ __align__(16) unsigned char sm_raw[];
    const SelectionArrays arrays = selection_arrays(sm_raw, sort_cap);
    float* qs = (float*)(sm_raw + selection_bytes(sort_cap));                 // [group][d]
    const int group = n_heads / n_kv;
    float* stat_m = qs + group * d;                      // [warps][kMaxGroup]
    float* stat_l = stat_m + kSelectWarps * kMaxGroup;   // [warps][kMaxGroup]
    const int t = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    int* list = lists + ((int64_t)t * n_kv + kvh) * list_cap;
    const int p = positions[t];
    if (p + 1 <= dense_len) {
        if (tid == 0) list[0] = -2;
        return;
    }
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int per_page = kPageTokens / stride;
    const int n_vis = p + 1 >= kernel ? (p + 1 - kernel) / stride + 1 : 0;
    const Selection sel = selection_of(p, kernel, stride, block_size, init_blocks, local_blocks, sort_cap);
    if (tid == 0 && p / block_size - local_blocks + 1 - init_blocks > sort_cap) g_select_overflow = 1;
    clear_selection(sel, arrays);

    for (int i = tid; i < group * d; i += kSelectThreads)
        qs[i] = to_f32(q[((int64_t)t * n_heads + kvh * group) * d + i]);
    __syncthreads();

    // first walk: maximum and sum of exponentials per head (lane h keeps head h's)
    float dots[kMaxGroup];
    float my_m = -INFINITY, my_l = 0.f;
    for (int i = warp; i < n_vis; i += kSelectWarps) {
        group_dots<sizeof(T) == 2>(pooled_row(pooled, pages, i, stride, per_page, n_kv, kvh, d), qs, group, d, lane, scale, dots);
        float mine = -INFINITY;
#pragma unroll
        for (int h = 0; h < kMaxGroup; ++h)
            if (h == lane) mine = dots[h];
        if (lane < group) {
            const float m_new = fmaxf(my_m, mine);
            my_l = my_l * expf(my_m - m_new) + expf(mine - m_new);
            my_m = m_new;
        }
    }
    stat_m[warp * kMaxGroup + lane] = my_m;
    stat_l[warp * kMaxGroup + lane] = my_l;
    __syncthreads();
    float head_m = -INFINITY, head_inv = 0.f;           // of head ``lane``
    if (lane < group) {
        for (int w = 0; w < kSelectWarps; ++w) head_m = fmaxf(head_m, stat_m[w * kMaxGroup + lane]);
        float l = 0.f;
        for (int w = 0; w < kSelectWarps; ++w) {
            const float m = stat_m[w * kMaxGroup + lane];
            if (m != -INFINITY) l += stat_l[w * kMaxGroup + lane] * expf(m - head_m);
        }
        head_inv = l > 0.f ? 1.f / l : 0.f;
    }
    // second walk: probabilities, summed over the heads of the group
    for (int i = warp; i < n_vis; i += kSelectWarps) {
        group_dots<sizeof(T) == 2>(pooled_row(pooled, pages, i, stride, per_page, n_kv, kvh, d), qs, group, d, lane, scale, dots);
        float mine = 0.f;
#pragma unroll
        for (int h = 0; h < kMaxGroup; ++h)
            if (h == lane) mine = dots[h];
        const float prob = lane < group ? expf(mine - head_m) * head_inv : 0.f;
        const float total = warp_sum(prob);
        if (lane == 0) note_score(sel, arrays, init_blocks, i, total);
    }
    __syncthreads();

    finish_selection(sel, arrays, list, list_cap, init_blocks, topk);
}

// ---------------------------------------------------------------------------
// The same selection with the scores on the tensor cores (bf16 queries, groups of up to 16 heads).
// The 16 rows of an mma tile are the query heads of the group, the 8 columns pooled keys.  A pooled
// key enters as the sum of two bf16 numbers (the mean's rounding and the rounding of the remainder,
// stored so by pool_keys_kernel), so that the product with the bf16 query keeps about 16 bits beyond bf16.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mma_16816_sel(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// This thread's part of a pooled key: 8 consecutive dims of every 32-dim window, leading terms and residuals.
template <int D>
struct RawKey {
    uint4 lead[D / 32], rest[D / 32];
    __device__ __forceinline__ void load(const float* __restrict__ row, int j) {
        const bf16* terms = reinterpret_cast<const bf16*>(row);
#pragma unroll
        for (int w = 0; w < D / 32; ++w) {
            lead[w] = __ldg(reinterpret_cast<const uint4*>(terms + 32 * w + 8 * j));
            rest[w] = __ldg(reinterpret_cast<const uint4*>(terms + D + 32 * w + 8 * j));
        }
    }
};

// scaled scores (log2 domain) of the warp's tile: rows g, g+8; columns = pooled keys tile*8 + 2j, 2j+1
template <int D>
__device__ __forceinline__ void score_tile(float (&sc)[4], const uint4 (&qf)[2][D / 32], const RawKey<D>& raw,
                                           float scale_log2) {
    sc[0] = sc[1] = sc[2] = sc[3] = 0.f;
#pragma unroll
    for (int w = 0; w < D / 32; ++w) {
        const uint4 h = raw.lead[w], l = raw.rest[w];
        mma_16816_sel(sc, qf[0][w].x, qf[1][w].x, qf[0][w].y, qf[1][w].y, h.x, h.y);
        mma_16816_sel(sc, qf[0][w].x, qf[1][w].x, qf[0][w].y, qf[1][w].y, l.x, l.y);
        mma_16816_sel(sc, qf[0][w].z, qf[1][w].z, qf[0][w].w, qf[1][w].w, h.z, h.w);
        mma_16816_sel(sc, qf[0][w].z, qf[1][w].z, qf[0][w].w, qf[1][w].w, l.z, l.w);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) sc[i] *= scale_log2;
}

// kSelMmaWarps: 4 when there are many (token, kv head) pairs (prefill), 16 when there are few (decode).
template <int D, int kSelMmaWarps>
__global__ void __launch_bounds__(kSelMmaWarps * 32)
select_blocks_mma_kernel(const bf16* __restrict__ q, const float* __restrict__ pooled, const int* __restrict__ positions,
                         const int* __restrict__ token_seq, const int* __restrict__ slots,
                         const int* __restrict__ page_table, int max_pages, int* __restrict__ lists, int list_cap,
                         int n_heads, int n_kv, float scale_log2, int kernel, int stride, int block_size,
                         int init_blocks, int topk, int local_blocks, int dense_len, int sort_cap) {
    extern __shared__ __align__(16) unsigned char sm_raw[];
    const SelectionArrays arrays = selection_arrays(sm_raw, sort_cap);
    float* stat_m = (float*)(sm_raw + selection_bytes(sort_cap));            // [warps][16]
    float* stat_l = stat_m + kSelMmaWarps * 16;                              // [warps][16]
    const int t = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, j = lane & 3;
    int* list = lists + ((int64_t)t * n_kv + kvh) * list_cap;
    const int p = positions[t];
    if (p + 1 <= dense_len) {
        if (tid == 0) list[0] = -2;
        return;
    }
    const int group = n_heads / n_kv;
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int per_page = kPageTokens / stride;
    const int n_vis = p + 1 >= kernel ? (p + 1 - kernel) / stride + 1 : 0;
    const int n_tiles = (n_vis + 7) / 8;
    const Selection sel = selection_of(p, kernel, stride, block_size, init_blocks, local_blocks, sort_cap);
    if (tid == 0 && p / block_size - local_blocks + 1 - init_blocks > sort_cap) g_select_overflow = 1;
    clear_selection(sel, arrays);                       // the barrier between the two walks orders it

    uint4 qf[2][D / 32];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const bool ok = g + 8 * r < group;
        const bf16* qrow = q + ((int64_t)t * n_heads + kvh * group + (ok ? g + 8 * r : 0)) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
            qf[r][w] = ok ? v : make_uint4(0, 0, 0, 0);
        }
    }
    // first walk: maximum and sum of exponentials of every head (rows g and g + 8 of this thread)
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // As column g of a tile this thread loads pooled key tile*8 + g; the next tile's key is asked for
    // before the current one is worked on.
    // The page numbers of the keys two and three tiles ahead are asked for while the key one tile ahead is: a row's
    // address needs its page's number, and with both loads in one iteration a tile cost their two latencies in a row.
    const int page_shift = __ffs(per_page) - 1;             // the stride divides the page: per_page is a power of two
    auto page_of = [&](int tile) { return CPM_PAGE(pages, min(tile * 8 + g, n_vis - 1) >> page_shift, 0x7fffffff); };
    auto row_at = [&](int tile, int page) {
        return pooled + (((int64_t)page * n_kv + kvh) * per_page + (min(tile * 8 + g, n_vis - 1) & (per_page - 1))) * D;
    };
    RawKey<D> cur, nxt;
    int page1 = page_of(warp + kSelMmaWarps), page2 = page_of(warp + 2 * kSelMmaWarps);
    if (warp < n_tiles) cur.load(row_at(warp, page_of(warp)), j);
    for (int tile = warp; tile < n_tiles; tile += kSelMmaWarps) {
        if (tile + kSelMmaWarps < n_tiles) nxt.load(row_at(tile + kSelMmaWarps, page1), j);
        page1 = page2;
        page2 = page_of(tile + 3 * kSelMmaWarps);
        float sc[4];
        score_tile<D>(sc, qf, cur, scale_log2);
        cur = nxt;
        const int c0 = tile * 8 + 2 * j;
        if (c0 >= n_vis) sc[0] = sc[2] = -INFINITY;
        if (c0 + 1 >= n_vis) sc[1] = sc[3] = -INFINITY;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = fmaxf(sc[2 * r], sc[2 * r + 1]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m[r], mx);                       // finite: column 0 of a tile is always visible
            l[r] = l[r] * exp2f(m[r] - mn) + exp2f(sc[2 * r] - mn) + exp2f(sc[2 * r + 1] - mn);
            m[r] = mn;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (j == 0) {
            stat_m[warp * 16 + g + 8 * r] = m[r];
            stat_l[warp * 16 + g + 8 * r] = l[r];
        }
    }
    __syncthreads();
    float head_m[2], head_inv[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kSelMmaWarps; ++w) mx = fmaxf(mx, stat_m[w * 16 + row]);
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kSelMmaWarps; ++w) {
            const float mw = stat_m[w * 16 + row];
            if (mw != -INFINITY) sum += stat_l[w * 16 + row] * exp2f(mw - mx);
        }
        head_m[r] = mx;
        head_inv[r] = (row < group && sum > 0.f) ? 1.f / sum : 0.f;     // rows beyond the group count for nothing
    }
    // second walk: probabilities summed over the heads
    page1 = page_of(warp + kSelMmaWarps);
    page2 = page_of(warp + 2 * kSelMmaWarps);
    if (warp < n_tiles) cur.load(row_at(warp, page_of(warp)), j);
    for (int tile = warp; tile < n_tiles; tile += kSelMmaWarps) {
        if (tile + kSelMmaWarps < n_tiles) nxt.load(row_at(tile + kSelMmaWarps, page1), j);
        page1 = page2;
        page2 = page_of(tile + 3 * kSelMmaWarps);
        float sc[4];
        score_tile<D>(sc, qf, cur, scale_log2);
        cur = nxt;
        float col0 = exp2f(sc[0] - head_m[0]) * head_inv[0] + exp2f(sc[2] - head_m[1]) * head_inv[1];
        float col1 = exp2f(sc[1] - head_m[0]) * head_inv[0] + exp2f(sc[3] - head_m[1]) * head_inv[1];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            col0 += __shfl_xor_sync(0xffffffffu, col0, o);
            col1 += __shfl_xor_sync(0xffffffffu, col1, o);
        }
        const int c0 = tile * 8 + 2 * j;
        if (g == 0) {
            if (c0 < n_vis) note_score(sel, arrays, init_blocks, c0, col0);
            if (c0 + 1 < n_vis) note_score(sel, arrays, init_blocks, c0 + 1, col1);
        }
    }
    __syncthreads();
    finish_selection(sel, arrays, list, list_cap, init_blocks, topk);
}

// ---------------------------------------------------------------------------
// Few queries (decode): the pooled keys of one query are shared out over many blocks.
// With one block per (token, kv head) a decode step of two sequences keeps four SMs busy
// for the whole walk over some thousand pooled keys (measured 69 us a layer at 30,000
// cached tokens).  Here a first kernel, gridDim.x slices per (token, kv head), writes the
// raw scaled scores of its slice (log2 domain, [pooled key][16 heads]) and the slice's
// maximum and sum of exponentials per head; a second kernel, one block per (token, kv
// head), merges the statistics, turns scores into probabilities summed over the heads,
// and chooses the blocks as the one-kernel path does.
// ---------------------------------------------------------------------------
constexpr int kSliceWarps = 4;

template <int D>
__global__ void __launch_bounds__(kSliceWarps * 32)
select_scores_kernel(const bf16* __restrict__ q, const float* __restrict__ pooled, const int* __restrict__ positions,
                     const int* __restrict__ token_seq, const int* __restrict__ slots,
                     const int* __restrict__ page_table, int max_pages, int n_heads, int n_kv, float scale_log2,
                     int kernel, int stride, int dense_len, int max_entries, float* __restrict__ raw,
                     float* __restrict__ stats) {
    __shared__ float stat_m[kSliceWarps][16], stat_l[kSliceWarps][16];
    const int slice = blockIdx.x, n_slices = gridDim.x, kvh = blockIdx.y, t = blockIdx.z, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, j = lane & 3;
    pdl_launch_dependents();
    pdl_wait();
    const int p = positions[t];
    if (p + 1 <= dense_len) return;
    const int group = n_heads / n_kv;
    const int* pages = page_table + (int64_t)slots[token_seq[t]] * max_pages;
    const int per_page = kPageTokens / stride;
    const int n_vis = min(p + 1 >= kernel ? (p + 1 - kernel) / stride + 1 : 0, max_entries);
    const int n_tiles = (n_vis + 7) / 8;
    const int per_slice = (n_tiles + n_slices - 1) / n_slices;
    const int tile0 = slice * per_slice, tile1 = min(n_tiles, tile0 + per_slice);
    const int64_t unit = (int64_t)t * n_kv + kvh;
    float* my_raw = raw + unit * max_entries * 16;

    uint4 qf[2][D / 32];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const bool ok = g + 8 * r < group;
        const bf16* qrow = q + ((int64_t)t * n_heads + kvh * group + (ok ? g + 8 * r : 0)) * D + 8 * j;
#pragma unroll
        for (int w = 0; w < D / 32; ++w) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(qrow + 32 * w));
            qf[r][w] = ok ? v : make_uint4(0, 0, 0, 0);
        }
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    auto row_of = [&](int tile) {
        return pooled_row(pooled, pages, min(tile * 8 + g, n_vis - 1), stride, per_page, n_kv, kvh, D);
    };
    RawKey<D> cur, nxt;
    if (tile0 + warp < tile1) cur.load(row_of(tile0 + warp), j);
    for (int tile = tile0 + warp; tile < tile1; tile += kSliceWarps) {
        if (tile + kSliceWarps < tile1) nxt.load(row_of(tile + kSliceWarps), j);
        float sc[4];
        score_tile<D>(sc, qf, cur, scale_log2);
        cur = nxt;
        const int c0 = tile * 8 + 2 * j;
        if (c0 < n_vis) {
            my_raw[(int64_t)c0 * 16 + g] = sc[0];
            my_raw[(int64_t)c0 * 16 + g + 8] = sc[2];
        } else {
            sc[0] = sc[2] = -INFINITY;
        }
        if (c0 + 1 < n_vis) {
            my_raw[(int64_t)(c0 + 1) * 16 + g] = sc[1];
            my_raw[(int64_t)(c0 + 1) * 16 + g + 8] = sc[3];
        } else {
            sc[1] = sc[3] = -INFINITY;
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float mx = fmaxf(sc[2 * r], sc[2 * r + 1]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m[r], mx);                       // finite: column 0 of a tile is always visible
            l[r] = l[r] * exp2f(m[r] - mn) + exp2f(sc[2 * r] - mn) + exp2f(sc[2 * r + 1] - mn);
            m[r] = mn;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (j == 0) {
            stat_m[warp][g + 8 * r] = m[r];
            stat_l[warp][g + 8 * r] = l[r];
        }
    }
    __syncthreads();
    if (tid < 16) {
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kSliceWarps; ++w) mx = fmaxf(mx, stat_m[w][tid]);
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kSliceWarps; ++w)
            if (stat_m[w][tid] != -INFINITY) sum += stat_l[w][tid] * exp2f(stat_m[w][tid] - mx);
        float* out = stats + ((unit * n_slices + slice) * 16 + tid) * 2;
        out[0] = mx;
        out[1] = sum;
    }
}

constexpr int kFinishThreads = 512;

__global__ void __launch_bounds__(kFinishThreads)
select_finish_kernel(const float* __restrict__ raw, const float* __restrict__ stats, int n_slices,
                     const int* __restrict__ positions, int* __restrict__ lists, int list_cap, int n_heads, int n_kv,
                     int kernel, int stride, int block_size, int init_blocks, int topk, int local_blocks, int dense_len,
                     int max_entries, int sort_cap) {
    extern __shared__ __align__(16) unsigned char sm_raw[];
    const SelectionArrays arrays = selection_arrays(sm_raw, sort_cap);
    __shared__ float head_m[16], head_inv[16];
    const int t = blockIdx.x, kvh = blockIdx.y, tid = threadIdx.x;
    int* list = lists + ((int64_t)t * n_kv + kvh) * list_cap;
    // The step's positions are written before the step's first kernel, by a launch that everything after it waits
    // for in full; the arrays cleared here are this block's own.  Only the scores need the kernel ahead.
    pdl_launch_dependents();
    const int p = positions[t];
    const int group = n_heads / n_kv;
    const int64_t unit = (int64_t)t * n_kv + kvh;
    const int n_vis = min(p + 1 >= kernel ? (p + 1 - kernel) / stride + 1 : 0, max_entries);
    const Selection sel = selection_of(p, kernel, stride, block_size, init_blocks, local_blocks, sort_cap);
    if (p + 1 > dense_len) clear_selection(sel, arrays);
    pdl_wait();
    if (p + 1 <= dense_len) {
        if (tid == 0) list[0] = -2;
        return;
    }
    if (tid == 0 && p / block_size - local_blocks + 1 - init_blocks > sort_cap) g_select_overflow = 1;
    {
        // The slices' statistics, merged by all threads: thread (head = tid % 16, lot = tid / 16) takes the slices
        // lot, lot + 32, ... (sixteen threads walking them one after the other waited for one load at a time:
        // 23 us at 74 slices), then sixteen threads merge the 32 lots.
        __shared__ float lot_m[kFinishThreads / 16][16], lot_l[kFinishThreads / 16][16];
        const int head = tid & 15, lot = tid >> 4;
        const float* st = stats + unit * n_slices * 32 + head * 2;
        float mx = -INFINITY, sum = 0.f;
        for (int s = lot; s < n_slices; s += kFinishThreads / 16) {
            const float m = st[s * 32], l = st[s * 32 + 1];
            if (m != -INFINITY) {
                const float mn = fmaxf(mx, m);
                sum = sum * exp2f(mx - mn) + l * exp2f(m - mn);
                mx = mn;
            }
        }
        lot_m[lot][head] = mx;
        lot_l[lot][head] = sum;
        __syncthreads();
        if (tid < 16) {
            float all_m = -INFINITY;
#pragma unroll
            for (int i = 0; i < kFinishThreads / 16; ++i) all_m = fmaxf(all_m, lot_m[i][tid]);
            float all_l = 0.f;
#pragma unroll
            for (int i = 0; i < kFinishThreads / 16; ++i)
                if (lot_m[i][tid] != -INFINITY) all_l += lot_l[i][tid] * exp2f(lot_m[i][tid] - all_m);
            head_m[tid] = all_m;
            head_inv[tid] = (tid < group && all_l > 0.f) ? 1.f / all_l : 0.f;   // rows beyond the group count for nothing
        }
    }
    __syncthreads();
    // a thread's next row is asked for before its current one is worked on
    const float* my_raw = raw + unit * max_entries * 16;
    float4 next[4];
    if (tid < n_vis) {
        const float4* row = reinterpret_cast<const float4*>(my_raw + (int64_t)tid * 16);
#pragma unroll
        for (int c = 0; c < 4; ++c) next[c] = row[c];
    }
    for (int i = tid; i < n_vis; i += kFinishThreads) {
        float4 v[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] = next[c];
        if (i + kFinishThreads < n_vis) {
            const float4* row = reinterpret_cast<const float4*>(my_raw + (int64_t)(i + kFinishThreads) * 16);
#pragma unroll
            for (int c = 0; c < 4; ++c) next[c] = row[c];
        }
        float total = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            total += exp2f(v[c].x - head_m[4 * c]) * head_inv[4 * c] + exp2f(v[c].y - head_m[4 * c + 1]) * head_inv[4 * c + 1]
                   + exp2f(v[c].z - head_m[4 * c + 2]) * head_inv[4 * c + 2] + exp2f(v[c].w - head_m[4 * c + 3]) * head_inv[4 * c + 3];
        }
        note_score(sel, arrays, init_blocks, i, total);
    }
    __syncthreads();
    finish_selection(sel, arrays, list, list_cap, init_blocks, topk);
}

// Floats of scratch the two-kernel path needs (raw scores and slice statistics).
CPM_API int64_t cpm_select_blocks_scratch_floats(int n_tokens, int n_kv, int max_entries, int n_slices) {
    return (int64_t)n_tokens * n_kv * ((int64_t)max_entries * 16 + (int64_t)n_slices * 32);
}

static int next_pow2(int n) {
    int v = 1;
    while (v < n) v <<= 1;
    return v;
}

template <int D>
static int launch_select_mma(const void* q, const float* pooled, const int* positions, const int* token_seq,
                             const int* slots, const int* page_table, int max_pages, int* lists, int list_cap,
                             int n_tokens, int n_heads, int n_kv, float scale, int kernel, int stride, int block_size,
                             int init_blocks, int topk, int local_blocks, int dense_len, int sort_cap,
                             cudaStream_t stream) {
    const size_t smem = selection_bytes(sort_cap) + 2 * 16 * 16 * sizeof(float);
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    const bool few = n_tokens * n_kv < 148;
    auto kern = few ? select_blocks_mma_kernel<D, 16> : select_blocks_mma_kernel<D, 4>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    kern<<<dim3(n_tokens, n_kv), few ? 512 : 128, smem, stream>>>((const bf16*)q, pooled, positions, token_seq, slots,
        page_table, max_pages, lists, list_cap, n_heads, n_kv, scale * 1.4426950408889634f, kernel, stride, block_size,
        init_blocks, topk, local_blocks, dense_len, sort_cap);
    return launch_status();
}

// max_entries: an upper bound on the pooled keys any query of the step sees (longest sequence / stride + 1); it
// sizes the keys of the candidate blocks (``sort_cap`` of them), 8 bytes of shared memory per block.
template <int D>
static int launch_select_sliced(const void* q, const float* pooled, const int* positions, const int* token_seq,
                                const int* slots, const int* page_table, int max_pages, int* lists, int list_cap,
                                int n_tokens, int n_heads, int n_kv, float scale, int kernel, int stride, int block_size,
                                int init_blocks, int topk, int local_blocks, int dense_len, int max_entries, int sort_cap,
                                float* scratch, int n_slices, cudaStream_t stream) {
    const size_t smem = selection_bytes(sort_cap);
    if (smem > 200 * 1024 || n_tokens > 65535) return CPM_BAD_ARGUMENT;
    float* raw = scratch;
    float* stats = scratch + (int64_t)n_tokens * n_kv * max_entries * 16;
    cpm_launch(kLaunchAttention, select_scores_kernel<D>, dim3(n_slices, n_kv, n_tokens), kSliceWarps * 32, 0, stream,
               (const bf16*)q, pooled, positions, token_seq, slots, page_table, max_pages, n_heads, n_kv,
               scale * 1.4426950408889634f, kernel, stride, dense_len, max_entries, raw, stats);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(select_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    cpm_launch(kLaunchAttention, select_finish_kernel, dim3(n_tokens, n_kv), kFinishThreads, smem, stream,
               (const float*)raw, (const float*)stats, n_slices, positions, lists, list_cap, n_heads, n_kv, kernel, stride,
               block_size, init_blocks, topk, local_blocks, dense_len, max_entries, sort_cap);
    return launch_status();
}

// scratch/n_slices: with scratch of cpm_select_blocks_scratch_floats(n_tokens, n_kv, max_entries, n_slices) floats and
// n_slices >= 1, bf16 queries of groups up to 16 heads take the two-kernel path that shares a query's pooled keys out
// over n_slices blocks (for steps of few tokens); it launches two kernels.
CPM_API int cpm_select_blocks(const void* q, const float* pooled, const int* positions, const int* token_seq,
                              const int* slots, const int* page_table, int max_pages, int* lists, int list_cap,
                              int n_tokens, int n_heads, int n_kv, int d, float scale, int kernel, int stride,
                              int block_size, int init_blocks, int topk, int local_blocks, int dense_len,
                              int max_entries, int dtype, float* scratch, int n_slices, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (stride <= 0 || kernel % stride || block_size % stride || kPageTokens % stride || n_kv > 65535 ||
        n_heads % n_kv || n_heads / n_kv > kMaxGroup || d % 4 || list_cap < topk + local_blocks + 1 || max_entries < 1)
        return CPM_BAD_ARGUMENT;
    const int sort_cap = next_pow2(max_entries / (block_size / stride) + 2);
    const int group = n_heads / n_kv;
    if (dtype == CPM_BF16 && group <= 16 && scratch != nullptr && n_slices >= 1 && n_slices <= 65535) {
#define CPM_SELECT_SLICED(DD) return launch_select_sliced<DD>(q, pooled, positions, token_seq, slots, page_table, max_pages, \
        lists, list_cap, n_tokens, n_heads, n_kv, scale, kernel, stride, block_size, init_blocks, topk, local_blocks, \
        dense_len, max_entries, sort_cap, scratch, n_slices, stream)
        if (d == 32) CPM_SELECT_SLICED(32);
        if (d == 64) CPM_SELECT_SLICED(64);
        if (d == 96) CPM_SELECT_SLICED(96);
        if (d == 128) CPM_SELECT_SLICED(128);
#undef CPM_SELECT_SLICED
    }
    if (dtype == CPM_BF16 && group <= 16) {
#define CPM_SELECT_MMA(DD) return launch_select_mma<DD>(q, pooled, positions, token_seq, slots, page_table, max_pages, lists, \
        list_cap, n_tokens, n_heads, n_kv, scale, kernel, stride, block_size, init_blocks, topk, local_blocks, dense_len, \
        sort_cap, stream)
        if (d == 32) CPM_SELECT_MMA(32);
        if (d == 64) CPM_SELECT_MMA(64);
        if (d == 96) CPM_SELECT_MMA(96);
        if (d == 128) CPM_SELECT_MMA(128);
#undef CPM_SELECT_MMA
    }
    const size_t smem = selection_bytes(sort_cap)
                        + ((size_t)group * d + 2 * kSelectWarps * kMaxGroup) * sizeof(float);
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    dim3 grid(n_tokens, n_kv);
    cudaError_t e = cudaSuccess;
    if (dtype == CPM_BF16) {
        auto kern = select_blocks_kernel<bf16>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, kSelectThreads, smem, stream>>>((const bf16*)q, pooled, positions, token_seq, slots, page_table, max_pages,
            lists, list_cap, n_heads, n_kv, d, scale, kernel, stride, block_size, init_blocks, topk, local_blocks,
            dense_len, sort_cap);
    } else {
        auto kern = select_blocks_kernel<float>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, kSelectThreads, smem, stream>>>((const float*)q, pooled, positions, token_seq, slots, page_table, max_pages,
            lists, list_cap, n_heads, n_kv, d, scale, kernel, stride, block_size, init_blocks, topk, local_blocks,
            dense_len, sort_cap);
    }
    return launch_status();
}

CPM_BOUNDS_TU(sparse)
