// Choosing the next token from fp32 logits: greedy, or temperature with an optional
// nucleus (top-p).  One block per row.
//
// The reference samples with torch on a logits row of the storage type:
// argmax, or multinomial(softmax(logits / temperature)) (cpmcu/llm.py:282-285).
// Here the row is fp32, ties of the greedy choice go to the lowest index, and the
// random number of a row is a counter-based Philox value keyed by
// (seed, sequence key, step key), so a sequence's draws do not depend on what
// else is in the batch.
#include "common.cuh"
#include <math.h>

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ void philox_round(uint32_t& c0, uint32_t& c1, uint32_t& c2, uint32_t& c3,
                                             uint32_t k0, uint32_t k1) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
}

// Philox4x32-10; returns a uniform number in [0, 1) with 24 random bits.
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t a, uint32_t b) {
    uint32_t c0 = a, c1 = b, c2 = 0u, c3 = 0u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        philox_round(c0, c1, c2, c3, k0, k1);
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, int64_t ld, int vocab, int* __restrict__ out,
                   const float* __restrict__ temperature, const float* __restrict__ top_p,
                   uint64_t seed, const int* __restrict__ seq_key, const int* __restrict__ step_key) {
    __shared__ ArgMax am_scratch[33];
    __shared__ float f_scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float thread_sums[kSampleThreads];
    __shared__ int chosen;
    const int row = blockIdx.x;
    const float* z = logits + (int64_t)row * ld;
    const int tid = threadIdx.x;

    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += blockDim.x) best = better(best, ArgMax{z[i], i});
    best = block_argmax(best, am_scratch);
    const float temp = temperature ? temperature[row] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) out[row] = best.i;
        return;
    }
    const float mx = best.v;
    const float inv_t = 1.0f / temp;

    // total mass
    float part = 0.f;
    for (int i = tid; i < vocab; i += blockDim.x) part += expf((z[i] - mx) * inv_t);
    const float total = block_sum(part, f_scratch);

    // nucleus: the largest threshold whose kept mass still reaches top_p * total
    float threshold = 0.f;
    const float p_keep = top_p ? top_p[row] : 1.f;
    if (p_keep < 1.f) {
        const float need = p_keep * total;
        uint32_t lo = 0u, hi = __float_as_uint(1.0f) + 1u;    // mass(lo) >= need, mass(hi) < need
        while (hi - lo > 1u) {
            const uint32_t mid = lo + ((hi - lo) >> 1);
            const float th = __uint_as_float(mid);
            float s = 0.f;
            for (int i = tid; i < vocab; i += blockDim.x) {
                const float w = expf((z[i] - mx) * inv_t);
                if (w >= th) s += w;
            }
            s = block_sum(s, f_scratch);
            if (s >= need) lo = mid; else hi = mid;
        }
        threshold = __uint_as_float(lo);
    }

    // inverse CDF over the kept entries in index order; a thread owns a contiguous range
    const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = min(vocab, tid * chunk), end = min(vocab, begin + chunk);
    float mine = 0.f;
    for (int i = begin; i < end; ++i) {
        const float w = expf((z[i] - mx) * inv_t);
        if (w >= threshold) mine += w;
    }
    thread_sums[tid] = mine;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            const float s = thread_sums[t];
            thread_sums[t] = run;       // exclusive prefix
            run += s;
        }
        f_scratch[0] = run;             // kept mass
    }
    __syncthreads();
    const float kept = f_scratch[0];
    const float u = philox_uniform(seed, (uint32_t)seq_key[row], (uint32_t)step_key[row]);
    const float target = u * kept;
    const float before = thread_sums[tid];
    if (mine > 0.f && before <= target && target < before + mine) {
        float run = before;
        int pick = -1, last = -1;
        for (int i = begin; i < end; ++i) {
            const float w = expf((z[i] - mx) * inv_t);
            if (w >= threshold) {
                run += w;
                last = i;
                if (run > target) { pick = i; break; }
            }
        }
        chosen = pick >= 0 ? pick : last;
    }
    __syncthreads();
    if (tid == 0) out[row] = chosen >= 0 ? chosen : best.i;
}

CPM_API int cpm_sample_rows(const float* logits, int64_t ld, int n_rows, int vocab, int* out,
                            const float* temperature, const float* top_p, uint64_t seed,
                            const int* seq_key, const int* step_key, cudaStream_t stream) {
    if (n_rows <= 0) return CPM_OK;
    if (vocab <= 0) return CPM_BAD_ARGUMENT;
    if (temperature && (!seq_key || !step_key)) return CPM_BAD_ARGUMENT;
    cpm_launch(kLaunchOther, sample_rows_kernel, n_rows, kSampleThreads, 0, stream, logits, ld, vocab, out, temperature, top_p, seed,
               seq_key, step_key);
    return launch_status();
}
