// Row-wise kernels of a step: embedding lookup, residual add + RMS norm, the gated
// activation, and rotary position encoding fused with the store into the cache.
// All arithmetic is fp32; only loads and stores touch the storage type.
#include "common.cuh"

int g_cpm_pdl = kDefaultPdlMask;

// Which classes of kernels are launched with programmatic dependent launch (a mask over LaunchClass; 0: none;
// negative: the default mask).
CPM_API void cpm_set_pdl(int mask) { g_cpm_pdl = mask < 0 ? kDefaultPdlMask : mask; }

// ---------------------------------------------------------------------------
// Embedding rows times a scale, into the fp32 residual stream.
// The reference gathers rows (src/model/embedding.cuh:7-20) and scales them in a
// second kernel with the scale rounded to the storage type
// (src/model/elementwise.cuh:34-41); here the product is formed once in fp32.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                  float* __restrict__ out, int hidden, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t row = ids[blockIdx.x];
    const T* src = table + row * hidden;
    float* dst = out + (int64_t)blockIdx.x * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_f32(src[c]) * scale;
}

CPM_API int cpm_embed_rows(const int* ids, const void* table, float* out, int n_tokens, int hidden,
                           float scale, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchOther, embed_rows_kernel<bf16>, n_tokens, threads, 0, stream, ids, (const bf16*)table, out, hidden, scale);
    else
        cpm_launch(kLaunchOther, embed_rows_kernel<float>, n_tokens, threads, 0, stream, ids, (const float*)table, out, hidden, scale);
    return launch_status();
}

// ---------------------------------------------------------------------------
// x += alpha * delta (fp32 sum), y = x * rsqrt(mean(x^2) + eps) * w.
// The reference adds in the storage type inside its norm kernel
// (src/model/norm.cuh:53-99) after scaling the addend in a kernel of its own
// (src/model/layer.cuh:48-50, 63); here the scale, the add and the norm are one
// pass and the sum stays in fp32.
// rows != nullptr: only the listed rows are normed, y is compact [n_rows, hidden]
// and x is left as it is.
// ---------------------------------------------------------------------------
// Four consecutive elements (16-byte or 8-byte aligned) as floats, and back.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, typename W>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, float alpha,
                                   const W* __restrict__ w, T* __restrict__ y,
                                   const int* __restrict__ rows, int hidden, float eps, int write_back) {
    extern __shared__ float row_cache[];   // hidden floats + 33
    float* scratch = row_cache + hidden;
    pdl_launch_dependents();
    pdl_wait();
    const int64_t src_row = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + src_row * hidden;
    const T* dr = delta ? delta + src_row * hidden : nullptr;
    float ss = 0.f;
    if ((hidden & 3) == 0) {
        // four elements per thread and step: 16-byte loads of the fp32 stream, one load of the addend's four
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            float4 v = *reinterpret_cast<const float4*>(xr + c);
            if (dr) {
                const float4 d4 = load4(dr + c);
                v.x = fmaf(alpha, d4.x, v.x);
                v.y = fmaf(alpha, d4.y, v.y);
                v.z = fmaf(alpha, d4.z, v.z);
                v.w = fmaf(alpha, d4.w, v.w);
                if (write_back) *reinterpret_cast<float4*>(xr + c) = v;
            }
            *reinterpret_cast<float4*>(row_cache + c) = v;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            float v = xr[c];
            if (dr) {
                v = fmaf(alpha, to_f32(dr[c]), v);
                if (write_back) xr[c] = v;
            }
            row_cache[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float r = rsqrtf(total / (float)hidden + eps);
    T* yr = y + (int64_t)blockIdx.x * hidden;
    if ((hidden & 3) == 0) {
        for (int c = 4 * threadIdx.x; c < hidden; c += 4 * blockDim.x) {
            const float4 v = *reinterpret_cast<const float4*>(row_cache + c);
            const float4 w4 = load4(w + c);
            store4(yr + c, make_float4(v.x * r * w4.x, v.y * r * w4.y, v.z * r * w4.z, v.w * r * w4.w));
        }
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x)
            yr[c] = from_f32<T>(row_cache[c] * r * to_f32(w[c]));
    }
}

template <typename T, typename W>
static int launch_add_rmsnorm(float* x, const void* delta, float alpha, const void* w, void* y, const int* rows,
                              int n_rows, int hidden, float eps, int write_back, cudaStream_t stream) {
    const size_t smem = (size_t)(hidden + 33) * sizeof(float);
    if (smem > 227 * 1024) return CPM_BAD_ARGUMENT;
    auto kern = add_rmsnorm_kernel<T, W>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : 128);
    cpm_launch(kLaunchNorm, kern, n_rows, threads, smem, stream, x, (const T*)delta, alpha, (const W*)w, (T*)y, rows, hidden, eps, write_back);
    return launch_status();
}

CPM_API int cpm_add_rmsnorm(float* x, const void* delta, float alpha, const void* w, int w_is_f32, void* y,
                            const int* rows, int n_rows, int hidden, float eps, int write_back, int dtype,
                            cudaStream_t stream) {
    if (n_rows <= 0) return CPM_OK;
    if (dtype == CPM_BF16) {
        if (w_is_f32) return launch_add_rmsnorm<bf16, float>(x, delta, alpha, w, y, rows, n_rows, hidden, eps, write_back, stream);
        return launch_add_rmsnorm<bf16, bf16>(x, delta, alpha, w, y, rows, n_rows, hidden, eps, write_back, stream);
    }
    if (!w_is_f32) return CPM_BAD_ARGUMENT;
    return launch_add_rmsnorm<float, float>(x, delta, alpha, w, y, rows, n_rows, hidden, eps, write_back, stream);
}

// x += alpha * delta, for a residual that no norm follows.
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ x, const T* __restrict__ delta, float alpha, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = fmaf(alpha, to_f32(delta[i]), x[i]);
}

CPM_API int cpm_residual_add(float* x, const void* delta, float alpha, int64_t n, int dtype, cudaStream_t stream) {
    if (n <= 0) return CPM_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == CPM_BF16) residual_add_kernel<bf16><<<blocks, threads, 0, stream>>>(x, (const bf16*)delta, alpha, n);
    else residual_add_kernel<float><<<blocks, threads, 0, stream>>>(x, (const float*)delta, alpha, n);
    return launch_status();
}

// ---------------------------------------------------------------------------
// h[t, c] = silu(gu[t, c]) * gu[t, inter + c]; a row of gu is [gate | up]
// (src/model/activation.cuh:6-18, src/model/ffn.cuh:38-50).
// ---------------------------------------------------------------------------
// interleave == 0: a row is [gate(inter) | up(inter)].  interleave == 8: a row is made of blocks of
// 16, the 8 gate values of 8 features followed by their 8 up values (the layout the fused
// decode product wants).  Two features per thread.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ h, int inter, int interleave) {
    const int c = 2 * (blockIdx.y * blockDim.x + threadIdx.x);
    if (c >= inter) return;
    const T* row = gu + (int64_t)blockIdx.x * 2 * inter;
    T* out = h + (int64_t)blockIdx.x * inter;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int f = c + e;
        if (f >= inter) break;
        const int gi = interleave ? (f / interleave) * 2 * interleave + f % interleave : f;
        const int ui = interleave ? gi + interleave : inter + f;
        const float g = to_f32(row[gi]);
        const float u = to_f32(row[ui]);
        const float s = 1.0f / (1.0f + expf(-g));
        out[f] = from_f32<T>(g * s * u);
    }
}

// bf16 rows in the interleaved layout: a thread takes one block of 8 features with three 16-byte accesses.
__global__ void silu_mul_bf16_blocks_kernel(const bf16* __restrict__ gu, bf16* __restrict__ h, int inter) {
    const int blk = blockIdx.y * blockDim.x + threadIdx.x;          // block of 8 features
    if (blk * 8 >= inter) return;
    const uint4* src = reinterpret_cast<const uint4*>(gu + (int64_t)blockIdx.x * 2 * inter + (int64_t)blk * 16);
    const uint4 gv = src[0], uv = src[1];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
        const float a = g.x * (1.0f / (1.0f + expf(-g.x))) * u.x;
        const float b = g.y * (1.0f / (1.0f + expf(-g.y))) * u.y;
        o2[i] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<uint4*>(h + (int64_t)blockIdx.x * inter + (int64_t)blk * 8) = ov;
}

CPM_API int cpm_silu_mul(const void* gu, void* h, int n_tokens, int inter, int interleave, int dtype,
                         cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (interleave != 0 && (interleave != 8 || inter % 8 != 0)) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_BF16 && interleave == 8) {
        dim3 grid(n_tokens, (inter / 8 + 255) / 256);
        silu_mul_bf16_blocks_kernel<<<grid, 256, 0, stream>>>((const bf16*)gu, (bf16*)h, inter);
        return launch_status();
    }
    dim3 grid(n_tokens, (inter + 511) / 512);
    if (grid.y > 65535) return CPM_BAD_ARGUMENT;
    if (dtype == CPM_BF16) silu_mul_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)gu, (bf16*)h, inter, interleave);
    else silu_mul_kernel<float><<<grid, 256, 0, stream>>>((const float*)gu, (float*)h, inter, interleave);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Rotary encoding of queries and keys, and the store of keys and values into
// the paged cache.  Pairs are (c, c + rot_dim/2) inside the first rot_dim
// dimensions of a head, angle = position * inv_freq[c] formed and evaluated in
// fp32 with the accurate sincosf (src/model/rotary.cuh:6-34 uses the same pairing
// but the fast-math cos/sin).  cos and sin are multiplied by ``magnitude`` (the
// LongRoPE attention factor).  inv_freq == nullptr: no rotation.
// qkv row: [heads*d | kv_heads*d | kv_heads*d].
// ---------------------------------------------------------------------------
constexpr int kRopeHeadsPerBlock = 4;

template <typename T>
__global__ void rope_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const int* __restrict__ positions, const int* __restrict__ token_seq,
                                  const int* __restrict__ slots, const int* __restrict__ page_table,
                                  int max_pages, const float* __restrict__ inv_freq, float magnitude,
                                  int n_heads, int n_kv, int d, int rot_dim) {
    extern __shared__ float cs_table[];       // cos[half], sin[half] of this token
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rot_dim >> 1;
    const int64_t row_stride = (int64_t)(n_heads + 2 * n_kv) * d;
    const T* row = qkv + t * row_stride;
    const int n_all = n_heads + (k_cache ? 2 * n_kv : 0);       // q heads, then k heads, then v heads
    const int h_begin = blockIdx.y * kRopeHeadsPerBlock;
    const int h_end = min(n_all, h_begin + kRopeHeadsPerBlock);
    if (h_begin >= h_end) return;

    for (int c = threadIdx.x; c < half; c += blockDim.x) {
        float cs = 1.f, sn = 0.f;
        if (inv_freq) {
            const float angle = (float)pos * inv_freq[c];
            sincosf(angle, &sn, &cs);
            cs *= magnitude;
            sn *= magnitude;
        }
        cs_table[c] = cs;
        cs_table[half + c] = sn;
    }
    __syncthreads();

    int64_t k_base = 0, v_base = 0;
    if (k_cache) {
        const int slot = slots[token_seq[t]];
        const int page = CPM_PAGE(page_table + (int64_t)slot * max_pages, pos / kPageTokens, max_pages);
        k_base = page_row_offset(page, 0, pos % kPageTokens, n_kv, d);
        v_base = value_offset(page, 0, 0, pos % kPageTokens, n_kv, d);
    }
    const int64_t head_stride_in_page = (int64_t)kPageTokens * d;
    for (int h = h_begin; h < h_end; ++h) {
        const T* src = row + (int64_t)h * d;
        if (h >= n_heads + n_kv) {                               // a value head: transposed store
            const int kvh = h - n_heads - n_kv;
            for (int c = threadIdx.x; c < d; c += blockDim.x)
                v_cache[v_base + ((int64_t)kvh * d + c) * kPageTokens] = src[c];
            continue;
        }
        T* dst = h < n_heads ? q_out + ((int64_t)t * n_heads + h) * d
                             : k_cache + k_base + (int64_t)(h - n_heads) * head_stride_in_page;
        for (int c = threadIdx.x; c < half; c += blockDim.x) {
            const float cs = cs_table[c], sn = cs_table[half + c];
            const float a = to_f32(src[c]);
            const float b = to_f32(src[c + half]);
            dst[c] = from_f32<T>(a * cs - b * sn);
            dst[c + half] = from_f32<T>(a * sn + b * cs);
        }
        for (int c = rot_dim + threadIdx.x; c < d; c += blockDim.x) dst[c] = src[c];
    }
}

// The same for bf16 with all of a head rotated (rot_dim == d, a multiple of 16): a thread takes eight pairs,
// two 16-byte loads and two 16-byte stores; value heads are copied 16 elements per thread (their store is
// transposed, one element per 128 bytes).  heads_per_block: all heads of a token for prompts, a few for
// decode steps, where the tokens alone would not fill the GPU.
__global__ void rope_store_vec_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q_out,
                                      bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                      const int* __restrict__ positions, const int* __restrict__ token_seq,
                                      const int* __restrict__ slots, const int* __restrict__ page_table,
                                      int max_pages, const float* __restrict__ inv_freq, float magnitude,
                                      int n_heads, int n_kv, int d, int heads_per_block) {
    extern __shared__ float cs_table[];       // cos[half], sin[half] of this token
    pdl_launch_dependents();
    // Positions, slots and page tables were written before this step's kernels began; the angles and the page are
    // worked out from them while the product ahead of this kernel is still finishing.  Only qkv needs the wait.
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = d >> 1;
    const int64_t row_stride = (int64_t)(n_heads + 2 * n_kv) * d;
    const bf16* row = qkv + t * row_stride;
    const int n_all = n_heads + (k_cache ? 2 * n_kv : 0);
    const int h_begin = blockIdx.y * heads_per_block;
    const int h_end = min(n_all, h_begin + heads_per_block);
    if (h_begin >= h_end) return;

    for (int c = threadIdx.x; c < half; c += blockDim.x) {
        float cs = 1.f, sn = 0.f;
        if (inv_freq) {
            const float angle = (float)pos * inv_freq[c];
            sincosf(angle, &sn, &cs);
            cs *= magnitude;
            sn *= magnitude;
        }
        cs_table[c] = cs;
        cs_table[half + c] = sn;
    }

    int64_t k_base = 0, v_base = 0;
    if (k_cache && h_end > n_heads) {                            // only blocks with key or value heads look the page up
        const int slot = slots[token_seq[t]];
        const int page = CPM_PAGE(page_table + (int64_t)slot * max_pages, pos / kPageTokens, max_pages);
        k_base = page_row_offset(page, 0, pos % kPageTokens, n_kv, d);
        v_base = value_offset(page, 0, 0, pos % kPageTokens, n_kv, d);
    }
    __syncthreads();
    pdl_wait();
    const int per_head = d >> 4;                                 // items of 16 elements in a head
    const int items = (h_end - h_begin) * per_head;
    for (int item = threadIdx.x; item < items; item += blockDim.x) {
        const int h = h_begin + item / per_head, part = item % per_head;
        const bf16* src = row + (int64_t)h * d;
        if (h >= n_heads + n_kv) {                               // a value head: transposed store
            const int kvh = h - n_heads - n_kv;
            const uint4 a = *reinterpret_cast<const uint4*>(src + 16 * part);
            const uint4 b = *reinterpret_cast<const uint4*>(src + 16 * part + 8);
            const bf16* ea = reinterpret_cast<const bf16*>(&a);
            const bf16* eb = reinterpret_cast<const bf16*>(&b);
            bf16* dst = v_cache + v_base + ((int64_t)kvh * d + 16 * part) * kPageTokens;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                dst[(int64_t)e * kPageTokens] = ea[e];
                dst[(int64_t)(e + 8) * kPageTokens] = eb[e];
            }
            continue;
        }
        bf16* dst = h < n_heads ? q_out + ((int64_t)t * n_heads + h) * d
                                : k_cache + k_base + (int64_t)(h - n_heads) * kPageTokens * d;
        const int c = 8 * part;                                  // pairs (c + e, c + e + half)
        const uint4 lo = *reinterpret_cast<const uint4*>(src + c);
        const uint4 hi = *reinterpret_cast<const uint4*>(src + c + half);
        const __nv_bfloat162* lo2 = reinterpret_cast<const __nv_bfloat162*>(&lo);
        const __nv_bfloat162* hi2 = reinterpret_cast<const __nv_bfloat162*>(&hi);
        uint4 out_lo, out_hi;
        __nv_bfloat162* ol = reinterpret_cast<__nv_bfloat162*>(&out_lo);
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out_hi);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 a = __bfloat1622float2(lo2[e]), b = __bfloat1622float2(hi2[e]);
            const float c0 = cs_table[c + 2 * e], s0 = cs_table[half + c + 2 * e];
            const float c1 = cs_table[c + 2 * e + 1], s1 = cs_table[half + c + 2 * e + 1];
            ol[e] = __floats2bfloat162_rn(a.x * c0 - b.x * s0, a.y * c1 - b.y * s1);
            oh[e] = __floats2bfloat162_rn(a.x * s0 + b.x * c0, a.y * s1 + b.y * c1);
        }
        *reinterpret_cast<uint4*>(dst + c) = out_lo;
        *reinterpret_cast<uint4*>(dst + c + half) = out_hi;
    }
}

CPM_API int cpm_rope_store(const void* qkv, void* q_out, void* k_cache, void* v_cache, const int* positions,
                           const int* token_seq, const int* slots, const int* page_table, int max_pages,
                           const float* inv_freq, float magnitude, int n_tokens, int n_heads, int n_kv, int d,
                           int rot_dim, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return CPM_OK;
    if (rot_dim < 0 || rot_dim > d || (rot_dim & 1)) return CPM_BAD_ARGUMENT;
    if ((k_cache == nullptr) != (v_cache == nullptr)) return CPM_BAD_ARGUMENT;
    const int n_all = n_heads + (k_cache ? 2 * n_kv : 0);
    if (dtype == CPM_BF16 && rot_dim == d && d % 16 == 0 && d >= 16 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 &&
        ((uintptr_t)k_cache & 15) == 0) {
        const int heads_per_block = n_tokens >= 64 ? n_all : kRopeHeadsPerBlock;
        const int items = heads_per_block * (d / 16);
        const int threads = items >= 256 ? 256 : ((items + 31) / 32) * 32;
        dim3 vgrid(n_tokens, (n_all + heads_per_block - 1) / heads_per_block);
        if (vgrid.y > 65535) return CPM_BAD_ARGUMENT;
        cpm_launch(kLaunchRope, rope_store_vec_kernel, vgrid, threads, (size_t)d * sizeof(float), stream, (const bf16*)qkv, (bf16*)q_out,
                   (bf16*)k_cache, (bf16*)v_cache, positions, token_seq, slots, page_table, max_pages, inv_freq, magnitude,
                   n_heads, n_kv, d, heads_per_block);
        return launch_status();
    }
    dim3 grid(n_tokens, (n_all + kRopeHeadsPerBlock - 1) / kRopeHeadsPerBlock);
    if (grid.y > 65535) return CPM_BAD_ARGUMENT;
    const int threads = d >= 128 ? 64 : 32;
    const size_t smem = (size_t)(rot_dim > 0 ? rot_dim : 2) * sizeof(float);
    if (dtype == CPM_BF16)
        cpm_launch(kLaunchRope, rope_store_kernel<bf16>, grid, threads, smem, stream, (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache,
            (bf16*)v_cache, positions, token_seq, slots, page_table, max_pages, inv_freq, magnitude, n_heads, n_kv, d, rot_dim);
    else
        cpm_launch(kLaunchRope, rope_store_kernel<float>, grid, threads, smem, stream, (const float*)qkv, (float*)q_out, (float*)k_cache,
            (float*)v_cache, positions, token_seq, slots, page_table, max_pages, inv_freq, magnitude, n_heads, n_kv, d, rot_dim);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Between two decode steps that run without the host: the sampled token becomes the
// next input, and the position, key count and draw counter of every live sequence
// go up by one.  Entries that only pad the batch (live == 0) stay where they are.
// ---------------------------------------------------------------------------
__global__ void advance_decode_kernel(int* __restrict__ ids, int* __restrict__ positions, int* __restrict__ kv_len,
                                      int* __restrict__ step_key, const int* __restrict__ sampled,
                                      const int* __restrict__ live, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (live[i]) {
        ids[i] = sampled[i];
        positions[i] += 1;
        kv_len[i] += 1;
        step_key[i] += 1;
    }
}

CPM_API int cpm_advance_decode(int* ids, int* positions, int* kv_len, int* step_key, const int* sampled,
                               const int* live, int n, cudaStream_t stream) {
    if (n <= 0) return CPM_OK;
    cpm_launch(kLaunchOther, advance_decode_kernel, (n + 127) / 128, 128, 0, stream, ids, positions, kv_len, step_key, sampled, live, n);
    return launch_status();
}

// Tokens per cache page these kernels were built for (the Python side compares it with its own constant).
CPM_API int cpm_page_tokens() { return kPageTokens; }

CPM_BOUNDS_TU(elementwise)
