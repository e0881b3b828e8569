// Shared helpers of the sm_100a kernel library: element types, conversions,
// reductions and the page geometry of the key-value cache.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <math.h>

#define CPM_API extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python side.
enum : int { CPM_F32 = 0, CPM_BF16 = 1 };

// Tokens per cache page.  A sequence's keys and values live in pages of this many
// tokens.  A key page is [kv_head][token_in_page][head_dim]; a value page is stored
// transposed, [kv_head][head_dim][token_in_page].  The tile of one head is contiguous
// in both, and both can feed tensor-core fragments with 16-byte loads along the
// contiguous axis (head_dim for the scores, tokens for the weighted sum).
constexpr int kPageTokens = 64;

// Status codes returned by the launchers (0 = launched; the CUDA error otherwise).
enum : int {
    CPM_OK = 0,
    CPM_BAD_ARGUMENT = -1,   // a size the kernel does not take
};

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Largest value with the lowest index among equals, over a warp and over a block.
struct ArgMax { float v; int i; };

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* scratch /* 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        ArgMax t = lane < n_warps ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax b;
            b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, b);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// A build with -DCPM_CHECK_BOUNDS checks every page number a kernel takes from a page table (the logical index
// against the table's width, the page against the number of pages the cache holds) before it is used as an
// address: a bad one is recorded (the first per source file and run: what, index, value, limit), page 0 is used
// in its place, and the host reads the record after the step (cpm_bounds_error_<file>).  It stands in for a
// memory checker where none can be run; the ordinary build has none of it.
#ifdef CPM_CHECK_BOUNDS
static __device__ int g_bounds_record[4];               // code (0 = none), index, value, limit
static __device__ int g_bounds_pages = 0x7fffffff;      // pages the cache in use holds (cpm_bounds_limit_<file>)
__device__ __forceinline__ int cpm_checked_page(const int* pages, int idx, int max_pages) {
    const bool idx_ok = idx >= 0 && idx < max_pages;
    const int v = idx_ok ? pages[idx] : -1;
    if (idx_ok && v >= 0 && v < g_bounds_pages) return v;
    if (atomicCAS(&g_bounds_record[0], 0, idx_ok ? 2 : 1) == 0) {
        g_bounds_record[1] = idx;
        g_bounds_record[2] = v;
        g_bounds_record[3] = idx_ok ? g_bounds_pages : max_pages;
    }
    return 0;
}
#define CPM_PAGE(pages, idx, max_pages) cpm_checked_page(pages, idx, max_pages)
// The host side of one source file's record: read-and-clear, and the page limit.
#define CPM_BOUNDS_TU(name)                                                                          \
    CPM_API int cpm_bounds_error_##name(int* out4) {                                                 \
        int zero[4] = {0, 0, 0, 0};                                                                  \
        if (cudaMemcpyFromSymbol(out4, g_bounds_record, sizeof(zero)) != cudaSuccess) return -1;     \
        if (out4[0]) cudaMemcpyToSymbol(g_bounds_record, zero, sizeof(zero));                        \
        return out4[0];                                                                              \
    }                                                                                                \
    CPM_API int cpm_bounds_limit_##name(int n_pages) {                                               \
        return cudaMemcpyToSymbol(g_bounds_pages, &n_pages, sizeof(int)) == cudaSuccess ? 0 : -1;    \
    }
#else
#define CPM_PAGE(pages, idx, max_pages) ((pages)[idx])
#define CPM_BOUNDS_TU(name)
#endif

// Address of the first element of (page, kv_head, token_in_page) in a cache lane.
__device__ __forceinline__ int64_t page_row_offset(int page, int kv_head, int in_page, int n_kv, int d) {
    return (((int64_t)page * n_kv + kv_head) * kPageTokens + in_page) * (int64_t)d;
}

// Address of value element (page, kv_head, dim, token_in_page) in a cache lane.
__device__ __forceinline__ int64_t value_offset(int page, int kv_head, int dim, int in_page, int n_kv, int d) {
    return (((int64_t)page * n_kv + kv_head) * d + dim) * (int64_t)kPageTokens + in_page;
}

// Programmatic dependent launch.  A kernel launched with the attribute may start while the
// kernel before it in the stream is still running; it must not touch anything that kernel
// (or an earlier one) writes before pdl_wait() returns, which is when the preceding kernel
// has completed and its writes are visible.  pdl_launch_dependents() lets the kernel after
// this one begin its own launch.  Both are no-ops for a kernel launched the ordinary way.
// What a kernel does before pdl_wait() here is only ever to prefetch weights, which no
// kernel writes.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Which kernels are launched with the attribute: a mask over the classes below (bit = 1 << class).  Measured on
// the 8B decode step (batch 8, 3.64 ms without): norms and products 3.47 ms, with the rotary kernel and the decode
// attention as well 3.45 ms; the kernel that combines the attention's shares must stay out (with it the gain is
// gone: 3.66 ms), and so does everything else (embedding, sampling, the step's bookkeeping).
enum LaunchClass : int { kLaunchOther = 0, kLaunchNorm = 1, kLaunchProduct = 2, kLaunchRope = 3, kLaunchAttention = 4,
                         kLaunchCombine = 5 };
constexpr int kDefaultPdlMask = (1 << kLaunchNorm) | (1 << kLaunchProduct) | (1 << kLaunchRope) | (1 << kLaunchAttention);
extern int g_cpm_pdl;      // the mask in force (cpm_set_pdl)

template <typename... KArgs, typename... Args>
static inline void cpm_launch(LaunchClass cls, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ((g_cpm_pdl >> (int)cls) & 1) ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Raises a kernel's dynamic shared-memory limit once per device (the attribute belongs to the device's
// context, so a process that uses several GPUs has to set it on each).  ``done`` is a zero-initialised
// array of kMaxDevices flags, one array per kernel.  Returns CPM_OK or the CUDA error.
constexpr int kMaxDevices = 64;
template <typename Kernel>
static inline int ensure_dynamic_smem(Kernel kernel, int bytes, bool* done) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return CPM_BAD_ARGUMENT;
    if (done[dev]) return CPM_OK;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return (int)e;
    done[dev] = true;
    return CPM_OK;
}

static inline int launch_status() {
    cudaError_t e = cudaPeekAtLastError();
    return e == cudaSuccess ? CPM_OK : (int)e;
}
