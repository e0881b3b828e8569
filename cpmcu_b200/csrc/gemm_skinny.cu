// C[M,N] = alpha * X[M,K] * W[N,K]^T for a handful of rows (decode: M = tokens of the
// step, up to 16): a weight-streaming kernel.  The weights are read exactly once, with
// 16-byte loads along K straight into tensor-core fragments; the activations are tiny and
// come from the caches.
//
// A block owns 16 weight rows (one m16 tile of mma.sync m16n8k16, the weight as the A
// operand, the tokens as the n8 columns) and its 8 warps take interleaved 32-element
// slices of K, so that together they walk each row contiguously; the warps' partial sums
// meet in shared memory.  A thread's 8 consecutive K elements stand for the k-slots of two
// mma instructions; the sum over K does not care about the order as long as both operands
// use the same assignment.
//
// Epilogues: bf16 output; fp32 output times alpha (the output head); SiLU(gate)*up for a
// gate_up matrix whose rows are interleaved in blocks of 8 (8 gate rows, then the 8 up
// rows of the same features), so that gate and up of a feature meet in one tile.
// The reference calls cublasGemmEx for every product (src/model/linear.cuh:8-37) and runs
// the gated activation as a kernel of its own (src/model/activation.cuh:6-18).
#include "common.cuh"

enum : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU = 2 };

__device__ __forceinline__ void mma_16816_s(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// weights are used once: keep them out of L1
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

constexpr int kSkinnyWarps = 8;

template <int NT, int EPI>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
skinny_gemm_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X, void* __restrict__ out, int M, int N, int K,
                   float alpha) {
    constexpr int MT = NT * 8;                          // token columns
    __shared__ float red[kSkinnyWarps][16][MT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int n0 = blockIdx.x * 16;
    const bool row_ok0 = n0 + g < N, row_ok1 = n0 + g + 8 < N;
    const bf16* w0 = W + (int64_t)(row_ok0 ? n0 + g : 0) * K + 8 * j;
    const bf16* w1 = W + (int64_t)(row_ok1 ? n0 + g + 8 : 0) * K + 8 * j;
    const bf16* xp[NT];
    bool tok_ok[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        tok_ok[nt] = nt * 8 + g < M;
        xp[nt] = X + (int64_t)(tok_ok[nt] ? nt * 8 + g : 0) * K + 8 * j;
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    const int steps = K / 32;
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 4
    for (int s = warp; s < steps; s += kSkinnyWarps) {
        const uint4 lo = row_ok0 ? ld_stream16(w0 + 32 * s) : zero;
        const uint4 hi = row_ok1 ? ld_stream16(w1 + 32 * s) : zero;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 b = tok_ok[nt] ? __ldg(reinterpret_cast<const uint4*>(xp[nt] + 32 * s)) : zero;
            mma_16816_s(acc[nt], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
            mma_16816_s(acc[nt], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][g][nt * 8 + 2 * j] = acc[nt][0];
        red[warp][g][nt * 8 + 2 * j + 1] = acc[nt][1];
        red[warp][g + 8][nt * 8 + 2 * j] = acc[nt][2];
        red[warp][g + 8][nt * 8 + 2 * j + 1] = acc[nt][3];
    }
    __syncthreads();
    if (EPI == EPI_SILU) {
        // rows 0..7 are gate, rows 8..15 up, of features (n0 / 2) + 0..7
        const int f = threadIdx.x & 7, tok = threadIdx.x >> 3;
        if (tok < M && tok < MT) {
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < kSkinnyWarps; ++w) {
                gate += red[w][f][tok];
                up += red[w][f + 8][tok];
            }
            const int feature = (n0 >> 1) + f;
            if (feature < (N >> 1)) {
                const float s = 1.0f / (1.0f + expf(-gate));
                reinterpret_cast<bf16*>(out)[(int64_t)tok * (N >> 1) + feature] = __float2bfloat16_rn(gate * s * up);
            }
        }
    } else {
        const int row = threadIdx.x & 15, tok = threadIdx.x >> 4;
        if (tok < M && tok < MT && n0 + row < N) {
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kSkinnyWarps; ++w) sum += red[w][row][tok];
            if (EPI == EPI_F32) reinterpret_cast<float*>(out)[(int64_t)tok * N + n0 + row] = alpha * sum;
            else reinterpret_cast<bf16*>(out)[(int64_t)tok * N + n0 + row] = __float2bfloat16_rn(alpha * sum);
        }
    }
}

template <int NT>
static int launch_skinny(const void* W, const void* X, void* out, int M, int N, int K, float alpha, int epilogue,
                         cudaStream_t stream) {
    const unsigned blocks = (unsigned)((N + 15) / 16);
    const int threads = kSkinnyWarps * 32;
    if (epilogue == EPI_BF16)
        skinny_gemm_kernel<NT, EPI_BF16><<<blocks, threads, 0, stream>>>((const bf16*)W, (const bf16*)X, out, M, N, K, alpha);
    else if (epilogue == EPI_F32)
        skinny_gemm_kernel<NT, EPI_F32><<<blocks, threads, 0, stream>>>((const bf16*)W, (const bf16*)X, out, M, N, K, alpha);
    else if (epilogue == EPI_SILU)
        skinny_gemm_kernel<NT, EPI_SILU><<<blocks, threads, 0, stream>>>((const bf16*)W, (const bf16*)X, out, M, N, K, alpha);
    else
        return CPM_BAD_ARGUMENT;
    return launch_status();
}

// W [N,K] bf16, X [M,K] bf16 (both contiguous); out [M,N] bf16 or fp32, or [M,N/2] bf16 for the gated
// epilogue.  Takes M <= 16 and K a multiple of 32; N is free (for the gated epilogue a multiple of 16).
CPM_API int cpm_gemm_skinny_bf16(const void* W, const void* X, void* out, int M, int N, int K, float alpha,
                                 int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return CPM_OK;
    if (M > 16 || K <= 0 || K % 32 != 0) return CPM_BAD_ARGUMENT;
    if (epilogue == EPI_SILU && N % 16 != 0) return CPM_BAD_ARGUMENT;
    if (M <= 8) return launch_skinny<1>(W, X, out, M, N, K, alpha, epilogue, stream);
    return launch_skinny<2>(W, X, out, M, N, K, alpha, epilogue, stream);
}
