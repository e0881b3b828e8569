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

// 128-byte lines of each weight row a block asks L2 for at its start (and, under programmatic dependent
// launch, before it waits for the kernel ahead of it).  Eight lines bring the first loads of the main loop
// forward and were worth 0.6 to 3.7 % of a decode step, depending on the machine; 16 and more cost time.
static int g_skinny_prefetch_lines = 8;

CPM_API void cpm_set_skinny_prefetch_lines(int n) { g_skinny_prefetch_lines = n < 0 ? 0 : n; }

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

// The second launch bound (one block per SM suffices) matters: it lets the compiler spend registers on
// keeping the loads of eight K steps in flight instead of saving them for occupancy; with it the kernel
// went from 4.5 to 6.1 TB/s on the down projection.  With two tiles of token columns (9 to 16 rows) the
// kernel would take 166 registers and lose the second block per SM, so there the bound is two blocks (53
// instead of 59 us on the gate_up shape, which is what cuBLAS with the activation kernel takes).  Every block
// reads all the activations from L1 and L2, so the engine hands it 9 to 16 rows only for the products whose
// blocks * rows * K stays small (QKV, O and down of the 8B sizes, not gate_up or the head).
template <int NT, int EPI, int kSkinnyWarps>
__global__ void __launch_bounds__(kSkinnyWarps * 32, NT == 1 ? 1 : 2)
skinny_gemm_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X, void* __restrict__ out, int M, int N, int K,
                   float alpha, int prefetch_lines) {
    constexpr int MT = NT * 8;                          // token columns
    __shared__ float red[kSkinnyWarps][16][MT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int n0 = blockIdx.x * 16;
    // Before the kernel ahead of this one in the stream has finished, this block already asks for its
    // 16 weight rows to be brought into L2: weights are never written, and the tail of one product then
    // overlaps with the start of the next.
    {
        const int lines = min(prefetch_lines, (K * 2 + 127) / 128);      // 128-byte lines per row
        for (int i = threadIdx.x; i < 16 * lines; i += kSkinnyWarps * 32) {
            const int r = i / lines, l = i - r * lines;
            const char* p = reinterpret_cast<const char*>(W + (int64_t)min(n0 + r, N - 1) * K) + l * 128;
            asm volatile("prefetch.global.L2 [%0];" :: "l"(p));
        }
    }
    pdl_wait();
    // Rows beyond N and token columns beyond M read a valid row instead and their results are never
    // stored: rows of the product are independent, so no load needs a predicate.
    const bf16* w0 = W + (int64_t)min(n0 + g, N - 1) * K + 8 * j;
    const bf16* w1 = W + (int64_t)min(n0 + g + 8, N - 1) * K + 8 * j;
    const bf16* xp[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xp[nt] = X + (int64_t)min(nt * 8 + g, M - 1) * K + 8 * j;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    const int steps = K / 32;
#pragma unroll 8
    for (int s = warp; s < steps; s += kSkinnyWarps) {
        const uint4 lo = ld_stream16(w0 + 32 * s);
        const uint4 hi = ld_stream16(w1 + 32 * s);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(xp[nt] + 32 * s));
            mma_16816_s(acc[nt], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
            mma_16816_s(acc[nt], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
        }
    }
    // Only now may the next kernel's blocks be placed: a grid of many waves would otherwise lose slots on the
    // SMs to blocks that do nothing but wait.
    pdl_launch_dependents();
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
        for (int o = threadIdx.x; o < 8 * MT; o += kSkinnyWarps * 32) {
            const int f = o & 7, tok = o >> 3;
            if (tok >= M) continue;
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
        for (int o = threadIdx.x; o < 16 * MT; o += kSkinnyWarps * 32) {
            const int row = o & 15, tok = o >> 4;
            if (tok >= M || n0 + row >= N) continue;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kSkinnyWarps; ++w) sum += red[w][row][tok];
            if (EPI == EPI_F32) reinterpret_cast<float*>(out)[(int64_t)tok * N + n0 + row] = alpha * sum;
            else reinterpret_cast<bf16*>(out)[(int64_t)tok * N + n0 + row] = __float2bfloat16_rn(alpha * sum);
        }
    }
}

template <int NT, int EPI>
static int launch_skinny_epi(const void* W, const void* X, void* out, int M, int N, int K, float alpha,
                             cudaStream_t stream) {
    const unsigned blocks = (unsigned)((N + 15) / 16);
    cpm_launch(kLaunchProduct, skinny_gemm_kernel<NT, EPI, 8>, blocks, 256, 0, stream, (const bf16*)W, (const bf16*)X, out, M, N, K, alpha, g_skinny_prefetch_lines);
    return launch_status();
}

template <int NT>
static int launch_skinny(const void* W, const void* X, void* out, int M, int N, int K, float alpha, int epilogue,
                         cudaStream_t stream) {
    if (epilogue == EPI_BF16) return launch_skinny_epi<NT, EPI_BF16>(W, X, out, M, N, K, alpha, stream);
    if (epilogue == EPI_F32) return launch_skinny_epi<NT, EPI_F32>(W, X, out, M, N, K, alpha, stream);
    if (epilogue == EPI_SILU) return launch_skinny_epi<NT, EPI_SILU>(W, X, out, M, N, K, alpha, stream);
    return CPM_BAD_ARGUMENT;
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
