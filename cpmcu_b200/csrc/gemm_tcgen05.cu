// C[M,N] = A[M,K] * W[N,K]^T in bf16 on the fifth-generation tensor cores (tcgen05), for the
// many-row products of prefill: operands travel global -> shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), one elected thread issues tcgen05.mma with both
// operands in shared memory, the fp32 accumulator lives in tensor memory (TMEM) and is read back
// with tcgen05.ld for the epilogue.
//
// A block is persistent and works on 128 x 256 output tiles.  Warp 0 is the TMA producer, warp 1
// allocates TMEM and issues the MMAs, warps 2..5 are the epilogue (each reads its own 32 TMEM
// lanes = 32 output rows).  Two accumulators of 256 columns (all 512 TMEM columns) let the
// epilogue of one tile overlap the main loop of the next; a ring of kStages shared-memory stages
// (16 KiB of A and 32 KiB of W per 64-wide K block) decouples TMA from the MMAs.  mbarriers carry
// every hand-over: full/empty per stage, accumulator full/empty per TMEM buffer.
//
// Epilogues: bf16 output, or SiLU(gate) * up for a gate_up weight whose rows are interleaved in
// blocks of 8 (the 32 accumulator columns a thread reads at a time hold 8 gate, 8 up, 8 gate, 8
// up values of 16 features), which saves the round trip of the [M, 2*inter] intermediate that the
// reference makes between cublasGemmEx and its activation kernel (src/model/ffn.cuh:38-50).
//
// Every wait on a barrier is bounded: when a bound is hit the block records an error code, stops
// taking work, frees its TMEM and returns, so a fault in the hand-over logic cannot hang the GPU.
// No TMA multicast and no clusters are used.
#include "common.cuh"
#include <cuda.h>

namespace tc5 {

constexpr int kBlockM = 128, kBlockN = 256, kBlockK = 64;      // K block = 128 bytes of bf16 = one swizzle row
constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kBlockK * 2;                  // 16 KiB
constexpr int kBBytes = kBlockN * kBlockK * 2;                  // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024;        // + room to align the stages to 1 KiB
constexpr int kThreads = 192;                                   // 6 warps
constexpr int kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 20;                       // tries of a bounded barrier wait (each try may block for a while)

enum : int { EPI_BF16 = 0, EPI_SILU = 2 };
enum : int { ERR_NONE = 0, ERR_FULL_WAIT = 1, ERR_EMPTY_WAIT = 2, ERR_ACC_FULL_WAIT = 3, ERR_ACC_EMPTY_WAIT = 4 };

__device__ int g_error = 0;      // first error code any block has recorded since the last reset

// ---- PTX wrappers ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase with this parity, at most kSpinLimit tries.  false = gave up.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void tmem_load_32cols(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                   "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// start address (>>4), leading byte offset 1 (unused for swizzled K-major), stride byte offset
// 1024 (8 rows), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBlockN >> 3) << 17) |
                                ((uint32_t)(kBlockM >> 4) << 24);

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    bf16* __restrict__ out, int M, int N, int K) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full_bar[2], acc_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t stages = (smem_u32(smem_raw) + 1023u) & ~1023u;        // swizzled tiles want 1 KiB alignment
    const int tiles_m = (M + kBlockM - 1) / kBlockM, tiles_n = (N + kBlockN - 1) / kBlockN;
    const int n_tiles = tiles_m * tiles_n, k_blocks = K / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full_bar[b]), 1);
            mbar_init(smem_u32(&acc_empty_bar[b]), 4);                    // one arrival per epilogue warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {                                                      // this warp owns the TMEM allocation
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

    if (warp == 0) {
        // ---- TMA producer (one elected lane) ----
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !*(volatile int*)&abort_flag; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * kBlockM, n0 = (tile / tiles_m) * kBlockN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), ((it / kStages) & 1) ^ 1)) { fail(ERR_EMPTY_WAIT); break; }
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    mbar_expect_tx(bar, kStageBytes);
                    tma_load_2d(stages + s * kStageBytes, &map_a, bar, kb * kBlockK, m0);
                    tma_load_2d(stages + s * kStageBytes + kABytes, &map_w, bar, kb * kBlockK, n0);
                }
            }
            if (*(volatile int*)&abort_flag) {
                // copies that were asked for must land before the block gives up its shared memory
                const uint32_t first = it > (uint32_t)kStages ? it - kStages : 0;
                for (uint32_t j = first; j < it; ++j)
                    mbar_wait_bounded(smem_u32(&full_bar[j % kStages]), (j / kStages) & 1);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (one elected lane) ----
        if (lane == 0) {
            uint32_t it = 0, local_tile = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !*(volatile int*)&abort_flag; tile += gridDim.x, ++local_tile) {
                const int acc = local_tile & 1;
                if (!mbar_wait_bounded(smem_u32(&acc_empty_bar[acc]), ((local_tile >> 1) & 1) ^ 1)) { fail(ERR_ACC_EMPTY_WAIT); break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * kBlockN;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (it / kStages) & 1)) { fail(ERR_FULL_WAIT); ok = false; break; }
                    tcgen05_fence_after();
                    const uint64_t da = smem_desc_sw128(stages + s * kStageBytes);
                    const uint64_t db = smem_desc_sw128(stages + s * kStageBytes + kABytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k)                // 32 bytes further along K per MMA: +2 in the address field
                        tcgen05_mma_f16(tmem_d, da + 2 * k, db + 2 * k, kInstrDesc, (kb | k) != 0);
                    tcgen05_commit(smem_u32(&empty_bar[s]));              // the stage is free when these MMAs are done
                }
                if (!ok) break;
                tcgen05_commit(smem_u32(&acc_full_bar[acc]));             // the accumulator is complete when all are done
            }
        }
    } else {
        // ---- epilogue: warps 2..5; a warp may touch TMEM lanes 32 * (warp % 4) .. + 31 only ----
        const int quarter = warp & 3;
        uint32_t local_tile = 0;
        for (int tile = blockIdx.x; tile < n_tiles && !*(volatile int*)&abort_flag; tile += gridDim.x, ++local_tile) {
            const int m0 = (tile % tiles_m) * kBlockM, n0 = (tile / tiles_m) * kBlockN;
            const int acc = local_tile & 1;
            if (!mbar_wait_bounded(smem_u32(&acc_full_bar[acc]), (local_tile >> 1) & 1)) { fail(ERR_ACC_FULL_WAIT); break; }
            tcgen05_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBlockN;
#pragma unroll 1
            for (int c = 0; c < kBlockN / 32; ++c) {
                uint32_t v[32];
                tmem_load_32cols(taddr + c * 32, v);
                tmem_load_wait();
                const int col = n0 + c * 32;
                if (row < M && col < N) {
                    if (EPI == EPI_SILU) {
                        // columns: 8 gate, 8 up, 8 gate, 8 up of features (col / 2) .. + 15
                        uint32_t packed[8];
#pragma unroll
                        for (int h = 0; h < 2; ++h)
#pragma unroll
                            for (int i = 0; i < 8; i += 2) {
                                const float g0 = __uint_as_float(v[16 * h + i]), g1 = __uint_as_float(v[16 * h + i + 1]);
                                const float u0 = __uint_as_float(v[16 * h + 8 + i]), u1 = __uint_as_float(v[16 * h + 9 + i]);
                                const float a = g0 * (1.0f / (1.0f + __expf(-g0))) * u0;
                                const float b = g1 * (1.0f / (1.0f + __expf(-g1))) * u1;
                                const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
                                packed[4 * h + i / 2] = *reinterpret_cast<const uint32_t*>(&p);
                            }
                        uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)row * (N >> 1) + (col >> 1));
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
                        uint32_t packed[16];
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                            packed[i / 2] = *reinterpret_cast<const uint32_t*>(&p);
                        }
                        bf16* dst_row = out + (int64_t)row * N + col;
                        if (col + 32 <= N) {
                            uint4* dst = reinterpret_cast<uint4*>(dst_row);
#pragma unroll
                            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
                        } else {
                            for (int i = 0; i < 32 && col + i < N; ++i)
                                dst_row[i] = __ushort_as_bfloat16((unsigned short)(packed[i / 2] >> (16 * (i & 1))));
                        }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty_bar[acc]));
        }
    }
    // ---- all roles meet; the allocating warp gives the TMEM back ----
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

// ---- host side ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Map of a row-major [rows, K] bf16 matrix, boxes of box_rows x 64 elements, 128-byte swizzle, zero fill outside.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBlockK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int EPI>
static int launch(const void* A, const void* W, void* out, int M, int N, int K, int n_blocks, cudaStream_t stream) {
    CUtensorMap map_a, map_w;
    if (!make_map(&map_a, A, M, K, kBlockM) || !make_map(&map_w, W, N, K, kBlockN)) return CPM_BAD_ARGUMENT;
    auto kern = gemm_tcgen05_kernel<EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tiles = ((M + kBlockM - 1) / kBlockM) * ((N + kBlockN - 1) / kBlockN);
    kern<<<tiles < n_blocks ? tiles : n_blocks, kThreads, kSmemBytes, stream>>>(map_a, map_w, (bf16*)out, M, N, K);
    return launch_status();
}

}  // namespace tc5

// A [M,K], W [N,K] bf16 row-major (16-byte aligned, K a multiple of 64); out [M,N] bf16, or [M,N/2] for the
// gated epilogue (N a multiple of 32, W rows interleaved in blocks of 8).  n_blocks: blocks to launch (one per SM).
CPM_API int cpm_gemm_bf16_tcgen05(const void* A, const void* W, void* out, int M, int N, int K, int epilogue,
                                  int n_blocks, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return CPM_OK;
    if (K <= 0 || K % tc5::kBlockK != 0 || n_blocks < 1 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)out & 15))
        return CPM_BAD_ARGUMENT;
    if (epilogue == tc5::EPI_SILU) {
        if (N % 32 != 0) return CPM_BAD_ARGUMENT;
        return tc5::launch<tc5::EPI_SILU>(A, W, out, M, N, K, n_blocks, stream);
    }
    if (epilogue != tc5::EPI_BF16 || N % 8 != 0) return CPM_BAD_ARGUMENT;
    return tc5::launch<tc5::EPI_BF16>(A, W, out, M, N, K, n_blocks, stream);
}

// Error code recorded by the kernel since the last call (0 = none), and reset.  Synchronises the device.
CPM_API int cpm_gemm_tcgen05_error() {
    int code = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&code, tc5::g_error, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(tc5::g_error, &zero, sizeof(int));
    return code;
}
