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
#include "tcgen05.cuh"

namespace tc5 {

constexpr int kBlockM = 128, kBlockN = 256, kBlockK = 64;      // K block = 128 bytes of bf16 = one swizzle row
constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kBlockK * 2;                  // 16 KiB
constexpr int kBBytes = kBlockN * kBlockK * 2;                  // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 4 * 4096;   // + room to align the stages to 1 KiB, + the epilogue warps' staging
// The single-block kernel also comes with tiles of 224 weight rows: with few rows of A (a decode batch: one row
// tile) the tiles are all there is to share out, and 32,768 weight rows are 128 tiles of 256 (20 of 148 SMs idle)
// but 147 tiles of 224.  The second accumulator always starts at TMEM column 256.
constexpr int kNarrowN = 224;
template <int BN> struct TileN {
    static constexpr int kB = BN * kBlockK * 2;
    static constexpr int kStage = kABytes + kB;
    static constexpr int kSmem = kStages * kStage + 1024 + 4 * 4096;
    static constexpr uint32_t kDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                      ((uint32_t)(kBlockM >> 4) << 24);
};
constexpr int kThreads = 192;                                   // 6 warps
constexpr int kTmemCols = 512;
constexpr int kBandTiles = 16;                                  // 2048 rows of A are shared by the blocks that run together

enum : int { EPI_BF16 = 0, EPI_SILU = 2 };
enum : int { ERR_NONE = 0, ERR_FULL_WAIT = 1, ERR_EMPTY_WAIT = 2, ERR_ACC_FULL_WAIT = 3, ERR_ACC_EMPTY_WAIT = 4 };

__device__ int g_error = 0;      // first error code any block has recorded since the last reset

// Instruction descriptor: D fp32, A and B bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBlockN >> 3) << 17) |
                                ((uint32_t)(kBlockM >> 4) << 24);

// Order of the tiles: bands of ``band`` row tiles, inside a band the row tile runs fastest.  The blocks that
// run at one time then share a few row tiles of A and a few of W, whatever the number of rows, and both
// stay in L2 (with all rows in one band, 8192 rows took A out of L2 between its uses).
struct TileCoord { int m, n; };
__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_m, int tiles_n, int band) {
    const int per_band = band * tiles_n;
    const int b = tile / per_band, in_band = tile - b * per_band;
    const int first = b * band, height = min(band, tiles_m - first);
    TileCoord c;
    c.n = in_band / height;
    c.m = first + (in_band - c.n * height);
    return c;
}

// One epilogue warp's 32 rows of a tile: accumulator columns from TMEM, converted (or gated) to bf16, through a
// 4 KiB staging area of the warp in shared memory, so that every store instruction writes whole 128-byte lines
// of four output rows.  (Stores of 16 bytes to 32 different rows, straight from the registers, cost the
// 128 x 256 kernel 12 % of its time.)  The staging rows are 128 bytes, their 16-byte chunks XOR-swizzled
// by the row, which keeps both the writes (one row per lane) and the reads (eight lanes per row) free of
// bank conflicts.  taddr: TMEM address of the warp's lanes and the tile's first column.
template <int EPI, int BN = kBlockN>
__device__ __forceinline__ void epilogue_tile(bf16* __restrict__ out, uint32_t taddr, unsigned char* staging, int row0, int n0,
                                              int M, int N, int lane) {
    constexpr int kLoadsPerPass = EPI == EPI_SILU ? 4 : 2;          // 32 accumulator columns each; a pass is 64 outputs
    constexpr int kLoads = BN / 32;                                 // the tile's accumulator columns, 32 at a time
    constexpr int kPasses = (kLoads + kLoadsPerPass - 1) / kLoadsPerPass;     // the last pass may be a part of one
    const int ldo = EPI == EPI_SILU ? N >> 1 : N;
    const int oc_tile = EPI == EPI_SILU ? n0 >> 1 : n0;
    uint4* my_row = reinterpret_cast<uint4*>(staging + lane * 128);
#pragma unroll 1
    for (int p = 0; p < kPasses; ++p) {
        if (oc_tile + p * 64 >= ldo) break;
        const int loads_here = min(kLoadsPerPass, kLoads - p * kLoadsPerPass);
#pragma unroll
        for (int h = 0; h < kLoadsPerPass; ++h) {
            if (h >= loads_here) break;                              // warp-uniform
            uint32_t v[32];
            tmem_load_32cols(taddr + (p * kLoadsPerPass + h) * 32, v);
            tmem_load_wait();
            if (EPI == EPI_SILU) {
                // columns: 8 gate, 8 up, 8 gate, 8 up of 16 consecutive features
                uint32_t packed[8];
#pragma unroll
                for (int q = 0; q < 2; ++q)
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const float g0 = __uint_as_float(v[16 * q + i]), g1 = __uint_as_float(v[16 * q + i + 1]);
                        const float u0 = __uint_as_float(v[16 * q + 8 + i]), u1 = __uint_as_float(v[16 * q + 9 + i]);
                        const float a = __fdividef(g0, 1.0f + __expf(-g0)) * u0;      // the result is rounded to bf16
                        const float b = __fdividef(g1, 1.0f + __expf(-g1)) * u1;
                        const __nv_bfloat162 pk = __floats2bfloat162_rn(a, b);
                        packed[4 * q + i / 2] = *reinterpret_cast<const uint32_t*>(&pk);
                    }
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    my_row[(2 * h + c) ^ (lane & 7)] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            } else {
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const __nv_bfloat162 pk = __floats2bfloat162_rn(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                    packed[i / 2] = *reinterpret_cast<const uint32_t*>(&pk);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    my_row[(4 * h + c) ^ (lane & 7)] = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            }
        }
        __syncwarp();
        const int j = lane & 7, col = oc_tile + p * 64 + j * 8;
        const bool chunk_valid = j < loads_here * (8 / kLoadsPerPass);       // 16-byte chunks this pass has filled
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = 4 * i + (lane >> 3);
            const uint4 val = *reinterpret_cast<const uint4*>(staging + r * 128 + ((j ^ (r & 7)) << 4));
            if (chunk_valid && row0 + r < M && col < ldo) *reinterpret_cast<uint4*>(out + (int64_t)(row0 + r) * ldo + col) = val;
        }
        __syncwarp();
    }
}

template <int EPI, int BN = kBlockN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    bf16* __restrict__ out, int M, int N, int K) {
    constexpr int kBlockN = BN;                                    // this instantiation's tile width
    constexpr int kStageBytes = TileN<BN>::kStage;
    constexpr uint32_t kInstrDesc = TileN<BN>::kDesc;
    constexpr int kAccStride = 256;                                // TMEM columns between the two accumulators
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full_bar[2], acc_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t stages = (smem_u32(smem_raw) + 1023u) & ~1023u;        // swizzled tiles want 1 KiB alignment
    unsigned char* staging = smem_raw + (stages - smem_u32(smem_raw)) + kStages * kStageBytes;
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

    // Both loops below start every tile at stage 0 and walk the ring in rounds with the stage index unrolled:
    // barrier addresses, shared-memory addresses and matrix descriptors are then loop invariants held in
    // registers.  (With a stage index computed per K block the issuing thread spent more time on a K block than
    // its four MMAs take to run: 0.45 us against 0.27 us at full clocks.)  A tile may end in the middle of a
    // round, so each stage keeps its own phase bit: bit s of ``phase`` is the parity of stage s's next use.
    if (warp == 0) {
        // ---- TMA producer (one elected lane) ----
        if (lane == 0) {
            // Under programmatic dependent launch this kernel may start while the one ahead of it still runs.
            // Weights are written by no kernel: the first stages' weight tiles are asked for at once, the
            // activations' tiles (which the kernel ahead writes) after the wait.  Nothing is written to global
            // memory before the wait either: the epilogue runs on accumulators that need the activations.
            int early = 0;
            if (blockIdx.x < n_tiles) {
                const TileCoord tc0 = tile_coord(blockIdx.x, tiles_m, tiles_n, kBandTiles);
                early = min(kStages, k_blocks);
#pragma unroll
                for (int s = 0; s < kStages; ++s) {
                    if (s >= early) break;
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    mbar_expect_tx(bar, kStageBytes);
                    tma_load_2d(stages + s * kStageBytes + kABytes, &map_w, bar, s * kBlockK, tc0.n * kBlockN);
                }
            }
            pdl_wait();
            uint32_t phase = 0, used = 0;              // per stage: parity of its next use; whether it has been filled before
            int pending = early;                       // stages of the first tile whose weight tile is on its way already
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok && !*(volatile int*)&abort_flag; tile += gridDim.x) {
                const TileCoord tc = tile_coord(tile, tiles_m, tiles_n, kBandTiles);
                const int m0 = tc.m * kBlockM, n0 = tc.n * kBlockN;
                for (int first = 0; first < k_blocks && ok; first += kStages) {
#pragma unroll
                    for (int s = 0; s < kStages; ++s) {
                        const int kb = first + s;
                        if (kb >= k_blocks) break;
                        const uint32_t bar = smem_u32(&full_bar[s]);
                        if (pending > 0) {                               // its weight tile went out before the wait
                            --pending;
                        } else {
                            if ((used >> s) & 1u) {
                                if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), ((phase >> s) & 1u) ^ 1u)) { fail(ERR_EMPTY_WAIT); ok = false; break; }
                            }
                            mbar_expect_tx(bar, kStageBytes);
                            tma_load_2d(stages + s * kStageBytes + kABytes, &map_w, bar, kb * kBlockK, n0);
                        }
                        tma_load_2d(stages + s * kStageBytes, &map_a, bar, kb * kBlockK, m0);
                        phase ^= 1u << s;
                        used |= 1u << s;
                    }
                }
            }
            if (*(volatile int*)&abort_flag) {
                // copies that were asked for must land before the block gives up its shared memory; stages whose
                // weight tile was asked for early still lack their activations' tile: ask for it, so that they complete
                if (pending > 0) {
                    const TileCoord tc0 = tile_coord(blockIdx.x, tiles_m, tiles_n, kBandTiles);
                    for (int s = early - pending; s < early; ++s) {
                        tma_load_2d(stages + s * kStageBytes, &map_a, smem_u32(&full_bar[s]), s * kBlockK, tc0.m * kBlockM);
                        phase ^= 1u << s;
                        used |= 1u << s;
                    }
                }
                for (int s = 0; s < kStages; ++s)                        // each stage's latest fill
                    if ((used >> s) & 1u) mbar_wait_bounded(smem_u32(&full_bar[s]), ((phase >> s) & 1u) ^ 1u);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer (one elected lane) ----
        if (lane == 0) {
            uint32_t phase = 0, local_tile = 0;
            bool ok = true;
            const uint64_t da0 = smem_desc_sw128(stages), db0 = smem_desc_sw128(stages + kABytes);
            constexpr uint64_t kStep = (uint64_t)(kStageBytes >> 4);      // the descriptor's address counts 16 bytes
            for (int tile = blockIdx.x; tile < n_tiles && ok && !*(volatile int*)&abort_flag; tile += gridDim.x, ++local_tile) {
                const int acc = local_tile & 1;
                if (!mbar_wait_bounded(smem_u32(&acc_empty_bar[acc]), ((local_tile >> 1) & 1) ^ 1)) { fail(ERR_ACC_EMPTY_WAIT); break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * kAccStride;
                for (int first = 0; first < k_blocks && ok; first += kStages) {
#pragma unroll
                    for (int s = 0; s < kStages; ++s) {
                        const int kb = first + s;
                        if (kb >= k_blocks) break;
                        if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (phase >> s) & 1u)) { fail(ERR_FULL_WAIT); ok = false; break; }
                        phase ^= 1u << s;
                        tcgen05_fence_after();
#pragma unroll
                        for (int k = 0; k < kBlockK / 16; ++k)            // 32 bytes further along K per MMA: +2 in the address field
                            tcgen05_mma_f16(tmem_d, da0 + s * kStep + 2 * k, db0 + s * kStep + 2 * k, kInstrDesc, (kb | k) != 0);
                        tcgen05_commit(smem_u32(&empty_bar[s]));          // the stage is free when these MMAs are done
                    }
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
            const TileCoord tc = tile_coord(tile, tiles_m, tiles_n, kBandTiles);
            const int m0 = tc.m * kBlockM, n0 = tc.n * kBlockN;
            const int acc = local_tile & 1;
            if (!mbar_wait_bounded(smem_u32(&acc_full_bar[acc]), (local_tile >> 1) & 1)) { fail(ERR_ACC_FULL_WAIT); break; }
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kAccStride;
            epilogue_tile<EPI, BN>(out, taddr, staging + quarter * 4096, m0 + quarter * 32, n0, M, N, lane);
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

// ---------------------------------------------------------------------------
// Two blocks on one 256 x 256 tile (thread-block cluster of 2, tcgen05 cta_group::2).  Each block of
// the pair loads its own 128 rows of A and its own 128 rows of W per 64-wide K block (32 KiB a stage,
// so 6 stages fit where the single-block kernel has 4) and holds the accumulator of its own 128
// output rows in its TMEM; the even block of the pair issues the MMAs for both.  Hand-overs: the
// "full" barriers live in the even block and collect the bytes of both blocks' TMA loads (the odd
// block reaches them through their cluster address); "empty" and "accumulator full" are
// raised in both blocks at once by tcgen05.commit with a cluster multicast; the epilogue warps of
// both blocks arrive on the even block's "accumulator empty".  The TMA loads carry no multicast.
// ---------------------------------------------------------------------------
constexpr int kStages2 = 6;
constexpr int kHalfN = kBlockN / 2;                              // W rows a block of the pair loads
constexpr int kABytes2 = kBlockM * kBlockK * 2;                  // 16 KiB
constexpr int kBBytes2 = kHalfN * kBlockK * 2;                   // 16 KiB
constexpr int kStageBytes2 = kABytes2 + kBBytes2;
constexpr int kSmemBytes2 = kStages2 * kStageBytes2 + 1024 + 4 * 4096;   // + the epilogue warps' staging
constexpr uint32_t kInstrDesc2 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBlockN >> 3) << 17) |
                                 ((uint32_t)((2 * kBlockM) >> 4) << 24);

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                     uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(bar) : "memory");
}
// The address, valid in the whole cluster, of this block's shared-memory location in the block of that rank.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         bf16* __restrict__ out, int M, int N, int K) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kStages2], empty_bar[kStages2], acc_full_bar[2], acc_empty_bar[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                                  // 0: issues the MMAs of the pair
    const uint32_t stages = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* staging = smem_raw + (stages - smem_u32(smem_raw)) + kStages2 * kStageBytes2;
    const int tiles_m = (M + 2 * kBlockM - 1) / (2 * kBlockM), tiles_n = (N + kBlockN - 1) / kBlockN;
    const int n_tiles = tiles_m * tiles_n, k_blocks = K / kBlockK;
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full_bar[b]), 1);
            mbar_init(smem_u32(&acc_empty_bar[b]), 8);                     // 4 epilogue warps of each block
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(&tmem_base_slot)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();                                                        // the partner's barriers exist before anything is sent to them
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    auto fail = [&](int code) {
        atomicCAS(&g_error, 0, code);
        atomicExch(&abort_flag, 1);
    };

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = pair; tile < n_tiles && !*(volatile int*)&abort_flag; tile += n_pairs) {
                const TileCoord tc = tile_coord(tile, tiles_m, tiles_n, kBandTiles / 2);
                const int m0 = tc.m * 2 * kBlockM + rank * kBlockM;
                const int n0 = tc.n * kBlockN + rank * kHalfN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages2;
                    if (!mbar_wait_bounded(smem_u32(&empty_bar[s]), ((it / kStages2) & 1) ^ 1)) { fail(ERR_EMPTY_WAIT); break; }
                    const uint32_t bar = map_to_rank(smem_u32(&full_bar[s]), 0);   // the even block's barrier
                    if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * kStageBytes2);
                    tma_load_2d_pair(stages + s * kStageBytes2, &map_a, bar, kb * kBlockK, m0);
                    tma_load_2d_pair(stages + s * kStageBytes2 + kABytes2, &map_w, bar, kb * kBlockK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            uint32_t it = 0, local_tile = 0;
            for (int tile = pair; tile < n_tiles && !*(volatile int*)&abort_flag; tile += n_pairs, ++local_tile) {
                const int acc = local_tile & 1;
                if (!mbar_wait_bounded(smem_u32(&acc_empty_bar[acc]), ((local_tile >> 1) & 1) ^ 1)) { fail(ERR_ACC_EMPTY_WAIT); break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * kBlockN;
                bool ok = true;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kStages2;
                    if (!mbar_wait_bounded(smem_u32(&full_bar[s]), (it / kStages2) & 1)) { fail(ERR_FULL_WAIT); ok = false; break; }
                    tcgen05_fence_after();
                    const uint64_t da = smem_desc_sw128(stages + s * kStageBytes2);
                    const uint64_t db = smem_desc_sw128(stages + s * kStageBytes2 + kABytes2);
#pragma unroll
                    for (int k = 0; k < kBlockK / 16; ++k)
                        tcgen05_mma_f16_pair(tmem_d, da + 2 * k, db + 2 * k, kInstrDesc2, (kb | k) != 0);
                    tcgen05_commit_pair(smem_u32(&empty_bar[s]));          // frees the stage in both blocks
                }
                if (!ok) break;
                tcgen05_commit_pair(smem_u32(&acc_full_bar[acc]));         // both blocks' epilogues may start
            }
        }
    } else {
        const int quarter = warp & 3;
        uint32_t local_tile = 0;
        for (int tile = pair; tile < n_tiles && !*(volatile int*)&abort_flag; tile += n_pairs, ++local_tile) {
            const TileCoord tc = tile_coord(tile, tiles_m, tiles_n, kBandTiles / 2);
            const int m0 = tc.m * 2 * kBlockM + rank * kBlockM, n0 = tc.n * kBlockN;
            const int acc = local_tile & 1;
            if (!mbar_wait_bounded(smem_u32(&acc_full_bar[acc]), (local_tile >> 1) & 1)) { fail(ERR_ACC_FULL_WAIT); break; }
            tcgen05_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kBlockN;
            epilogue_tile<EPI>(out, taddr, staging + quarter * 4096, m0 + quarter * 32, n0, M, N, lane);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty_bar[acc]), 0));
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();                                                        // nothing of the pair is in flight towards this block any more
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
    }
}

// ---- host side ----
// Map of a row-major [rows, K] bf16 matrix, boxes of box_rows x 64 elements, 128-byte swizzle, zero fill outside.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    return make_map_2d_bf16(map, base, (uint64_t)rows, (uint64_t)K, (uint64_t)K * 2, kBlockK, box_rows);
}

template <int EPI, int BN>
static int launch_tiles(const void* A, const void* W, void* out, int M, int N, int K, int n_blocks, cudaStream_t stream) {
    CUtensorMap map_a, map_w;
    if (!make_map(&map_a, A, M, K, kBlockM) || !make_map(&map_w, W, N, K, BN)) return CPM_BAD_ARGUMENT;
    auto kern = gemm_tcgen05_kernel<EPI, BN>;
    static bool configured[kMaxDevices] = {};            // per kernel and per device
    if (int st = ensure_dynamic_smem(kern, TileN<BN>::kSmem, configured)) return st;
    const int tiles = ((M + kBlockM - 1) / kBlockM) * ((N + BN - 1) / BN);
    cpm_launch(kLaunchProduct, kern, dim3(tiles < n_blocks ? tiles : n_blocks), dim3(kThreads), (size_t)TileN<BN>::kSmem, stream,
               map_a, map_w, (bf16*)out, M, N, K);
    return launch_status();
}

static int g_narrow_tiles = 1;       // cpm_set_tcgen05_narrow: 0 keeps every product on 256-row tiles

template <int EPI>
static int launch(const void* A, const void* W, void* out, int M, int N, int K, int n_blocks, cudaStream_t stream) {
    // One row tile of A (a decode batch): the weight tiles are all the work there is to share out; take the
    // narrower tiles where they need fewer rounds of the blocks times their width.
    if (g_narrow_tiles && M <= kBlockM) {
        auto cost = [&](int bn) { const int t = (N + bn - 1) / bn; return (int64_t)((t + n_blocks - 1) / n_blocks) * bn; };
        if (cost(kNarrowN) < cost(kBlockN)) return launch_tiles<EPI, kNarrowN>(A, W, out, M, N, K, n_blocks, stream);
    }
    return launch_tiles<EPI, kBlockN>(A, W, out, M, N, K, n_blocks, stream);
}

// The pair kernel: clusters of two blocks, n_blocks rounded down to an even number.
template <int EPI>
static int launch_pair(const void* A, const void* W, void* out, int M, int N, int K, int n_blocks, cudaStream_t stream) {
    CUtensorMap map_a, map_w;
    if (!make_map(&map_a, A, M, K, kBlockM) || !make_map(&map_w, W, N, K, kHalfN)) return CPM_BAD_ARGUMENT;
    auto kern = gemm_tcgen05_pair_kernel<EPI>;
    static bool configured[kMaxDevices] = {};            // per kernel and per device
    if (int st = ensure_dynamic_smem(kern, kSmemBytes2, configured)) return st;
    const int tiles = ((M + 2 * kBlockM - 1) / (2 * kBlockM)) * ((N + kBlockN - 1) / kBlockN);
    int pairs = n_blocks / 2;
    if (pairs < 1) return CPM_BAD_ARGUMENT;
    if (pairs > tiles) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes2;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_a, map_w, (bf16*)out, M, N, K);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

}  // namespace tc5

// The same product by pairs of blocks on 256 x 256 tiles (see the pair kernel); same arguments and limits.
CPM_API int cpm_gemm_bf16_tcgen05_pair(const void* A, const void* W, void* out, int M, int N, int K, int epilogue,
                                       int n_blocks, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return CPM_OK;
    if (K <= 0 || K % tc5::kBlockK != 0 || n_blocks < 2 || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) || ((uintptr_t)out & 15))
        return CPM_BAD_ARGUMENT;
    if (epilogue == tc5::EPI_SILU) {
        if (N % 32 != 0) return CPM_BAD_ARGUMENT;
        return tc5::launch_pair<tc5::EPI_SILU>(A, W, out, M, N, K, n_blocks, stream);
    }
    if (epilogue != tc5::EPI_BF16 || N % 8 != 0) return CPM_BAD_ARGUMENT;
    return tc5::launch_pair<tc5::EPI_BF16>(A, W, out, M, N, K, n_blocks, stream);
}

// A [M,K], W [N,K] bf16 row-major (16-byte aligned, K a multiple of 64); out [M,N] bf16, or [M,N/2] for the
// gated epilogue (N a multiple of 32, W rows interleaved in blocks of 8).  n_blocks: blocks to launch (one per SM).
CPM_API void cpm_set_tcgen05_narrow(int on) { tc5::g_narrow_tiles = on ? 1 : 0; }

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
