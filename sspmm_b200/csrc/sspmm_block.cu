// Block variant of the vector-sparse SpMM for matrices whose vector rows are
// dense-ish (most columns present): the compressed operand is expanded once into
// a dense, zero-filled, TRANSPOSED copy  At[K][M']  (M' = m_vec*V), and
//     C[M'][N] = A * B
// runs as a tiled tensor-core GEMM.  Executes 2*M'*K*N flops instead of
// 2*nvec*V*N, but at the full tcgen05 rate (MMA N = 128/256 instead of 16) and
// with every B row read once per 128 output rows instead of once per vector.
//
// Same entry contract as the gather kernel (reference entry:
// SSpMM/src/sspmm.cu:626-649); the choice between the two is made by the host
// from the density nvec / (m_vec*K).
//
// GEMM structure (per CTA, persistent over tiles, m-tile fastest):
//   tile        128 rows of C  x  BN (256 or 128) columns, K step 64
//   MMA A       At tile [64 k][128 m], M-major, 128-byte swizzle  (TMA 2-D boxes 64 x 64)
//   MMA B       B  tile [64 k][BN n],  N-major, 128-byte swizzle  (TMA 2-D boxes 64 x 64)
//   D           TMEM, lane = row of C, column = column of C, two accumulators
//   warps       0 TMA producer, 1 MMA issuer / TMEM owner, 4-7 epilogue
//   epilogue    tcgen05.ld 32 columns at a time -> fp16/fp32 -> 64-byte rows in a swizzled
//               staging tile -> TMA store (clips the M and N tails, keeps stores off the LSU)
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch.h"
#include "ptx.cuh"

namespace sspmm_b200 {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kBlockThreads = 256;

// Process-wide switch for the CTA-pair kernel (tests and profiling compare the two variants through
// sspmm_set_kernel).  Every launch of this file is an ordinary stream-ordered launch.
std::atomic<bool> g_block_pairs{true};

// ---- expansion of the compressed operand ------------------------------------
// At[k][i*V .. i*V+V) = values of the vector of row i at column k, or zeros.
// One CTA per (vector row i, chunk of kExpandChunk columns): the row's column
// list is turned into a column -> vector map in shared memory, then every
// column of the chunk is written (value vector or zeros), so no separate zero
// fill of At is needed.
constexpr int kExpandChunk = 1024;

template <int V>
__global__ void __launch_bounds__(256)
expand_transposed_kernel(int m_vec, int K, const int* __restrict__ row_offsets, const int* __restrict__ col,
                         const __half* __restrict__ values, __half* __restrict__ at) {
    __shared__ int slot[kExpandChunk];
    const int64_t mp = (int64_t)m_vec * V;
    const int k_begin = blockIdx.x * kExpandChunk;
    const int k_end = min(K, k_begin + kExpandChunk);
    for (int i = blockIdx.y; i < m_vec; i += gridDim.y) {
        for (int k = threadIdx.x; k < kExpandChunk; k += blockDim.x) slot[k] = -1;
        __syncthreads();
        const int j0 = row_offsets[i], j1 = row_offsets[i + 1];
        // four independent loads in flight per thread: the kernel is a chain of dependent reads otherwise
        for (int j = j0 + threadIdx.x; j < j1; j += 4 * blockDim.x) {
            int c[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) c[q] = (j + q * (int)blockDim.x < j1) ? __ldg(col + j + q * blockDim.x) : -1;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (c[q] >= k_begin && c[q] < k_end) slot[c[q] - k_begin] = j + q * blockDim.x;   // duplicates: one of them wins
        }
        __syncthreads();
        for (int k = k_begin + threadIdx.x; k < k_end; k += 4 * blockDim.x) {
            int js[4];
            uint4 v[4][V / 8];
#pragma unroll
            for (int q = 0; q < 4; ++q) js[q] = (k + q * (int)blockDim.x < k_end) ? slot[k + q * blockDim.x - k_begin] : -1;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4* src = reinterpret_cast<const uint4*>(values + (int64_t)(js[q] >= 0 ? js[q] : 0) * V);
#pragma unroll
                for (int h = 0; h < V / 8; ++h) v[q][h] = js[q] >= 0 ? __ldg(src + h) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int kq = k + q * (int)blockDim.x;
                if (kq < k_end) {
                    uint4* dst = reinterpret_cast<uint4*>(at + (int64_t)kq * mp + (int64_t)i * V);
#pragma unroll
                    for (int h = 0; h < V / 8; ++h) dst[h] = v[q][h];
                }
            }
        }
        __syncthreads();
    }
}

template <int BN, int STAGES>
struct BlockLayout {
    static constexpr int kAStage = kBM * kBK * 2;                // 16 KB: 2 chunks of [64 k][64 m]
    static constexpr int kBStage = BN * kBK * 2;                 // 4 or 2 chunks of [64 k][64 n]
    static constexpr int kChunk = kBK * 128;                     // 8 KB
    static constexpr int kAOff = 0;
    static constexpr int kBOff = STAGES * kAStage;
    static constexpr int kOutBuf = kBM * 64;                     // 128 rows x 64 bytes
    static constexpr int kOutOff = kBOff + STAGES * kBStage;     // two staging buffers for the TMA store
    static constexpr int kBarOff = kOutOff + 2 * kOutBuf;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemPtrOff + 8;
    static constexpr int kBytes = kAbortOff + 8;
    static constexpr int kDynamic = kBytes + 1024;
    static constexpr uint32_t kTmemCols = 2 * BN;                // two accumulators (power of two: 256 or 512)
};

struct BlockProblem {
    int Mp, N, K;            // rows of C (m_vec*V), columns, reduction length
    int m_tiles, n_tiles, total_tiles;
    int splits, steps_per_split;   // split-K: work item z = split, its K steps [z*steps_per_split, ...); 1 = off
    int wide;                // 1: the operand maps are chunked ({64, K, width/64[, batch]}), so ONE TMA instruction
                             // per operand and stage brings all 64-wide chunks; 0: one instruction per chunk
    int64_t out_stride;      // per batch, elements
};

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(kBlockThreads, 1)
sspmm_block_kernel(const __grid_constant__ CUtensorMap tmap_at, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c, BlockProblem p) {
    using L = BlockLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + L::kBarOff;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_at);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), L::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    const int k_steps = (p.K + kBK - 1) / kBK;
    const int tiles_per_batch = p.m_tiles * p.n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (int T = blockIdx.x; T < p.total_tiles; T += gridDim.x) {
                const int z = T / tiles_per_batch, r = T % tiles_per_batch;
                const int m0 = (r % p.m_tiles) * kBM, n0 = (r / p.m_tiles) * BN;
                const int b = p.splits > 1 ? 0 : z;
                const int ks0 = p.splits > 1 ? z * p.steps_per_split : 0;
                const int ks1 = p.splits > 1 ? min(k_steps, ks0 + p.steps_per_split) : k_steps;
                bool ok = true;
                for (int ks = ks0; ks < ks1; ++ks) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitBlock)) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_arrive_expect_tx(full, L::kAStage + L::kBStage);
                    const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                    if (p.wide) {
                        tma_load_3d(a_s, &tmap_at, 0, ks * kBK, m0 >> 6, full);
                        tma_load_4d(b_s, &tmap_b, 0, ks * kBK, n0 >> 6, b, full);
                    } else {
#pragma unroll
                        for (int c = 0; c < kBM / 64; ++c) tma_load_2d(a_s + c * L::kChunk, &tmap_at, m0 + 64 * c, ks * kBK, full);
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)
                            tma_load_3d(b_s + c * L::kChunk, &tmap_b, n0 + 64 * c, ks * kBK, b, full);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        constexpr uint32_t idesc = make_idesc_f16_f32(kBM, BN, true, true);
        uint32_t stage = 0, phase = 0, acc_it = 0;
        bool ok = true;
        for (int T = blockIdx.x; ok && T < p.total_tiles; T += gridDim.x) {
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            if (!mbar_wait(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag, kStatusWaitBlock)) break;
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * BN;
            const int z = T / tiles_per_batch;
            const int ks0 = p.splits > 1 ? z * p.steps_per_split : 0;
            const int ks1 = p.splits > 1 ? min(k_steps, ks0 + p.steps_per_split) : k_steps;
            for (int ks = ks0; ks < ks1; ++ks) {
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, kStatusWaitBlock)) { ok = false; break; }
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                    // K tail: rows past K are zero-filled by TMA in both operands, so whole 16-row MMAs are safe
                    const int rows = min(kBK, p.K - ks * kBK);
                    const int nk = (rows + 15) >> 4;
                    for (int kk = 0; kk < nk; ++kk) {
                        const uint64_t a_desc = make_smem_desc(a_s + kk * 2048, L::kChunk, 1024, 2);
                        const uint64_t b_desc = make_smem_desc(b_s + kk * 2048, L::kChunk, 1024, 2);
                        tc_mma_f16(d_tmem, a_desc, b_desc, idesc, (ks > ks0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty + 8 * stage);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (!ok) break;
            if (lane == 0) tc_commit(bar_acc_full + 8 * buf);
            __syncwarp();
            ++acc_it;
        }
    } else if (warp >= 4) {
        // Each thread owns one row of the 128-row tile.  Per 32 accumulator columns: TMEM -> registers ->
        // 64-byte row pieces in a staging tile (64-byte swizzle, conflict-free) -> one TMA store.
        constexpr int kColsPerStore = 64 / (int)sizeof(OutT);          // 32 (fp16) or 16 (fp32)
        constexpr int kStoresPerLoad = 32 / kColsPerStore;
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool issuer = (threadIdx.x == 128);
        const uint32_t swz = (uint32_t)((row >> 1) & 3);
        uint32_t acc_it = 0, st_it = 0;
        bool ok = true;
        for (int T = blockIdx.x; ok && T < p.total_tiles; T += gridDim.x) {
            const int b = T / tiles_per_batch, r = T % tiles_per_batch;
            const int m0 = (r % p.m_tiles) * kBM, n0 = (r / p.m_tiles) * BN;
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            // the four warps must agree on leaving: they meet at named barriers below
            if (!named_barrier_and(2, 128, mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kStatusWaitBlock))) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            uint32_t v[2][32];
            tmem_ld_x32(taddr, v[0]);
#pragma unroll
            for (int cc = 0; cc < BN / 32; ++cc) {
                tc_wait_ld();
                if (cc + 1 < BN / 32) {
                    tmem_ld_x32(taddr + (cc + 1) * 32, v[(cc + 1) & 1]);       // in flight while this chunk is stored
                } else {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);        // accumulator drained
                }
                const uint32_t(&w)[32] = v[cc & 1];
#pragma unroll
                for (int h = 0; h < kStoresPerLoad; ++h) {
                    const uint32_t sb = st_it & 1u;
                    uint8_t* stage_row = smem + L::kOutOff + sb * L::kOutBuf + row * 64;
                    named_barrier_sync(1, 128);          // the issuer has seen the store that last read this buffer finish
                    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 o;
                            __half2 h0 = __floats2half2_rn(__uint_as_float(w[g * 8 + 0]), __uint_as_float(w[g * 8 + 1]));
                            __half2 h1 = __floats2half2_rn(__uint_as_float(w[g * 8 + 2]), __uint_as_float(w[g * 8 + 3]));
                            __half2 h2 = __floats2half2_rn(__uint_as_float(w[g * 8 + 4]), __uint_as_float(w[g * 8 + 5]));
                            __half2 h3 = __floats2half2_rn(__uint_as_float(w[g * 8 + 6]), __uint_as_float(w[g * 8 + 7]));
                            o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                            o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(stage_row + (((uint32_t)g ^ swz) << 4)) = o;
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int e = h * 16 + g * 4;
                            *reinterpret_cast<uint4*>(stage_row + (((uint32_t)g ^ swz) << 4)) =
                                make_uint4(w[e], w[e + 1], w[e + 2], w[e + 3]);
                        }
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(1, 128);          // the staging tile is complete
                    if (issuer) {
                        tma_store_3d(&tmap_c, sbase + L::kOutOff + sb * L::kOutBuf, n0 + cc * 32 + h * kColsPerStore, m0, b);
                        tma_store_commit();
                        tma_store_wait_read<1>();        // the other buffer's store has finished reading
                    }
                    ++st_it;
                }
            }
            ++acc_it;
        }
        if (issuer) tma_store_wait_all<0>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
}

// ---- CTA-pair variant ------------------------------------------------------------
// Two CTAs (a cluster of two, on neighbouring SMs) share one 256-row x BN-column tile: each holds its
// own 128 rows of A and HALF of the B tile, and one tcgen05.mma.cta_group::2 (issued by the even CTA)
// reads both halves, so every SM pulls BN/2 instead of BN columns of B per step from L2 -- the block
// kernel is limited by what one SM can pull from L2, not by the tensor pipe.  Each CTA's TMEM receives
// its own 128 rows of D and its own epilogue warps store them.
//   even CTA   owns the "stage filled" barriers (both CTAs' TMA loads report their bytes there) and
//              the "accumulator drained" barriers (both CTAs' epilogue warps arrive there)
//   both CTAs  own a copy of the "stage free" and "accumulator ready" barriers; the MMA thread's
//              tcgen05.commit arrives on both copies
template <int BN, int STAGES>
struct PairLayout {
    static constexpr int kBH = BN / 2;                           // columns of B held by one CTA
    static constexpr int kAStage = kBM * kBK * 2;                // 16 KB
    static constexpr int kBStage = kBH * kBK * 2;                // 16 or 8 KB
    static constexpr int kChunk = kBK * 128;
    static constexpr int kAOff = 0;
    static constexpr int kBOff = STAGES * kAStage;
    static constexpr int kOutBuf = kBM * 64;
    static constexpr int kOutOff = kBOff + STAGES * kBStage;
    static constexpr int kBarOff = kOutOff + 2 * kOutBuf;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemPtrOff + 8;
    static constexpr int kBytes = kAbortOff + 8;
    static constexpr int kDynamic = kBytes + 1024;
    static constexpr uint32_t kTmemCols = 2 * BN;
};

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(kBlockThreads, 1)
sspmm_block_pair_kernel(const __grid_constant__ CUtensorMap tmap_at, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_c, BlockProblem p) {
    using L = PairLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + L::kBarOff;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);            // the even CTA's producer; bytes come from both CTAs
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 8);       // four epilogue warps in each CTA
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_at);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_c);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), L::kTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                // the other CTA's barriers exist before anything is signalled to them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    const int k_steps = (p.K + kBK - 1) / kBK;
    const int tiles_per_batch = p.m_tiles * p.n_tiles;        // m_tiles counts 256-row pair tiles here

    if (warp == 0) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            for (int T = pair; T < p.total_tiles; T += pairs) {
                const int z = T / tiles_per_batch, r = T % tiles_per_batch;
                const int m0 = (r % p.m_tiles) * (2 * kBM) + (int)rank * kBM;
                const int n0 = (r / p.m_tiles) * BN + (int)rank * L::kBH;
                const int b = p.splits > 1 ? 0 : z;
                const int ks0 = p.splits > 1 ? z * p.steps_per_split : 0;
                const int ks1 = p.splits > 1 ? min(k_steps, ks0 + p.steps_per_split) : k_steps;
                bool ok = true;
                for (int ks = ks0; ks < ks1; ++ks) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitBlock)) { ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * (L::kAStage + L::kBStage));
                    const uint32_t full = cluster_map_shared(bar_full + 8 * stage, 0);
                    const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                    if (p.wide) {
                        tma_load_3d_pair(a_s, &tmap_at, 0, ks * kBK, m0 >> 6, full);
                        tma_load_4d_pair(b_s, &tmap_b, 0, ks * kBK, n0 >> 6, b, full);
                    } else {
#pragma unroll
                        for (int c = 0; c < kBM / 64; ++c)
                            tma_load_2d_pair(a_s + c * L::kChunk, &tmap_at, m0 + 64 * c, ks * kBK, full);
#pragma unroll
                        for (int c = 0; c < L::kBH / 64; ++c)
                            tma_load_3d_pair(b_s + c * L::kChunk, &tmap_b, n0 + 64 * c, ks * kBK, b, full);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            constexpr uint32_t idesc = make_idesc_f16_f32(2 * kBM, BN, true, true);
            uint32_t stage = 0, phase = 0, acc_it = 0;
            bool ok = true;
                for (int T = pair; ok && T < p.total_tiles; T += pairs) {
                const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
                if (!mbar_wait(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag, kStatusWaitBlock)) break;
                    tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const int z = T / tiles_per_batch;
                const int ks0 = p.splits > 1 ? z * p.steps_per_split : 0;
                const int ks1 = p.splits > 1 ? min(k_steps, ks0 + p.steps_per_split) : k_steps;
                for (int ks = ks0; ks < ks1; ++ks) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, kStatusWaitBlock)) { ok = false; break; }
                        tc_fence_after_sync();
                    if (lane == 0) {
                        const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                        const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                        const int rows = min(kBK, p.K - ks * kBK);
                        const int nk = (rows + 15) >> 4;
                        for (int kk = 0; kk < nk; ++kk) {
                            const uint64_t a_desc = make_smem_desc(a_s + kk * 2048, L::kChunk, 1024, 2);
                            const uint64_t b_desc = make_smem_desc(b_s + kk * 2048, L::kChunk, 1024, 2);
                            tc_mma_f16_pair(d_tmem, a_desc, b_desc, idesc, (ks > ks0 || kk > 0) ? 1u : 0u);
                        }
                        tc_commit_pair(bar_empty + 8 * stage, 3);          // the stage is free in both CTAs
                    }
                    __syncwarp();
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (lane == 0) tc_commit_pair(bar_acc_full + 8 * buf, 3);  // both CTAs' epilogues may read D
                __syncwarp();
                ++acc_it;
            }
            }
    } else if (warp >= 4) {
        constexpr int kColsPerStore = 64 / (int)sizeof(OutT);
        constexpr int kStoresPerLoad = 32 / kColsPerStore;
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool issuer = (threadIdx.x == 128);
        const uint32_t swz = (uint32_t)((row >> 1) & 3);
        uint32_t acc_it = 0, st_it = 0;
        for (int T = pair; T < p.total_tiles; T += pairs) {
            const int b = T / tiles_per_batch, r = T % tiles_per_batch;
            const int m0 = (r % p.m_tiles) * (2 * kBM) + (int)rank * kBM, n0 = (r / p.m_tiles) * BN;
            const bool rows_exist = m0 < p.Mp;                   // an odd number of 128-row tiles leaves the last half empty
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            if (!named_barrier_and(2, 128, mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kStatusWaitBlock))) break;
            tc_fence_after_sync();
            const uint32_t drained = cluster_map_shared(bar_acc_empty + 8 * buf, 0);
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            uint32_t v[2][32];
            tmem_ld_x32(taddr, v[0]);
#pragma unroll
            for (int cc = 0; cc < BN / 32; ++cc) {
                tc_wait_ld();
                if (cc + 1 < BN / 32) {
                    tmem_ld_x32(taddr + (cc + 1) * 32, v[(cc + 1) & 1]);
                } else {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(drained);
                }
                const uint32_t(&w)[32] = v[cc & 1];
#pragma unroll
                for (int h = 0; h < kStoresPerLoad; ++h) {
                    const uint32_t sb = st_it & 1u;
                    uint8_t* stage_row = smem + L::kOutOff + sb * L::kOutBuf + row * 64;
                    named_barrier_sync(1, 128);
                    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 o;
                            __half2 h0 = __floats2half2_rn(__uint_as_float(w[g * 8 + 0]), __uint_as_float(w[g * 8 + 1]));
                            __half2 h1 = __floats2half2_rn(__uint_as_float(w[g * 8 + 2]), __uint_as_float(w[g * 8 + 3]));
                            __half2 h2 = __floats2half2_rn(__uint_as_float(w[g * 8 + 4]), __uint_as_float(w[g * 8 + 5]));
                            __half2 h3 = __floats2half2_rn(__uint_as_float(w[g * 8 + 6]), __uint_as_float(w[g * 8 + 7]));
                            o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                            o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(stage_row + (((uint32_t)g ^ swz) << 4)) = o;
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            const int e = h * 16 + g * 4;
                            *reinterpret_cast<uint4*>(stage_row + (((uint32_t)g ^ swz) << 4)) =
                                make_uint4(w[e], w[e + 1], w[e + 2], w[e + 3]);
                        }
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(1, 128);
                    if (issuer) {
                        if (rows_exist) {
                            tma_store_3d(&tmap_c, sbase + L::kOutOff + sb * L::kOutBuf, n0 + cc * 32 + h * kColsPerStore, m0, b);
                            tma_store_commit();
                        }
                        tma_store_wait_read<1>();
                    }
                    ++st_it;
                }
            }
            ++acc_it;
        }
        if (issuer) tma_store_wait_all<0>();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                // neither CTA leaves while the other may still signal it or read its memory
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, L::kTmemCols);
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn block_encode_fn() {
    static EncodeFn cached = [] {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<EncodeFn>(fn);
    }();
    return cached;
}

bool encode_2d(EncodeFn enc, CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint32_t box_inner,
               uint32_t box_outer) {
    const cuuint64_t gdim[2] = {inner, outer};
    const cuuint64_t gstride[1] = {inner * sizeof(__half)};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1u, 1u};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D map {inner, rows, batch} with a 64 x `box_rows` x 1 box (in elements: box_inner x box_rows x 1).
bool encode_3d(EncodeFn enc, CUtensorMap* m, CUtensorMapDataType dt, size_t es, const void* base, uint64_t inner,
               uint64_t rows, uint64_t batch, uint64_t batch_stride_elems, uint32_t box_inner, uint32_t box_rows,
               CUtensorMapSwizzle swz) {
    const cuuint64_t gdim[3] = {inner, rows, batch};
    const cuuint64_t gstride[2] = {inner * es, (batch > 1 ? batch_stride_elems : inner * rows) * es};
    const cuuint32_t box[3] = {box_inner, box_rows, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(m, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Chunked views for the one-instruction loads: a row-major [rows][width] fp16 matrix (width % 64 == 0) seen as
// {64, rows, width / 64[, batch]}; a box {64, 64, chunks[, 1]} lands as `chunks` consecutive [64 rows][128 B]
// swizzled blocks, the layout the MMA descriptors expect.
bool encode_chunked(EncodeFn enc, CUtensorMap* m, const void* base, uint64_t width, uint64_t rows, uint64_t batch,
                    uint64_t batch_stride_elems, uint32_t chunks, bool with_batch) {
    const cuuint64_t gdim[4] = {64, rows, width / 64, batch};
    const cuuint64_t gstride[3] = {width * 2, 128, (batch > 1 ? batch_stride_elems : width * rows) * 2};
    const cuuint32_t box[4] = {64, 64, chunks, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, with_batch ? 4 : 3, const_cast<void*>(base), gdim, gstride, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES, typename OutT>
cudaError_t launch_block(const SpmmArgs& a, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                         const BlockProblem& p, int sms, bool setup_only) {
    using L = BlockLayout<BN, STAGES>;
    auto kern = sspmm_block_kernel<BN, STAGES, OutT>;
    static DeviceOnce attr_once;                      // one flag set per instantiation
    if (!attr_once.done()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e != cudaSuccess) return e;
        attr_once.mark();
    }
    if (setup_only) return cudaSuccess;
    // as few CTAs as finish in the same number of rounds: the SMs left over go to products on other streams
    const int rounds = (p.total_tiles + sms - 1) / sms;
    const int grid = (p.total_tiles + rounds - 1) / rounds;
    kern<<<grid, kBlockThreads, L::kDynamic, a.stream>>>(ta, tb, tc, p);
    return cudaGetLastError();
}

// Launch of the CTA-pair kernel: clusters of two CTAs; the persistent grid holds as many pairs as the
// device can keep resident (asked from the occupancy calculator once per device and instantiation).
template <int BN, int STAGES, typename OutT>
cudaError_t launch_block_pair(const SpmmArgs& a, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                              const BlockProblem& p, int sms, bool setup_only) {
    using L = PairLayout<BN, STAGES>;
    auto kern = sspmm_block_pair_kernel<BN, STAGES, OutT>;
    static DeviceOnce attr_once;
    static std::atomic<int> resident_pairs[64];
    int dev = 0;
    cudaGetDevice(&dev);
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kBlockThreads); cfg.dynamicSmemBytes = L::kDynamic; cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (!attr_once.done()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e != cudaSuccess) return e;
        cfg.gridDim = dim3(2 * (sms / 2));
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess) return e;
        if (n <= 0) {
            set_error("no CTA pair of the block kernel fits on this device");
            return cudaErrorLaunchOutOfResources;
        }
        if (dev >= 0 && dev < 64) resident_pairs[dev].store(n, std::memory_order_release);
        attr_once.mark();
    }
    if (setup_only) return cudaSuccess;
    int cap = (dev >= 0 && dev < 64) ? resident_pairs[dev].load(std::memory_order_acquire) : 0;
    if (cap <= 0 || cap > sms / 2) cap = sms / 2;
    const int rounds = (p.total_tiles + cap - 1) / cap;
    const int pairs = (p.total_tiles + rounds - 1) / rounds;     // same number of rounds with fewer pairs, see launch_block
    cfg.gridDim = dim3(2 * pairs);
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, p);
}

// out[i] = sum over splits of partial[s][i], converted once.
template <typename OutT>
__global__ void __launch_bounds__(256)
reduce_splits_kernel(const float* __restrict__ partial, OutT* __restrict__ out, int64_t elems, int splits) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= elems) return;                                      // elems is a multiple of 4 (N % 8 == 0)
    float4 acc = *reinterpret_cast<const float4*>(partial + i);
    for (int s2 = 1; s2 < splits; ++s2) {
        const float4 v = *reinterpret_cast<const float4*>(partial + (int64_t)s2 * elems + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if constexpr (sizeof(OutT) == 2) {
        __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
        uint2 w;
        w.x = *reinterpret_cast<uint32_t*>(&lo); w.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + i) = w;
    } else {
        *reinterpret_cast<float4*>(out + i) = acc;
    }
}

struct BlockPlan {
    bool pair;               // CTA-pair kernel: m_tiles counts 256-row tiles
    int BN, m_tiles, n_tiles, splits, steps_per_split;
    size_t at_bytes, partial_bytes;
};

// Kernel variant, tile shape and split-K factor.  A "unit" is what holds one tile: an SM, or a pair of
// SMs for the CTA-pair kernel (used when C has at least two 128-row tiles and pairing wastes little).
// With fewer tiles than units every CTA is limited by what one SM can pull from L2, so the K range of a
// tile is cut into `splits` work items whose fp32 partial tiles are summed by reduce_splits_kernel;
// `budget` is the scratch the caller can provide.
BlockPlan plan_block(const SpmmArgs& a, int sms, size_t budget) {
    BlockPlan pl;
    const int Mp = a.m_vec * a.V;
    const int m128 = (Mp + kBM - 1) / kBM;
    // The pair kernel pays a cluster launch and two cluster barriers, and both epilogues gate the next
    // tile; measured on B200 it wins once every pair of SMs has a 256 x 256 tile and the K loop is long
    // enough (K >= 512 with fp16 output, K >= 2048 with fp32 output).
    const int m_pairs = (m128 + 1) / 2;
    const int64_t pair_tiles256 = (int64_t)m_pairs * ((a.N + 255) / 256) * a.batch;
    pl.pair = g_block_pairs && m128 >= 2 && (m128 % 2 == 0 || m128 >= 9) && pair_tiles256 >= sms / 2 &&
              a.K >= (a.out_f16 ? 512 : 2048);
    pl.m_tiles = pl.pair ? m_pairs : m128;
    const int units = pl.pair ? sms / 2 : sms;
    const int64_t tiles256 = (int64_t)pl.m_tiles * ((a.N + 255) / 256) * a.batch;
    pl.BN = tiles256 >= units ? 256 : 128;
    pl.n_tiles = (a.N + pl.BN - 1) / pl.BN;
    pl.splits = 1;
    const int k_steps = (a.K + kBK - 1) / kBK;
    pl.steps_per_split = k_steps;
    pl.at_bytes = (((size_t)a.K * Mp * sizeof(__half)) + 255) & ~(size_t)255;
    pl.partial_bytes = 0;
    if (pl.pair || a.batch != 1 || tiles256 >= units || k_steps < 8) return pl;
    // Fewer 256-column tiles than SMs: pick tile width and split-K factor by a small time model
    // (microseconds, constants measured on B200): a work item costs 2 + steps * 0.40 (128 columns) or
    // 2 + steps * 0.45 (256 columns); items run in waves of one per SM; summing fp32 partial tiles costs
    // 3 + their bytes at 4 TB/s.
    double best = 1e30;
    for (int bn = 128; bn <= 256; bn += 128) {
        const int n_tiles = (a.N + bn - 1) / bn;
        const int64_t tiles = (int64_t)pl.m_tiles * n_tiles;
        for (int want = 1; want <= 8; ++want) {
            const int sps = (k_steps + want - 1) / want;
            if (want > 1 && sps < 4) break;
            const int splits = (k_steps + sps - 1) / sps;                // every split gets at least one step
            if (splits != want) continue;
            const size_t bytes = splits > 1 ? (size_t)splits * Mp * a.N * sizeof(float) : 0;
            if (pl.at_bytes + bytes > budget) continue;
            const int64_t waves = (tiles * splits + units - 1) / units;
            double t = (double)waves * (2.0 + sps * (bn == 256 ? 0.45 : 0.40));
            if (splits > 1) t += 3.0 + ((double)bytes + (double)Mp * a.N * 2.0) / 4.0e6;
            if (t < best) {
                best = t;
                pl.BN = bn; pl.n_tiles = n_tiles; pl.splits = splits; pl.steps_per_split = sps; pl.partial_bytes = bytes;
            }
        }
    }
    return pl;
}

}  // namespace

void sspmm_block_allow_pairs(bool allow) { g_block_pairs.store(allow); }

size_t sspmm_block_scratch_bytes(const SpmmArgs& a) {
    const BlockPlan pl = plan_block(a, current_device_sm_count() > 0 ? current_device_sm_count() : 148, ~(size_t)0);
    return pl.at_bytes + pl.partial_bytes;
}

// `scratch` (scratch_bytes long, owned by the caller) holds the transposed dense copy of A
// (K * m_vec*V halfs) and, when split-K is used, the fp32 partial tiles after it.
// Every check and every tensor-map encode comes before the first launch: an error return has
// enqueued nothing and written nothing to `scratch`.
cudaError_t launch_sspmm_block(const SpmmArgs& a, void* scratch, size_t scratch_bytes) {
    EncodeFn enc = block_encode_fn();
    if (!enc) {
        set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
        return cudaErrorNotSupported;
    }
    if (a.values_stride != 0 && a.batch > 1) {
        set_error("the block kernel shares one value array across the batch");
        return cudaErrorInvalidValue;
    }
    const int Mp = a.m_vec * a.V;
    __half* at = static_cast<__half*>(scratch);
    const int sms = current_device_sm_count();
    if (sms <= 0) return cudaErrorNoDevice;
    if (!scratch || (size_t)a.K * Mp * sizeof(__half) > scratch_bytes) {
        set_error("scratch too small for the block kernel");
        return cudaErrorInvalidValue;
    }
    const BlockPlan pl = plan_block(a, sms, scratch_bytes);
    BlockProblem p;
    p.Mp = Mp; p.N = a.N; p.K = a.K;
    p.m_tiles = pl.m_tiles; p.n_tiles = pl.n_tiles;
    p.splits = pl.splits; p.steps_per_split = pl.steps_per_split;
    const int64_t total = (int64_t)p.m_tiles * p.n_tiles * (pl.splits > 1 ? pl.splits : a.batch);
    if (total > 0x7fffffffLL) {
        set_error("problem too large for 32-bit tile ids");
        return cudaErrorInvalidValue;
    }
    p.total_tiles = (int)total;
    p.out_stride = a.out_stride;
    CUtensorMap ta, tb, tc;
    const bool split = pl.splits > 1;
    if (split && pl.at_bytes + pl.partial_bytes > scratch_bytes) {
        set_error("scratch too small for the split-K partial tiles");
        return cudaErrorInvalidValue;
    }
    float* partial = split ? reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + pl.at_bytes) : nullptr;
    const bool c_f16 = a.out_f16 && !split;                       // partial tiles are fp32
    const size_t oes = c_f16 ? 2 : 4;
    // one TMA instruction per operand and stage when both widths are whole 64-element chunks
    const uint32_t b_chunks = (uint32_t)(pl.pair ? pl.BN / 128 : pl.BN / 64);
    p.wide = (Mp % 64 == 0 && a.N % 64 == 0 &&
              encode_chunked(enc, &ta, at, (uint64_t)Mp, (uint64_t)a.K, 1, 0, 2, false) &&
              encode_chunked(enc, &tb, a.rhs, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)a.batch, (uint64_t)a.rhs_stride,
                             b_chunks, true)) ? 1 : 0;
    if ((!p.wide && (!encode_2d(enc, &ta, at, (uint64_t)Mp, (uint64_t)a.K, 64, 64) ||
                     !encode_3d(enc, &tb, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.rhs, (uint64_t)a.N, (uint64_t)a.K,
                                (uint64_t)a.batch, (uint64_t)a.rhs_stride, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B))) ||
        !encode_3d(enc, &tc, c_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, oes,
                   split ? static_cast<void*>(partial) : a.out, (uint64_t)a.N, (uint64_t)Mp,
                   (uint64_t)(split ? pl.splits : a.batch), (uint64_t)(split ? (int64_t)Mp * a.N : a.out_stride),
                   (uint32_t)(64 / oes), 128, CU_TENSOR_MAP_SWIZZLE_64B)) {
        set_error("cuTensorMapEncodeTiled failed (Mp=%d N=%d K=%d batch=%d)", Mp, a.N, a.K, a.batch);
        return cudaErrorInvalidValue;
    }
    // one-time function attributes first (setup_only), then the expansion, then the GEMM
    auto gemm = [&](bool setup_only) -> cudaError_t {
        if (pl.pair)                                              // always 256-column tiles, never split
            return c_f16 ? launch_block_pair<256, 6, __half>(a, ta, tb, tc, p, sms, setup_only)
                         : launch_block_pair<256, 6, float>(a, ta, tb, tc, p, sms, setup_only);
        if (pl.BN == 256)
            return c_f16 ? launch_block<256, 4, __half>(a, ta, tb, tc, p, sms, setup_only)
                         : launch_block<256, 4, float>(a, ta, tb, tc, p, sms, setup_only);
        return c_f16 ? launch_block<128, 6, __half>(a, ta, tb, tc, p, sms, setup_only)
                     : launch_block<128, 6, float>(a, ta, tb, tc, p, sms, setup_only);
    };
    cudaError_t e = gemm(true);
    if (e != cudaSuccess) return e;
    {
        const int by = a.m_vec < 32768 ? a.m_vec : 32768;
        const dim3 grid((a.K + kExpandChunk - 1) / kExpandChunk, by);
        if (a.V == 16) expand_transposed_kernel<16><<<grid, 256, 0, a.stream>>>(a.m_vec, a.K, a.row_offsets, a.column_indices, a.values, at);
        else expand_transposed_kernel<8><<<grid, 256, 0, a.stream>>>(a.m_vec, a.K, a.row_offsets, a.column_indices, a.values, at);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    e = gemm(false);
    if (e != cudaSuccess || !split) return e;
    const int64_t elems = (int64_t)Mp * a.N;
    const unsigned rgrid = (unsigned)((elems / 4 + 255) / 256);
    if (a.out_f16) reduce_splits_kernel<__half><<<rgrid, 256, 0, a.stream>>>(partial, static_cast<__half*>(a.out), elems, pl.splits);
    else reduce_splits_kernel<float><<<rgrid, 256, 0, a.stream>>>(partial, static_cast<float*>(a.out), elems, pl.splits);
    return cudaGetLastError();
}

}  // namespace sspmm_b200
