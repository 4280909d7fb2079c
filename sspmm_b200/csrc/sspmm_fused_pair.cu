// CTA-pair form of the grouped SpMM kernel (sspmm_fused.cu, expanded mode): a cluster of two CTAs on neighbouring SMs
// owns a tile of 256 rows x 256 columns.  Each CTA fetches its own 128 rows of A and only HALF of the B tile by TMA
// (32 KB per K step and SM instead of 48 KB, so six stages fit where the one-CTA kernel has four), the even CTA issues
// tcgen05.mma.cta_group::2 (M = 256) which reads both halves, and each CTA's epilogue stores its own 128 rows.
// The one-CTA kernel waits for TMA data about 40 % of the time (a request is under way for ~3000 cycles under load
// and four stages of 48 KB do not cover that); this form moves a third fewer bytes per flop through L2 -> SM.
//
// Same work-item list, queue, in-kernel expansion of A by the loader warps, split-tile summation and bounded waits as
// the one-CTA kernel; the even CTA's scheduler publishes every item to both CTAs' rings.
//   even CTA   owns the "stage filled" barriers (both CTAs' TMA requests report their bytes there), the
//              "accumulator drained" barriers (both epilogues arrive there) and the "ring slot free" barriers
//   both CTAs  own a copy of the "stage free", "accumulator ready" and "item published" barriers
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch.h"
#include "ptx.cuh"

namespace sspmm_b200 {
namespace fused {

constexpr int kPairStages = 6;
constexpr int kPairBN = 256;

struct PairSmem {
    static constexpr int kAStage = kBM * kBK * 2;                // 16 KB: this CTA's 128 rows of A
    static constexpr int kBStage = (kPairBN / 2) * kBK * 2;      // 16 KB: this CTA's 128 columns of B
    static constexpr int kChunk = kBK * 128;
    static constexpr int kAOff = 0;
    static constexpr int kBOff = kPairStages * kAStage;
    static constexpr int kOutBuf = kBM * 64;
    static constexpr int kOutOff = kBOff + kPairStages * kBStage;
    static constexpr int kBarOff = kOutOff + 2 * kOutBuf;
    static constexpr int kNumBars = 2 * kPairStages + 4 + 2 * kRing;
    static constexpr int kRingOff = kBarOff + kNumBars * 8;
    static constexpr int kTmemPtrOff = kRingOff + kRing * 32;
    static constexpr int kAbortOff = kTmemPtrOff + 8;
    static constexpr int kBcastOff = kAbortOff + 8;
    static constexpr int kBytes = kBcastOff + 8;
    static constexpr int kDynamic = kBytes + 1024;
    static constexpr uint32_t kTmemCols = 2 * kPairBN;
    static_assert(kDynamic <= 227 * 1024, "shared memory of one CTA");
};

template <typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
sspmm_fused_pair_kernel(const __grid_constant__ Params gp) {
    using L = PairSmem;
    constexpr int STAGES = kPairStages, BN = kPairBN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + L::kBarOff;                 // even CTA's copy is the one in use
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;          // even CTA's copy
    const uint32_t bar_item_full = bar_acc_empty + 2 * 8;
    const uint32_t bar_item_empty = bar_item_full + kRing * 8;    // even CTA's copy
    volatile int* ring = reinterpret_cast<volatile int*>(smem + L::kRingOff);
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
    volatile int* bcast = reinterpret_cast<volatile int*>(smem + L::kBcastOff);
    volatile int* bcast2 = bcast + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);            // the even CTA's producer; bytes come from both CTAs
            mbar_init(bar_empty + 8 * s, 1);           // tcgen05.commit (arrives in both CTAs)
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 8);       // four epilogue warps in each CTA
        }
        for (int r = 0; r < kRing; ++r) {
            mbar_init(bar_item_full + 8 * r, 1);
            mbar_init(bar_item_empty + 8 * r, 11);     // even CTA: producer, MMA, 4 epilogue warps; odd CTA: producer, 4 epilogue warps
        }
        *abort_flag = 0;
        mbar_fence_init();
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

    auto problem_of = [&](int prob) -> const Problem* { return gp.probs + prob; };
    // Item n of the pair sits in ring slot n % kRing of BOTH CTAs; "slot free" is counted in the even CTA.
    auto take_item = [&](uint32_t n, Item& it, bool whole_warp) -> bool {
        const uint32_t slot = n % kRing, ph = (n / kRing) & 1u;
        bool ok = mbar_wait_cluster(bar_item_full + 8 * slot, ph, abort_flag, kStatusWaitFused);
        if (whole_warp) ok = __all_sync(0xffffffffu, ok);
        if (!ok) { it.prob = -1; return false; }
        volatile int* e = ring + slot * 8;
        it.prob = e[0]; it.m_tile = e[1]; it.n_tile = e[2]; it.ks0 = e[3]; it.ks1 = e[4];
        it.pslot = e[5]; it.pp = e[6]; it.cslot = e[7];
        if (whole_warp) __syncwarp();
        if (!whole_warp || lane == 0) mbar_arrive_cluster(cluster_map_shared(bar_item_empty + 8 * slot, 0));
        return it.prob >= 0;
    };

    if (warp < 4) {
      if (warp == 0) {
        // ------------------------------------------------------------------ scheduler (even CTA) + TMA producer
        if (lane == 0) {
            uint32_t n_pub = 0;
            bool sched_done = false;
            int idx = pair, raw_next = 0;
            auto publish = [&](uint32_t upto, bool must) -> bool {
                while (!sched_done && n_pub < upto) {
                    const uint32_t slot = n_pub % kRing, ph = (n_pub / kRing) & 1u;
                    if (must) {
                        if (!mbar_wait(bar_item_empty + 8 * slot, ph ^ 1u, abort_flag, kStatusWaitFused)) return false;
                    } else if (!mbar_test_wait(bar_item_empty + 8 * slot, ph ^ 1u)) {
                        return true;
                    }
                    if (n_pub > 0) idx = pairs + raw_next;
                    int w[8] = {-1, 0, 0, 0, 0, 0, 0, 0};
                    if (idx < gp.n_items) {
                        const int4* src = reinterpret_cast<const int4*>(gp.items + idx);
                        const int4 lo = __ldg(src), hi = __ldg(src + 1);
                        w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w; w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
                    }
                    volatile int* e = ring + slot * 8;
                    const uint32_t remote = cluster_map_shared(sbase + L::kRingOff + slot * 32, 1);
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        e[q] = w[q];
                        st_shared_cluster_u32(remote + 4 * q, (uint32_t)w[q]);
                    }
                    mbar_arrive(bar_item_full + 8 * slot);
                    mbar_arrive_cluster(cluster_map_shared(bar_item_full + 8 * slot, 1));
                    ++n_pub;
                    if (w[0] < 0) sched_done = true;
                    else raw_next = atomicAdd(gp.queue, 1);
                }
                return true;
            };
            uint32_t stage = 0, phase = 0;
            int last_prob = -1;
            bool ok = true;
            Item it;
            for (uint32_t n = 0; ok; ++n) {
                if (rank == 0) {
                    if (!publish(n + 1, true)) break;
                    publish(n + 1 + kPublishAheadTma, false);
                }
                if (!take_item(n, it, false)) break;
                const Problem* P = problem_of(it.prob);
                if (it.prob != last_prob) {
                    fence_tensormap_acquire(&P->tmap_a);
                    fence_tensormap_acquire(&P->tmap_b);
                    fence_tensormap_acquire(&P->tmap_b1);
                    // the dense copy of this product's A is written by loader warps of this and other CTAs
                    const int need = P->expand_blocks;
                    const int* done = gp.expand_state + 2 + it.prob;
                    const long long t0 = clock64();
                    while (ld_acquire_gpu(done) < need) {
                        if (*abort_flag) { ok = false; break; }
                        if (clock64() - t0 > g_wait_cycle_limit) {
                            *abort_flag = 1;
                            atomicCAS(&g_device_status, 0, kStatusWaitFused);
                            ok = false;
                            break;
                        }
                    }
                    if (!ok) break;
                    fence_proxy_async_all();
                    last_prob = it.prob;
                }
                const int wide = P->wide;
                const int n0 = it.n_tile * BN;
                const int n_valid = min(BN, P->N - n0);
                const int half = ((n_valid + 15) & ~15) >> 1;                  // columns of B each CTA supplies
                const bool whole = (wide & 1) && n_valid == BN;
                const int chunks = whole ? BN / 128 : (half + 63) >> 6;
                const int m0 = it.m_tile * (2 * kBM) + (int)rank * kBM;
                for (int ks = it.ks0; ks < it.ks1; ++ks) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitFused)) { ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, 2u * (L::kAStage + (uint32_t)chunks * L::kChunk));
                    const uint32_t full = cluster_map_shared(bar_full + 8 * stage, 0);
                    const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                    if (wide & 2) {
                        tma_load_3d_pair(a_s, &P->tmap_a, 0, ks * kBK, m0 >> 6, full);
                    } else {
                        for (int c = 0; c < kBM / 64; ++c) tma_load_3d_pair(a_s + c * L::kChunk, &P->tmap_a, m0 + 64 * c, ks * kBK, 0, full);
                    }
                    if (whole) {
                        tma_load_3d_pair(b_s, &P->tmap_b, 0, ks * kBK, (n0 >> 6) + (int)rank * (BN / 128), full);
                    } else {
                        for (int c = 0; c < chunks; ++c)
                            tma_load_3d_pair(b_s + c * L::kChunk, &P->tmap_b1, n0 + (int)rank * half + 64 * c, ks * kBK, 0, full);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    if (rank == 0 && (ks & 7) == 7) publish(n + 1 + kPublishAheadTma, false);
                }
            }
        }
      } else if (warp == 1 && rank == 0) {
        // ------------------------------------------------------------------ MMA issuer (even CTA)
        uint32_t stage = 0, phase = 0, acc_it = 0;
        bool ok = true;
        Item it;
        for (uint32_t n = 0; ok && take_item(n, it, true); ++n) {
            const Problem* P = problem_of(it.prob);
            const int n_valid = min(BN, P->N - it.n_tile * BN);
            const uint32_t idesc = make_idesc_f16_f32(2 * kBM, (n_valid + 15) & ~15, true, true);
            const int K = P->K;
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag, kStatusWaitFused))) break;
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (int ks = it.ks0; ks < it.ks1; ++ks) {
                if (!__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, kStatusWaitFused))) { ok = false; break; }
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                    const int rows = min(kBK, K - ks * kBK);
                    const int nk = (rows + 15) >> 4;
                    for (int kk = 0; kk < nk; ++kk) {
                        const uint64_t a_desc = make_smem_desc(a_s + kk * 2048, L::kChunk, 1024, 2);
                        const uint64_t b_desc = make_smem_desc(b_s + kk * 2048, L::kChunk, 1024, 2);
                        tc_mma_f16_pair(d_tmem, a_desc, b_desc, idesc, (ks > it.ks0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit_pair(bar_empty + 8 * stage, 3);              // the stage is free in both CTAs
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (!ok) break;
            if (lane == 0) tc_commit_pair(bar_acc_full + 8 * buf, 3);      // both CTAs' epilogues may read D
            __syncwarp();
            ++acc_it;
        }
      }
    } else if (warp >= kLoaderWarp0) {
        // ------------------------------------------------------------------ expansion of A (see sspmm_fused.cu)
        const int t = threadIdx.x - kLoaderWarp0 * 32;
        constexpr int kExpandThreads = kLoaderGroups * kGroupThreads;
        for (;;) {
            if (t == 0) *bcast2 = atomicAdd(gp.expand_state, 1);
            named_barrier_sync(3, kExpandThreads);
            const int vb = *bcast2;
            named_barrier_sync(3, kExpandThreads);
            if (vb >= gp.expand_blocks) break;
            int lo = 0, hi = gp.n_jobs - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (__ldg(&gp.jobs[mid].block_base) <= vb) lo = mid; else hi = mid - 1;
            }
            const ExpandJob job = gp.jobs[lo];
            const int id = (vb - job.block_base) * kExpandThreads + t;
            if (job.V == 16) expand_slots<16>(job, id); else expand_slots<8>(job, id);
            __threadfence();
            named_barrier_sync(3, kExpandThreads);
            if (t == 0) atomicAdd(gp.expand_state + 2 + job.prob, 1);
        }
    } else {
        // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        constexpr int kColsPerStore = 64 / (int)sizeof(OutT);
        constexpr int kStoresPerLoad = 32 / kColsPerStore;
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool issuer = (threadIdx.x == kEpilogueWarp0 * 32);
        const uint32_t swz = (uint32_t)((row >> 1) & 3);
        uint32_t acc_it = 0, st_it = 0;
        int last_prob = -1;
        Item it;
        for (uint32_t n = 0;; ++n) {
            if (!named_barrier_and(2, 128, take_item(n, it, true))) break;
            const Problem* P = problem_of(it.prob);
            const int m0 = it.m_tile * (2 * kBM) + (int)rank * kBM, n0 = it.n_tile * BN;
            const int N = P->N;
            const bool rows_exist = m0 < P->Mp;                  // an odd number of 128-row tiles leaves the last half empty
            const int chunks = (min(BN, N - n0) + 31) >> 5;
            const int parts = it.pp >> 8;
            if (issuer && it.prob != last_prob) fence_tensormap_acquire(&P->tmap_c);
            last_prob = it.prob;
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            if (!named_barrier_and(2, 128, mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kStatusWaitFused))) break;
            tc_fence_after_sync();
            const uint32_t drained = cluster_map_shared(bar_acc_empty + 8 * buf, 0);
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            uint32_t v[2][32];
            tmem_ld_x32(taddr, v[0]);
            if (parts == 1) {
#pragma unroll
                for (int cc = 0; cc < BN / 32; ++cc) {
                    if (cc < chunks) {
                        tc_wait_ld();
                        if (cc + 1 < chunks) {
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
                                    tma_store_3d(&P->tmap_c, sbase + L::kOutOff + sb * L::kOutBuf, n0 + cc * 32 + h * kColsPerStore, m0, 0);
                                    tma_store_commit();
                                }
                                tma_store_wait_read<1>();
                            }
                            ++st_it;
                        }
                    }
                }
            } else {
                // part of a tile's K range: fp32 partial of this CTA's 128 rows to scratch; the last part to arrive for
                // this half of the tile adds all parts in part order and writes C (see sspmm_fused.cu)
                float4* mine = reinterpret_cast<float4*>(gp.partials) + ((int64_t)it.pslot * 2 + rank) * (BN * 32);
#pragma unroll
                for (int cc = 0; cc < BN / 32; ++cc) {
                    if (cc < chunks) {
                        tc_wait_ld();
                        if (cc + 1 < chunks) {
                            tmem_ld_x32(taddr + (cc + 1) * 32, v[(cc + 1) & 1]);
                        } else {
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive_cluster(drained);
                        }
                        const uint32_t(&w)[32] = v[cc & 1];
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            __stcg(mine + (cc * 8 + i) * kBM + row,
                                   make_float4(__uint_as_float(w[4 * i]), __uint_as_float(w[4 * i + 1]),
                                               __uint_as_float(w[4 * i + 2]), __uint_as_float(w[4 * i + 3])));
                    }
                }
                __threadfence();
                named_barrier_sync(1, 128);
                if (issuer) *bcast = atomicAdd(gp.counters + it.cslot * 2 + rank, 1);
                named_barrier_sync(1, 128);
                if (*bcast == parts - 1) {
                    __threadfence();
                    const float4* first = reinterpret_cast<const float4*>(gp.partials) +
                                          ((int64_t)(it.pslot - (it.pp & 0xff)) * 2 + rank) * (BN * 32);
                    const int gm = m0 + row;
                    OutT* crow = static_cast<OutT*>(P->out) + (int64_t)gm * N + n0;
                    for (int cc = 0; cc < chunks; ++cc) {
                        float4 acc[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] = __ldcg(first + (cc * 8 + i) * kBM + row);
                        for (int p = 1; p < parts; ++p) {
                            const float4* src = first + (int64_t)p * 2 * (BN * 32);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float4 x = __ldcg(src + (cc * 8 + i) * kBM + row);
                                acc[i].x += x.x; acc[i].y += x.y; acc[i].z += x.z; acc[i].w += x.w;
                            }
                        }
                        if (gm < P->Mp) {
                            if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                                for (int g = 0; g < 4; ++g) {
                                    if (n0 + cc * 32 + g * 8 < N) {
                                        __half2 h0 = __floats2half2_rn(acc[2 * g].x, acc[2 * g].y);
                                        __half2 h1 = __floats2half2_rn(acc[2 * g].z, acc[2 * g].w);
                                        __half2 h2 = __floats2half2_rn(acc[2 * g + 1].x, acc[2 * g + 1].y);
                                        __half2 h3 = __floats2half2_rn(acc[2 * g + 1].z, acc[2 * g + 1].w);
                                        uint4 o;
                                        o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
                                        o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
                                        *reinterpret_cast<uint4*>(crow + cc * 32 + g * 8) = o;
                                    }
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    if (n0 + cc * 32 + i * 4 < N) *reinterpret_cast<float4*>(crow + cc * 32 + i * 4) = acc[i];
                            }
                        }
                    }
                    if (issuer) gp.counters[it.cslot * 2 + rank] = 0;
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
    // The CTA that leaves last puts the queue and the expansion counters back to zero for the next run.
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(gp.queue + 1, 1) == (int)gridDim.x - 1) {
            gp.queue[0] = 0;
            gp.queue[1] = 0;
            for (int i = 0; i < 2 + gp.n_jobs; ++i) gp.expand_state[i] = 0;
            __threadfence();
        }
    }
}

cudaError_t launch_pair(const Params& p, bool out_f16, int pairs, cudaStream_t st, bool setup_only) {
    using L = PairSmem;
    auto kern_h = sspmm_fused_pair_kernel<__half>;
    auto kern_f = sspmm_fused_pair_kernel<float>;
    static DeviceOnce once;
    if (!once.done()) {
        cudaError_t e = cudaFuncSetAttribute(kern_h, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(kern_f, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e != cudaSuccess) return e;
        once.mark();
    }
    if (setup_only) return cudaSuccess;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = L::kDynamic; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return out_f16 ? cudaLaunchKernelEx(&cfg, kern_h, p) : cudaLaunchKernelEx(&cfg, kern_f, p);
}

}  // namespace fused
}  // namespace sspmm_b200
