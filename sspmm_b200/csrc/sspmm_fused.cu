// Vector-sparse SpMM as ONE persistent tensor-core launch, for one product or for a whole group of
// products (the layers of a model step), straight from the compressed operand: no dense copy of A,
// no scratch for it, no second kernel.
//
//   C[M'][N] = A_vs * B      M' = m_vec * V        (reference entry: SSpMM/src/sspmm.cu:548-649,
//                                                   one launch per product, no scratch)
//
// What makes the compressed operand directly usable is a PLAN, built once per weight STRUCTURE
// (row_offsets / column_indices; values may change freely): for every 128-row tile of A, every 64-column
// step and every vector row of the tile, a 64-bit mask of the columns that carry a vector and the
// position of the first of them in column order (16 bytes).  A loader thread that owns slot (vector
// row, column k) of a stage then knows, without reading a column id, whether a vector exists and where:
// values[start + popc(mask below k)], through a permutation when the row's list is not ascending.
//
// Per CTA (persistent, one per SM), tile 128 rows x BN columns, K step 64:
//   warp 0        TMA producer of the B tile [64 k][BN n] (N-major, 128-byte swizzle)
//   warp 1        MMA issuer / TMEM owner: tcgen05.mma kind::f16, M = 128, N <= BN, K = 16, accumulators
//                 2 x BN TMEM columns
//   warp 2        scheduler: takes work items (static stride, or an atomic queue shared by the grid) and
//                 publishes them to the other warps through a small shared-memory ring
//   warps 4-7     epilogue: TMEM -> registers -> swizzled staging -> TMA store; or, for a tile whose K range
//                 was cut into parts, fp32 partial tile to scratch and the LAST part to arrive adds all parts
//                 in part order and writes C (no CTA ever waits for another)
//   warps 8-15    two loader groups that build the A tile [64 k][128 m] (M-major, 128-byte swizzle) of
//                 alternate stages from the value vectors with 16-byte loads and stores
// Every wait is bounded and unwinds with a status code (see ptx.cuh).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <new>
#include <vector>

#include "../../include/sspmm_b200.h"
#include "launch.h"
#include "ptx.cuh"

namespace sspmm_b200 {
namespace fused {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 512;
constexpr int kRing = 4;
constexpr int kLoaderGroups = 2;
constexpr int kGroupThreads = 128;

// One product, as the kernel sees it.  Lives in kernel parameter space (single product) or in device
// memory (group); 64-byte aligned because of the tensor maps.
struct alignas(64) Problem {
    CUtensorMap tmap_b;        // B  {N, K, 1}   fp16, box 64 x 64, 128-byte swizzle
    CUtensorMap tmap_c;        // C  {N, M', 1}  fp16/fp32, box (64 bytes) x 128 rows, 64-byte swizzle
    const uint4* meta;         // plan: [m_tile][k_step][row in tile] {mask lo, mask hi, start, 0}
    const int* perm;           // plan: position in column order -> index of the vector (null = identity)
    const __half* values;
    void* out;
    int Mp, N, K, V;
    int k_steps, m_tiles, n_tiles, reserved;
};
static_assert(sizeof(Problem) % 64 == 0, "Problem must keep the tensor maps 64-byte aligned in arrays");

// A unit of work: K steps [ks0, ks1) of one tile.  parts > 1: the tile's K range was cut; this is part
// `part`, its fp32 partial tile is slot pslot of the scratch (parts of a tile are consecutive slots) and
// cslot is the tile's arrival counter.
struct Item {
    int prob, m_tile, n_tile, ks0, ks1, pslot, pp /* part | parts << 8 */, cslot;
};

struct Params {
    const Problem* probs;      // device array, or null: inline_prob
    const Item* items;         // device array, or null: every tile of inline_prob once, whole K range
    int n_items;
    int dynamic;               // 1: items are taken from queue[0] (grid-wide atomic), else CTA b takes b, b + grid, ...
    int* queue;                // [0] next item, [1] CTAs that finished taking items (the last one resets both)
    float* partials;
    int* counters;
    Problem inline_prob;
};

template <int BN, int STAGES>
struct Layout {
    static constexpr int kAStage = kBM * kBK * 2;                // 16 KB: 2 chunks of [64 k][64 m]
    static constexpr int kBStage = BN * kBK * 2;                 // BN/64 chunks of [64 k][64 n]
    static constexpr int kChunk = kBK * 128;                     // 8 KB
    static constexpr int kAOff = 0;
    static constexpr int kBOff = STAGES * kAStage;
    static constexpr int kOutBuf = kBM * 64;                     // 128 rows x 64 bytes
    static constexpr int kOutOff = kBOff + STAGES * kBStage;
    static constexpr int kBarOff = kOutOff + 2 * kOutBuf;
    static constexpr int kNumBars = 2 * STAGES + 4 + 2 * kRing;
    static constexpr int kRingOff = kBarOff + kNumBars * 8;
    static constexpr int kTmemPtrOff = kRingOff + kRing * 32;
    static constexpr int kAbortOff = kTmemPtrOff + 8;
    static constexpr int kBcastOff = kAbortOff + 8;
    static constexpr int kBytes = kBcastOff + 8;
    static constexpr int kDynamic = kBytes + 1024;
    static constexpr uint32_t kTmemCols = 2 * BN;                // 128, 256 or 512
};

__device__ __forceinline__ void fence_tensormap_acquire(const void* tmap) {
    // a tensor map that was written to global memory by a copy is read through its own proxy
    asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// Loads the value vectors of one A stage (vector rows of tile m_tile, columns [64 ks, 64 ks + 64)) into
// registers: thread t of the 128 of a loader group owns vector row t / TPR and columns t % TPR + TPR * q.
template <int V>
struct AStage {
    static constexpr int R = kBM / V;             // vector rows per tile: 8 or 16
    static constexpr int TPR = kGroupThreads / R; // threads per vector row: 16 or 8
    static constexpr int SLOTS = kBK / TPR;       // columns per thread: 4 or 8
    static constexpr int H = V / 8;               // 16-byte pieces per vector: 2 or 1
    uint4 v[SLOTS][H];

    __device__ __forceinline__ void load(const Problem* P, uint4 meta, int t) {
        const unsigned long long mask = (unsigned long long)meta.x | ((unsigned long long)meta.y << 32);
        const int start = (int)meta.z;
        const int kb = t % TPR;
        int jj[SLOTS];
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int kk = kb + TPR * q;
            const bool present = (mask >> kk) & 1ull;
            jj[q] = present ? start + __popcll(mask & ((1ull << kk) - 1ull)) : -1;
        }
        if (P->perm) {
#pragma unroll
            for (int q = 0; q < SLOTS; ++q)
                if (jj[q] >= 0) jj[q] = __ldg(P->perm + jj[q]);
        }
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const uint4* src = reinterpret_cast<const uint4*>(P->values + (int64_t)(jj[q] >= 0 ? jj[q] : 0) * V);
#pragma unroll
            for (int h = 0; h < H; ++h) v[q][h] = jj[q] >= 0 ? __ldg(src + h) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // a_s: the stage's A tile; rows of 128 bytes (64 m of one k), 16-byte pieces XOR-swizzled by k & 7
    __device__ __forceinline__ void store(uint8_t* a_s, int t) const {
        const int r = t / TPR, kb = t % TPR;
        uint8_t* base = a_s + (r / (R / 2)) * (kBK * 128);
        const int piece0 = (r % (R / 2)) * H;
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int kk = kb + TPR * q;
#pragma unroll
            for (int h = 0; h < H; ++h)
                *reinterpret_cast<uint4*>(base + kk * 128 + (((piece0 + h) ^ (kk & 7)) << 4)) = v[q][h];
        }
    }
    static __device__ __forceinline__ uint4 load_meta(const Problem* P, int m_tile, int ks, int t) {
        return __ldg(P->meta + ((int64_t)m_tile * P->k_steps + ks) * R + t / TPR);
    }
};

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
sspmm_fused_kernel(const __grid_constant__ Params gp) {
    using L = Layout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + L::kBarOff;
    const uint32_t bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    const uint32_t bar_item_full = bar_acc_empty + 2 * 8;
    const uint32_t bar_item_empty = bar_item_full + kRing * 8;
    volatile int* ring = reinterpret_cast<volatile int*>(smem + L::kRingOff);
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
    volatile int* bcast = reinterpret_cast<volatile int*>(smem + L::kBcastOff);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1 + kGroupThreads / 32);   // producer's expect_tx + the loader group's warps
            mbar_init(bar_empty + 8 * s, 1);                       // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);
        }
        for (int r = 0; r < kRing; ++r) {
            mbar_init(bar_item_full + 8 * r, 1);
            mbar_init(bar_item_empty + 8 * r, 14);                 // warps 0, 1, 4-7, 8-15
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), L::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    // Item n of this CTA sits in ring slot n % kRing; everyone but the scheduler reads it the same way.
    auto problem_of = [&](int prob) -> const Problem* { return gp.probs ? gp.probs + prob : &gp.inline_prob; };
    // whole_warp: every lane of the calling warp takes part and all of them get the same answer.
    auto take_item = [&](uint32_t n, Item& it, bool whole_warp) -> bool {
        const uint32_t slot = n % kRing, ph = (n / kRing) & 1u;
        bool ok = mbar_wait(bar_item_full + 8 * slot, ph, abort_flag, kStatusWaitFused);
        if (whole_warp) ok = __all_sync(0xffffffffu, ok);
        if (!ok) { it.prob = -1; return false; }
        volatile int* e = ring + slot * 8;
        it.prob = e[0]; it.m_tile = e[1]; it.n_tile = e[2]; it.ks0 = e[3]; it.ks1 = e[4];
        it.pslot = e[5]; it.pp = e[6]; it.cslot = e[7];
        if (whole_warp) __syncwarp();
        if (!whole_warp || lane == 0) mbar_arrive(bar_item_empty + 8 * slot);
        return it.prob >= 0;
    };

    if (warp == 2) {
        // ------------------------------------------------------------------ scheduler
        if (lane == 0) {
            int idx = blockIdx.x;
            for (uint32_t n = 0;; ++n) {
                const uint32_t slot = n % kRing, ph = (n / kRing) & 1u;
                if (!mbar_wait(bar_item_empty + 8 * slot, ph ^ 1u, abort_flag, kStatusWaitFused)) break;
                Item it;
                if (idx < gp.n_items) {
                    if (gp.items) {
                        const int4* src = reinterpret_cast<const int4*>(gp.items + idx);
                        const int4 lo = __ldg(src), hi = __ldg(src + 1);
                        it.prob = lo.x; it.m_tile = lo.y; it.n_tile = lo.z; it.ks0 = lo.w;
                        it.ks1 = hi.x; it.pslot = hi.y; it.pp = hi.z; it.cslot = hi.w;
                    } else {
                        it.prob = 0; it.m_tile = idx % gp.inline_prob.m_tiles; it.n_tile = idx / gp.inline_prob.m_tiles;
                        it.ks0 = 0; it.ks1 = gp.inline_prob.k_steps; it.pslot = 0; it.pp = 1 << 8; it.cslot = 0;
                    }
                } else {
                    it.prob = -1; it.m_tile = it.n_tile = it.ks0 = it.ks1 = it.pslot = it.pp = it.cslot = 0;
                }
                volatile int* e = ring + slot * 8;
                e[0] = it.prob; e[1] = it.m_tile; e[2] = it.n_tile; e[3] = it.ks0; e[4] = it.ks1;
                e[5] = it.pslot; e[6] = it.pp; e[7] = it.cslot;
                mbar_arrive(bar_item_full + 8 * slot);
                if (it.prob < 0) break;
                idx = gp.dynamic ? (int)gridDim.x + atomicAdd(gp.queue, 1) : idx + (int)gridDim.x;
            }
            if (gp.dynamic) {
                __threadfence();
                const int done = atomicAdd(gp.queue + 1, 1);
                if (done == (int)gridDim.x - 1) {            // every CTA has taken its last item: ready for the next launch
                    gp.queue[0] = 0;
                    gp.queue[1] = 0;
                    __threadfence();
                }
            }
        }
    } else if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer of B
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            int last_prob = -1;
            bool ok = true;
            Item it;
            for (uint32_t n = 0; ok && take_item(n, it, false); ++n) {
                const Problem* P = problem_of(it.prob);
                if (gp.probs && it.prob != last_prob) {
                    fence_tensormap_acquire(&P->tmap_b);
                    last_prob = it.prob;
                }
                const int n0 = it.n_tile * BN;
                const int chunks = min(BN / 64, (P->N - n0 + 63) >> 6);
                for (int ks = it.ks0; ks < it.ks1; ++ks) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitFused)) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_arrive_expect_tx(full, (uint32_t)chunks * L::kChunk);
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                    for (int c = 0; c < chunks; ++c) tma_load_3d(b_s + c * L::kChunk, &P->tmap_b, n0 + 64 * c, ks * kBK, 0, full);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        uint32_t stage = 0, phase = 0, acc_it = 0;
        bool ok = true;
        Item it;
        for (uint32_t n = 0; ok && take_item(n, it, true); ++n) {
            const Problem* P = problem_of(it.prob);
            const int n_valid = min(BN, P->N - it.n_tile * BN);
            const uint32_t idesc = make_idesc_f16_f32(kBM, (n_valid + 15) & ~15, true, true);
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
                    // K tail: columns of A past K carry no vector and rows of B past K are zero-filled by TMA
                    const int rows = min(kBK, K - ks * kBK);
                    const int nk = (rows + 15) >> 4;
                    for (int kk = 0; kk < nk; ++kk) {
                        const uint64_t a_desc = make_smem_desc(a_s + kk * 2048, L::kChunk, 1024, 2);
                        const uint64_t b_desc = make_smem_desc(b_s + kk * 2048, L::kChunk, 1024, 2);
                        tc_mma_f16(d_tmem, a_desc, b_desc, idesc, (ks > it.ks0 || kk > 0) ? 1u : 0u);
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
    } else if (warp >= 8) {
        // ------------------------------------------------------------------ A loaders
        const int group = (warp - 8) >> 2;
        const int t = threadIdx.x - (256 + kGroupThreads * group);
        uint32_t it_count = 0;
        bool ok = true;
        Item it;
        for (uint32_t n = 0; ok && take_item(n, it, true); ++n) {
            const Problem* P = problem_of(it.prob);
            const int steps = it.ks1 - it.ks0;
            // first step of this item that belongs to this group (groups alternate over the CTA's stage sequence)
            int s = ((int)(it_count & 1u) == group) ? 0 : 1;
            if (P->V == 16) {
                uint4 meta = s < steps ? AStage<16>::load_meta(P, it.m_tile, it.ks0 + s, t) : make_uint4(0, 0, 0, 0);
                for (; s < steps; s += kLoaderGroups) {
                    const uint32_t c = it_count + (uint32_t)s;
                    const uint32_t stage = c % STAGES, phase = (c / STAGES) & 1u;
                    AStage<16> a;
                    a.load(P, meta, t);
                    if (s + kLoaderGroups < steps) meta = AStage<16>::load_meta(P, it.m_tile, it.ks0 + s + kLoaderGroups, t);
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitFused))) { ok = false; break; }
                    a.store(smem + L::kAOff + stage * L::kAStage, t);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * stage);
                }
            } else {
                uint4 meta = s < steps ? AStage<8>::load_meta(P, it.m_tile, it.ks0 + s, t) : make_uint4(0, 0, 0, 0);
                for (; s < steps; s += kLoaderGroups) {
                    const uint32_t c = it_count + (uint32_t)s;
                    const uint32_t stage = c % STAGES, phase = (c / STAGES) & 1u;
                    AStage<8> a;
                    a.load(P, meta, t);
                    if (s + kLoaderGroups < steps) meta = AStage<8>::load_meta(P, it.m_tile, it.ks0 + s + kLoaderGroups, t);
                    if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitFused))) { ok = false; break; }
                    a.store(smem + L::kAOff + stage * L::kAStage, t);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * stage);
                }
            }
            it_count += (uint32_t)steps;
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue
        // Each thread owns one row of the 128-row tile and handles 32 accumulator columns at a time.
        constexpr int kColsPerStore = 64 / (int)sizeof(OutT);          // 32 (fp16) or 16 (fp32)
        constexpr int kStoresPerLoad = 32 / kColsPerStore;
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool issuer = (threadIdx.x == 128);
        const uint32_t swz = (uint32_t)((row >> 1) & 3);
        uint32_t acc_it = 0, st_it = 0;
        int last_prob = -1;
        Item it;
        for (uint32_t n = 0;; ++n) {
            // the four warps must agree on leaving: they meet at named barriers below
            if (!named_barrier_and(2, 128, take_item(n, it, true))) break;
            const Problem* P = problem_of(it.prob);
            const int m0 = it.m_tile * kBM, n0 = it.n_tile * BN;
            const int N = P->N;
            const int chunks = (min(BN, N - n0) + 31) >> 5;
            const int parts = it.pp >> 8;
            if (issuer && gp.probs && it.prob != last_prob) fence_tensormap_acquire(&P->tmap_c);
            last_prob = it.prob;
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            if (!named_barrier_and(2, 128, mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kStatusWaitFused))) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            uint32_t v[2][32];
            tmem_ld_x32(taddr, v[0]);
            if (parts == 1) {
#pragma unroll
                for (int cc = 0; cc < BN / 32; ++cc) {
                    if (cc < chunks) {
                        tc_wait_ld();
                        if (cc + 1 < chunks) {
                            tmem_ld_x32(taddr + (cc + 1) * 32, v[(cc + 1) & 1]);   // in flight while this chunk is stored
                        } else {
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);    // accumulator drained
                        }
                        const uint32_t(&w)[32] = v[cc & 1];
#pragma unroll
                        for (int h = 0; h < kStoresPerLoad; ++h) {
                            const uint32_t sb = st_it & 1u;
                            uint8_t* stage_row = smem + L::kOutOff + sb * L::kOutBuf + row * 64;
                            named_barrier_sync(1, 128);      // the issuer has seen the store that last read this buffer finish
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
                            named_barrier_sync(1, 128);      // the staging tile is complete
                            if (issuer) {
                                tma_store_3d(&P->tmap_c, sbase + L::kOutOff + sb * L::kOutBuf, n0 + cc * 32 + h * kColsPerStore, m0, 0);
                                tma_store_commit();
                                tma_store_wait_read<1>();    // the other buffer's store has finished reading
                            }
                            ++st_it;
                        }
                    }
                }
            } else {
                // This item covers a part of the tile's K range.  Its fp32 partial tile goes to scratch as
                // [32-column chunk][float4 index][row] (coalesced); then the tile's arrival counter tells whether
                // this was the last part, in which case all parts are added in part order and C is written.
                float4* mine = reinterpret_cast<float4*>(gp.partials) + (int64_t)it.pslot * (BN * 32);
#pragma unroll
                for (int cc = 0; cc < BN / 32; ++cc) {
                    if (cc < chunks) {
                        tc_wait_ld();
                        if (cc + 1 < chunks) {
                            tmem_ld_x32(taddr + (cc + 1) * 32, v[(cc + 1) & 1]);
                        } else {
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
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
                if (issuer) *bcast = atomicAdd(gp.counters + it.cslot, 1);
                named_barrier_sync(1, 128);
                if (*bcast == parts - 1) {
                    __threadfence();
                    const float4* first = reinterpret_cast<const float4*>(gp.partials) + (int64_t)(it.pslot - (it.pp & 0xff)) * (BN * 32);
                    const int gm = m0 + row;
                    OutT* crow = static_cast<OutT*>(P->out) + (int64_t)gm * N + n0;
                    for (int cc = 0; cc < chunks; ++cc) {
                        float4 acc[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[i] = __ldcg(first + (cc * 8 + i) * kBM + row);
                        for (int p = 1; p < parts; ++p) {
                            const float4* src = first + (int64_t)p * (BN * 32);
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
                                    if (n0 + cc * 32 + g * 8 < N) {              // N % 8 == 0: a piece is all in or all out
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
                    if (issuer) gp.counters[it.cslot] = 0;         // ready for the next launch
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

// ---- plan construction ------------------------------------------------------------------
// One CTA per vector row: bitmap of the row's columns in shared memory -> masks, starts, permutation.
// flags: [0] irregular (column outside [0, K) or listed twice in a vector row), [1] some row is not ascending,
//        [2] longest vector row.
template <int V>
__global__ void __launch_bounds__(256)
plan_build_kernel(int m_vec, int K, int k_steps, const int* __restrict__ row_offsets, const int* __restrict__ col,
                  uint4* __restrict__ meta, int* __restrict__ perm, int* __restrict__ flags) {
    extern __shared__ unsigned int sm[];
    unsigned int* bm = sm;                       // 2 * k_steps words
    int* pre = reinterpret_cast<int*>(sm + 2 * k_steps);     // k_steps exclusive prefix
    __shared__ int carry, warp_tot[8];
    constexpr int R = kBM / V;
    const int i = blockIdx.x;
    const int j0 = row_offsets[i], j1 = row_offsets[i + 1];
    for (int w = threadIdx.x; w < 2 * k_steps; w += 256) bm[w] = 0u;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    bool bad = j1 < j0;
    for (int j = j0 + threadIdx.x; j < j1; j += 256) {
        const int c = col[j];
        if ((unsigned)c >= (unsigned)K) { bad = true; continue; }
        const unsigned bit = 1u << (c & 31);
        if (atomicOr(&bm[c >> 5], bit) & bit) bad = true;
    }
    __syncthreads();
    // exclusive prefix of popc over the k steps, 256 at a time
    const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
    for (int base = 0; base < k_steps; base += 256) {
        const int ks = base + threadIdx.x;
        const int pc = ks < k_steps ? __popc(bm[2 * ks]) + __popc(bm[2 * ks + 1]) : 0;
        int inc = pc;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int x = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += x;
        }
        if (lane == 31) warp_tot[wp] = inc;
        __syncthreads();
        int before = carry;
        for (int w = 0; w < wp; ++w) before += warp_tot[w];
        if (ks < k_steps) pre[ks] = before + inc - pc;
        __syncthreads();
        if (threadIdx.x == 255) carry = before + inc;
        __syncthreads();
    }
    const int64_t tile = i / R, r = i % R;
    for (int ks = threadIdx.x; ks < k_steps; ks += 256)
        meta[(tile * k_steps + ks) * R + r] = make_uint4(bm[2 * ks], bm[2 * ks + 1], (unsigned)(j0 + pre[ks]), 0u);
    bool unsorted = false;
    for (int j = j0 + threadIdx.x; j < j1; j += 256) {
        const int c = col[j];
        if ((unsigned)c >= (unsigned)K) continue;
        const int rank = pre[c >> 6] + (((c >> 5) & 1) ? __popc(bm[2 * (c >> 6)]) : 0) + __popc(bm[c >> 5] & ((1u << (c & 31)) - 1u));
        if (rank != j - j0) unsorted = true;
        if (rank < j1 - j0) perm[j0 + rank] = j;
    }
    if (bad) atomicOr(flags + 0, 1);
    if (unsorted) atomicOr(flags + 1, 1);
    if (threadIdx.x == 0) atomicMax(flags + 2, j1 - j0);
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
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

// {inner, rows, 1} with a box_inner x box_rows x 1 box.
bool encode_map(EncodeFn enc, CUtensorMap* m, CUtensorMapDataType dt, size_t es, const void* base, uint64_t inner,
                uint64_t rows, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swz) {
    const cuuint64_t gdim[3] = {inner, rows, 1};
    const cuuint64_t gstride[2] = {inner * es, inner * rows * es};
    const cuuint32_t box[3] = {box_inner, box_rows, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(m, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace fused
}  // namespace sspmm_b200

// ---- C ABI ----------------------------------------------------------------------------------
using namespace sspmm_b200;

struct sspmm_plan {
    int m_vec, V, K, device;
    long long nvec;
    int max_len;
    int m_tiles, k_steps;
    bool fused;                // metadata built and the structure is regular: the one-launch kernel applies
    bool sorted;
    const int* row_offsets;    // the caller's arrays (not owned)
    const int* column_indices;
    uint4* meta;               // owned
    int* perm;                 // owned, null when every row is ascending
};

struct sspmm_group {
    int device, count, BN;
    bool out_f16;
    int n_items, grid;
    void* dev_block;           // one allocation: problems | items | queue | counters | partials
    fused::Params params;
    size_t partial_bytes;
};

namespace sspmm_b200 {
namespace fused {

constexpr size_t kMaxMetaBytes = (size_t)256 << 20;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int BN, int STAGES, typename OutT>
cudaError_t launch_typed(const Params& p, int grid, cudaStream_t st, bool setup_only) {
    using L = Layout<BN, STAGES>;
    auto kern = sspmm_fused_kernel<BN, STAGES, OutT>;
    static DeviceOnce once;
    if (!once.done()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e != cudaSuccess) return e;
        once.mark();
    }
    if (setup_only) return cudaSuccess;
    kern<<<grid, kThreads, L::kDynamic, st>>>(p);
    return cudaGetLastError();
}

cudaError_t launch(const Params& p, int BN, bool out_f16, int grid, cudaStream_t st, bool setup_only = false) {
    if (BN == 256) return out_f16 ? launch_typed<256, 4, __half>(p, grid, st, setup_only) : launch_typed<256, 4, float>(p, grid, st, setup_only);
    if (BN == 128) return out_f16 ? launch_typed<128, 6, __half>(p, grid, st, setup_only) : launch_typed<128, 6, float>(p, grid, st, setup_only);
    return out_f16 ? launch_typed<64, 8, __half>(p, grid, st, setup_only) : launch_typed<64, 8, float>(p, grid, st, setup_only);
}

// Fills everything of a Problem but nothing that lives on the device.  Returns false with the error set.
bool fill_problem(Problem* P, const sspmm_plan* plan, const void* values, const void* rhs, void* out, int N, bool out_f16,
                  int BN) {
    EncodeFn enc = encode_fn();
    if (!enc) { set_error("cuTensorMapEncodeTiled is not available from the CUDA driver"); return false; }
    if (!plan || !plan->fused) { set_error("the plan does not support the one-launch kernel"); return false; }
    if (N <= 0 || N % 8 != 0 || !values || !rhs || !out || !aligned16(values) || !aligned16(rhs) || !aligned16(out)) {
        set_error("the planned SpMM needs N > 0, N %% 8 == 0 and 16-byte aligned values, rhs and output");
        return false;
    }
    const int Mp = plan->m_vec * plan->V;
    const size_t oes = out_f16 ? 2 : 4;
    if (!encode_map(enc, &P->tmap_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, rhs, (uint64_t)N, (uint64_t)plan->K, 64, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B) ||
        !encode_map(enc, &P->tmap_c, out_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, oes, out,
                    (uint64_t)N, (uint64_t)Mp, (uint32_t)(64 / oes), 128, CU_TENSOR_MAP_SWIZZLE_64B)) {
        set_error("cuTensorMapEncodeTiled failed (Mp=%d N=%d K=%d)", Mp, N, plan->K);
        return false;
    }
    P->meta = plan->meta; P->perm = plan->perm;
    P->values = static_cast<const __half*>(values); P->out = out;
    P->Mp = Mp; P->N = N; P->K = plan->K; P->V = plan->V;
    P->k_steps = plan->k_steps; P->m_tiles = plan->m_tiles; P->n_tiles = (N + BN - 1) / BN; P->reserved = 0;
    return true;
}

}  // namespace fused
}  // namespace sspmm_b200

extern "C" {

int sspmm_plan_create(int m_vec, int vec_length, int K, const int* d_row_offsets, const int* d_column_indices,
                      void* stream, sspmm_plan** plan) {
    set_error("%s", "");
    if (!plan) { set_error("null output pointer"); return (int)cudaErrorInvalidValue; }
    *plan = nullptr;
    if (vec_length != 8 && vec_length != 16) {
        set_error("vec_length must be 8 or 16 (got %d)", vec_length);
        return (int)cudaErrorInvalidValue;
    }
    if (m_vec < 0 || K < 0 || (m_vec > 0 && !d_row_offsets)) {
        set_error("bad plan arguments (m_vec=%d K=%d)", m_vec, K);
        return (int)cudaErrorInvalidValue;
    }
    sspmm_plan* pl = new (std::nothrow) sspmm_plan();
    if (!pl) return (int)cudaErrorMemoryAllocation;
    pl->m_vec = m_vec; pl->V = vec_length; pl->K = K;
    cudaGetDevice(&pl->device);
    pl->row_offsets = d_row_offsets; pl->column_indices = d_column_indices;
    pl->m_tiles = (m_vec * vec_length + fused::kBM - 1) / fused::kBM;
    pl->k_steps = (K + fused::kBK - 1) / fused::kBK;
    pl->nvec = 0; pl->max_len = 0; pl->fused = false; pl->sorted = true; pl->meta = nullptr; pl->perm = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto failed = [&](cudaError_t e, const char* what) {
        if (pl->meta) cudaFree(pl->meta);
        if (pl->perm) cudaFree(pl->perm);
        delete pl;
        set_error("%s: %s", what, cudaGetErrorString(e));
        return (int)e;
    };
    if (m_vec == 0) { *plan = pl; return 0; }
    int nvec = 0;
    cudaError_t e = cudaMemcpyAsync(&nvec, d_row_offsets + m_vec, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return failed(e, "reading the vector count");
    pl->nvec = nvec;
    const int R = fused::kBM / vec_length;
    const size_t meta_bytes = (size_t)pl->m_tiles * pl->k_steps * R * sizeof(uint4);
    // The one-launch kernel does dense-tile work: it pays off when a fair share of the (vector row, column)
    // slots carry a vector.  Sparse structures (and empty ones) keep the gather kernels.
    const double density = (K > 0 && m_vec > 0) ? (double)nvec / ((double)m_vec * K) : 0.0;
    if (nvec <= 0 || K <= 0 || !d_column_indices || meta_bytes > fused::kMaxMetaBytes || density < 1.0 / 16 ||
        (size_t)pl->k_steps * 12 > 160 * 1024) {
        *plan = pl;
        return 0;
    }
    int* flags = nullptr;
    e = cudaMalloc(&pl->meta, meta_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&pl->perm, (size_t)nvec * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&flags, 4 * sizeof(int));
    if (e == cudaSuccess) e = cudaMemsetAsync(pl->meta, 0, meta_bytes, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(flags, 0, 4 * sizeof(int), st);
    if (e == cudaSuccess) {
        const size_t smem = (size_t)pl->k_steps * 12;
        auto kern = vec_length == 16 ? fused::plan_build_kernel<16> : fused::plan_build_kernel<8>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) {
            kern<<<m_vec, 256, smem, st>>>(m_vec, K, pl->k_steps, d_row_offsets, d_column_indices, pl->meta, pl->perm, flags);
            e = cudaGetLastError();
        }
    }
    int h[4] = {0, 0, 0, 0};
    if (e == cudaSuccess) e = cudaMemcpyAsync(h, flags, sizeof h, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (flags) cudaFree(flags);
    if (e != cudaSuccess) return failed(e, "building the plan");
    pl->fused = h[0] == 0;
    pl->sorted = h[1] == 0;
    pl->max_len = h[2];
    if (pl->sorted || !pl->fused) { cudaFree(pl->perm); pl->perm = nullptr; }
    if (!pl->fused) { cudaFree(pl->meta); pl->meta = nullptr; }
    *plan = pl;
    return 0;
}

int sspmm_plan_destroy(sspmm_plan* plan) {
    if (!plan) return 0;
    if (plan->meta) cudaFree(plan->meta);
    if (plan->perm) cudaFree(plan->perm);
    delete plan;
    return 0;
}

int sspmm_plan_info(const sspmm_plan* plan, int64_t* nvec, int* one_launch, int* ascending, int64_t* device_bytes) {
    if (!plan) return (int)cudaErrorInvalidValue;
    if (nvec) *nvec = plan->nvec;
    if (one_launch) *one_launch = plan->fused ? 1 : 0;
    if (ascending) *ascending = plan->sorted ? 1 : 0;
    if (device_bytes) {
        const int R = fused::kBM / plan->V;
        *device_bytes = (plan->meta ? (int64_t)plan->m_tiles * plan->k_steps * R * 16 : 0) + (plan->perm ? plan->nvec * 4 : 0);
    }
    return 0;
}

int sspmm_planned(const sspmm_plan* plan, const void* values_f16, const void* rhs_f16, void* out, int N, int out_is_f16,
                  void* stream) {
    set_error("%s", "");
    if (!plan) { set_error("null plan"); return (int)cudaErrorInvalidValue; }
    if (N < 0) { set_error("negative N"); return (int)cudaErrorInvalidValue; }
    if (plan->m_vec == 0 || N == 0) return 0;
    if (!plan->fused) {
        // sparse or irregular structure: the regular entry points (gather kernels) take it
        if (out_is_f16)
            return sspmm_f16_f16(plan->m_vec, plan->V, N, plan->K, nullptr, plan->row_offsets, plan->column_indices, values_f16,
                                 rhs_f16, out, stream);
        return sspmm_f16_f32(plan->m_vec, plan->V, N, plan->K, nullptr, plan->row_offsets, plan->column_indices, values_f16,
                             rhs_f16, static_cast<float*>(out), stream);
    }
    const int sms = current_device_sm_count();
    if (sms <= 0) return (int)cudaErrorNoDevice;
    // widest tile that still gives every SM a tile
    int BN = 256;
    while (BN > 64 && (int64_t)plan->m_tiles * ((N + BN - 1) / BN) < sms) BN >>= 1;
    fused::Params p;
    p.probs = nullptr; p.items = nullptr; p.dynamic = 0; p.queue = nullptr; p.partials = nullptr; p.counters = nullptr;
    if (!fused::fill_problem(&p.inline_prob, plan, values_f16, rhs_f16, out, N, out_is_f16 != 0, BN)) return (int)cudaErrorInvalidValue;
    const int64_t tiles = (int64_t)p.inline_prob.m_tiles * p.inline_prob.n_tiles;
    if (tiles > 0x7fffffffLL) { set_error("problem too large for 32-bit tile ids"); return (int)cudaErrorInvalidValue; }
    p.n_items = (int)tiles;
    const int rounds = (int)((tiles + sms - 1) / sms);
    const int grid = (int)((tiles + rounds - 1) / rounds);
    cudaError_t e = fused::launch(p, BN, out_is_f16 != 0, grid, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { set_error("SpMM launch: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

int sspmm_group_create(const sspmm_group_item* items, int count, int out_is_f16, sspmm_group** group) {
    set_error("%s", "");
    if (!group) { set_error("null output pointer"); return (int)cudaErrorInvalidValue; }
    *group = nullptr;
    if (!items || count <= 0) { set_error("a group needs at least one product"); return (int)cudaErrorInvalidValue; }
    const int sms = current_device_sm_count();
    if (sms <= 0) return (int)cudaErrorNoDevice;
    int dev = 0;
    cudaGetDevice(&dev);
    for (int i = 0; i < count; ++i) {
        const sspmm_plan* pl = items[i].plan;
        if (!pl || !pl->fused) { set_error("product %d: the plan does not support the one-launch kernel", i); return (int)cudaErrorInvalidValue; }
        if (pl->device != dev) { set_error("product %d: plan was built on device %d, current device is %d", i, pl->device, dev); return (int)cudaErrorInvalidValue; }
        if (items[i].N <= 0) { set_error("product %d: N must be positive", i); return (int)cudaErrorInvalidValue; }
    }
    // tile width: the widest that gives the grid at least two tiles per SM
    int BN = 256;
    for (;; BN >>= 1) {
        int64_t tiles = 0;
        for (int i = 0; i < count; ++i) tiles += (int64_t)items[i].plan->m_tiles * ((items[i].N + BN - 1) / BN);
        if (tiles >= 2 * sms || BN == 64) break;
    }
    std::vector<fused::Problem> probs((size_t)count);
    int64_t tiles = 0;
    double work = 0;                                   // K steps, with a fixed cost of two steps per tile
    for (int i = 0; i < count; ++i) {
        if (!fused::fill_problem(&probs[i], items[i].plan, items[i].values_f16, items[i].rhs_f16, items[i].out, items[i].N,
                                 out_is_f16 != 0, BN))
            return (int)cudaErrorInvalidValue;
        const int64_t t = (int64_t)probs[i].m_tiles * probs[i].n_tiles;
        tiles += t;
        work += (double)t * (probs[i].k_steps + 2);
    }
    if (tiles > (1 << 26)) { set_error("group too large (%lld tiles)", (long long)tiles); return (int)cudaErrorInvalidValue; }
    // Tiles longer than `cut` K steps are cut into parts so that no single item is a large share of an
    // SM's work; the parts' fp32 partial tiles are summed by whichever part finishes last.
    const double per_sm = work / sms;
    int cut = (int)(per_sm / 3.0);
    if (cut < 8) cut = 8;
    std::vector<fused::Item> list;
    list.reserve((size_t)tiles + 1024);
    int pslots = 0, cslots = 0;
    // longest items first (a greedy queue then balances itself); inside a product, tiles that share a panel of B
    // (same n tile) are neighbours, so CTAs running side by side reuse it from L2
    std::vector<int> order((size_t)count);
    for (int i = 0; i < count; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return probs[a].k_steps > probs[b].k_steps; });
    for (int oi = 0; oi < count; ++oi) {
        const int i = order[oi];
        const fused::Problem& P = probs[i];
        int parts = (tiles < 8 * (int64_t)sms && P.k_steps > cut) ? (P.k_steps + cut - 1) / cut : 1;
        if (parts > 16) parts = 16;
        const int sps = (P.k_steps + parts - 1) / parts;
        parts = (P.k_steps + sps - 1) / sps;
        for (int nt = 0; nt < P.n_tiles; ++nt)
            for (int mt = 0; mt < P.m_tiles; ++mt) {
                if (parts == 1) {
                    list.push_back(fused::Item{i, mt, nt, 0, P.k_steps, 0, 1 << 8, 0});
                } else {
                    for (int z = 0; z < parts; ++z)
                        list.push_back(fused::Item{i, mt, nt, z * sps, std::min(P.k_steps, (z + 1) * sps), pslots + z,
                                                   z | (parts << 8), cslots});
                    pslots += parts;
                    ++cslots;
                }
            }
    }
    std::stable_sort(list.begin(), list.end(),
                     [](const fused::Item& a, const fused::Item& b) { return (a.ks1 - a.ks0) > (b.ks1 - b.ks0); });
    sspmm_group* g = new (std::nothrow) sspmm_group();
    if (!g) return (int)cudaErrorMemoryAllocation;
    g->device = dev; g->count = count; g->BN = BN; g->out_f16 = out_is_f16 != 0;
    g->n_items = (int)list.size();
    g->grid = g->n_items < sms ? g->n_items : sms;
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t off_items = up(probs.size() * sizeof(fused::Problem));
    const size_t off_queue = off_items + up(list.size() * sizeof(fused::Item));
    const size_t off_counters = off_queue + 256;
    const size_t off_partials = off_counters + up((size_t)(cslots + 1) * sizeof(int));
    g->partial_bytes = (size_t)pslots * fused::kBM * BN * sizeof(float);
    const size_t total = off_partials + g->partial_bytes;
    cudaError_t e = cudaMalloc(&g->dev_block, total);
    if (e == cudaSuccess) e = cudaMemset(g->dev_block, 0, off_partials);
    uint8_t* base = static_cast<uint8_t*>(g->dev_block);
    if (e == cudaSuccess) e = cudaMemcpy(base, probs.data(), probs.size() * sizeof(fused::Problem), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(base + off_items, list.data(), list.size() * sizeof(fused::Item), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = fused::launch(g->params, BN, g->out_f16, 1, nullptr, true);
    if (e != cudaSuccess) {
        if (g->dev_block) cudaFree(g->dev_block);
        delete g;
        set_error("group set-up: %s", cudaGetErrorString(e));
        return (int)e;
    }
    g->params.probs = reinterpret_cast<const fused::Problem*>(base);
    g->params.items = reinterpret_cast<const fused::Item*>(base + off_items);
    g->params.n_items = g->n_items;
    g->params.dynamic = 1;
    g->params.queue = reinterpret_cast<int*>(base + off_queue);
    g->params.counters = reinterpret_cast<int*>(base + off_counters);
    g->params.partials = reinterpret_cast<float*>(base + off_partials);
    *group = g;
    return 0;
}

int sspmm_group_run(sspmm_group* group, void* stream) {
    set_error("%s", "");
    if (!group) { set_error("null group"); return (int)cudaErrorInvalidValue; }
    cudaError_t e = fused::launch(group->params, group->BN, group->out_f16, group->grid, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { set_error("group launch: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

int sspmm_group_info(const sspmm_group* group, int* tile_columns, int* work_items, int* ctas, int64_t* device_bytes) {
    if (!group) return (int)cudaErrorInvalidValue;
    if (tile_columns) *tile_columns = group->BN;
    if (work_items) *work_items = group->n_items;
    if (ctas) *ctas = group->grid;
    if (device_bytes) *device_bytes = (int64_t)group->partial_bytes;
    return 0;
}

int sspmm_group_destroy(sspmm_group* group) {
    if (!group) return 0;
    if (group->dev_block) cudaFree(group->dev_block);
    delete group;
    return 0;
}

}  // extern "C"
