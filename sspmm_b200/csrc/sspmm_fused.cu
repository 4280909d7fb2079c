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
// values[start + popc(mask below k)].  When some row's column list is not ascending the plan holds the positions
// themselves instead (4 bytes per slot), laid out so that a loader thread reads its own in one or two loads.
//
// Per CTA (persistent, one per SM), tile 128 rows x BN columns, K step 64:
//   warp 0        one thread: scheduler (takes work items -- static stride, or an atomic queue shared by the grid --
//                 and publishes them to the other warps through a shared-memory ring, well ahead of their use)
//                 and TMA producer of the B tile [64 k][BN n] (N-major, 128-byte swizzle)
//   warp 1        MMA issuer / TMEM owner: tcgen05.mma kind::f16, M = 128, N <= BN, K = 16, accumulators
//                 2 x BN TMEM columns
//   warps 4-7     epilogue: TMEM -> registers -> swizzled staging -> TMA store; or, for a tile whose K range
//                 was cut into parts, fp32 partial tile to scratch and the LAST part to arrive adds all parts
//                 in part order and writes C (no CTA ever waits for another)
//   warps 8-15    two loader groups that build the A tile [64 k][128 m] (M-major, 128-byte swizzle) of
//                 alternate stages from the value vectors: 16-byte loads into registers, requested well
//                 ahead of the 16-byte stores into the tile
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
// Warps: 0 scheduler + TMA producer (one thread), 1 MMA issuer, 2-3 idle, 4-7 epilogue, 8-15 two loader groups
// of four warps.  Sixteen warps are four per scheduler partition: 128 registers per thread.  (Measured on B200:
// a third loader group caps every thread at 96 registers and made the kernel slower, not faster.)
constexpr int kLoaderGroups = 2;
constexpr int kGroupThreads = 128;
constexpr int kEpilogueWarp0 = 4;
constexpr int kLoaderWarp0 = 8;
constexpr int kPublishAhead = 16;       // items the scheduler keeps published ahead of the B producer (< kRing)
// With A fetched by TMA nobody looks further ahead than the next item, and every item published early is an item
// claimed early: sixteen claimed items per CTA is the whole work list of a small group, dealt out before anybody
// knows who will be free.  (Measured on the conv step at the 8-GPU shard width: CTAs ended between 112 and 156 us.)
constexpr int kPublishAheadTma = 2;
constexpr int kThreads = kLoaderWarp0 * 32 + kLoaderGroups * kGroupThreads;
// Work items are published ahead of their use.  A loader thread looks four of its own stages ahead, which with
// one-step items is a dozen items past the stage it is about to store, while the epilogue may still hold the
// item two before that one; the scheduler keeps kPublishAhead items published beyond the one the B producer is
// loading, and the ring is deeper than both spans together, so a loader never waits for an item that could
// only be published after the loader itself has stored.
constexpr int kRing = 32;

// One product, as the kernel sees it.  Lives in kernel parameter space (single product) or in device
// memory (group); 64-byte aligned because of the tensor maps.
struct alignas(64) Problem {
    CUtensorMap tmap_a;        // expanded mode only: At {M', K, 1} fp16 (dense transposed copy of A), box 64 x 64, 128-byte swizzle
    CUtensorMap tmap_b;        // B  {N, K, 1}   fp16, box 64 x 64, 128-byte swizzle (or the chunked view, see `wide`)
    CUtensorMap tmap_b1;       // B {N, K, 1}, box 64 x 64 at any column that is a multiple of 8: the last, partly filled column tile fetches only its own chunks
    CUtensorMap tmap_c;        // C  {N, M', 1}  fp16/fp32, box (64 bytes) x 128 rows, 64-byte swizzle
    const uint4* meta;         // plan, ascending rows: [m_tile][k_step][row in tile] {mask lo, mask hi, start, 0}
    const int* posmap;         // plan, other structures: [m_tile][k_step][loader thread][slot] index of the vector or -1
    const __half* values;
    void* out;
    int Mp, N, K, V;
    int k_steps, m_tiles, n_tiles;
    int expand_blocks;         // expanded mode: blocks of the expansion of this product's A (see ExpandJob)
    int wide;                  // bit 0: tmap_b, bit 1: tmap_a are chunked views {64, rows, width / 64}: one TMA request brings all chunks of a tile
};
static_assert(sizeof(Problem) % 64 == 0, "Problem must keep the tensor maps 64-byte aligned in arrays");

// A unit of work: K steps [ks0, ks1) of one tile.  parts > 1: the tile's K range was cut; this is part
// `part`, its fp32 partial tile is slot pslot of the scratch (parts of a tile are consecutive slots) and
// cslot is the tile's arrival counter.
struct Item {
    int prob, m_tile, n_tile, ks0, ks1, pslot, pp /* part | parts << 8 */, cslot;
};

struct ExpandJob;

struct Params {
    const Problem* probs;      // device array, or null: inline_prob
    const Item* items;         // device array, or null: every tile of inline_prob once, whole K range
    int n_items;
    int dynamic;               // 1: items are taken from queue[0] (grid-wide atomic), else CTA b takes b, b + grid, ...
    int* queue;                // [0] next item, [1] CTAs that have left (the last one resets both, and expand_state)
    float* partials;
    int* counters;
    // expanded mode: the loader warps write the dense copies of A block by block (expand_state[0] = next block),
    // expand_state[2 + p] counts the finished blocks of product p, expand_state[1] the CTAs that have left
    const ExpandJob* jobs;
    int n_jobs, expand_blocks;
    int* expand_state;
    Problem inline_prob;
};

// Shared memory: a ring of stages, each an A tile (filled by the loader warps, or by TMA) and a B tile (filled
// by TMA); one tcgen05.commit per K step releases both.
template <int BN, int STAGES>
struct Layout {
    static constexpr int kAStages = STAGES, BSTAGES = STAGES;
    static constexpr int kAStage = kBM * kBK * 2;                // 16 KB: 2 chunks of [64 k][64 m]
    static constexpr int kBStage = BN * kBK * 2;                 // BN/64 chunks of [64 k][64 n]
    static constexpr int kChunk = kBK * 128;                     // 8 KB
    static constexpr int kAOff = 0;
    static constexpr int kBOff = kAStages * kAStage;
    static constexpr int kOutBuf = kBM * 64;                     // 128 rows x 64 bytes
    static constexpr int kOutOff = kBOff + BSTAGES * kBStage;
    static constexpr int kBarOff = kOutOff + 2 * kOutBuf;
    static constexpr int kNumBars = 3 * STAGES + 4 + 2 * kRing;
    static constexpr int kRingOff = kBarOff + kNumBars * 8;
    static constexpr int kTmemPtrOff = kRingOff + kRing * 32;
    static constexpr int kAbortOff = kTmemPtrOff + 8;
    static constexpr int kBcastOff = kAbortOff + 8;
    static constexpr int kBytes = kBcastOff + 8;
    static constexpr int kDynamic = kBytes + 1024;
    static constexpr uint32_t kTmemCols = 2 * BN;                // 128, 256 or 512
    static_assert(kDynamic <= 227 * 1024, "shared memory of one CTA");
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// orders earlier generic-proxy accesses (made visible to this thread) before later async-proxy (TMA) accesses, global memory included
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void fence_tensormap_acquire(const void* tmap) {
    // a tensor map that was written to global memory by a copy is read through its own proxy
    asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// The A tile of one stage (vector rows of tile m_tile, columns [64 ks, 64 ks + 64)) is built by the 128
// threads of a loader group: thread t owns vector row t / TPR and columns t % TPR + TPR * q.  Positions,
// loads and stores are separate steps so that a loader keeps several stages in flight (see the loader role).
template <int V>
struct ATile {
    static constexpr int R = kBM / V;             // vector rows per tile: 8 or 16
    static constexpr int TPR = kGroupThreads / R; // threads per vector row: 16 or 8
    static constexpr int SLOTS = kBK / TPR;       // columns per thread: 4 or 8
    static constexpr int H = V / 8;               // 16-byte pieces per vector: 2 or 1

    // positions of this thread's vectors in the value array (-1: no vector) from the row's column mask
    static __device__ __forceinline__ void positions(uint4 meta, int t, int (&jj)[8]) {
        const unsigned long long mask = (unsigned long long)meta.x | ((unsigned long long)meta.y << 32);
        const int start = (int)meta.z;
        const int kb = t % TPR;
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int kk = kb + TPR * q;
            const bool present = (mask >> kk) & 1ull;
            jj[q] = present ? start + __popcll(mask & ((1ull << kk) - 1ull)) : -1;
        }
    }
    static __device__ __forceinline__ void load(const __half* __restrict__ values, const int (&jj)[8], uint4 (&v)[8]) {
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const uint4* src = reinterpret_cast<const uint4*>(values + (int64_t)(jj[q] >= 0 ? jj[q] : 0) * V);
#pragma unroll
            for (int h = 0; h < H; ++h) v[q * H + h] = jj[q] >= 0 ? __ldg(src + h) : make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // a_s: the stage's A tile; rows of 128 bytes (64 m of one k), 16-byte pieces XOR-swizzled by k & 7
    static __device__ __forceinline__ void store(uint8_t* a_s, int t, const uint4 (&v)[8]) {
        const int r = t / TPR, kb = t % TPR;
        uint8_t* base = a_s + (r / (R / 2)) * (kBK * 128);
        const int piece0 = (r % (R / 2)) * H;
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int kk = kb + TPR * q;
#pragma unroll
            for (int h = 0; h < H; ++h)
                *reinterpret_cast<uint4*>(base + kk * 128 + (((piece0 + h) ^ (kk & 7)) << 4)) = v[q * H + h];
        }
    }
};

// One stage of the CTA's stage sequence, as a loader thread carries it while the stage is in flight.
struct StageDesc {
    const __half* values;
    int V;               // 8 or 16, + 32 when the metadata words are positions; 0 = no stage (end of the sequence)
};

// ---- expansion of the compressed operands of a group ---------------------------------------
// At[k][i*V .. i*V+V) = value vector of vector row i at column k, or zeros; every element of At is written, so
// nothing from an earlier run survives.  One thread per (vector row i, eight columns of a 64-column step): the
// plan's metadata tells it which of its columns carry a vector and where, so a thread is two dependent reads
// (metadata, value vectors) and its stores; consecutive threads have consecutive i, so the stores of a warp to a
// row of At are contiguous.  The work is cut into blocks of 256 threads, which the loader warps of the tensor-core
// kernel (idle when A tiles come by TMA) take from a counter while the other warps already multiply.
struct ExpandJob {
    const uint4* meta;             // the plan's column masks, or null
    const int* posmap;             // the plan's positions (when meta is null)
    const __half* values;
    __half* at;
    int m_vec, K, V, k_steps;
    int block_base;                // first block of this job (jobs are sorted by it)
    int prob;                      // the product whose copy this job writes
};

template <int V>
__device__ __forceinline__ void expand_slots(const ExpandJob& job, int id) {
    using A = ATile<V>;
    const int i = id % job.m_vec;
    const int g = (id / job.m_vec) & 7;
    const int ks = id / (job.m_vec * 8);
    if (ks >= job.k_steps) return;
    const int tile = i / A::R, r = i % A::R;
    const int64_t stage = (int64_t)tile * job.k_steps + ks;
    int jj[8];
    if (job.meta) {
        const uint4 m = __ldg(job.meta + stage * A::R + r);
        const unsigned long long mask = (unsigned long long)m.x | ((unsigned long long)m.y << 32);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int kk = g * 8 + q;
            jj[q] = ((mask >> kk) & 1ull) ? (int)m.z + __popcll(mask & ((1ull << kk) - 1ull)) : -1;
        }
    } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int kk = g * 8 + q;
            jj[q] = __ldg(job.posmap + (stage * kGroupThreads + r * A::TPR + kk % A::TPR) * A::SLOTS + kk / A::TPR);
        }
    }
    uint4 v[8][V / 8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const uint4* src = reinterpret_cast<const uint4*>(job.values + (int64_t)(jj[q] >= 0 ? jj[q] : 0) * V);
#pragma unroll
        for (int h = 0; h < V / 8; ++h) v[q][h] = jj[q] >= 0 ? __ldg(src + h) : make_uint4(0u, 0u, 0u, 0u);
    }
    const int64_t mp = (int64_t)job.m_vec * V;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
        const int k = ks * kBK + g * 8 + q;
        if (k < job.K) {
            uint4* dst = reinterpret_cast<uint4*>(job.at + (int64_t)k * mp + (int64_t)i * V);
#pragma unroll
            for (int h = 0; h < V / 8; ++h) dst[h] = v[q][h];
        }
    }
}

// ATMA = true: the A tiles come by TMA from a dense transposed copy of A (written by expand_group_kernel just
// before; the loader warps then have nothing to do).  ATMA = false: the loader warps build them from the
// compressed operand.
template <int BN, int STAGES, typename OutT, bool ATMA>
__global__ void __launch_bounds__(kThreads, 1)
sspmm_fused_kernel(const __grid_constant__ Params gp) {
    using L = Layout<BN, STAGES>;
    constexpr int kAStages = STAGES, BSTAGES = STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_a_full = sbase + L::kBarOff;          // A tile of the stage written (loader warps; unused with A by TMA)
    const uint32_t bar_b_full = bar_a_full + STAGES * 8;      // B tile (and, with A by TMA, the A tile) of the stage has landed
    const uint32_t bar_empty = bar_b_full + STAGES * 8;       // the MMAs that read the stage have completed
    const uint32_t bar_a_empty = bar_empty, bar_b_empty = bar_empty;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    const uint32_t bar_item_full = bar_acc_empty + 2 * 8;
    const uint32_t bar_item_empty = bar_item_full + kRing * 8;
    volatile int* ring = reinterpret_cast<volatile int*>(smem + L::kRingOff);
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);
    volatile int* bcast = reinterpret_cast<volatile int*>(smem + L::kBcastOff);
    volatile int* bcast2 = bcast + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_a_full + 8 * s, kGroupThreads / 32);     // the warps of the loader group that owns the stage
            mbar_init(bar_b_full + 8 * s, 1);                      // producer's expect_tx
            mbar_init(bar_empty + 8 * s, 1);                       // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);
        }
        for (int r = 0; r < kRing; ++r) {
            mbar_init(bar_item_full + 8 * r, 1);
            mbar_init(bar_item_empty + 8 * r, 6 + (ATMA ? 0 : kLoaderGroups * kGroupThreads / 32));   // producer, MMA, epilogue and loader warps
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), L::kTmemCols);
        tmem_relinquish();
    }
    // The number of the first expansion block is asked for now: the answer is on its way while the barriers are set up.
    int first_expand_block = 0;
    if (ATMA && gp.jobs && threadIdx.x == kLoaderWarp0 * 32) first_expand_block = atomicAdd(gp.expand_state, 1);
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

    if (warp < 4) {
      if (warp == 0) {
        // ------------------------------------------------------------------ scheduler + TMA producer of B
        if (lane == 0) {
            // scheduler state: items 0 .. n_pub-1 of this CTA are in the ring; raw_next is the answer of the
            // queue to the request made when the previous item was published (used only at the next publish,
            // so the thread does not wait for it)
            uint32_t n_pub = 0;
            bool sched_done = false;
            int idx = blockIdx.x, raw_next = 0;
            // publishes items until `upto` are in the ring (or the list ends); must = false: gives up when the ring is full
            auto publish = [&](uint32_t upto, bool must) -> bool {
                while (!sched_done && n_pub < upto) {
                    const uint32_t slot = n_pub % kRing, ph = (n_pub / kRing) & 1u;
                    if (must) {
                        if (!mbar_wait(bar_item_empty + 8 * slot, ph ^ 1u, abort_flag, kStatusWaitFused)) return false;
                    } else if (!mbar_test_wait(bar_item_empty + 8 * slot, ph ^ 1u)) {
                        return true;
                    }
                    if (n_pub > 0) idx = gp.dynamic ? (int)gridDim.x + raw_next : idx + (int)gridDim.x;
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
                    ++n_pub;
                    if (it.prob < 0) sched_done = true;
                    else if (gp.dynamic) raw_next = atomicAdd(gp.queue, 1);
                }
                return true;
            };
            uint32_t stage = 0, phase = 0;
            int last_prob = -1;
            bool ok = true;
            Item it;
            for (uint32_t n = 0; ok; ++n) {
                if (!publish(n + 1, true)) break;                // the item this thread is about to load
                // and, ring permitting, the ones further ahead: at once when the loader warps look ahead to them;
                // with A by TMA only after this item's first loads are on their way (fetching a work item is a
                // round trip to L2 that nothing else of this thread waits for)
                publish(n + 1 + (ATMA ? kPublishAheadTma : kPublishAhead), false);
                if (!take_item(n, it, false)) break;
                const Problem* P = problem_of(it.prob);
                if (gp.probs && it.prob != last_prob) {
                    fence_tensormap_acquire(&P->tmap_b);
                    fence_tensormap_acquire(&P->tmap_b1);
                    if constexpr (ATMA) {
                        fence_tensormap_acquire(&P->tmap_a);
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
                        fence_proxy_async_all();      // those were ordinary stores; TMA reads through the async proxy
                    }
                    last_prob = it.prob;
                }
                const int n0 = it.n_tile * BN;
                const int wide = P->wide;
                const int chunks = min(BN / 64, (P->N - n0 + 63) >> 6);
                for (int ks = it.ks0; ks < it.ks1; ++ks) {
                    if (!mbar_wait(bar_b_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitFused)) { ok = false; break; }
                    const uint32_t full = bar_b_full + 8 * stage;
                    mbar_arrive_expect_tx(full, (uint32_t)chunks * L::kChunk + (ATMA ? L::kAStage : 0));
                    if constexpr (ATMA) {
                        const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                        if (wide & 2) {
                            tma_load_3d(a_s, &P->tmap_a, 0, ks * kBK, it.m_tile * (kBM / 64), full);
                        } else {
                            for (int c = 0; c < kBM / 64; ++c)
                                tma_load_3d(a_s + c * L::kChunk, &P->tmap_a, it.m_tile * kBM + 64 * c, ks * kBK, 0, full);
                        }
                    }
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
                    if ((wide & 1) && chunks == BN / 64) {
                        tma_load_3d(b_s, &P->tmap_b, 0, ks * kBK, n0 >> 6, full);
                    } else if (wide & 1) {
                        for (int c = 0; c < chunks; ++c) tma_load_3d(b_s + c * L::kChunk, &P->tmap_b1, n0 + 64 * c, ks * kBK, 0, full);
                    } else {
                        for (int c = 0; c < chunks; ++c) tma_load_3d(b_s + c * L::kChunk, &P->tmap_b, n0 + 64 * c, ks * kBK, 0, full);
                    }
                    if (++stage == BSTAGES) { stage = 0; phase ^= 1u; }
                    if ((ks & 7) == 7)
                        publish(n + 1 + (ATMA ? kPublishAheadTma : kPublishAhead), false);
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
                if (!__all_sync(0xffffffffu, (ATMA || mbar_wait(bar_a_full + 8 * stage, phase, abort_flag, kStatusWaitFused)) &&
                                            mbar_wait(bar_b_full + 8 * stage, phase, abort_flag, kStatusWaitFused))) { ok = false; break; }
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
      }
    } else if (warp >= kLoaderWarp0) {
      if constexpr (ATMA) {
        // ------------------------------------------------------------------ expansion (A tiles come by TMA)
        // The 256 loader threads act as one block of the expansion: they take block numbers from a counter, write
        // their part of a dense copy of A and count the block as done for its product.  They wait for nothing but
        // each other, so the copies are always completed, whichever CTAs are resident.
        if (gp.jobs) {
            const int t = threadIdx.x - kLoaderWarp0 * 32;
            constexpr int kExpandThreads = kLoaderGroups * kGroupThreads;
            // The request for the next block number is made while the current block is written (its answer is
            // only needed in the next round), and the job of a block is found by walking on from the last one: a
            // round is then one chain of metadata -> value vectors -> stores, not three.
            int claimed = first_expand_block, job_at = 0;
            for (;;) {
                if (t == 0) *bcast2 = claimed;
                named_barrier_sync(3, kExpandThreads);
                const int vb = *bcast2;
                named_barrier_sync(3, kExpandThreads);            // everyone has read the number before the next one is written
                if (vb >= gp.expand_blocks) break;
                if (t == 0) claimed = atomicAdd(gp.expand_state, 1);
                while (job_at + 1 < gp.n_jobs && __ldg(&gp.jobs[job_at + 1].block_base) <= vb) ++job_at;
                const ExpandJob job = gp.jobs[job_at];
                const int id = (vb - job.block_base) * kExpandThreads + t;
                if (job.V == 16) expand_slots<16>(job, id); else expand_slots<8>(job, id);
                __threadfence();
                named_barrier_sync(3, kExpandThreads);
                if (t == 0) atomicAdd(gp.expand_state + 2 + job.prob, 1);
            }
        }
      } else {
        // ------------------------------------------------------------------ A loaders
        // The groups take the stages of the CTA's stage sequence in turn.  A stage goes through three steps,
        // each of which waits for memory: metadata, value vectors, shared-memory slot.  Under load a request
        // to L2 is under way for well over a thousand cycles, longer than the group's turn comes round, so a
        // thread keeps four of its stages in flight (two with metadata requested, two with value vectors
        // requested) and runs ahead across item boundaries: the latencies overlap instead of adding up.
        const int group = (warp - kLoaderWarp0) >> 2;
        const int t = threadIdx.x - (kLoaderWarp0 * 32 + kGroupThreads * group);
        uint32_t n_item = 0, it_count = 0;
        uint32_t c_finish = (uint32_t)group;    // this group's stages are group, group + kLoaderGroups, ... in order
        int s_next = 0, steps = 0, item_v = 0;
        bool have_item = false, done = false;
        Item it;
        const __half* item_values = nullptr;
        const uint4* item_meta = nullptr;       // this thread's metadata word of the item's first stage
        int meta_stride = 0;                    // uint4 words between consecutive K steps
        // next stage of this group; meta_at = where its metadata for this thread lives
        auto next_stage = [&](const uint4*& meta_at) -> StageDesc {
            StageDesc d;
            d.values = nullptr; d.V = 0;
            for (;;) {
                if (done) return d;
                if (!have_item) {
                    if (!take_item(n_item, it, true)) { done = true; return d; }
                    ++n_item;
                    have_item = true;
                    const Problem* P = problem_of(it.prob);
                    steps = it.ks1 - it.ks0;
                    s_next = (group + kLoaderGroups - (int)(it_count % kLoaderGroups)) % kLoaderGroups;
                    const int V = P->V;
                    item_values = P->values;
                    if (P->posmap) {
                        // kGroupThreads threads x (4 or 8) ints per stage: one or two 16-byte words per thread
                        item_v = V + 32;
                        meta_stride = kGroupThreads * (V == 16 ? 1 : 2);
                        item_meta = reinterpret_cast<const uint4*>(P->posmap) +
                                    ((int64_t)it.m_tile * P->k_steps + it.ks0) * meta_stride + t * (V == 16 ? 1 : 2);
                    } else {
                        item_v = V;
                        meta_stride = kBM / V;
                        item_meta = P->meta + ((int64_t)it.m_tile * P->k_steps + it.ks0) * meta_stride + t / (kGroupThreads / meta_stride);
                    }
                }
                if (s_next < steps) {
                    d.values = item_values; d.V = item_v;
                    meta_at = item_meta + (int64_t)s_next * meta_stride;
                    s_next += kLoaderGroups;
                    return d;
                }
                it_count += (uint32_t)steps;
                have_item = false;
            }
        };
        // metadata words of a stage: one (masks; positions at V = 16) or two (positions at V = 8)
        auto load_meta = [&](const StageDesc& d, const uint4* meta_at, uint4 (&m)[2]) {
            m[0] = __ldg(meta_at);
            if (d.V == 32 + 8) m[1] = __ldg(meta_at + 1);
        };
        // requests the value vectors of a stage whose metadata has arrived
        auto load = [&](const StageDesc& d, const uint4 (&m)[2], uint4 (&v)[8]) {
            int jj[8];
            if (d.V == 16) { ATile<16>::positions(m[0], t, jj); ATile<16>::load(d.values, jj, v); }
            else if (d.V == 8) { ATile<8>::positions(m[0], t, jj); ATile<8>::load(d.values, jj, v); }
            else if (d.V == 32 + 16) {
                jj[0] = (int)m[0].x; jj[1] = (int)m[0].y; jj[2] = (int)m[0].z; jj[3] = (int)m[0].w;
                ATile<16>::load(d.values, jj, v);
            } else {
                jj[0] = (int)m[0].x; jj[1] = (int)m[0].y; jj[2] = (int)m[0].z; jj[3] = (int)m[0].w;
                jj[4] = (int)m[1].x; jj[5] = (int)m[1].y; jj[6] = (int)m[1].z; jj[7] = (int)m[1].w;
                ATile<8>::load(d.values, jj, v);
            }
        };
        // the group's next stage in order: waits for its slot, stores the tile, hands it to the MMA
        auto finish = [&](const StageDesc& d, const uint4 (&v)[8]) -> bool {
            const uint32_t stage = c_finish % kAStages, phase = (c_finish / kAStages) & 1u;
            c_finish += kLoaderGroups;
            if (!__all_sync(0xffffffffu, mbar_wait(bar_a_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitFused))) return false;
            uint8_t* a_s = smem + L::kAOff + stage * L::kAStage;
            if ((d.V & 31) == 16) ATile<16>::store(a_s, t, v); else ATile<8>::store(a_s, t, v);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_a_full + 8 * stage);
            return true;
        };
        uint4 v0[8], v1[8], m0[2], m1[2];
        const uint4* meta_at = nullptr;
        // invariant at the top of the loop: v0 / v1 = value vectors of d0 / d1 (requested), m0 / m1 = metadata of d2 / d3 (requested)
        StageDesc d0 = next_stage(meta_at);
        if (d0.V) { load_meta(d0, meta_at, m0); load(d0, m0, v0); }
        StageDesc d1 = next_stage(meta_at);
        if (d1.V) { load_meta(d1, meta_at, m1); load(d1, m1, v1); }
        StageDesc d2 = next_stage(meta_at);
        if (d2.V) load_meta(d2, meta_at, m0);
        StageDesc d3 = next_stage(meta_at);
        if (d3.V) load_meta(d3, meta_at, m1);
        while (d0.V) {
            if (!finish(d0, v0)) break;
            if (d2.V) load(d2, m0, v0);
            StageDesc d4 = next_stage(meta_at);
            if (d4.V) load_meta(d4, meta_at, m0);
            if (!d1.V) break;
            if (!finish(d1, v1)) break;
            if (d3.V) load(d3, m1, v1);
            StageDesc d5 = next_stage(meta_at);
            if (d5.V) load_meta(d5, meta_at, m1);
            d0 = d2; d1 = d3; d2 = d4; d3 = d5;
        }
      }
    } else {
        // ------------------------------------------------------------------ epilogue
        // Each thread owns one row of the 128-row tile and handles 32 accumulator columns at a time.
        constexpr int kColsPerStore = 64 / (int)sizeof(OutT);          // 32 (fp16) or 16 (fp32)
        constexpr int kStoresPerLoad = 32 / kColsPerStore;
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const bool issuer = (threadIdx.x == kEpilogueWarp0 * 32);
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
    // The CTA that leaves last puts the queue and the expansion counters back to zero for the next run.
    if (threadIdx.x == 0 && gp.dynamic) {
        __threadfence();
        if (atomicAdd(gp.queue + 1, 1) == (int)gridDim.x - 1) {
            gp.queue[0] = 0;
            gp.queue[1] = 0;
            if (gp.expand_state)
                for (int i = 0; i < 2 + gp.n_jobs; ++i) gp.expand_state[i] = 0;
            __threadfence();
        }
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

// Positions for structures with rows that are not ascending: posmap[((tile * k_steps + ks) * 128 + t) * SLOTS + q] =
// index of the vector that loader thread t puts into its slot q of that stage, or -1.
template <int V>
__global__ void __launch_bounds__(256)
plan_posmap_kernel(long long slots, const uint4* __restrict__ meta, const int* __restrict__ perm, int* __restrict__ posmap) {
    using A = ATile<V>;
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= slots) return;
    const int q = (int)(idx % A::SLOTS);
    const int t = (int)((idx / A::SLOTS) % kGroupThreads);
    const long long stage = idx / (A::SLOTS * kGroupThreads);
    const int kk = t % A::TPR + A::TPR * q;
    const uint4 m = meta[stage * A::R + t / A::TPR];
    const unsigned long long mask = (unsigned long long)m.x | ((unsigned long long)m.y << 32);
    posmap[idx] = ((mask >> kk) & 1ull) ? perm[(int)m.z + __popcll(mask & ((1ull << kk) - 1ull))] : -1;
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

// Chunked view of a row-major [rows][width] fp16 matrix (width % 64 == 0): {64, rows, width / 64}; a box
// {64, 64, chunks} lands as `chunks` consecutive [64 rows][128 B] swizzled blocks, the layout the MMA descriptors expect.
bool encode_chunked(EncodeFn enc, CUtensorMap* m, const void* base, uint64_t width, uint64_t rows, uint32_t chunks) {
    const cuuint64_t gdim[3] = {64, rows, width / 64};
    const cuuint64_t gstride[2] = {width * 2, 128};
    const cuuint32_t box[3] = {64, 64, chunks};
    const cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), gdim, gstride, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
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
    uint4* meta;               // owned: column masks (every row ascending)
    int* posmap;               // owned: positions (some row not ascending); exactly one of the two is set when fused
};

struct sspmm_group {
    int device, count, BN;
    bool out_f16;
    bool pair;                 // CTA-pair kernel (tiles of 256 x 256); always expanded
    bool expanded;             // A tiles by TMA from dense transposed copies that the kernel's loader warps write at every run
    int n_items, grid;
    void* dev_block;           // one allocation: problems | items | queue | counters | expansion jobs | partials | copies of A
    fused::Params params;
    int expand_units;
    size_t scratch_bytes;      // partial tiles + copies of A
};

namespace sspmm_b200 {
namespace fused {

constexpr size_t kMaxMetaBytes = (size_t)256 << 20;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int BN, int STAGES, typename OutT, bool ATMA>
cudaError_t launch_typed(const Params& p, int grid, cudaStream_t st, bool setup_only) {
    using L = Layout<BN, STAGES>;
    auto kern = sspmm_fused_kernel<BN, STAGES, OutT, ATMA>;
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

template <typename OutT, bool ATMA>
cudaError_t launch_bn(const Params& p, int BN, int grid, cudaStream_t st, bool setup_only) {
    if (BN == 256) return launch_typed<256, 4, OutT, ATMA>(p, grid, st, setup_only);
    if (BN == 128) return launch_typed<128, 6, OutT, ATMA>(p, grid, st, setup_only);
    return launch_typed<64, 8, OutT, ATMA>(p, grid, st, setup_only);
}

// CTA-pair kernel (sspmm_fused_pair.cu)
cudaError_t launch_pair(const Params& p, bool out_f16, int pairs, cudaStream_t st, bool setup_only);
constexpr bool kAutoPairs = false;

cudaError_t launch(const Params& p, int BN, bool out_f16, bool a_tma, int grid, cudaStream_t st, bool setup_only = false) {
    if (a_tma) return out_f16 ? launch_bn<__half, true>(p, BN, grid, st, setup_only) : launch_bn<float, true>(p, BN, grid, st, setup_only);
    return out_f16 ? launch_bn<__half, false>(p, BN, grid, st, setup_only) : launch_bn<float, false>(p, BN, grid, st, setup_only);
}

// Fills everything of a Problem but nothing that lives on the device.  Returns false with the error set.
bool fill_problem(Problem* P, const sspmm_plan* plan, const void* values, const void* rhs, void* out, int N, bool out_f16,
                  int BN, bool pair = false) {
    EncodeFn enc = encode_fn();
    if (!enc) { set_error("cuTensorMapEncodeTiled is not available from the CUDA driver"); return false; }
    if (!plan || !plan->fused) { set_error("the plan does not support the one-launch kernel"); return false; }
    if (N <= 0 || N % 8 != 0 || !values || !rhs || !out || !aligned16(values) || !aligned16(rhs) || !aligned16(out)) {
        set_error("the planned SpMM needs N > 0, N %% 8 == 0 and 16-byte aligned values, rhs and output");
        return false;
    }
    const int Mp = plan->m_vec * plan->V;
    const size_t oes = out_f16 ? 2 : 4;
    // a CTA pair fetches the B tile in two halves, one per CTA
    P->wide = (N % 64 == 0 && encode_chunked(enc, &P->tmap_b, rhs, (uint64_t)N, (uint64_t)plan->K, (uint32_t)(pair ? BN / 128 : BN / 64))) ? 1 : 0;
    if (!encode_map(enc, &P->tmap_b1, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, rhs, (uint64_t)N, (uint64_t)plan->K, 64, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B) ||
        (!P->wide && !encode_map(enc, &P->tmap_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, rhs, (uint64_t)N, (uint64_t)plan->K, 64, 64,
                                 CU_TENSOR_MAP_SWIZZLE_128B)) ||
        !encode_map(enc, &P->tmap_c, out_f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, oes, out,
                    (uint64_t)N, (uint64_t)Mp, (uint32_t)(64 / oes), 128, CU_TENSOR_MAP_SWIZZLE_64B)) {
        set_error("cuTensorMapEncodeTiled failed (Mp=%d N=%d K=%d)", Mp, N, plan->K);
        return false;
    }
    P->meta = plan->meta; P->posmap = plan->posmap;
    P->values = static_cast<const __half*>(values); P->out = out;
    P->Mp = Mp; P->N = N; P->K = plan->K; P->V = plan->V;
    P->k_steps = plan->k_steps; P->m_tiles = pair ? (plan->m_tiles + 1) / 2 : plan->m_tiles; P->n_tiles = (N + BN - 1) / BN; P->expand_blocks = 0;
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
    pl->nvec = 0; pl->max_len = 0; pl->fused = false; pl->sorted = true; pl->meta = nullptr; pl->posmap = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int* perm = nullptr;       // position in column order -> index of the vector; only needed to build posmap
    auto failed = [&](cudaError_t e, const char* what) {
        if (pl->meta) cudaFree(pl->meta);
        if (pl->posmap) cudaFree(pl->posmap);
        if (perm) cudaFree(perm);
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
    if (e == cudaSuccess) e = cudaMalloc(&perm, (size_t)nvec * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&flags, 4 * sizeof(int));
    if (e == cudaSuccess) e = cudaMemsetAsync(pl->meta, 0, meta_bytes, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(flags, 0, 4 * sizeof(int), st);
    if (e == cudaSuccess) {
        const size_t smem = (size_t)pl->k_steps * 12;
        auto kern = vec_length == 16 ? fused::plan_build_kernel<16> : fused::plan_build_kernel<8>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) {
            kern<<<m_vec, 256, smem, st>>>(m_vec, K, pl->k_steps, d_row_offsets, d_column_indices, pl->meta, perm, flags);
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
    if (pl->fused && !pl->sorted) {
        // some row is not ascending: replace the masks by explicit positions
        const int slots_per_thread = vec_length == 16 ? 4 : 8;
        const long long slots = (long long)pl->m_tiles * pl->k_steps * fused::kGroupThreads * slots_per_thread;
        if ((size_t)slots * sizeof(int) > fused::kMaxMetaBytes) {
            pl->fused = false;
        } else {
            e = cudaMalloc(&pl->posmap, (size_t)slots * sizeof(int));
            if (e == cudaSuccess) {
                const unsigned blocks = (unsigned)((slots + 255) / 256);
                if (vec_length == 16) fused::plan_posmap_kernel<16><<<blocks, 256, 0, st>>>(slots, pl->meta, perm, pl->posmap);
                else fused::plan_posmap_kernel<8><<<blocks, 256, 0, st>>>(slots, pl->meta, perm, pl->posmap);
                e = cudaGetLastError();
            }
            if (e == cudaSuccess) e = cudaStreamSynchronize(st);
            if (e != cudaSuccess) return failed(e, "building the plan's position table");
        }
    }
    cudaFree(perm);
    perm = nullptr;
    if (!pl->fused || pl->posmap) { cudaFree(pl->meta); pl->meta = nullptr; }
    *plan = pl;
    return 0;
}

int sspmm_plan_destroy(sspmm_plan* plan) {
    if (!plan) return 0;
    if (plan->meta) cudaFree(plan->meta);
    if (plan->posmap) cudaFree(plan->posmap);
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
        *device_bytes = plan->meta ? (int64_t)plan->m_tiles * plan->k_steps * R * 16
                                   : (plan->posmap ? (int64_t)plan->m_tiles * plan->k_steps * fused::kGroupThreads * (plan->V == 16 ? 4 : 8) * 4 : 0);
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
    p.jobs = nullptr; p.n_jobs = 0; p.expand_blocks = 0; p.expand_state = nullptr;
    if (!fused::fill_problem(&p.inline_prob, plan, values_f16, rhs_f16, out, N, out_is_f16 != 0, BN)) return (int)cudaErrorInvalidValue;
    const int64_t tiles = (int64_t)p.inline_prob.m_tiles * p.inline_prob.n_tiles;
    if (tiles > 0x7fffffffLL) { set_error("problem too large for 32-bit tile ids"); return (int)cudaErrorInvalidValue; }
    p.n_items = (int)tiles;
    const int rounds = (int)((tiles + sms - 1) / sms);
    const int grid = (int)((tiles + rounds - 1) / rounds);
    cudaError_t e = fused::launch(p, BN, out_is_f16 != 0, false, grid, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { set_error("SpMM launch: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

int sspmm_group_create(const sspmm_group_item* items, int count, int out_is_f16, int mode, sspmm_group** group) {
    set_error("%s", "");
    if (!group) { set_error("null output pointer"); return (int)cudaErrorInvalidValue; }
    *group = nullptr;
    if (!items || count <= 0) { set_error("a group needs at least one product"); return (int)cudaErrorInvalidValue; }
    if (mode < 0 || mode > 3) { set_error("group mode must be 0 (automatic), 1 (compressed), 2 (expanded) or 3 (expanded, CTA pairs)"); return (int)cudaErrorInvalidValue; }
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
    // CTA pairs (tiles of 256 x 256, see sspmm_fused_pair.cu) when asked for, or when the group is large enough for
    // 256-column tiles and for the expanded mode
    bool pair = mode == 3;
    if (mode == 0 && BN == 256 && fused::kAutoPairs) {
        double est = 0;
        for (int i = 0; i < count; ++i)
            est += (double)items[i].plan->m_tiles * ((items[i].N + 255) / 256) * (items[i].plan->k_steps + 2);
        pair = est / sms >= 48.0;
    }
    if (pair) BN = 256;
    const int units = pair ? sms / 2 : sms;            // what holds one tile: an SM, or a pair of SMs
    std::vector<fused::Problem> probs((size_t)count);
    int64_t tiles = 0;
    double work = 0;                                   // K steps, with a fixed cost of two steps per tile
    for (int i = 0; i < count; ++i) {
        if (!fused::fill_problem(&probs[i], items[i].plan, items[i].values_f16, items[i].rhs_f16, items[i].out, items[i].N,
                                 out_is_f16 != 0, BN, pair))
            return (int)cudaErrorInvalidValue;
        const int64_t t = (int64_t)probs[i].m_tiles * probs[i].n_tiles;
        tiles += t;
        work += (double)t * (probs[i].k_steps + 2);
    }
    if (tiles > (1 << 26)) { set_error("group too large (%lld tiles)", (long long)tiles); return (int)cudaErrorInvalidValue; }
    // Tiles longer than `cut` K steps are cut into parts so that no single item is a large share of an
    // SM's work; the parts' fp32 partial tiles are summed by whichever part finishes last.
    const double per_sm = work / units;
    int cut = (int)(per_sm / 3.0);
    if (cut < 8) cut = 8;
    std::vector<fused::Item> list;
    list.reserve((size_t)tiles + 1024);
    int pslots = 0, cslots = 0;
    // longest items first (a greedy queue then balances itself).  Products that multiply the same dense operand
    // (same pointer, width and depth) form a bundle whose tiles are emitted panel by panel: all tiles of all
    // bundle members that read one column panel of B are neighbours in the list, so CTAs running side by side
    // fetch the panel from HBM once and from L2 afterwards.
    std::vector<int> order((size_t)count);
    for (int i = 0; i < count; ++i) order[i] = i;
    // Among products of equal depth those with the longer vectors go first: their dense copies take half as many
    // expansion blocks per tile, so the CTAs that start on them wait less for the first copies.
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
        if (probs[a].k_steps != probs[b].k_steps) return probs[a].k_steps > probs[b].k_steps;
        return items[a].plan->V > items[b].plan->V;
    });
    std::vector<char> placed((size_t)count, 0);
    for (int oi = 0; oi < count; ++oi) {
        if (placed[(size_t)order[oi]]) continue;
        const int lead = order[oi];
        std::vector<int> bundle;
        for (int oj = oi; oj < count; ++oj) {
            const int j = order[oj];
            if (placed[(size_t)j]) continue;
            if (items[j].rhs_f16 == items[lead].rhs_f16 && items[j].N == items[lead].N && probs[j].K == probs[lead].K &&
                probs[j].k_steps == probs[lead].k_steps && probs[j].n_tiles == probs[lead].n_tiles) {
                bundle.push_back(j);
                placed[(size_t)j] = 1;
            }
        }
        const fused::Problem& L = probs[lead];
        int parts = (tiles < 8 * (int64_t)units && L.k_steps > cut) ? (L.k_steps + cut - 1) / cut : 1;
        if (parts > 16) parts = 16;
        if (count == 1) {
            // One product: the number of parts that gives the shortest critical path.  An item costs its K steps
            // plus two for the hand-over, and a cut tile pays for its fp32 partial tiles (written once, read once:
            // measured about 17 K steps' worth per part for a 128 x 256 tile when every SM does it at once).
            const int64_t t = (int64_t)L.m_tiles * L.n_tiles;
            const int64_t extra = 17 * BN / 256 + 1;
            int64_t best = -1;
            for (int q = 1; q <= 16 && q <= L.k_steps; ++q) {
                const int64_t rounds = (t * q + units - 1) / units;
                const int64_t cost = rounds * ((L.k_steps + q - 1) / q + 2 + (q > 1 ? extra : 0));
                if (best < 0 || cost < best) { best = cost; parts = q; }
            }
        }
        const int sps = (L.k_steps + parts - 1) / parts;
        parts = (L.k_steps + sps - 1) / sps;
        for (int nt = 0; nt < L.n_tiles; ++nt)
            for (int i : bundle) {
                const fused::Problem& P = probs[i];
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
    }
    std::stable_sort(list.begin(), list.end(),
                     [](const fused::Item& a, const fused::Item& b) { return (a.ks1 - a.ks0) > (b.ks1 - b.ks0); });
    sspmm_group* g = new (std::nothrow) sspmm_group();
    if (!g) return (int)cudaErrorMemoryAllocation;
    g->device = dev; g->count = count; g->BN = BN; g->out_f16 = out_is_f16 != 0;
    g->n_items = (int)list.size();
    g->grid = g->n_items < units ? g->n_items : units;  // CTAs, or CTA pairs
    g->pair = pair;
    // Measured on B200: with the A tiles built by the loader warps a K step takes about 1150 cycles, with A tiles
    // fetched by TMA from a dense copy about 700-750; writing the copies costs one more launch and a few tens of
    // microseconds.  So groups with much work per SM expand, small ones (latency matters) do not.
    g->expanded = pair || mode == 2 || (mode == 0 && per_sm >= 48.0);
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    std::vector<fused::ExpandJob> jobs;
    std::vector<size_t> at_off((size_t)count, 0);
    size_t at_bytes = 0;
    g->expand_units = 0;
    if (g->expanded) {
        jobs.resize((size_t)count);
        for (int i = 0; i < count; ++i) {
            const sspmm_plan* pl = items[i].plan;
            at_off[i] = at_bytes;
            at_bytes += up((size_t)pl->K * pl->m_vec * pl->V * sizeof(__half));
            fused::ExpandJob& j = jobs[i];
            j.meta = pl->meta; j.posmap = pl->posmap;
            j.values = static_cast<const __half*>(items[i].values_f16); j.at = nullptr;
            j.m_vec = pl->m_vec; j.K = pl->K; j.V = pl->V; j.k_steps = pl->k_steps;
            j.prob = i;
            probs[i].expand_blocks = (int)(((int64_t)pl->m_vec * 8 * pl->k_steps + 255) / 256);
        }
    }
    const size_t off_items = up(probs.size() * sizeof(fused::Problem));
    const size_t off_queue = off_items + up(list.size() * sizeof(fused::Item));
    const size_t off_counters = off_queue + 256;
    const size_t off_state = off_counters + up((size_t)(2 * cslots + 2) * sizeof(int));
    const size_t off_jobs = off_state + up((size_t)(count + 2) * sizeof(int));
    const size_t off_partials = off_jobs + up(jobs.size() * sizeof(fused::ExpandJob));
    const size_t partial_bytes = up((size_t)pslots * (pair ? 2 : 1) * fused::kBM * BN * sizeof(float));
    const size_t off_at = off_partials + partial_bytes;
    g->scratch_bytes = partial_bytes + at_bytes;
    const size_t total = off_at + at_bytes;
    cudaError_t e = cudaMalloc(&g->dev_block, total);
    if (e == cudaSuccess) e = cudaMemset(g->dev_block, 0, off_partials);
    uint8_t* base = static_cast<uint8_t*>(g->dev_block);
    bool maps_ok = true;
    if (e == cudaSuccess && g->expanded) {
        fused::EncodeFn enc = fused::encode_fn();
        for (int i = 0; i < count && maps_ok; ++i) {
            jobs[i].at = reinterpret_cast<__half*>(base + off_at + at_off[i]);
            if (enc && probs[i].Mp % 64 == 0 &&
                fused::encode_chunked(enc, &probs[i].tmap_a, jobs[i].at, (uint64_t)probs[i].Mp, (uint64_t)probs[i].K, fused::kBM / 64)) {
                probs[i].wide |= 2;
                continue;
            }
            maps_ok = enc && fused::encode_map(enc, &probs[i].tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, jobs[i].at,
                                               (uint64_t)probs[i].Mp, (uint64_t)probs[i].K, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
        }
        // the copies are written in the order the products are multiplied (longest K first)
        std::vector<fused::ExpandJob> sorted;
        sorted.reserve((size_t)count);
        for (int oi = 0; oi < count; ++oi) {
            fused::ExpandJob j = jobs[order[oi]];
            j.block_base = g->expand_units;
            g->expand_units += probs[order[oi]].expand_blocks;
            sorted.push_back(j);
        }
        if (maps_ok) e = cudaMemcpy(base + off_jobs, sorted.data(), sorted.size() * sizeof(fused::ExpandJob), cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) e = cudaMemcpy(base, probs.data(), probs.size() * sizeof(fused::Problem), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(base + off_items, list.data(), list.size() * sizeof(fused::Item), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = pair ? fused::launch_pair(g->params, g->out_f16, 1, nullptr, true)
                                   : fused::launch(g->params, BN, g->out_f16, g->expanded, 1, nullptr, true);
    if (e == cudaSuccess && !maps_ok) {
        cudaFree(g->dev_block);
        delete g;
        set_error("cuTensorMapEncodeTiled failed for a dense copy of A");
        return (int)cudaErrorInvalidValue;
    }
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
    g->params.jobs = g->expanded ? reinterpret_cast<const fused::ExpandJob*>(base + off_jobs) : nullptr;
    g->params.n_jobs = g->expanded ? count : 0;
    g->params.expand_blocks = g->expand_units;
    g->params.expand_state = g->expanded ? reinterpret_cast<int*>(base + off_state) : nullptr;
    *group = g;
    return 0;
}

int sspmm_group_run(sspmm_group* group, void* stream) {
    set_error("%s", "");
    if (!group) { set_error("null group"); return (int)cudaErrorInvalidValue; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = group->pair ? fused::launch_pair(group->params, group->out_f16, group->grid, st, false)
                                : fused::launch(group->params, group->BN, group->out_f16, group->expanded, group->grid, st);
    if (e != cudaSuccess) { set_error("group launch: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}

int sspmm_group_info(const sspmm_group* group, int* tile_columns, int* work_items, int* ctas, int* launches,
                     int64_t* scratch_bytes) {
    if (!group) return (int)cudaErrorInvalidValue;
    if (tile_columns) *tile_columns = group->BN;
    if (work_items) *work_items = group->n_items;
    if (ctas) *ctas = group->pair ? 2 * group->grid : group->grid;
    if (launches) *launches = 1;
    if (scratch_bytes) *scratch_bytes = (int64_t)group->scratch_bytes;
    return 0;
}

int sspmm_group_destroy(sspmm_group* group) {
    if (!group) return 0;
    if (group->dev_block) cudaFree(group->dev_block);
    delete group;
    return 0;
}

}  // extern "C"
