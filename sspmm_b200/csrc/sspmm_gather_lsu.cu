// Vector-sparse SpMM on the tensor cores, second gather variant: the rows of B are fetched by
// ordinary 16-byte loads of twelve producer warps (instead of TMA row-gather requests) and written
// into the same 128-byte-swizzled M-major layout the MMA reads.  Measured reason: the TMA gather
// path sustains about one 128-byte row per 19 cycles per SM; loads issued from many threads keep
// far more requests in flight and run at L2 speed.
//
// Also splits very long vector rows: a row with more than `chunk` vectors is cut into chunks that
// are separate work items; their fp32 partial tiles go to scratch, and whichever chunk of a row
// finishes last adds them up, in chunk order, and writes C once (one rounding).  Without this a
// power-law matrix is as slow as its longest row.
//
// Same contract as the other SpMM kernels (reference entry: SSpMM/src/sspmm.cu:626-649).
//
// Warps (672 threads): 0-3 epilogue, 4-7 MMA issuers (4 owns the TMEM allocation), 8 scheduler,
// 9-20 three producer groups of four warps that fill pipeline stages in turn.
//
// Four MMA issuers, not one: an MMA of this shape (128 x 16 x 16) is a few cycles of tensor-core work, but
// the thread that issues it is held about 130 cycles per tcgen05.mma and about 100 per tcgen05.commit
// (measured), so one issuer caps the kernel near 1100 cycles per 64-vector stage.  The issuers take the
// stages in turn, each into its own TMEM accumulator, and the epilogue adds the accumulators up.
//
// The scheduler warp is what keeps the dependent loads of the work list (row order -> row pointers
// -> number of 64-vector stages) off everybody else's critical path: it looks up 32 work items at a
// time, one per lane, and publishes one 32-byte descriptor per pipeline stage in a shared-memory
// ring that all other warps read.  A producer group therefore knows its next stage without touching
// global memory, loads that stage's column ids while the B rows of the current one are in flight,
// and carries the stage's value vectors along (no separate value loader whose one-stage-at-a-time
// latency would bound the pipeline).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch.h"
#include "ptx.cuh"

namespace sspmm_b200 {
namespace lsu {

constexpr int kTileN = 128;
constexpr int kMmaN = 16;
constexpr int kKS = 64;                // gathered rows per stage
constexpr int kStages = 8;
constexpr int kIssuers = 4;
constexpr int kFirstProducerWarp = 4 + kIssuers + 1;
constexpr int kThreads = (kFirstProducerWarp + 4 * 3) * 32;
constexpr int kTmemCols = 2 * kIssuers * kMmaN;   // two tiles in flight, one accumulator per issuer
constexpr int kProducerGroups = 3;
constexpr int kRing = 64;              // stage descriptors in the ring: two batches of 32
constexpr int kRingConsumers = 4 + kIssuers + 4 * kProducerGroups;   // warps that read the ring
constexpr int kEpiStride = 36;         // floats per row of an epilogue warp's staging tile (32 + padding)

constexpr int kAChunk = kKS * 128;
constexpr int kAStage = 2 * kAChunk;   // 16 KB
constexpr int kVChunk = kKS * 16;
constexpr int kVStage = 2 * kVChunk;   // 2 KB
constexpr int kAOff = 0;
constexpr int kVOff = kStages * kAStage;
constexpr int kRingOff = kVOff + kStages * kVStage;
constexpr int kEpiOff = kRingOff + kRing * 32;
constexpr int kBarOff = kEpiOff + 4 * 16 * kEpiStride * 4;
constexpr int kNumBars = 2 * kStages + 4 + 4;
constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
constexpr int kAbortOff = kTmemPtrOff + 8;
constexpr int kSmemBytes = kAbortOff + 8 + 1024;

struct Problem {
    int m_vec, N, K, n_tiles, base_tiles;   // base_tiles = m_vec * n_tiles * batch
    int chunk;                              // rows longer than this are split (0 = never)
    int cap;                                // capacity of the entry list
    const int* row_indices;
    const int* row_offsets;
    const int* col;
    const __half* values;
    const __half* rhs;
    int64_t values_stride, rhs_stride, out_stride;
    const int* n_entries;                   // device: number of (row, chunk) entries (null when chunk == 0)
    const int2* entries;                    // device: x = vector row, y = chunk index
    float* partial;                         // device: [entry][n_tile][V][128] fp32
    int* arrivals;                          // device: [entry][n_tile][4] finished chunks per split row and warp slice, zero at launch
    int* queue;                             // device: work counter, zero at launch (null: items are dealt out round robin)
};

struct Item {
    int row;        // vector row (-1: nothing to do)
    int j0, len;    // vectors [j0, j0 + len) of the value / column arrays
    int n0, batch;  // batch: for chunk entries (slot >= 0) instead (chunks of the row << 16) | chunk number
    int slot;       // >= 0: partial-tile slot (entry * n_tiles + n_tile); -1: store to C
};

__device__ __forceinline__ Item get_item(const Problem& p, int T, int extra_entries, int chunk) {
    Item it;
    it.slot = -1;
    if (T < p.base_tiles) {
        const int sched = T % p.m_vec;
        const int rest = T / p.m_vec;
        it.n0 = (rest % p.n_tiles) * kTileN;
        it.batch = rest / p.n_tiles;
        const int i = p.row_indices ? __ldg(p.row_indices + sched) : sched;
        if ((unsigned)i >= (unsigned)p.m_vec) { it.row = -1; it.j0 = 0; it.len = 0; return it; }
        it.row = i;
        it.j0 = __ldg(p.row_offsets + i);
        it.len = max(0, __ldg(p.row_offsets + i + 1) - it.j0);
        if (chunk > 0 && it.len > chunk) { it.row = -1; it.len = 0; }          // done as chunk entries
        return it;
    }
    const int x = T - p.base_tiles;
    const int e = x / p.n_tiles;
    it.batch = 0;
    it.n0 = (x % p.n_tiles) * kTileN;
    if (e >= extra_entries) { it.row = -1; it.j0 = 0; it.len = 0; return it; }
    const int2 en = p.entries[e];
    it.row = en.x;
    const int j0 = __ldg(p.row_offsets + en.x);
    const int len = __ldg(p.row_offsets + en.x + 1) - j0;
    it.j0 = j0 + en.y * chunk;
    it.len = max(0, min(chunk, len - en.y * chunk));
    it.slot = x;
    it.batch = (((len + chunk - 1) / chunk) << 16) | en.y;       // split rows: chunks of the row and this chunk's number
    return it;
}

// One pipeline stage of one work item, as published by the scheduler warp.
struct __align__(16) StageDesc {
    int j;          // first vector of the stage in the column / value arrays
    int count;      // vectors in the stage (0: the item is an empty vector row, whose tile is zero-filled)
    int flags;      // kFirst | kLast | kEnd, and from bit 8 up the number of stages of the item (saturating)
    int pipe;       // running number of the stage inside this CTA (picks the smem stage and the producer group)
    int row;        // vector row
    int n0;         // first column of the tile
    int batch;
    int slot;       // >= 0: partial-tile slot; -1: store to C
};
constexpr int kFirst = 1, kLast = 2, kEnd = 4;
static_assert(sizeof(StageDesc) == 32, "descriptor size");

// Ring bookkeeping shared by all readers: descriptor number r lives in slot r % kRing; the batch of 32 that
// holds it is published through ring_full[(r / 32) & 1] and handed back through ring_empty[(r / 32) & 1].
struct RingReader {
    uint32_t r = 0;
    const StageDesc* ring;
    uint32_t bar_full, bar_empty;
    volatile int* abort_flag;
    // Makes descriptor r readable.  Blocking: false means the wait was abandoned.  Non-blocking: false means the
    // batch has not been published yet.
    __device__ __forceinline__ bool acquire(bool blocking) {
        if ((r & 31u) != 0u) return true;
        const uint32_t bar = bar_full + 8u * ((r >> 5) & 1u), parity = (r >> 6) & 1u;
        if (!blocking) return mbar_test_wait(bar, parity);
        return mbar_wait(bar, parity, abort_flag, kStatusWaitFull);
    }
    __device__ __forceinline__ StageDesc read() const {
        const int4* q = reinterpret_cast<const int4*>(ring + (r & (kRing - 1)));
        const int4 a = q[0], b = q[1];
        StageDesc d;
        d.j = a.x; d.count = a.y; d.flags = a.z; d.pipe = a.w;
        d.row = b.x; d.n0 = b.y; d.batch = b.z; d.slot = b.w;
        return d;
    }
    // Moves past descriptor r (whose contents the caller has copied); the whole warp calls it.
    __device__ __forceinline__ void release(int lane) {
        ++r;
        if ((r & 31u) == 0u) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8u * (((r - 1u) >> 5) & 1u));
        }
    }
};

template <int V, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
sspmm_gather_lsu_kernel(Problem p, OutT* __restrict__ out, int vec_store_ok) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + kBarOff;
    const uint32_t bar_empty = bar_full + kStages * 8;
    const uint32_t bar_acc_full = bar_empty + kStages * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    const uint32_t bar_ring_full = bar_acc_empty + 2 * 8;
    const uint32_t bar_ring_empty = bar_ring_full + 2 * 8;
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kAbortOff);
    StageDesc* ring = reinterpret_cast<StageDesc*>(smem + kRingOff);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 4);      // the four warps of the producer group that owns the stage
            mbar_init(bar_empty + 8 * s, 1);     // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, kIssuers);   // every issuer commits at the end of a tile
            mbar_init(bar_acc_empty + 8 * b, 4);
            mbar_init(bar_ring_full + 8 * b, 1);
            mbar_init(bar_ring_empty + 8 * b, kRingConsumers);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (V == 8) {
        // the upper half of every value stage (rows 8..15 of the MMA's N = 16) stays zero
        for (int o = threadIdx.x * 16; o < kStages * kVChunk; o += kThreads * 16) {
            const int s = o / kVChunk, r = o % kVChunk;
            *reinterpret_cast<uint4*>(smem + kVOff + s * kVStage + kVChunk + r) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
    }
    if (warp == 4) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;
    // The entry list was sized from a remembered vector count; if this call's matrix needs more
    // entries than fit, splitting is switched off for the whole launch (every row is then done whole).
    int extra_entries = p.n_entries ? *p.n_entries : 0;
    const int chunk = (p.chunk > 0 && extra_entries <= p.cap) ? p.chunk : 0;
    if (chunk == 0) extra_entries = 0;
    const int total = p.base_tiles + extra_entries * p.n_tiles;

    RingReader rd;
    rd.ring = ring; rd.bar_full = bar_ring_full; rd.bar_empty = bar_ring_empty; rd.abort_flag = abort_flag;

    if (warp == 4 + kIssuers) {
        // ---------------------------------------------------------------- scheduler
        // Work items in the order they are handed out: the chunks of split rows first (they are the longest),
        // then the vector rows in the caller's order.  With a work counter the CTAs take them in small batches
        // as they go (vector rows of a power-law matrix differ in length by orders of magnitude, so dealing
        // them out round robin leaves most SMs idle at the end); without one, round robin.
        const int n_entry_tiles = extra_entries * p.n_tiles;
        int take = 32;
        if (p.queue) take = max(1, min(32, total / ((int)gridDim.x * 8)));
        int dealt = 0;
        auto grab = [&](Item& it) {
            int u = total;
            bool any;
            if (p.queue) {
                int u0 = 0;
                if (lane == 0) u0 = atomicAdd(p.queue, take);
                u0 = __shfl_sync(0xffffffffu, u0, 0);
                any = u0 < total;
                if (lane < take && u0 < total - lane) u = u0 + lane;
            } else {
                const long long first = (long long)blockIdx.x + (long long)dealt * gridDim.x;
                any = first < total;
                const long long mine_u = first + (long long)lane * gridDim.x;
                if (mine_u < total) u = (int)mine_u;
                dealt += 32;
            }
            it.row = -1; it.j0 = 0; it.len = 0; it.n0 = 0; it.batch = 0; it.slot = -1;
            if (u < total) it = get_item(p, u < n_entry_tiles ? p.base_tiles + u : u - n_entry_tiles, extra_entries, chunk);
            return any;
        };
        uint32_t w = 0;                 // descriptors written
        int pipe = 0;
        bool ok = true;
        // makes ring slot w writable (at the start of a batch: waits until every reader left the batch two back)
        auto open_slot = [&]() {
            if ((w & 31u) != 0u) return true;
            return mbar_wait(bar_ring_empty + 8u * ((w >> 5) & 1u), ((w >> 6) & 1u) ^ 1u, abort_flag, kStatusWaitEmpty);
        };
        // after `n` descriptors were written starting at w: publishes the batch if it is complete
        auto wrote = [&](uint32_t n) {
            w += n;
            if ((w & 31u) == 0u) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_ring_full + 8u * (((w - 1u) >> 5) & 1u));
            }
        };
        Item mine;
        bool have = grab(mine);
        while (have && ok) {
            const Item cur = mine;
            have = grab(mine);                            // the next look-ups overlap the emission of these
            for (int i = 0; i < take && ok; ++i) {
                const int row = __shfl_sync(0xffffffffu, cur.row, i);
                if (row < 0) continue;
                const int len = __shfl_sync(0xffffffffu, cur.len, i);
                const int j0 = __shfl_sync(0xffffffffu, cur.j0, i);
                const int n0 = __shfl_sync(0xffffffffu, cur.n0, i);
                const int batch = __shfl_sync(0xffffffffu, cur.batch, i);
                const int slot = __shfl_sync(0xffffffffu, cur.slot, i);
                const int ns = len > 0 ? (len + kKS - 1) / kKS : 1;
                for (int s0 = 0; s0 < ns && ok;) {
                    if (!open_slot()) { ok = false; break; }
                    const int n = min(min(32, ns - s0), 32 - (int)(w & 31u));
                    if (lane < n) {
                        const int s = s0 + lane;
                        StageDesc d;
                        d.j = j0 + s * kKS;
                        d.count = len > 0 ? min(kKS, len - s * kKS) : 0;
                        d.flags = (s == 0 ? kFirst : 0) | (s == ns - 1 ? kLast : 0) | (min(ns, 1 << 20) << 8);
                        d.pipe = pipe + s;
                        d.row = row; d.n0 = n0; d.batch = batch; d.slot = slot;
                        int4* q = reinterpret_cast<int4*>(ring + ((w + lane) & (kRing - 1)));
                        q[0] = make_int4(d.j, d.count, d.flags, d.pipe);
                        q[1] = make_int4(d.row, d.n0, d.batch, d.slot);
                    }
                    wrote((uint32_t)n);
                    s0 += n;
                }
                if (len > 0) pipe += ns;
            }
        }
        // end marks up to the end of the batch (a full batch of them when the last one was just published)
        if (ok && open_slot()) {
            const int n = 32 - (int)(w & 31u);
            if (lane < n) {
                int4* q = reinterpret_cast<int4*>(ring + ((w + lane) & (kRing - 1)));
                q[0] = make_int4(0, 0, kEnd, 0);
                q[1] = make_int4(-1, 0, 0, -1);
            }
            wrote((uint32_t)n);
        }
    } else if (warp >= kFirstProducerWarp) {
        // ---------------------------------------------------------------- producers
        const int group = (warp - kFirstProducerWarp) >> 2;
        const int t = threadIdx.x - (kFirstProducerWarp + 4 * group) * 32;        // 0..127 inside the group
        const int cc = t & 15;                                   // 16-byte piece of the 256-byte row segment
        const int rsub = t >> 4;                                 // row inside each block of 8 rows
        const int half_sel = cc >> 3, c16 = cc & 7;
        constexpr int kChunksPerRow = V / 8;                     // 16-byte pieces of one value vector
        const int vr = t / kChunksPerRow, vc = t % kChunksPerRow;   // this thread's piece of the stage's value vectors
        const bool has_vpiece = t < kKS * kChunksPerRow;

        // Finds the next stage this group owns.  0 = found (in `d`), 1 = end of the list, 2 = the ring batch
        // is not published yet (non-blocking calls only), 3 = a wait was abandoned.
        auto advance = [&](StageDesc& d, bool blocking) {
            for (;;) {
                if (!rd.acquire(blocking)) return blocking ? 3 : 2;
                d = rd.read();
                if (d.flags & kEnd) return 1;
                rd.release(lane);
                if (d.count > 0 && d.pipe % kProducerGroups == group) return 0;
            }
        };
        auto load_cols = [&](const StageDesc& d, int (&c)[8]) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int r = 8 * q + rsub;
                c[q] = -1;
                if (r < d.count) c[q] = __ldg(p.col + d.j + r);
            }
        };
        StageDesc nxt;
        int cols[8];
        int st = advance(nxt, true);
        if (st == 0) load_cols(nxt, cols);
        while (st == 0) {
            const StageDesc cur = nxt;
            int cur_cols[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) cur_cols[q] = cols[q];
            // the B rows and value vectors of this stage
            const int cur_batch = cur.slot >= 0 ? 0 : cur.batch;          // chunk entries carry their chunk numbers there
            const __half* bbase = p.rhs + (int64_t)cur_batch * p.rhs_stride + cur.n0 + cc * 8;
            const bool col_ok = cur.n0 + cc * 8 < p.N;
            uint4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                v[q] = make_uint4(0, 0, 0, 0);
                if (col_ok && (unsigned)cur_cols[q] < (unsigned)p.K)
                    v[q] = __ldg(reinterpret_cast<const uint4*>(bbase + (int64_t)cur_cols[q] * p.N));
            }
            uint4 vv = make_uint4(0, 0, 0, 0);
            if (has_vpiece && vr < cur.count)
                vv = __ldg(reinterpret_cast<const uint4*>(p.values + (int64_t)cur_batch * p.values_stride +
                                                          ((int64_t)cur.j + vr) * V + vc * 8));
            // while they are in flight: the column ids of the next owned stage, if its descriptor is out already
            st = advance(nxt, false);
            if (st == 0) load_cols(nxt, cols);
            const uint32_t stage = (uint32_t)cur.pipe % kStages, phase = ((uint32_t)cur.pipe / kStages) & 1u;
            if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitEmpty)) break;
            uint8_t* a_s = smem + kAOff + stage * kAStage + half_sel * kAChunk;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int r = 8 * q + rsub;
                *reinterpret_cast<uint4*>(a_s + r * 128 + ((c16 ^ (r & 7)) << 4)) = v[q];
            }
            if (has_vpiece) *reinterpret_cast<uint4*>(smem + kVOff + stage * kVStage + vc * kVChunk + vr * 16) = vv;
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full + 8 * stage);
            if (st == 2) {
                // nothing of this group is pending now, so waiting for the scheduler cannot hold anybody up
                st = advance(nxt, true);
                if (st == 0) load_cols(nxt, cols);
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- MMA issuers (warps 4 .. 4 + kIssuers - 1)
        constexpr uint32_t idesc = make_idesc_f16_f32(kTileN, kMmaN, true, true);
        const int me = warp - 4;
        uint32_t acc_it = 0;
        bool started = false;            // has this issuer written its accumulator for the current tile?
        for (;;) {
            if (!rd.acquire(true)) break;
            const StageDesc d = rd.read();
            if (d.flags & kEnd) break;
            rd.release(lane);
            if (d.count <= 0) continue;
            const uint32_t buf = acc_it & 1u;
            if (d.flags & kFirst) {
                if (!mbar_wait(bar_acc_empty + 8 * buf, ((acc_it >> 1) & 1u) ^ 1u, abort_flag, kStatusWaitAccEmpty)) break;
                tc_fence_after_sync();
                started = false;
            }
            if (d.pipe % kIssuers == me) {
                const uint32_t stage = (uint32_t)d.pipe % kStages, phase = ((uint32_t)d.pipe / kStages) & 1u;
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, kStatusWaitFull)) break;
                tc_fence_after_sync();
                if (lane == 0) {
                    const uint32_t d_tmem = tmem_base + (buf * kIssuers + me) * kMmaN;
                    const int nk = (d.count + 15) >> 4;
                    const uint32_t a_addr = sbase + kAOff + stage * kAStage;
                    const uint32_t v_addr = sbase + kVOff + stage * kVStage;
                    for (int kk = 0; kk < nk; ++kk) {
                        const uint64_t a_desc = make_smem_desc(a_addr + kk * 2048, kAChunk, 1024, 2);
                        const uint64_t b_desc = make_smem_desc(v_addr + kk * 256, 128, kVChunk, 0);
                        tc_mma_f16(d_tmem, a_desc, b_desc, idesc, (started || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty + 8 * stage);
                }
                started = true;
            }
            if (d.flags & kLast) {
                // a commit covers the MMAs its own thread issued, so every issuer reports the end of the tile
                if (lane == 0) tc_commit(bar_acc_full + 8 * buf);
                ++acc_it;
            }
            __syncwarp();
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 0-3)
        const int q = warp & 3;
        float* stg = reinterpret_cast<float*>(smem + kEpiOff) + q * 16 * kEpiStride;   // this warp's V x 32 tile
        uint32_t acc_it = 0;
        for (;;) {
            if (!rd.acquire(true)) break;
            const StageDesc d = rd.read();
            if (d.flags & kEnd) break;
            rd.release(lane);
            if (!(d.flags & kLast)) continue;
            uint32_t r[V];
            if (d.count > 0) {
                const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
                if (!mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kStatusWaitAccFull)) break;
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (kIssuers * kMmaN);
                // the accumulators that received a stage: those of the issuers of stages first .. last of the item
                const int ns = d.flags >> 8;
                const int n_acc = min(ns, kIssuers);
                const int a0 = d.pipe - ns + 1;
                const uint32_t t0 = taddr + (uint32_t)(a0 % kIssuers) * kMmaN;
                if constexpr (V == 16) tmem_ld_x16(t0, r); else tmem_ld_x8(t0, r);
                tc_wait_ld();
                for (int a = 1; a < n_acc; ++a) {
                    uint32_t r2[V];
                    const uint32_t ta = taddr + (uint32_t)((a0 + a) % kIssuers) * kMmaN;
                    if constexpr (V == 16) tmem_ld_x16(ta, r2); else tmem_ld_x8(ta, r2);
                    tc_wait_ld();
#pragma unroll
                    for (int v = 0; v < V; ++v) r[v] = __float_as_uint(__uint_as_float(r[v]) + __uint_as_float(r2[v]));
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
                ++acc_it;
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) r[v] = 0u;
            }
            const int nl = q * 32 + lane;
            int batch = d.batch;
            if (d.slot >= 0) {
                // A chunk of a split row.  Every epilogue warp looks after its own 32 columns: it stores its slice
                // of the partial tile, counts itself in, and the warp that finds all other chunks already counted
                // adds the slices up in chunk order (so the sum does not depend on who does it).
                const int n_chunks = d.batch >> 16, my_chunk = d.batch & 0xffff;
                const int slot0 = d.slot - my_chunk * p.n_tiles;              // slot of the row's chunk 0 for this tile
                batch = 0;
                float* o = p.partial + (int64_t)d.slot * V * kTileN + nl;
#pragma unroll
                for (int v = 0; v < V; ++v) o[v * kTileN] = __uint_as_float(r[v]);
                __threadfence();
                __syncwarp();
                int seen = 0;
                if (lane == 0) seen = atomicAdd(p.arrivals + (int64_t)slot0 * 4 + q, 1);
                seen = __shfl_sync(0xffffffffu, seen, 0);
                if (seen != n_chunks - 1) continue;
                __threadfence();
                float acc[V];
#pragma unroll
                for (int v = 0; v < V; ++v) acc[v] = 0.f;
                for (int c = 0; c < n_chunks; ++c) {
                    const float* src = p.partial + ((int64_t)slot0 + (int64_t)c * p.n_tiles) * V * kTileN + nl;
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[v] += __ldcg(src + v * kTileN);
                }
#pragma unroll
                for (int v = 0; v < V; ++v) r[v] = __float_as_uint(acc[v]);
            }
            if (vec_store_ok && d.n0 + q * 32 + 32 <= p.N) {
                // 16-byte stores: the warp's V x 32 tile goes through shared memory so that every lane owns
                // one 16-byte piece of a row of C
#pragma unroll
                for (int v = 0; v < V; ++v) stg[v * kEpiStride + lane] = __uint_as_float(r[v]);
                __syncwarp();
                constexpr int kCols = 16 / (int)sizeof(OutT);        // columns per piece
                constexpr int kPieces = 32 / kCols;                  // pieces per row
                OutT* obase = out + (int64_t)batch * p.out_stride + (int64_t)d.row * V * p.N + d.n0 + q * 32;
#pragma unroll
                for (int pc0 = 0; pc0 < V * kPieces; pc0 += 32) {
                    const int pc = pc0 + lane;
                    const int row = pc / kPieces, piece = pc % kPieces;
                    const float* src = stg + row * kEpiStride + piece * kCols;
                    const float4 f0 = *reinterpret_cast<const float4*>(src);
                    OutT* dst = obase + (int64_t)row * p.N + piece * kCols;
                    if constexpr (sizeof(OutT) == 2) {
                        const float4 f1 = *reinterpret_cast<const float4*>(src + 4);
                        const __half2 h0 = __floats2half2_rn(f0.x, f0.y), h1 = __floats2half2_rn(f0.z, f0.w);
                        const __half2 h2 = __floats2half2_rn(f1.x, f1.y), h3 = __floats2half2_rn(f1.z, f1.w);
                        uint4 u;
                        u.x = *reinterpret_cast<const uint32_t*>(&h0); u.y = *reinterpret_cast<const uint32_t*>(&h1);
                        u.z = *reinterpret_cast<const uint32_t*>(&h2); u.w = *reinterpret_cast<const uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>(dst) = u;
                    } else {
                        *reinterpret_cast<float4*>(dst) = f0;
                    }
                }
                __syncwarp();
            } else if (d.n0 + nl < p.N) {
                OutT* o = out + (int64_t)batch * p.out_stride + (int64_t)d.row * V * p.N + d.n0 + nl;
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    const float f = __uint_as_float(r[v]);
                    if constexpr (sizeof(OutT) == 2) o[(int64_t)v * p.N] = __float2half_rn(f);
                    else o[(int64_t)v * p.N] = f;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- splitting of long rows ---------------------------------------------------
// counter[0] = number of entries; entries of one row are consecutive, chunk 0 first.
__global__ void __launch_bounds__(256)
build_chunk_entries_kernel(int m_vec, int chunk, int cap, const int* __restrict__ row_offsets, int* __restrict__ counter,
                           int2* __restrict__ entries) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m_vec) return;
    const int len = row_offsets[i + 1] - row_offsets[i];
    if (len <= chunk) return;
    const int n = (len + chunk - 1) / chunk;
    const int base = atomicAdd(counter, n);
    for (int c = 0; c < n && base + c < cap; ++c) entries[base + c] = make_int2(i, c);
}

template <int V, typename OutT>
cudaError_t launch_typed(const SpmmArgs& a, Problem p, int cap, void* scratch, int grid) {
    auto kern = sspmm_gather_lsu_kernel<V, OutT>;
    static DeviceOnce once;
    if (!once.done()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        once.mark();
    }
    if (scratch) {
        // [0] number of chunk entries, [1] the work counter of the main kernel
        int* counter = static_cast<int*>(scratch);
        cudaError_t e = cudaMemsetAsync(counter, 0, 16 + (p.chunk > 0 ? (size_t)cap * p.n_tiles * 16 : 0), a.stream);
        if (e != cudaSuccess) return e;
        if (p.chunk > 0) {
            build_chunk_entries_kernel<<<(a.m_vec + 255) / 256, 256, 0, a.stream>>>(a.m_vec, p.chunk, cap, a.row_offsets,
                                                                                   counter, const_cast<int2*>(p.entries));
            e = cudaGetLastError();
            if (e != cudaSuccess) return e;
        }
    }
    // 16-byte stores need every row of C to start on a 16-byte boundary
    const size_t es = sizeof(OutT);
    const int vec_ok = (reinterpret_cast<uintptr_t>(a.out) % 16 == 0 && ((size_t)a.N * es) % 16 == 0 &&
                        ((size_t)a.out_stride * es) % 16 == 0) ? 1 : 0;
    kern<<<grid, kThreads, kSmemBytes, a.stream>>>(p, static_cast<OutT*>(a.out), vec_ok);
    return cudaGetLastError();
}

}  // namespace lsu

// Scratch layout: [16 B: entry counter, work counter][cap * n_tiles * 4 arrival counters][cap entries of int2]
// [partials].  cap = 0 disables row splitting; the first 16 bytes alone still give the kernel its work counter.
void sspmm_gather_lsu_plan(const SpmmArgs& a, long long nvec, int* chunk, int* cap, size_t* scratch_bytes) {
    *chunk = 0; *cap = 0; *scratch_bytes = 0;
    if (nvec <= 0 || a.batch != 1) return;
    *scratch_bytes = 256;
    const int sms = current_device_sm_count();
    const long long n_tiles = (a.N + lsu::kTileN - 1) / lsu::kTileN;
    // a chunk is about an eighth of an SM's share of the vectors, and at least eight pipeline stages
    long long c = nvec * n_tiles / ((long long)sms * 8);
    if (c < 512) c = 512;
    c = (c + 63) / 64 * 64;
    if (c >= a.K || c > 0x3fffffff) return;                 // no row can be longer than K vectors
    const long long n_cap = 2 * nvec / c + 1;
    const size_t bytes = 16 + (size_t)n_cap * n_tiles * 16 + (size_t)n_cap * 8 + (size_t)n_cap * n_tiles * a.V * lsu::kTileN * 4;
    if (n_cap > 60000 || bytes > ((size_t)1 << 30) || a.K / c >= 65535) return;
    *chunk = (int)c; *cap = (int)n_cap; *scratch_bytes = (bytes + 255) & ~(size_t)255;
}

cudaError_t launch_sspmm_gather_lsu(const SpmmArgs& a, int chunk, int cap, void* scratch) {
    const int n_tiles = (a.N + lsu::kTileN - 1) / lsu::kTileN;
    const int64_t base = (int64_t)a.m_vec * n_tiles * a.batch;
    const int64_t worst = base + (int64_t)cap * n_tiles;
    if (worst > 0x7fffffffLL) {
        set_error("problem too large for 32-bit tile ids");
        return cudaErrorInvalidValue;
    }
    lsu::Problem p;
    p.m_vec = a.m_vec; p.N = a.N; p.K = a.K; p.n_tiles = n_tiles; p.base_tiles = (int)base;
    p.chunk = chunk; p.cap = cap;
    p.row_indices = a.row_indices; p.row_offsets = a.row_offsets; p.col = a.column_indices;
    p.values = a.values; p.rhs = a.rhs;
    p.values_stride = a.values_stride; p.rhs_stride = a.rhs_stride; p.out_stride = a.out_stride;
    p.n_entries = nullptr; p.entries = nullptr; p.partial = nullptr; p.arrivals = nullptr;
    p.queue = scratch ? static_cast<int*>(scratch) + 1 : nullptr;
    if (chunk > 0) {
        uint8_t* s = static_cast<uint8_t*>(scratch);
        const size_t arrivals_bytes = (size_t)cap * n_tiles * 16;
        p.n_entries = reinterpret_cast<const int*>(s);
        p.arrivals = reinterpret_cast<int*>(s + 16);
        p.entries = reinterpret_cast<const int2*>(s + 16 + arrivals_bytes);
        p.partial = reinterpret_cast<float*>(s + 16 + arrivals_bytes + (size_t)cap * 8);
    }
    const int sms = current_device_sm_count();
    if (sms <= 0) return cudaErrorNoDevice;
    const int grid = (int)(worst < sms ? worst : sms);
    if (a.V == 16)
        return a.out_f16 ? lsu::launch_typed<16, __half>(a, p, cap, scratch, grid) : lsu::launch_typed<16, float>(a, p, cap, scratch, grid);
    return a.out_f16 ? lsu::launch_typed<8, __half>(a, p, cap, scratch, grid) : lsu::launch_typed<8, float>(a, p, cap, scratch, grid);
}

}  // namespace sspmm_b200
