// Sparse vector compression kernels.
//
// Reference behaviour (RowMerge/sparse_matrix_format.py:100-123): for vector row i,
//     cols = []
//     for j in 0..V-1 (rows below M only):  cols = list(set(cols + row[V*i+j]))
// and the vector row pointer is the running sum of len(cols).  The order of `cols`
// is CPython's set order, which for small non-negative ints is decided by an
// open-addressing table: hash(x) = x; start slot x & mask; probe the nine following
// slots when that window fits inside the table, else jump to (5*i + 1 + perturb) & mask
// with perturb >>= 5; after an insertion with 5*fill >= 3*mask the table is rebuilt
// with the power-of-two length above 4*used (2*used beyond 50 000), re-inserting
// the old entries in slot order; iteration is in slot order.
//
// A "team" (one warp, or one CTA) works on one vector row; the V rows of a group
// are one contiguous CSR range.
//   svc_count_kernel   marks the group's columns in a shared-memory bitmap with
//                      atomicOr, counts first-time bits by popc of the returned
//                      words, and decides per group whether ascending order is
//                      already the exact answer: it is when the largest column id
//                      is below the final table length (every key then sits in its
//                      home slot).
//   svc_scan_*         exclusive scans (vector row pointers, scratch offsets) and a
//                      histogram of replay classes.
//   svc_emit_sorted    bitmap -> ascending column list by a popc prefix scan; value
//                      vectors placed with prefix[word] + popc(lower bits).
//   svc_emit_replay    exact replay of the V set rebuilds.  Insertion into a table of
//                      fixed length is "first come, first served" along each key's
//                      probe path, which has a unique fixed point: slot = the first
//                      one on my path not held by an earlier element.  The team finds
//                      it in parallel with atomicMin on the element's sequence number (an
//                      element pushed out of a slot by an earlier one starts its path again);
//                      table growth steps are replayed level by level (8, 32, 128, ...).
// The replay kernels take their groups from per-class lists (written by the scan kernel)
// through a work counter, so a CTA never walks over groups of other classes and the
// groups of a class, whose cost differs by an order of magnitude, balance themselves.
#include "svc.cuh"

#include <mutex>

#include "launch.h"

namespace sspmm_b200 {

__device__ int g_svc_bad_column = 0;

namespace {

constexpr int kMinTable = 8;
constexpr int kLinearProbes = 9;
constexpr int kPerturbShift = 5;
constexpr int kEmptyPrio = 0x7fffffff;

// Replay classes by number of distinct columns u (and final table length):
constexpr int kClassSorted = 0;   // no replay
constexpr int kClassS = 1;        // u <= 306   (table <= 512):   warp team, everything in shared memory
constexpr int kClassM1 = 2;       // u <= 1228  (table <= 2048):  CTA team, everything in shared memory
constexpr int kClassM2 = 3;       // u <= 4914  (table <= 8192):  CTA team, everything in shared memory
constexpr int kClassL = 4;        // table <= 32768:              CTA team, table in shared memory, lists in global
constexpr int kClassXL = 5;       // larger:                      CTA team, table and lists in global
constexpr int kClassXS = 6;       // u <= 76    (table <= 128):   warp team, small enough for 48 resident teams per SM
constexpr int kNumClasses = kSvcClasses;
static_assert(kNumClasses == 7, "class numbering");

constexpr int kXSCapU = 76, kXSCapT = 128;
constexpr int kSCapU = 306, kSCapT = 512;
constexpr int kM1CapU = 1228, kM1CapT = 2048;
constexpr int kM2CapU = 4914, kM2CapT = 8192;
constexpr int kLCapT = 32768;
constexpr int kLCapU = 19660;   // most keys a table of kLCapT slots holds
constexpr int kLSeqInts = 19664;    // a table of kLCapT slots holds fewer than 19661 keys; class L keeps the level's sequence in shared memory
constexpr int kListsPerGroup = 4;   // X2, NEW, P, Q (the fifth list is the output slice)

__host__ __device__ inline void next_level(int size, long long& trig, int& next_size) {
    const long long mask = size - 1;
    trig = (3 * mask + 4) / 5;                         // smallest fill with 5*fill >= 3*mask
    const long long minused = trig > 50000 ? trig * 2 : trig * 4;
    long long ns = kMinTable;
    while (ns <= minused) ns <<= 1;
    next_size = (int)(ns > (1ll << 30) ? (1ll << 30) : ns);
}

// Table length after `distinct` different keys were added to an empty set.
__host__ __device__ inline int final_table_len(int distinct) {
    int size = kMinTable;
    for (;;) {
        long long trig;
        int ns;
        next_level(size, trig, ns);
        if (distinct < trig || size >= (1 << 30)) return size;
        size = ns;
    }
}

__host__ __device__ inline int replay_class(int u, int tbl_len) {
    if (tbl_len <= 0) return kClassSorted;
    if (u <= kXSCapU) return kClassXS;
    if (u <= kSCapU) return kClassS;
    if (u <= kM1CapU) return kClassM1;
    if (u <= kM2CapU) return kClassM2;
    if (tbl_len <= kLCapT) return kClassL;
    return kClassXL;
}

// The list of replayed groups is written segment by segment.  A segment is a class, or a part of one: the groups
// of a class differ in cost by the ratio of their sizes (up to four), and with only a few groups per team the order
// in which the work counter hands them out decides how long the last team runs.  So the classes with few, long
// groups are cut into four size ranges (two for S) that are listed largest first.
constexpr int kNumSegs = kSvcSegs;
constexpr int kSegS = 1, kSegM1 = 3, kSegM2 = 7, kSegL = 11, kSegXL = 15, kSegXS = 16, kSegSortedBig = 17;
static_assert(kNumSegs == 18, "segment numbering");
// Groups in ascending order with more than kBigGroup entries get a CTA each; the counting pass marks them
// (table length -1) and the last segment lists them.
__host__ __device__ inline int size_quarter(int u, int cap) {       // 0 = the largest sizes of a class whose largest is cap
    if (u > (int)((long long)cap * 181 / 256)) return 0;            // cap / sqrt(2)
    if (u > cap / 2) return 1;
    if (u > (int)((long long)cap * 91 / 256)) return 2;             // cap / (2 sqrt(2))
    return 3;
}
__host__ __device__ inline int list_segment(int u, int tbl_len) {
    switch (replay_class(u, tbl_len)) {
        case kClassS: return kSegS + (u > kSCapU / 2 ? 0 : 1);
        case kClassM1: return kSegM1 + size_quarter(u, kM1CapU);
        case kClassM2: return kSegM2 + size_quarter(u, kM2CapU);
        case kClassL: return kSegL + size_quarter(u, kLCapU);
        case kClassXL: return kSegXL;
        case kClassXS: return kSegXS;
        default: return tbl_len < 0 ? kSegSortedBig : 0;
    }
}
// first segment of a class and one past its last
__host__ inline void class_segments(int c, int& s0, int& s1) {
    switch (c) {
        case kClassS: s0 = kSegS; s1 = kSegM1; break;
        case kClassM1: s0 = kSegM1; s1 = kSegM2; break;
        case kClassM2: s0 = kSegM2; s1 = kSegL; break;
        case kClassL: s0 = kSegL; s1 = kSegXL; break;
        case kClassXL: s0 = kSegXL; s1 = kSegXS; break;
        case kClassXS: s0 = kSegXS; s1 = kSegSortedBig; break;
        default: s0 = 0; s1 = 1; break;
    }
}

// Global scratch ints of one replayed group.
__host__ __device__ inline long long group_scratch_ints(int u, int tbl_len) {
    const int c = replay_class(u, tbl_len);
    if (c == kClassL) return (long long)kListsPerGroup * u;
    if (c == kClassXL) return (long long)kListsPerGroup * u + tbl_len;
    return 0;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_max(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

// ---- teams -------------------------------------------------------------------
struct WarpTeam {
    static constexpr int kSize = 32;
    static constexpr int kPerBlock = 8;
    __device__ static int tid() { return threadIdx.x & 31; }
    __device__ static int index_in_block() { return threadIdx.x >> 5; }
    __device__ static void sync() { __syncwarp(); }
    __device__ static bool any(bool p, int*) { return __any_sync(0xffffffffu, p); }
    __device__ static int sum(int v, int*) { return warp_sum(v); }
    __device__ static int max_of(int v, int*) { return warp_max(v); }
    __device__ static int broadcast(int v, int*) { return __shfl_sync(0xffffffffu, v, 0); }   // value of thread 0
    // rank of this thread among the flagged threads of the team, in thread order
    __device__ static int rank(bool flag, int& total, int*) {
        const unsigned b = __ballot_sync(0xffffffffu, flag);
        total = __popc(b);
        return __popc(b & ((1u << (threadIdx.x & 31)) - 1u));
    }
};

template <int THREADS>
struct BlockTeam {
    static constexpr int kSize = THREADS;
    static constexpr int kPerBlock = 1;
    __device__ static int tid() { return threadIdx.x; }
    __device__ static int index_in_block() { return 0; }
    __device__ static void sync() { __syncthreads(); }
    __device__ static bool any(bool p, int*) { return __syncthreads_or(p ? 1 : 0) != 0; }
    __device__ static int sum(int v, int* scratch) {            // scratch: 33 ints of shared memory
        v = warp_sum(v);
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
        __syncthreads();
        int t = 0;
        for (int w = 0; w < THREADS / 32; ++w) t += scratch[w];
        __syncthreads();
        return t;
    }
    __device__ static int max_of(int v, int* scratch) {
        v = warp_max(v);
        if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
        __syncthreads();
        int t = scratch[0];
        for (int w = 1; w < THREADS / 32; ++w) t = max(t, scratch[w]);
        __syncthreads();
        return t;
    }
    __device__ static int broadcast(int v, int* scratch) {     // value of thread 0
        if (threadIdx.x == 0) scratch[32] = v;
        __syncthreads();
        const int r = scratch[32];
        __syncthreads();
        return r;
    }
    // exclusive prefix sum of v over the threads of the block, in thread order
    __device__ static int scan_exclusive(int v, int& total, int* scratch) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int inc = warp_incl_scan(v, lane);
        if (lane == 31) scratch[warp] = inc;
        __syncthreads();
        int before = 0, all = 0;
        for (int w = 0; w < THREADS / 32; ++w) {
            const int c = scratch[w];
            if (w < warp) before += c;
            all += c;
        }
        __syncthreads();
        total = all;
        return before + inc - v;
    }
    __device__ static int rank(bool flag, int& total, int* scratch) {
        const unsigned b = __ballot_sync(0xffffffffu, flag);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        if (lane == 0) scratch[warp] = __popc(b);
        __syncthreads();
        int before = 0, all = 0;
        for (int w = 0; w < THREADS / 32; ++w) {
            const int c = scratch[w];
            if (w < warp) before += c;
            all += c;
        }
        __syncthreads();
        total = all;
        return before + __popc(b & ((1u << lane) - 1u));
    }
};

// Groups with many entries get a whole CTA, the others a warp: two launches of the same kernel,
// each taking the groups that pass its filter (0 = all, 1 = at most kBigGroup entries, 2 = more).
constexpr int kBigGroup = 1024;
__device__ __forceinline__ bool group_passes(int filter, int entries) {
    return filter == 0 || (filter == 1) == (entries <= kBigGroup);
}

// ---------------------------------------------------------------- pass 1: count
template <class Team>
__global__ void __launch_bounds__(256)
svc_count_kernel(SvcProblem p, int words, int filter, int* __restrict__ counts, int* __restrict__ mode,
                 int* __restrict__ tbl_len) {
    extern __shared__ unsigned int sm_words[];
    __shared__ int red[33];
    unsigned int* bm = sm_words + (size_t)Team::index_in_block() * words;
    const int tid = Team::tid();
    for (int i = blockIdx.x * Team::kPerBlock + Team::index_in_block(); i < p.m_vec; i += gridDim.x * Team::kPerBlock) {
        const int r0 = min(i * p.V, p.M), r1 = min(i * p.V + p.V, p.M);
        const int e0 = p.row_ptr[r0], e1 = p.row_ptr[r1];
        if (!group_passes(filter, e1 - e0)) continue;
        if (e1 - e0 < words) {
            for (int e = e0 + tid; e < e1; e += Team::kSize) {
                const unsigned c = (unsigned)p.col_idx[e];
                if (c < (unsigned)p.K) bm[c >> 5] = 0u;
            }
        } else {
            for (int w = tid; w < words; w += Team::kSize) bm[w] = 0u;
        }
        Team::sync();
        int cnt = 0, mx = -1, bad = 0;
        for (int e = e0 + tid; e < e1; e += Team::kSize) {
            const int c = p.col_idx[e];
            if ((unsigned)c < (unsigned)p.K) {
                const unsigned bit = 1u << (c & 31);
                const unsigned old = atomicOr(&bm[c >> 5], bit);
                cnt += (old & bit) ? 0 : 1;
                mx = max(mx, c);
            } else {
                bad = 1;
            }
        }
        cnt = Team::sum(cnt, red);
        mx = Team::max_of(mx, red);
        bad = Team::max_of(bad, red);
        if (tid == 0) {
            counts[i] = cnt;
            const int len = final_table_len(cnt);
            const int replay = (mx >= len) ? 1 : 0;
            mode[i] = replay;
            tbl_len[i] = replay ? len : ((e1 - e0) > kBigGroup ? -1 : 0);     // -1: ascending order, and large enough for a CTA
            if (bad) g_svc_bad_column = 1;
        }
        Team::sync();
    }
}

// ---------------------------------------------------------------- scans
// Exclusive scans over the groups (vector row pointers from the counts, scratch offsets) and the lists of replayed
// groups per class, in three small launches: per-block sums, a scan of the block sums by one CTA, and the final
// positions.  A block covers kScanBlock groups; a block sum is kScanFields numbers: vectors, scratch ints, and
// the groups of each replay class.
// totals: [0] nvec, [1] scratch ints, [2..2+kNumSegs) groups per list segment, then the bad-column flag
constexpr int kScanThreads = 1024;
constexpr int kScanPerThread = 4;
constexpr int kScanBlock = kScanThreads * kScanPerThread;
constexpr int kScanFields = 2 + kNumSegs;
static_assert(kScanFields == kSvcScanFields, "scan fields");

// Sums `v` over the block; the result is valid in every thread.  sh: 32 long longs.
__device__ __forceinline__ long long block_sum_ll(long long v, long long* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    long long t = 0;
    for (int w = 0; w < kScanThreads / 32; ++w) t += sh[w];
    __syncthreads();
    return t;
}
// Exclusive prefix of `v` over the threads of the block, in thread order.  sh: 32 long longs.
__device__ __forceinline__ long long block_prefix_ll(long long v, long long* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const long long t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) sh[warp] = inc;
    __syncthreads();
    long long before = 0;
    for (int w = 0; w < warp; ++w) before += sh[w];
    __syncthreads();
    return before + inc - v;
}

__global__ void __launch_bounds__(kScanThreads)
svc_scan_sums_kernel(int m_vec, const int* __restrict__ counts, const int* __restrict__ tbl_len,
                     long long* __restrict__ block_sums) {
    __shared__ long long sh[32];
    long long f[kScanFields];
#pragma unroll
    for (int k = 0; k < kScanFields; ++k) f[k] = 0;
    const int first = blockIdx.x * kScanBlock + threadIdx.x * kScanPerThread;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
        const int i = first + j;
        if (i >= m_vec) break;
        const int u = counts[i], len = tbl_len[i];
        f[0] += u;
        f[1] += group_scratch_ints(u, len);
        const int c = list_segment(u, len);
#pragma unroll
        for (int k = 0; k < kNumSegs; ++k) f[2 + k] += (c == k) ? 1 : 0;
    }
#pragma unroll
    for (int k = 0; k < kScanFields; ++k) {
        const long long t = block_sum_ll(f[k], sh);
        if (threadIdx.x == 0) block_sums[(size_t)blockIdx.x * kScanFields + k] = t;
    }
}

// One CTA: block_sums -> exclusive prefixes in place, and the totals.
__global__ void __launch_bounds__(kScanThreads)
svc_scan_blocks_kernel(int n_blocks, long long* __restrict__ block_sums, long long* __restrict__ totals) {
    __shared__ long long sh[32];
    __shared__ long long carry[kScanFields];
    if (threadIdx.x < kScanFields) carry[threadIdx.x] = 0;
    __syncthreads();
    for (int b0 = 0; b0 < n_blocks; b0 += kScanThreads) {
        const int b = b0 + threadIdx.x;
        for (int k = 0; k < kScanFields; ++k) {
            const long long v = (b < n_blocks) ? block_sums[(size_t)b * kScanFields + k] : 0;
            const long long ex = block_prefix_ll(v, sh);
            const long long c0 = carry[k];
            if (b < n_blocks) block_sums[(size_t)b * kScanFields + k] = c0 + ex;
            __syncthreads();
            if (threadIdx.x == kScanThreads - 1) carry[k] = c0 + ex + v;
            __syncthreads();
        }
    }
    if (threadIdx.x == 0) {
        for (int k = 0; k < kScanFields; ++k) totals[k] = carry[k];
        totals[kScanFields] = g_svc_bad_column;          // reported with the totals, then cleared
        g_svc_bad_column = 0;
    }
}

// vec_ptr: counts in, exclusive scan out (and the total at [m_vec]); tbl_off: scratch offsets; class_list: the
// replayed groups segment by segment (see list_segment), inside a segment in ascending order.
__global__ void __launch_bounds__(kScanThreads)
svc_scan_place_kernel(int m_vec, int* __restrict__ vec_ptr, const int* __restrict__ tbl_len,
                      long long* __restrict__ tbl_off, const long long* __restrict__ block_sums,
                      const long long* __restrict__ totals, int* __restrict__ class_list) {
    __shared__ long long sh[32];
    const int first = blockIdx.x * kScanBlock + threadIdx.x * kScanPerThread;
    int u[kScanPerThread], cls[kScanPerThread];
    long long scr[kScanPerThread];
    long long f[kScanFields];
#pragma unroll
    for (int k = 0; k < kScanFields; ++k) f[k] = 0;
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
        const int i = first + j;
        u[j] = 0; scr[j] = 0; cls[j] = -1;
        if (i < m_vec) {
            u[j] = vec_ptr[i];
            const int len = tbl_len[i];
            scr[j] = group_scratch_ints(u[j], len);
            cls[j] = list_segment(u[j], len);
            f[0] += u[j];
            f[1] += scr[j];
#pragma unroll
            for (int k = 0; k < kNumSegs; ++k) f[2 + k] += (cls[j] == k) ? 1 : 0;
        }
    }
    // where segment k starts in the list: after all groups of the segments before it (segment 0 is not replayed)
    long long at[kScanFields];
#pragma unroll
    for (int k = 0; k < kScanFields; ++k)
        at[k] = block_sums[(size_t)blockIdx.x * kScanFields + k] + block_prefix_ll(f[k], sh);
    long long class_base = 0;
#pragma unroll
    for (int k = 1; k < kNumSegs; ++k) {
        at[2 + k] += class_base;
        class_base += totals[2 + k];
    }
#pragma unroll
    for (int j = 0; j < kScanPerThread; ++j) {
        const int i = first + j;
        if (i >= m_vec) break;
        vec_ptr[i] = (int)at[0];
        tbl_off[i] = at[1];
        at[0] += u[j];
        at[1] += scr[j];
#pragma unroll
        for (int k = 1; k < kNumSegs; ++k)
            if (cls[j] == k) class_list[at[2 + k]++] = i;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        vec_ptr[m_vec] = (int)totals[0];
        tbl_off[m_vec] = totals[1];
    }
}

// ---------------------------------------------------------------- pass 2a: ascending order
template <class Team>
__global__ void __launch_bounds__(256)
svc_emit_sorted_kernel(SvcProblem p, int words, int filter, const int* __restrict__ vec_ptr,
                       const int* __restrict__ mode, int* __restrict__ out_col, __half* __restrict__ out_vals,
                       const int* __restrict__ list, int n_list) {
    extern __shared__ unsigned int sm_words[];
    __shared__ int red[33];
    unsigned int* bm = sm_words + (size_t)Team::index_in_block() * words * 2;
    unsigned int* pre = bm + words;
    const int tid = Team::tid();
    // with a list: only the groups it names; else every group
    const int n_loop = list ? n_list : p.m_vec;
    for (int k = blockIdx.x * Team::kPerBlock + Team::index_in_block(); k < n_loop; k += gridDim.x * Team::kPerBlock) {
        const int i = list ? list[k] : k;
        if (mode[i] != 0) continue;
        const int r0 = min(i * p.V, p.M), r1 = min(i * p.V + p.V, p.M);
        const int e0 = p.row_ptr[r0], e1 = p.row_ptr[r1];
        const int base = vec_ptr[i];
        if (e1 == e0 || !group_passes(filter, e1 - e0)) continue;
        for (int w = tid; w < words; w += Team::kSize) bm[w] = 0u;
        Team::sync();
        for (int e = e0 + tid; e < e1; e += Team::kSize) {
            const int c = p.col_idx[e];
            if ((unsigned)c < (unsigned)p.K) atomicOr(&bm[c >> 5], 1u << (c & 31));
        }
        Team::sync();
        int running = 0;
        for (int w0 = 0; w0 < words; w0 += Team::kSize) {
            const int w = w0 + tid;
            unsigned word = (w < words) ? bm[w] : 0u;
            const int pc = __popc(word);
            // exclusive prefix of pc over the team, in thread order
            int incl = warp_incl_scan(pc, tid & 31);
            int chunk_total;
            if constexpr (Team::kSize == 32) {
                chunk_total = __shfl_sync(0xffffffffu, incl, 31);
            } else {
                const int wp = tid >> 5;
                if ((tid & 31) == 31) red[wp] = incl;
                __syncthreads();
                int before = 0, all = 0;
                for (int x = 0; x < Team::kSize / 32; ++x) {
                    const int c = red[x];
                    if (x < wp) before += c;
                    all += c;
                }
                __syncthreads();
                incl += before;
                chunk_total = all;
            }
            int o = running + incl - pc;
            if (w < words) pre[w] = (unsigned)o;
            o += base;
            while (word) {
                const int b = __ffs(word) - 1;
                out_col[o++] = w * 32 + b;
                word &= word - 1;
            }
            running += chunk_total;
        }
        if (out_vals) {
            Team::sync();
            // all entries of the group, flat; the matrix row of entry e is found by walking the (at most V) row ends
            for (int e = e0 + tid; e < e1; e += Team::kSize) {
                int r = r0;
                while (r + 1 < r1 && e >= p.row_ptr[r + 1]) ++r;
                const int c = p.col_idx[e];
                if ((unsigned)c < (unsigned)p.K) {
                    const int pos = (int)pre[c >> 5] + __popc(bm[c >> 5] & ((1u << (c & 31)) - 1u));
                    out_vals[((int64_t)base + pos) * p.V + (r - i * p.V)] = p.vals[e];
                }
            }
        }
        Team::sync();
    }
}

// ---------------------------------------------------------------- pass 2b: hash-table replay
struct Probe {            // position on a key's probe path
    unsigned i;           // start of the current window
    unsigned w;           // offset inside the window
    unsigned perturb;
};
__device__ __forceinline__ Probe probe_begin(int key, unsigned mask) {
    Probe p;
    p.i = (unsigned)key & mask; p.w = 0; p.perturb = (unsigned)key;
    return p;
}
// Returns true when the step was a jump to a new window.
__device__ __forceinline__ bool probe_advance(Probe& p, unsigned mask) {
    const unsigned window = (p.i + kLinearProbes <= mask) ? kLinearProbes : 0;
    if (p.w < window) {
        ++p.w;
        return false;
    }
    p.perturb >>= kPerturbShift;
    p.i = (p.i * 5u + 1u + p.perturb) & mask;
    p.w = 0;
    return true;
}
// Table of KEYS (-1 = free): slot holding `key`, or -1 when the path reaches a free slot first.
// Every probe loop is bounded (a table is never more than 60 % full, so a free slot is near).
__device__ __forceinline__ int find_key(const int* tab, unsigned mask, int key) {
    Probe p = probe_begin(key, mask);
    for (unsigned n = 0; n <= 8u * mask + 64u; ++n) {
        const int e = tab[p.i + p.w];
        if (e == key) return (int)(p.i + p.w);
        if (e == -1) return -1;
        probe_advance(p, mask);
    }
    return -1;
}
// Same, returning the first free slot when the key is absent (sequential insertion).
__device__ __forceinline__ int find_slot(const int* tab, unsigned mask, int key) {
    Probe p = probe_begin(key, mask);
    for (unsigned n = 0; n <= 8u * mask + 64u; ++n) {
        const int e = tab[p.i + p.w];
        if (e == key || e == -1) return (int)(p.i + p.w);
        probe_advance(p, mask);
    }
    return (int)(p.i + p.w);
}

struct ReplayBuffers {
    int* table;      // cap ints
    int* lists[4];   // lists of u ints: X2 (alternates with the output slice as the ordered list), NEW, P, Q
    int* seq_local;  // non-null: u ints of shared memory that hold the insertion sequence of the current level
                     // (the lists are then in global memory and are only streamed through)
};

// Ordered extraction: keys of `tab` in slot order into dst; returns how many.  With seq != null the
// table holds sequence numbers (kEmptyPrio = free) and is rewritten in place to hold keys (-1 = free).
template <class Team>
__device__ int extract_ordered(int* tab, int size, const int* seq, int* dst, int* red) {
    const int tid = Team::tid();
    if constexpr (Team::kSize >= 256) {
        // Large table, CTA team: every warp owns a contiguous run of size / warps slots and walks it 32
        // slots at a time (one ballot gives the occupancy of a row), so the whole table needs one prefix sum
        // over warp totals instead of a block-wide one per kSize slots, and the key lookups of four rows
        // are in flight together.
        if (size >= Team::kSize) {
            const int lane = tid & 31, warp = tid >> 5;
            const int rows = size / Team::kSize;                    // rows of 32 slots per warp
            const int first = warp * rows * 32 + lane;
            int cnt = 0;
            for (int j = 0; j < rows; ++j) {
                const int e = tab[first + j * 32];
                cnt += __popc(__ballot_sync(0xffffffffu, seq ? (e != kEmptyPrio) : (e != -1)));
            }
            if (lane == 0) red[warp] = cnt;
            Team::sync();
            int pos = 0, total = 0;
            for (int w = 0; w < Team::kSize / 32; ++w) {
                const int c = red[w];
                if (w < warp) pos += c;
                total += c;
            }
            Team::sync();
            for (int j0 = 0; j0 < rows; j0 += 4) {
                int e4[4], k4[4];
                bool f4[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    e4[b] = (j0 + b < rows) ? tab[first + (j0 + b) * 32] : (seq ? kEmptyPrio : -1);
                    f4[b] = seq ? (e4[b] != kEmptyPrio) : (e4[b] != -1);
                }
#pragma unroll
                for (int b = 0; b < 4; ++b) k4[b] = f4[b] ? (seq ? seq[e4[b]] : e4[b]) : -1;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    if (j0 + b < rows) {
                        const unsigned m = __ballot_sync(0xffffffffu, f4[b]);
                        if (f4[b]) dst[pos + __popc(m & ((1u << lane) - 1u))] = k4[b];
                        if (seq) tab[first + (j0 + b) * 32] = k4[b];
                        pos += __popc(m);
                    }
                }
            }
            Team::sync();
            return total;
        }
    }
    int n = 0;
    for (int s0 = 0; s0 < size; s0 += Team::kSize) {
        const int s = s0 + tid;
        int key = -1;
        if (s < size) {
            const int e = tab[s];
            if (seq) {
                key = (e == kEmptyPrio) ? -1 : seq[e];
                tab[s] = key;
            } else {
                key = e;
            }
        }
        int total;
        const int rk = Team::rank(key != -1, total, red);
        if (key != -1) dst[n + rk] = key;
        n += total;
    }
    Team::sync();
    return n;
}

// Sequential replay by one thread (used when a matrix row lists a column twice; rare).  tab holds keys.
__device__ int replay_sequential(const SvcProblem& p, int r0, int r1, int* tab, int cap, int* xa, int* xb, int* tmp) {
    int n_cur = 0;
    int* x = xa;
    int* xn = xb;
    unsigned mask = kMinTable - 1;
    for (int r = r0; r < r1; ++r) {
        const int rs = p.row_ptr[r], rlen = p.row_ptr[r + 1] - rs;
        int size = kMinTable, used = 0;
        mask = kMinTable - 1;
        for (int s = 0; s < size; ++s) tab[s] = -1;
        for (int t = 0; t < n_cur + rlen; ++t) {
            const int key = (t < n_cur) ? x[t] : p.col_idx[rs + t - n_cur];
            if ((unsigned)key >= (unsigned)p.K) continue;
            const int s = find_slot(tab, mask, key);
            if (tab[s] == key) continue;
            tab[s] = key;
            ++used;
            if ((long long)used * 5 >= (long long)mask * 3) {
                long long trig; int nsize;
                next_level(size, trig, nsize);
                if (nsize > cap) nsize = cap;
                int cnt = 0;
                for (int q = 0; q < size; ++q) if (tab[q] != -1) tmp[cnt++] = tab[q];
                for (int q = 0; q < nsize; ++q) tab[q] = -1;
                const unsigned nmask = (unsigned)nsize - 1u;
                for (int q = 0; q < cnt; ++q) tab[find_slot(tab, nmask, tmp[q])] = tmp[q];
                size = nsize; mask = nmask;
            }
        }
        int cnt = 0;
        for (int q = 0; q < size; ++q) if (tab[q] != -1) xn[cnt++] = tab[q];
        n_cur = cnt;
        int* t2 = x; x = xn; xn = t2;
    }
    return (int)mask;      // the ordered list is in `x` = xa if (r1-r0) is even else xb; caller arranges parity
}

template <class Team>
__device__ void replay_group(const SvcProblem& p, int i, int u_final, int cap, int base, ReplayBuffers bufs,
                             int* __restrict__ out_col, __half* __restrict__ out_vals, int* red) {
    const int tid = Team::tid();
    const int r0 = min(i * p.V, p.M), r1 = min(i * p.V + p.V, p.M);
    const int n_rebuilds = r1 - r0;
    int* const tab = bufs.table;
    // the ordered list alternates between two buffers; arrange that the last rebuild writes the output slice
    int* const out_slice = out_col + base;
    int* x = (n_rebuilds & 1) ? bufs.lists[0] : out_slice;      // list before the first rebuild (empty)
    int* xn = (n_rebuilds & 1) ? out_slice : bufs.lists[0];     // written by the first rebuild
    int* const fresh = bufs.lists[1];                           // NEW: columns of the row not yet in the set
    // insertion sequence of the current level, and the list the next level's head is extracted into: two lists
    // that swap roles, or (seq_local) a fixed shared-memory sequence refilled from one extraction list
    int* seq = bufs.seq_local ? bufs.seq_local : bufs.lists[2];
    int* ext = bufs.seq_local ? bufs.lists[2] : bufs.lists[3];

    int n_cur = 0;
    unsigned mask_prev = kMinTable - 1;
    if (tid < kMinTable) tab[tid] = -1;
    Team::sync();
    bool duplicate = false;

    for (int r = r0; r < r1 && !duplicate; ++r) {
        const int rs = p.row_ptr[r], rlen = p.row_ptr[r + 1] - rs;
        // ---- columns of this row that are not in the current set, in row order
        int n_new = 0;
        for (int t0 = 0; t0 < rlen; t0 += Team::kSize) {
            const int t = t0 + tid;
            const int key = (t < rlen) ? p.col_idx[rs + t] : -1;
            const bool isnew = (t < rlen) && (unsigned)key < (unsigned)p.K && find_key(tab, mask_prev, key) < 0;
            int total;
            const int rk = Team::rank(isnew, total, red);
            if (isnew && n_cur + n_new + rk < u_final) fresh[n_new + rk] = key;
            n_new += total;
        }
        Team::sync();
        const int n_total = n_cur + n_new;
        if (n_total > u_final) { duplicate = true; break; }     // only possible when the row repeats a column

        // ---- replay  set(list)  for the sequence  D = x[0..n_cur) ++ fresh[0..n_new), level by level.
        // Inside a level the table length is fixed and insertion is first come, first served: an element
        // takes a slot with atomicMin on its sequence number; if that displaces a later element, the same
        // thread carries the displaced element on from the slot it had recorded, so one pass settles all.
        int size = kMinTable, e_len = 0;
        unsigned mask = kMinTable - 1;
        for (;;) {
            long long trig_ll; int next_size;
            next_level(size, trig_ll, next_size);
            const int trig = (int)(trig_ll > 0x7fffffff ? 0x7fffffff : trig_ll);
            const int n_l = min(trig, n_total);
            mask = (unsigned)size - 1u;
            if (size >= 4 * Team::kSize) {
                const int4 fill = make_int4(kEmptyPrio, kEmptyPrio, kEmptyPrio, kEmptyPrio);
                int4* t4 = reinterpret_cast<int4*>(tab);
                for (int s = tid; s < size / 4; s += Team::kSize) t4[s] = fill;
            } else {
                for (int s = tid; s < size; s += Team::kSize) tab[s] = kEmptyPrio;
            }
            if (bufs.seq_local)                                                  // head of the sequence: last level's table order
                for (int q = tid; q < e_len; q += Team::kSize) seq[q] = ext[q];
            for (int q = e_len + tid; q < n_l; q += 4 * Team::kSize) {          // four loads in flight
                int v4[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int qq = q + b * Team::kSize;
                    v4[b] = (qq < n_l) ? ((qq < n_cur) ? x[qq] : fresh[qq - n_cur]) : 0;
                }
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    if (q + b * Team::kSize < n_l) seq[q + b * Team::kSize] = v4[b];
            }
            Team::sync();
            const int first_new = max(e_len, n_cur);
            bool dup_here = false;          // also raised when a bound is hit: the group is then redone sequentially
            volatile int* vtab = tab;
            for (int q4 = tid; q4 < n_l && !dup_here; q4 += 4 * Team::kSize) {
              int k4[4];
#pragma unroll
              for (int b = 0; b < 4; ++b) k4[b] = (q4 + b * Team::kSize < n_l) ? seq[q4 + b * Team::kSize] : 0;
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const int q = q4 + b * Team::kSize;
                if (q >= n_l || dup_here) break;
                int e = q, key = k4[b];
                Probe pr = probe_begin(key, mask);
                for (unsigned tries = 0;; ++tries) {
                    const int slot = (int)(pr.i + pr.w);
                    // Slot values only ever decrease during a level, so a slot seen with an earlier element stays
                    // out of reach; only a slot that looks free or later is worth the atomic.
                    int cur = vtab[slot];
                    if (cur > e) cur = atomicMin(&tab[slot], e);
                    if (cur > e) {
                        if (cur == kEmptyPrio) break;            // free slot taken: this chain ends
                        // a later element sat here: the same thread carries it on, from the start of its own path
                        // (every slot it passed before still holds an earlier element, so it walks to the same
                        // place and beyond)
                        e = cur;
                        key = seq[e];
                        pr = probe_begin(key, mask);
                        continue;
                    }
                    if ((e >= first_new && seq[cur] == key) || tries > 16u * mask + 256u) {
                        dup_here = true;
                        break;
                    }
                    probe_advance(pr, mask);
                }
              }
            }
            Team::sync();
            if (Team::any(dup_here, red)) { duplicate = true; break; }
            if (n_total < trig) {
                // no further growth: this table is final; keys in place, ordered list out
                n_cur = extract_ordered<Team>(tab, size, seq, xn, red);
                break;
            }
            e_len = extract_ordered<Team>(tab, size, seq, ext, red);
            if (!bufs.seq_local) { int* t3 = seq; seq = ext; ext = t3; }
            size = (next_size > cap) ? cap : next_size;
        }
        if (duplicate) break;
        int* t2 = x; x = xn; xn = t2;
        mask_prev = mask;
    }

    if (duplicate) {
        // rare: fall back to the sequential replay of the whole group by one thread
        int* xa = (n_rebuilds & 1) ? bufs.lists[0] : out_slice;
        int* xb = (n_rebuilds & 1) ? out_slice : bufs.lists[0];
        int m = 0;
        if (tid == 0) m = replay_sequential(p, r0, r1, tab, cap, xa, xb, bufs.lists[2]);
        Team::sync();
        mask_prev = (unsigned)Team::max_of(m, red);
        n_cur = u_final;
    }
    // here: out_slice holds the ordered list, tab holds its keys at their slots
    if (out_vals && n_cur > 0) {
        const int size = (int)mask_prev + 1;
        // a list that is free by now (the group is finished with its sequences)
        unsigned* const state = reinterpret_cast<unsigned*>(bufs.seq_local ? bufs.seq_local : bufs.lists[1]);
        int n = 0;
        for (int s0 = 0; s0 < size; s0 += Team::kSize) {        // slot -> position
            const int s = s0 + tid;
            const int key = (s < size) ? tab[s] : -1;
            int total;
            const int rk = Team::rank(key != -1, total, red);
            if (key != -1) state[n + rk] = (unsigned)s;          // position -> slot (ascending), searched below
            n += total;
        }
        Team::sync();
        const int e0 = p.row_ptr[r0], e1 = p.row_ptr[r1];
        for (int e = e0 + tid; e < e1; e += Team::kSize) {
            int r = r0;
            while (r + 1 < r1 && e >= p.row_ptr[r + 1]) ++r;
            const int c = p.col_idx[e];
            if ((unsigned)c >= (unsigned)p.K) continue;
            const int s = find_key(tab, mask_prev, c);
            if (s < 0) continue;
            // position of slot s = number of occupied slots before it: binary search in the slot list
            int lo = 0, hi = n - 1;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if ((int)state[mid] < s) lo = mid + 1; else hi = mid;
            }
            out_vals[((int64_t)base + lo) * p.V + (r - i * p.V)] = p.vals[e];
        }
    }
    Team::sync();
}

template <class Team, int CLASS>
__global__ void __launch_bounds__(Team::kSize * Team::kPerBlock,
                                  ((CLASS == kClassM1 || CLASS == kClassXS) ? 1536 : 1024) / (Team::kSize * Team::kPerBlock))
svc_emit_replay_kernel(SvcProblem p, const int* __restrict__ vec_ptr, const int* __restrict__ tbl_len,
                       const long long* __restrict__ tbl_off, int* __restrict__ scratch, int* __restrict__ out_col,
                       __half* __restrict__ out_vals, int smem_table_ints, int smem_list_ints,
                       const int* __restrict__ groups, int n_groups, int* __restrict__ queue) {
    extern __shared__ int sm_ints[];
    __shared__ int red[34];
    const int per_team = smem_table_ints + kListsPerGroup * smem_list_ints;
    int* mine = sm_ints + (size_t)Team::index_in_block() * per_team;
    for (;;) {
        int k = 0;
        if (Team::tid() == 0) k = atomicAdd(queue, 1);
        k = Team::broadcast(k, red);
        if (k >= n_groups) break;
        const int i = groups[k];
        const int base = vec_ptr[i];
        const int u = vec_ptr[i + 1] - base;
        const int cap = tbl_len[i];
        ReplayBuffers b;
        b.seq_local = nullptr;
        if (CLASS == kClassXS || CLASS == kClassS || CLASS == kClassM1 || CLASS == kClassM2) {
            b.table = mine;
            for (int l = 0; l < kListsPerGroup; ++l) b.lists[l] = mine + smem_table_ints + l * smem_list_ints;
        } else {
            int* g = scratch + tbl_off[i];
            for (int l = 0; l < kListsPerGroup; ++l) b.lists[l] = g + (size_t)l * u;
            b.table = (CLASS == kClassL) ? mine : g + (size_t)kListsPerGroup * u;
            if (CLASS == kClassL) b.seq_local = mine + smem_table_ints;
        }
        replay_group<Team>(p, i, u, cap, base, b, out_col, out_vals, red);
    }
}

int device_sm_count() { return current_device_sm_count(); }

// Side streams so that launches working on disjoint groups overlap (fork from / join into the caller's stream).
constexpr int kAuxStreams = 6;
struct Aux {
    cudaStream_t stream[kAuxStreams];
    cudaEvent_t fork, join[kAuxStreams];
    bool ready = false;
};
std::mutex g_aux_mu;                 // serialises enqueueing through the shared events
Aux g_aux[64];

Aux* aux_for_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    Aux& a = g_aux[dev];
    if (!a.ready) {
        for (int k = 0; k < kAuxStreams; ++k) {
            if (cudaStreamCreateWithFlags(&a.stream[k], cudaStreamNonBlocking) != cudaSuccess) return nullptr;
            if (cudaEventCreateWithFlags(&a.join[k], cudaEventDisableTiming) != cudaSuccess) return nullptr;
        }
        if (cudaEventCreateWithFlags(&a.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        a.ready = true;
    }
    return &a;
}

struct Fork {
    Aux* aux;
    cudaStream_t main;
    int used = 0;
    cudaError_t err = cudaSuccess;
    Fork(Aux* a, cudaStream_t m) : aux(a), main(m) {
        if (aux) err = cudaEventRecord(aux->fork, main);
    }
    // stream for the next independent launch (the caller's stream when side streams are unavailable)
    cudaStream_t next() {
        if (!aux || used >= kAuxStreams || err != cudaSuccess) return main;
        cudaStream_t s = aux->stream[used++];
        err = cudaStreamWaitEvent(s, aux->fork, 0);
        return err == cudaSuccess ? s : main;
    }
    cudaError_t join() {
        if (!aux) return err;
        for (int k = 0; k < used && err == cudaSuccess; ++k) {
            err = cudaEventRecord(aux->join[k], aux->stream[k]);
            if (err == cudaSuccess) err = cudaStreamWaitEvent(main, aux->join[k], 0);
        }
        return err;
    }
};

template <class Team, int CLASS>
cudaError_t launch_replay(const SvcProblem& p, const SvcScratch& s, int* out_col, __half* out_vals, long long groups,
                          long long first, int table_ints, int list_ints, cudaStream_t stream) {
    if (groups <= 0) return cudaSuccess;
    auto kern = svc_emit_replay_kernel<Team, CLASS>;
    const size_t smem = ((size_t)Team::kPerBlock * (table_ints + (size_t)kListsPerGroup * list_ints) +
                         (CLASS == kClassL ? kLSeqInts : 0)) * sizeof(int);
    static DeviceOnce once;
    if (!once.done()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // without this the driver may size the shared-memory carve-out for a single resident block
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        once.mark();
    }
    const int sms = device_sm_count();
    long long want = (groups + Team::kPerBlock - 1) / Team::kPerBlock;
    // as many blocks as can be resident: the groups are handed out through the class's work counter
    const long long cap_blocks = (long long)sms * (smem > 113 * 1024 ? 1 : (smem > 75 * 1024 ? 2 : (smem > 56 * 1024 ? 3 : (smem > 45 * 1024 ? 4 : (smem > 28 * 1024 ? 6 : 8)))));
    int grid = (int)(want < cap_blocks ? want : cap_blocks);
    if (grid < 1) grid = 1;
    kern<<<grid, Team::kSize * Team::kPerBlock, smem, stream>>>(p, s.vec_ptr, s.tbl_len, s.tbl_off, s.tables, out_col,
                                                                 out_vals, table_ints, list_ints, s.class_list + first,
                                                                 (int)groups, s.queue + CLASS);
    return cudaGetLastError();
}

template <class Kern>
cudaError_t allow_big_smem(Kern kern, DeviceOnce& once, int bytes) {
    if (once.done()) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) once.mark();
    return e;
}

}  // namespace

cudaError_t svc_count_and_scan(const SvcProblem& p, const SvcScratch& s, bool /*with_values*/, cudaStream_t stream) {
    if (p.m_vec > 0) {
        const int words = (p.K + 31) / 32;
        const int sms = device_sm_count();
        static DeviceOnce once_block, once_warp;
        cudaError_t e = allow_big_smem(svc_count_kernel<BlockTeam<256>>, once_block, 200 * 1024);
        if (e == cudaSuccess) e = allow_big_smem(svc_count_kernel<WarpTeam>, once_warp, 200 * 1024);
        if (e != cudaSuccess) return e;
        const size_t warp_smem = (size_t)WarpTeam::kPerBlock * words * 4;
        if (p.m_vec <= 16 * sms || warp_smem > 200 * 1024) {
            // few groups (or bitmaps too large for eight per block): one CTA per group
            const int grid = p.m_vec < sms * 16 ? p.m_vec : sms * 16;
            svc_count_kernel<BlockTeam<256>><<<grid, 256, (size_t)words * 4, stream>>>(p, words, 0, s.vec_ptr, s.mode, s.tbl_len);
            e = cudaGetLastError();
        } else {
            std::lock_guard<std::mutex> lk(g_aux_mu);
            Fork f(aux_for_device(), stream);
            int grid = (p.m_vec + WarpTeam::kPerBlock - 1) / WarpTeam::kPerBlock;
            if (grid > sms * 8) grid = sms * 8;
            svc_count_kernel<WarpTeam><<<grid, 256, warp_smem, f.next()>>>(p, words, 1, s.vec_ptr, s.mode, s.tbl_len);
            svc_count_kernel<BlockTeam<256>><<<sms * 4, 256, (size_t)words * 4, f.next()>>>(p, words, 2, s.vec_ptr, s.mode, s.tbl_len);
            e = cudaGetLastError();
            if (e == cudaSuccess) e = f.join();
        }
        if (e != cudaSuccess) return e;
    }
    const int n_blocks = p.m_vec > 0 ? (p.m_vec + kScanBlock - 1) / kScanBlock : 1;
    svc_scan_sums_kernel<<<n_blocks, kScanThreads, 0, stream>>>(p.m_vec, s.vec_ptr, s.tbl_len, s.block_sums);
    svc_scan_blocks_kernel<<<1, kScanThreads, 0, stream>>>(n_blocks, s.block_sums, s.totals);
    svc_scan_place_kernel<<<n_blocks, kScanThreads, 0, stream>>>(p.m_vec, s.vec_ptr, s.tbl_len, s.tbl_off, s.block_sums, s.totals,
                                                                 s.class_list);
    return cudaGetLastError();
}

cudaError_t svc_emit(const SvcProblem& p, const SvcScratch& s, const long long* seg_groups, int* out_col,
                     __half* out_vals, cudaStream_t stream) {
    if (p.m_vec == 0) return cudaSuccess;
    const int sms = device_sm_count();
    const int words = (p.K + 31) / 32;
    static DeviceOnce once_block, once_warp;
    cudaError_t e = allow_big_smem(svc_emit_sorted_kernel<BlockTeam<256>>, once_block, 208 * 1024);
    if (e == cudaSuccess) e = allow_big_smem(svc_emit_sorted_kernel<WarpTeam>, once_warp, 208 * 1024);
    if (e != cudaSuccess) return e;

    // the work counters of the replay classes, cleared before the side streams fork off
    e = cudaMemsetAsync(s.queue, 0, 8 * sizeof(int), stream);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lk(g_aux_mu);
    Fork f(aux_for_device(), stream);
    // groups per class and where the class starts in the list of replayed groups
    long long class_groups[kNumClasses] = {0}, first[kNumClasses] = {0};
    class_groups[kClassSorted] = seg_groups[0] + seg_groups[kSegSortedBig];
    long long big_first = 0;                       // the ascending groups that may need a CTA: last segment of the list
    for (int k = 1; k < kSegSortedBig; ++k) big_first += seg_groups[k];
    const int* big_list = s.class_list + big_first;
    const int n_big = (int)seg_groups[kSegSortedBig];
    for (int c = 1; c < kNumClasses; ++c) {
        int s0, s1;
        class_segments(c, s0, s1);
        for (int k = 1; k < s0; ++k) first[c] += seg_groups[k];
        for (int k = s0; k < s1; ++k) class_groups[c] += seg_groups[k];
    }
    if (class_groups[kClassSorted] > 0) {
        const size_t warp_smem = (size_t)WarpTeam::kPerBlock * words * 8;
        if (p.m_vec <= 16 * sms || warp_smem > 200 * 1024) {
            const int grid = p.m_vec < sms * 16 ? p.m_vec : sms * 16;
            svc_emit_sorted_kernel<BlockTeam<256>><<<grid, 256, (size_t)words * 8, stream>>>(p, words, 0, s.vec_ptr, s.mode, out_col, out_vals,
                                                                                             nullptr, 0);
        } else {
            int grid = (p.m_vec + WarpTeam::kPerBlock - 1) / WarpTeam::kPerBlock;
            if (grid > sms * 8) grid = sms * 8;
            svc_emit_sorted_kernel<WarpTeam><<<grid, 256, warp_smem, stream>>>(p, words, 1, s.vec_ptr, s.mode, out_col, out_vals, nullptr, 0);
            if (n_big > 0) {
                const int big_grid = n_big < sms * 2 ? n_big : sms * 2;
                svc_emit_sorted_kernel<BlockTeam<256>><<<big_grid, 256, (size_t)words * 8, f.next()>>>(p, words, 2, s.vec_ptr, s.mode, out_col,
                                                                                                     out_vals, big_list, n_big);
            }
        }
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    // where each class starts in the list of replayed groups (the order svc_scan_place_kernel writes them in)
    // the largest groups first: they are the critical path
    e = launch_replay<BlockTeam<1024>, kClassXL>(p, s, out_col, out_vals, class_groups[kClassXL], first[kClassXL], 0, 0, f.next());
    if (e == cudaSuccess)
        e = launch_replay<BlockTeam<1024>, kClassL>(p, s, out_col, out_vals, class_groups[kClassL], first[kClassL], kLCapT, 0, f.next());
    if (e == cudaSuccess)
        e = launch_replay<BlockTeam<512>, kClassM2>(p, s, out_col, out_vals, class_groups[kClassM2], first[kClassM2], kM2CapT, kM2CapU + 2, f.next());
    if (e == cudaSuccess)
        e = launch_replay<BlockTeam<256>, kClassM1>(p, s, out_col, out_vals, class_groups[kClassM1], first[kClassM1], kM1CapT, kM1CapU + 4, f.next());
    if (e == cudaSuccess)
        e = launch_replay<WarpTeam, kClassS>(p, s, out_col, out_vals, class_groups[kClassS], first[kClassS], kSCapT, kSCapU + 2, f.next());
    if (e == cudaSuccess)
        e = launch_replay<WarpTeam, kClassXS>(p, s, out_col, out_vals, class_groups[kClassXS], first[kClassXS], kXSCapT, kXSCapU + 2, stream);
    if (e != cudaSuccess) return e;
    return f.join();
}


// ---- batches -------------------------------------------------------------------------------
namespace {
// index of the matrix that owns position x, for a table whose `base` member is ascending
template <class F>
__device__ __forceinline__ int owner_of(long long x, int count, F base_of) {
    int lo = 0, hi = count - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (base_of(mid) <= x) lo = mid; else hi = mid - 1;
    }
    return lo;
}

__global__ void __launch_bounds__(256)
svc_stack_kernel(const SvcBatchEntry* __restrict__ tab, int count, long long rows, long long entries, int* __restrict__ row_ptr,
                 int* __restrict__ col_idx, __half* __restrict__ vals) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (long long r = t0; r <= rows; r += stride) {
        if (r == rows) { row_ptr[r] = (int)entries; continue; }
        const int m = owner_of(r, count, [&](int k) { return tab[k].row_base; });
        const long long lr = r - tab[m].row_base;
        row_ptr[r] = (int)(tab[m].nnz_base + (lr < tab[m].M ? tab[m].row_ptr[lr] : tab[m].nnz));
    }
    for (long long e = t0; e < entries; e += stride) {
        const int m = owner_of(e, count, [&](int k) { return tab[k].nnz_base; });
        const long long le = e - tab[m].nnz_base;
        col_idx[e] = tab[m].col_idx[le];
        if (vals) vals[e] = tab[m].vals[le];
    }
}

__global__ void svc_batch_cuts_kernel(const SvcBatchEntry* __restrict__ tab, int count, const int* __restrict__ vec_ptr,
                                      long long* __restrict__ cuts) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m <= count) cuts[m] = vec_ptr[tab[m].vec_row_base];
}

__global__ void __launch_bounds__(256)
svc_batch_row_ptrs_kernel(const SvcBatchEntry* __restrict__ tab, int count, long long vec_rows, const int* __restrict__ vec_ptr,
                          const long long* __restrict__ cuts, int* __restrict__ out) {
    // output position x = (stacked vector row) + (matrix index): each matrix has one pointer more than vector rows
    const long long total = vec_rows + count;
    for (long long x = (long long)blockIdx.x * blockDim.x + threadIdx.x; x < total; x += (long long)gridDim.x * blockDim.x) {
        const int m = owner_of(x, count, [&](int k) { return tab[k].vec_row_base + k; });
        const long long lv = x - tab[m].vec_row_base - m;
        out[x] = (int)(vec_ptr[tab[m].vec_row_base + lv] - cuts[m]);
    }
}
}  // namespace

cudaError_t svc_stack(const SvcBatchEntry* tab, int count, long long rows, long long entries, int V, int* row_ptr,
                      int* col_idx, __half* vals, cudaStream_t stream) {
    (void)V;
    const long long work = (rows + 1 > entries ? rows + 1 : entries);
    long long blocks = (work + 255) / 256;
    const long long cap = (long long)device_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    svc_stack_kernel<<<(int)blocks, 256, 0, stream>>>(tab, count, rows, entries, row_ptr, col_idx, vals);
    return cudaGetLastError();
}

cudaError_t svc_batch_cuts(const SvcBatchEntry* tab, int count, const int* vec_ptr, long long* cuts, cudaStream_t stream) {
    svc_batch_cuts_kernel<<<(count + 1 + 255) / 256, 256, 0, stream>>>(tab, count, vec_ptr, cuts);
    return cudaGetLastError();
}

cudaError_t svc_batch_row_ptrs(const SvcBatchEntry* tab, int count, long long vec_rows, const int* vec_ptr,
                               const long long* cuts, int* out, cudaStream_t stream) {
    long long blocks = (vec_rows + count + 255) / 256;
    const long long cap = (long long)device_sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    svc_batch_row_ptrs_kernel<<<(int)blocks, 256, 0, stream>>>(tab, count, vec_rows, vec_ptr, cuts, out);
    return cudaGetLastError();
}

cudaError_t svc_read_and_clear_bad_column_flag(int* flag, cudaStream_t stream) {
    cudaError_t e = cudaMemcpyFromSymbolAsync(flag, g_svc_bad_column, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*flag) {
        const int zero = 0;
        e = cudaMemcpyToSymbolAsync(g_svc_bad_column, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    }
    return e;
}

}  // namespace sspmm_b200
