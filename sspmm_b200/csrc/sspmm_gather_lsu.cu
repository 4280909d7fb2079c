// Vector-sparse SpMM on the tensor cores, second gather variant: the rows of B are fetched by
// ordinary 16-byte loads of eight producer warps (instead of TMA row-gather requests) and written
// into the same 128-byte-swizzled M-major layout the MMA reads.  Measured reason: the TMA gather
// path sustains about one 128-byte row per 19 cycles per SM; loads issued from many threads keep
// far more requests in flight and run at L2 speed.
//
// Also splits very long vector rows: a row with more than `chunk` vectors is cut into chunks that
// are separate work items; their fp32 partial tiles go to scratch and a small kernel adds them up
// and writes C once (one rounding).  Without this a power-law matrix is as slow as its longest row.
//
// Same contract as the other SpMM kernels (reference entry: SSpMM/src/sspmm.cu:626-649).
//
// Warps (576 threads): 0-3 epilogue, 4 MMA issuer / TMEM owner, 5 value-vector loader,
// 6-17 three gather-producer groups of four warps that fill pipeline stages in turn; each group
// loads the column ids of its next stage before the B rows of the current one, so that the two
// dependent memory latencies overlap.
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
constexpr int kThreads = 576;
constexpr int kTmemCols = 32;
constexpr int kProducerGroups = 3;
constexpr int kGroupThreads = 128;

constexpr int kAChunk = kKS * 128;
constexpr int kAStage = 2 * kAChunk;   // 16 KB
constexpr int kVChunk = kKS * 16;
constexpr int kVStage = 2 * kVChunk;   // 2 KB
constexpr int kAOff = 0;
constexpr int kVOff = kStages * kAStage;
constexpr int kBarOff = kVOff + kStages * kVStage;
constexpr int kNumBars = 2 * kStages + 4;
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
};

struct Item {
    int row;        // vector row (-1: nothing to do)
    int j0, len;    // vectors [j0, j0 + len) of the value / column arrays
    int n0, batch;
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
    return it;
}

template <int V, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
sspmm_gather_lsu_kernel(Problem p, OutT* __restrict__ out) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + kBarOff;
    const uint32_t bar_empty = bar_full + kStages * 8;
    const uint32_t bar_acc_full = bar_empty + kStages * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 2 * 8;
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kAbortOff);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 5);      // four producer warps + the value loader
            mbar_init(bar_empty + 8 * s, 1);     // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (V == 8) {
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

    if (warp >= 6) {
        // ---------------------------------------------------------------- gather producers
        const int group = (warp - 6) >> 2;
        const int t = threadIdx.x - (6 + 4 * group) * 32;        // 0..127 inside the group
        const int cc = t & 15;                                   // 16-byte piece of the 256-byte row segment
        const int rsub = t >> 4;                                 // row inside each block of 8 rows
        const int half_sel = cc >> 3, c16 = cc & 7;

        // cursor over the pipeline stages this group owns (every kProducerGroups-th stage of the CTA)
        int T = blockIdx.x;
        Item item;
        int k0 = 0;
        uint32_t it_count = 0;
        bool valid = false;
        // positions the cursor on the first stage at or after the current one that belongs to this group
        auto settle = [&](bool fresh_tile) {
            for (;;) {
                if (fresh_tile) {
                    valid = false;
                    while (T < total) {
                        item = get_item(p, T, extra_entries, chunk);
                        if (item.len > 0) { valid = true; break; }
                        T += gridDim.x;
                    }
                    if (!valid) return;
                    k0 = 0;
                    fresh_tile = false;
                }
                if ((int)(it_count % kProducerGroups) == group) return;
                k0 += kKS; ++it_count;
                if (k0 >= item.len) { T += gridDim.x; fresh_tile = true; }
            }
        };
        auto step = [&]() {                     // leave the current stage, go to the next owned one
            k0 += kKS; ++it_count;
            const bool fresh = k0 >= item.len;
            if (fresh) T += gridDim.x;
            settle(fresh);
        };
        auto load_cols = [&](int (&c)[8]) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int r = 8 * q + rsub;
                c[q] = -1;
                if (k0 + r < item.len) c[q] = __ldg(p.col + item.j0 + k0 + r);
            }
        };
        settle(true);
        int cols[8];
        if (valid) load_cols(cols);
        while (valid) {
            const Item cur = item;
            const uint32_t stage = it_count % kStages, phase = (it_count / kStages) & 1u;
            int cur_cols[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) cur_cols[q] = cols[q];
            step();
            if (valid) load_cols(cols);                          // column ids of the next owned stage
            const __half* bbase = p.rhs + (int64_t)cur.batch * p.rhs_stride + cur.n0 + cc * 8;
            const bool col_ok = cur.n0 + cc * 8 < p.N;
            uint4 v[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                v[q] = make_uint4(0, 0, 0, 0);
                if (col_ok && (unsigned)cur_cols[q] < (unsigned)p.K)
                    v[q] = __ldg(reinterpret_cast<const uint4*>(bbase + (int64_t)cur_cols[q] * p.N));
            }
            if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitEmpty)) break;
            uint8_t* a_s = smem + kAOff + stage * kAStage + half_sel * kAChunk;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int r = 8 * q + rsub;
                *reinterpret_cast<uint4*>(a_s + r * 128 + ((c16 ^ (r & 7)) << 4)) = v[q];
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full + 8 * stage);
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------------- value-vector loader
        constexpr int kChunksPerRow = V / 8;
        constexpr int kPerLane = kKS * kChunksPerRow / 32;
        uint32_t it_count = 0;
        bool ok = true;
        for (int T = blockIdx.x; ok && T < total; T += gridDim.x) {
            const Item item = get_item(p, T, extra_entries, chunk);
            if (item.len <= 0) continue;
            const __half* vbase = p.values + (int64_t)item.batch * p.values_stride + (int64_t)item.j0 * V;
            for (int k0 = 0; k0 < item.len; k0 += kKS, ++it_count) {
                const uint32_t stage = it_count % kStages, phase = (it_count / kStages) & 1u;
                uint4 v[kPerLane];
#pragma unroll
                for (int q = 0; q < kPerLane; ++q) {
                    const int id = lane + 32 * q;
                    const int r = id / kChunksPerRow, c = id % kChunksPerRow;
                    v[q] = make_uint4(0, 0, 0, 0);
                    if (k0 + r < item.len) v[q] = __ldg(reinterpret_cast<const uint4*>(vbase + (int64_t)(k0 + r) * V + c * 8));
                }
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitEmpty)) { ok = false; break; }
                uint8_t* vs = smem + kVOff + stage * kVStage;
#pragma unroll
                for (int q = 0; q < kPerLane; ++q) {
                    const int id = lane + 32 * q;
                    const int r = id / kChunksPerRow, c = id % kChunksPerRow;
                    *reinterpret_cast<uint4*>(vs + c * kVChunk + r * 16) = v[q];
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * stage);
            }
        }
    } else if (warp == 4) {
        // ---------------------------------------------------------------- MMA issuer
        constexpr uint32_t idesc = make_idesc_f16_f32(kTileN, kMmaN, true, true);
        uint32_t it_count = 0, acc_it = 0;
        bool ok = true;
        for (int T = blockIdx.x; ok && T < total; T += gridDim.x) {
            const Item item = get_item(p, T, extra_entries, chunk);
            if (item.len <= 0) continue;
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            if (!mbar_wait(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag, kStatusWaitAccEmpty)) break;
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * kMmaN;
            for (int k0 = 0; k0 < item.len; k0 += kKS, ++it_count) {
                const uint32_t stage = it_count % kStages, phase = (it_count / kStages) & 1u;
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, kStatusWaitFull)) { ok = false; break; }
                tc_fence_after_sync();
                if (lane == 0) {
                    const int rows = min(kKS, item.len - k0);
                    const int nk = (rows + 15) >> 4;
                    const uint32_t a_addr = sbase + kAOff + stage * kAStage;
                    const uint32_t v_addr = sbase + kVOff + stage * kVStage;
                    for (int kk = 0; kk < nk; ++kk) {
                        const uint64_t a_desc = make_smem_desc(a_addr + kk * 2048, kAChunk, 1024, 2);
                        const uint64_t b_desc = make_smem_desc(v_addr + kk * 256, 128, kVChunk, 0);
                        tc_mma_f16(d_tmem, a_desc, b_desc, idesc, (k0 > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_empty + 8 * stage);
                }
                __syncwarp();
            }
            if (!ok) break;
            if (lane == 0) tc_commit(bar_acc_full + 8 * buf);
            __syncwarp();
            ++acc_it;
        }
    } else {
        // ---------------------------------------------------------------- epilogue (warps 0-3)
        const int q = warp & 3;
        uint32_t acc_it = 0;
        for (int T = blockIdx.x; T < total; T += gridDim.x) {
            const Item item = get_item(p, T, extra_entries, chunk);
            if (item.row < 0) continue;
            uint32_t r[V];
            if (item.len > 0) {
                const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
                if (!mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kStatusWaitAccFull)) break;
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * kMmaN;
                if constexpr (V == 16) tmem_ld_x16(taddr, r); else tmem_ld_x8(taddr, r);
                tc_wait_ld();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
                ++acc_it;
            } else {
#pragma unroll
                for (int v = 0; v < V; ++v) r[v] = 0u;
            }
            const int nl = q * 32 + lane;
            if (item.slot >= 0) {
                float* o = p.partial + (int64_t)item.slot * V * kTileN + nl;
#pragma unroll
                for (int v = 0; v < V; ++v) o[v * kTileN] = __uint_as_float(r[v]);
            } else if (item.n0 + nl < p.N) {
                OutT* o = out + (int64_t)item.batch * p.out_stride + (int64_t)item.row * V * p.N + item.n0 + nl;
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

// One block per (column tile, entry); the block of a row's chunk 0 adds up all chunks of that row.
template <int V, typename OutT>
__global__ void __launch_bounds__(128)
sum_chunks_kernel(int N, int n_tiles, int chunk, int cap, const int* __restrict__ row_offsets,
                  const int* __restrict__ n_entries, const int2* __restrict__ entries, const float* __restrict__ partial,
                  OutT* __restrict__ out) {
    const int total = *n_entries;
    if (total > cap) return;
    const int t = blockIdx.x;
    const int n = t * kTileN + threadIdx.x;
    if (n >= N) return;
    // the entry list is usually far shorter than its capacity: a bounded grid walks it
    for (int e = blockIdx.y; e < total; e += gridDim.y) {
        const int2 en = entries[e];
        if (en.y != 0) continue;
        const int len = row_offsets[en.x + 1] - row_offsets[en.x];
        const int n_chunks = (len + chunk - 1) / chunk;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            float acc = 0.f;
            for (int c = 0; c < n_chunks; ++c)
                acc += partial[((int64_t)(e + c) * n_tiles + t) * V * kTileN + v * kTileN + threadIdx.x];
            const int64_t o = ((int64_t)en.x * V + v) * N + n;
            if constexpr (sizeof(OutT) == 2) out[o] = __float2half_rn(acc);
            else out[o] = acc;
        }
    }
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
    if (p.chunk > 0) {
        int* counter = static_cast<int*>(scratch);
        cudaError_t e = cudaMemsetAsync(counter, 0, 16, a.stream);
        if (e != cudaSuccess) return e;
        build_chunk_entries_kernel<<<(a.m_vec + 255) / 256, 256, 0, a.stream>>>(a.m_vec, p.chunk, cap, a.row_offsets,
                                                                               counter, const_cast<int2*>(p.entries));
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    kern<<<grid, kThreads, kSmemBytes, a.stream>>>(p, static_cast<OutT*>(a.out));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (p.chunk > 0) {
        dim3 g(p.n_tiles, cap < 592 ? cap : 592);
        sum_chunks_kernel<V, OutT><<<g, 128, 0, a.stream>>>(a.N, p.n_tiles, p.chunk, cap, a.row_offsets, p.n_entries, p.entries,
                                                            p.partial, static_cast<OutT*>(a.out));
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace lsu

// Scratch layout: [16 B counter][cap entries of int2][partials].  cap = 0 disables row splitting.
void sspmm_gather_lsu_plan(const SpmmArgs& a, long long nvec, int* chunk, int* cap, size_t* scratch_bytes) {
    *chunk = 0; *cap = 0; *scratch_bytes = 0;
    if (nvec <= 0 || a.batch != 1) return;
    const int sms = current_device_sm_count();
    const long long n_tiles = (a.N + lsu::kTileN - 1) / lsu::kTileN;
    long long c = nvec * n_tiles / ((long long)sms * 4);
    if (c < 1024) c = 1024;
    c = (c + 63) / 64 * 64;
    if (c >= a.K || c > 0x3fffffff) return;                 // no row can be longer than K vectors
    const long long n_cap = 2 * nvec / c + 1;
    const size_t bytes = 16 + (size_t)n_cap * 8 + (size_t)n_cap * n_tiles * a.V * lsu::kTileN * 4;
    if (n_cap > 60000 || bytes > ((size_t)1 << 30)) return;
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
    p.n_entries = nullptr; p.entries = nullptr; p.partial = nullptr;
    if (chunk > 0) {
        uint8_t* s = static_cast<uint8_t*>(scratch);
        p.n_entries = reinterpret_cast<const int*>(s);
        p.entries = reinterpret_cast<const int2*>(s + 16);
        p.partial = reinterpret_cast<float*>(s + 16 + (size_t)cap * 8);
    }
    const int sms = current_device_sm_count();
    if (sms <= 0) return cudaErrorNoDevice;
    const int grid = (int)(worst < sms ? worst : sms);
    if (a.V == 16)
        return a.out_f16 ? lsu::launch_typed<16, __half>(a, p, cap, scratch, grid) : lsu::launch_typed<16, float>(a, p, cap, scratch, grid);
    return a.out_f16 ? lsu::launch_typed<8, __half>(a, p, cap, scratch, grid) : lsu::launch_typed<8, float>(a, p, cap, scratch, grid);
}

}  // namespace sspmm_b200
