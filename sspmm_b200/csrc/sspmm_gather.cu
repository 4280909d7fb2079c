// Vector-sparse SpMM  C = A_vs * B  on the sm_100a tensor cores.
//
// Replaces the reference kernels SSpMM_V8 / SSpMM_V16 (SSpMM/src/sspmm.cu:222-439)
// and their launcher SSpMM_ex (SSpMM/src/sspmm.cu:548-623).  Same operands, same
// result; nothing of their one-warp mma.sync structure is kept.
//
// Mapping.  For one vector row i (V matrix rows sharing the column list
// cols[j0 .. j0+L)) and one tile of 128 output columns n0..n0+127 the kernel
// computes the transposed tile
//     D[n][v] = sum_j  B[cols[j]][n0+n] * values[j][v]          (128 x V, fp32)
// as a chain of tcgen05.mma (M=128, N=16, K=16, kind::f16):
//   * MMA operand A (128 x 16, M-major) = 16 gathered rows of B.  TMA row-gather
//     loads (tile::gather4, 64-column boxes, 128-byte swizzle) drop the rows
//     straight into the canonical M-major swizzled layout, so no thread touches B.
//   * MMA operand B (16 x 16, N-major) = 16 value vectors.  They are copied by a
//     loader warp into the canonical unswizzled N-major layout (two 8-wide
//     column blocks; for V=8 the second block is a constant zero block).
//   * D lives in tensor memory, lane = output column, column = v; two
//     accumulators so the epilogue of one tile overlaps the next tile's MMAs.
// A persistent CTA walks tiles T = blockIdx.x, +gridDim.x, ... with the vector row
// varying fastest, so that CTAs running at the same time gather from the same
// 128-column panel of B (it stays in L2).
//
// Warp roles (256 threads): 0 gather producer, 1 MMA issuer (+ TMEM owner),
// 2 value-vector loader, 3 idle, 4-7 epilogue (TMEM -> registers -> global).
// smem stages cycle through full/empty mbarriers; every wait is bounded.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "launch.h"
#include "ptx.cuh"

namespace sspmm_b200 {

namespace {

constexpr int kTileN = 128;      // output columns per tile (= MMA M)
constexpr int kMmaN = 16;        // MMA N (V padded to 16)
constexpr int kAccBufs = 2;
constexpr int kTmemCols = 32;    // 2 accumulators x 16 columns
constexpr int kThreads = 256;

template <int KS, int STAGES>
struct Layout {
    static constexpr int kAChunk = KS * 128;         // 64 columns x KS rows, 128-byte rows
    static constexpr int kAStage = 2 * kAChunk;
    static constexpr int kVChunk = KS * 16;          // 8 lanes of V x KS rows, 16-byte rows
    static constexpr int kVStage = 2 * kVChunk;
    static constexpr int kAOff = 0;
    static constexpr int kVOff = STAGES * kAStage;
    static constexpr int kBarOff = kVOff + STAGES * kVStage;
    static constexpr int kNumBars = 2 * STAGES + 2 * kAccBufs;
    static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemPtrOff + 8;
    static constexpr int kBytes = kAbortOff + 8;
    static constexpr int kDynamic = kBytes + 1024;   // slack for manual 1024-byte alignment
};

struct Tile {
    int row;       // vector row, -1 if the scheduling entry is out of range
    int j0;        // first vector of the row
    int len;       // vectors in the row
    int n0;        // first output column
    int batch;
};

struct Problem {
    int m_vec, N, K, n_tiles, total_tiles;
    const int* row_indices;
    const int* row_offsets;
    const int* col;
    const __half* values;
    int64_t values_stride, out_stride;
};

__device__ __forceinline__ Tile get_tile(const Problem& p, int T) {
    Tile t;
    const int sched = T % p.m_vec;
    const int rest = T / p.m_vec;
    t.n0 = (rest % p.n_tiles) * kTileN;
    t.batch = rest / p.n_tiles;
    int i = p.row_indices ? __ldg(p.row_indices + sched) : sched;
    if ((unsigned)i >= (unsigned)p.m_vec) {
        t.row = -1; t.j0 = 0; t.len = 0;
        return t;
    }
    t.row = i;
    t.j0 = __ldg(p.row_offsets + i);
    t.len = __ldg(p.row_offsets + i + 1) - t.j0;
    if (t.len < 0) t.len = 0;
    return t;
}

template <int V, typename OutT, int KS, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
sspmm_gather_kernel(const __grid_constant__ CUtensorMap tmap_rhs, Problem p, OutT* __restrict__ out) {
    using L = Layout<KS, STAGES>;
    static_assert(KS % 64 == 0, "stage = multiple of 64 gathered rows");
    constexpr int kGroupsPerLane = KS / 64;          // 4-row gather groups handled by one lane

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + L::kBarOff;                    // [STAGES]
    const uint32_t bar_empty = bar_full + STAGES * 8;                // [STAGES]
    const uint32_t bar_acc_full = bar_empty + STAGES * 8;            // [kAccBufs]
    const uint32_t bar_acc_empty = bar_acc_full + kAccBufs * 8;      // [kAccBufs]
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 2);    // gather producer (with tx bytes) + value loader
            mbar_init(bar_empty + 8 * s, 1);   // tcgen05.commit
        }
        for (int b = 0; b < kAccBufs; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);   // tcgen05.commit
            mbar_init(bar_acc_empty + 8 * b, 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_rhs);
    }
    if (V == 8) {
        // constant zero block standing in for value lanes 8..15
        for (int o = threadIdx.x * 16; o < STAGES * L::kVChunk; o += kThreads * 16) {
            const int s = o / L::kVChunk, r = o % L::kVChunk;
            *reinterpret_cast<uint4*>(smem + L::kVOff + s * L::kVStage + L::kVChunk + r) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (warp == 0) {
        // ------------------------------------------------------------------ gather producer
        uint32_t stage = 0, phase = 0;
        int T = blockIdx.x;
        Tile nt;             // tile of the next stage to issue
        int nk0 = 0;
        bool nvalid = false;
        while (T < p.total_tiles) {
            nt = get_tile(p, T);
            if (nt.len > 0) { nvalid = true; break; }
            T += gridDim.x;
        }
        int nidx[kGroupsPerLane][4];
        auto load_idx = [&](const Tile& t, int k0, int (&idx)[kGroupsPerLane][4]) {
#pragma unroll
            for (int u = 0; u < kGroupsPerLane; ++u) {
                const int g = (lane >> 1) + 16 * u;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int jj = k0 + 4 * g + e;
                    int c = 0;
                    if (jj < t.len) c = __ldg(p.col + t.j0 + jj);
                    idx[u][e] = c + t.batch * p.K;
                }
            }
        };
        if (nvalid) load_idx(nt, nk0, nidx);
        while (nvalid) {
            const Tile ct = nt;
            const int ck0 = nk0;
            int cidx[kGroupsPerLane][4];
#pragma unroll
            for (int u = 0; u < kGroupsPerLane; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e) cidx[u][e] = nidx[u][e];
            // look one stage ahead so the index loads overlap the wait below
            nk0 += KS;
            if (nk0 >= nt.len) {
                nk0 = 0;
                nvalid = false;
                T += gridDim.x;
                while (T < p.total_tiles) {
                    nt = get_tile(p, T);
                    if (nt.len > 0) { nvalid = true; break; }
                    T += gridDim.x;
                }
            }
            if (nvalid) load_idx(nt, nk0, nidx);

            if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitEmpty)) break;
            const int rows = min(KS, ct.len - ck0);
            const int groups = ((rows + 15) & ~15) >> 2;
            if (lane == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, (uint32_t)groups * 2u * 512u);
            __syncwarp();
            const int c = lane & 1;
            const uint32_t a_stage = sbase + L::kAOff + stage * L::kAStage + c * L::kAChunk;
#pragma unroll
            for (int u = 0; u < kGroupsPerLane; ++u) {
                const int g = (lane >> 1) + 16 * u;
                if (g < groups)
                    tma_gather4(a_stage + g * 512, &tmap_rhs, ct.n0 + c * 64, cidx[u][0], cidx[u][1], cidx[u][2],
                                cidx[u][3], bar_full + 8 * stage);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ value-vector loader
        constexpr int kChunksPerRow = V / 8;
        constexpr int kPerLane = KS * kChunksPerRow / 32;
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int T = blockIdx.x; ok && T < p.total_tiles; T += gridDim.x) {
            const Tile t = get_tile(p, T);
            if (t.len <= 0) continue;
            const __half* vbase = p.values + (int64_t)t.batch * p.values_stride + (int64_t)t.j0 * V;
            for (int k0 = 0; k0 < t.len; k0 += KS) {
                uint4 v[kPerLane];
#pragma unroll
                for (int q = 0; q < kPerLane; ++q) {
                    const int id = lane + 32 * q;
                    const int r = id / kChunksPerRow, c = id % kChunksPerRow;
                    v[q] = make_uint4(0, 0, 0, 0);
                    if (k0 + r < t.len)
                        v[q] = __ldg(reinterpret_cast<const uint4*>(vbase + (int64_t)(k0 + r) * V + c * 8));
                }
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitEmpty)) { ok = false; break; }
                uint8_t* vs = smem + L::kVOff + stage * L::kVStage;
#pragma unroll
                for (int q = 0; q < kPerLane; ++q) {
                    const int id = lane + 32 * q;
                    const int r = id / kChunksPerRow, c = id % kChunksPerRow;
                    *reinterpret_cast<uint4*>(vs + c * L::kVChunk + r * 16) = v[q];
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = make_idesc_f16_f32(kTileN, kMmaN, /*A M-major*/ true, /*B N-major*/ true);
        uint32_t stage = 0, phase = 0;
        uint32_t acc_it = 0;
        bool ok = true;
        for (int T = blockIdx.x; ok && T < p.total_tiles; T += gridDim.x) {
            const Tile t = get_tile(p, T);
            if (t.len <= 0) continue;
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            if (!mbar_wait(bar_acc_empty + 8 * buf, acc_phase ^ 1u, abort_flag, kStatusWaitAccEmpty)) break;
            tc_fence_after_sync();
            const uint32_t d_tmem = tmem_base + buf * kMmaN;
            for (int k0 = 0; k0 < t.len; k0 += KS) {
                if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, kStatusWaitFull)) { ok = false; break; }
                tc_fence_after_sync();
                if (lane == 0) {
                    const int rows = min(KS, t.len - k0);
                    const int nk = (rows + 15) >> 4;
                    const uint32_t a_addr = sbase + L::kAOff + stage * L::kAStage;
                    const uint32_t v_addr = sbase + L::kVOff + stage * L::kVStage;
                    for (int kk = 0; kk < nk; ++kk) {
                        // A: 128-byte swizzle, M-major: 64-column blocks kAChunk apart, 8-row groups 1024 B apart
                        const uint64_t a_desc = make_smem_desc(a_addr + kk * 2048, L::kAChunk, 1024, 2);
                        // B: no swizzle, N-major: 8-lane blocks kVChunk apart, 8-row groups 128 B apart
                        const uint64_t b_desc = make_smem_desc(v_addr + kk * 256, 128, L::kVChunk, 0);
                        tc_mma_f16(d_tmem, a_desc, b_desc, idesc, (k0 > 0 || kk > 0) ? 1u : 0u);
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
        // ------------------------------------------------------------------ epilogue
        const int q = warp & 3;                      // TMEM lane quarter this warp may read
        uint32_t acc_it = 0;
        for (int T = blockIdx.x; T < p.total_tiles; T += gridDim.x) {
            const Tile t = get_tile(p, T);
            if (t.row < 0) continue;
            uint32_t r[V];
            if (t.len > 0) {
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
            const int n = t.n0 + q * 32 + lane;
            if (n < p.N) {
                OutT* o = out + (int64_t)t.batch * p.out_stride + (int64_t)t.row * V * p.N + n;
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
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- host side --------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}


template <int V, typename OutT, int KS, int STAGES>
cudaError_t launch_one(const SpmmArgs& a, const CUtensorMap& tmap, const Problem& p, int grid) {
    using L = Layout<KS, STAGES>;
    auto kern = sspmm_gather_kernel<V, OutT, KS, STAGES>;
    static DeviceOnce attr_once;                      // one flag set per instantiation
    if (!attr_once.done()) {
        cudaError_t attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (attr_err != cudaSuccess) return attr_err;
        attr_once.mark();
    }
    kern<<<grid, kThreads, L::kDynamic, a.stream>>>(tmap, p, static_cast<OutT*>(a.out));
    return cudaGetLastError();
}

}  // namespace

int current_device_sm_count() {
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

cudaError_t launch_sspmm_gather(const SpmmArgs& a) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) {
        set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
        return cudaErrorNotSupported;
    }
    const int n_tiles = (a.N + kTileN - 1) / kTileN;
    const int64_t total = (int64_t)a.m_vec * n_tiles * a.batch;
    if (total > 0x7fffffffLL || (int64_t)a.K * a.batch > 0x7fffffffLL) {
        set_error("problem too large for 32-bit tile ids");
        return cudaErrorInvalidValue;
    }
    CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.N, (cuuint64_t)a.K * (cuuint64_t)a.batch};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.N * sizeof(__half)};
    const cuuint32_t box[2] = {64u, 1u};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(a.rhs), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (N=%d K=%d)", (int)r, a.N, a.K);
        return cudaErrorInvalidValue;
    }
    Problem p;
    p.m_vec = a.m_vec; p.N = a.N; p.K = a.K; p.n_tiles = n_tiles; p.total_tiles = (int)total;
    p.row_indices = a.row_indices; p.row_offsets = a.row_offsets; p.col = a.column_indices; p.values = a.values;
    p.values_stride = a.values_stride; p.out_stride = a.out_stride;
    const int sms = current_device_sm_count();
    if (sms <= 0) return cudaErrorNoDevice;
    const int grid = (int)(total < sms ? total : sms);

    if (a.V == 16) {
        return a.out_f16 ? launch_one<16, __half, 64, 6>(a, tmap, p, grid) : launch_one<16, float, 64, 6>(a, tmap, p, grid);
    } else {
        return a.out_f16 ? launch_one<8, __half, 64, 6>(a, tmap, p, grid) : launch_one<8, float, 64, 6>(a, tmap, p, grid);
    }
}

}  // namespace sspmm_b200
