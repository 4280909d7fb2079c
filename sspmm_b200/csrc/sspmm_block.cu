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
//   epilogue    tcgen05.ld 32 columns at a time -> fp16/fp32 -> 16-byte stores
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch.h"
#include "ptx.cuh"

namespace sspmm_b200 {
namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kBlockThreads = 256;

// ---- expansion of the compressed operand ------------------------------------
// blockIdx.y = vector row, blockIdx.x strides over its vectors; each thread
// writes the V values of one vector as one or two 16-byte stores into row
// column_indices[j] of At.
template <int V>
__global__ void __launch_bounds__(256)
expand_transposed_kernel(int m_vec, int K, const int* __restrict__ row_offsets, const int* __restrict__ col,
                         const __half* __restrict__ values, __half* __restrict__ at) {
    const int64_t mp = (int64_t)m_vec * V;
    for (int i = blockIdx.y; i < m_vec; i += gridDim.y) {
        const int j0 = row_offsets[i], j1 = row_offsets[i + 1];
        for (int j = j0 + blockIdx.x * blockDim.x + threadIdx.x; j < j1; j += gridDim.x * blockDim.x) {
            const unsigned c = (unsigned)col[j];
            if (c >= (unsigned)K) continue;
            const uint4* src = reinterpret_cast<const uint4*>(values + (int64_t)j * V);
            uint4* dst = reinterpret_cast<uint4*>(at + (int64_t)c * mp + (int64_t)i * V);
#pragma unroll
            for (int q = 0; q < V / 8; ++q) dst[q] = __ldg(src + q);
        }
    }
}

template <int BN, int STAGES>
struct BlockLayout {
    static constexpr int kAStage = kBM * kBK * 2;                // 16 KB: 2 chunks of [64 k][64 m]
    static constexpr int kBStage = BN * kBK * 2;                 // 4 or 2 chunks of [64 k][64 n]
    static constexpr int kChunk = kBK * 128;                     // 8 KB
    static constexpr int kAOff = 0;
    static constexpr int kBOff = STAGES * kAStage;
    static constexpr int kBarOff = kBOff + STAGES * kBStage;
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
    int64_t out_stride;      // per batch, elements
};

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(kBlockThreads, 1)
sspmm_block_kernel(const __grid_constant__ CUtensorMap tmap_at, const __grid_constant__ CUtensorMap tmap_b,
                   BlockProblem p, OutT* __restrict__ out) {
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
                const int b = T / tiles_per_batch, r = T % tiles_per_batch;
                const int m0 = (r % p.m_tiles) * kBM, n0 = (r / p.m_tiles) * BN;
                bool ok = true;
                for (int ks = 0; ks < k_steps; ++ks) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, kStatusWaitBlock)) { ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_arrive_expect_tx(full, L::kAStage + L::kBStage);
                    const uint32_t a_s = sbase + L::kAOff + stage * L::kAStage;
                    const uint32_t b_s = sbase + L::kBOff + stage * L::kBStage;
#pragma unroll
                    for (int c = 0; c < kBM / 64; ++c) tma_load_2d(a_s + c * L::kChunk, &tmap_at, m0 + 64 * c, ks * kBK, full);
#pragma unroll
                    for (int c = 0; c < BN / 64; ++c)
                        tma_load_2d(b_s + c * L::kChunk, &tmap_b, n0 + 64 * c, b * p.K + ks * kBK, full);
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
            for (int ks = 0; ks < k_steps; ++ks) {
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
                        tc_mma_f16(d_tmem, a_desc, b_desc, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
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
        const int q = warp & 3;
        uint32_t acc_it = 0;
        for (int T = blockIdx.x; T < p.total_tiles; T += gridDim.x) {
            const int b = T / tiles_per_batch, r = T % tiles_per_batch;
            const int m0 = (r % p.m_tiles) * kBM, n0 = (r / p.m_tiles) * BN;
            const uint32_t buf = acc_it & 1u, acc_phase = (acc_it >> 1) & 1u;
            const int m = m0 + q * 32 + lane;
            OutT* orow = out + (int64_t)b * p.out_stride + (int64_t)m * p.N;
            if (k_steps > 0) {
                if (!mbar_wait(bar_acc_full + 8 * buf, acc_phase, abort_flag, kStatusWaitBlock)) break;
                tc_fence_after_sync();
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                uint32_t v[32];
                if (k_steps > 0) {
                    tmem_ld_x32(taddr + cc * 32, v);
                    tc_wait_ld();
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = 0u;
                }
                if (cc == BN / 32 - 1 && k_steps > 0) {
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
                }
                const int n = n0 + cc * 32;
                if (m < p.Mp) {
                    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (n + g * 8 + 8 <= p.N) {
                                uint4 w;
                                __half2 h0 = __floats2half2_rn(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
                                __half2 h1 = __floats2half2_rn(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
                                __half2 h2 = __floats2half2_rn(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
                                __half2 h3 = __floats2half2_rn(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
                                w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
                                w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
                                *reinterpret_cast<uint4*>(orow + n + g * 8) = w;
                            }
                        }
                    } else {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            if (n + g * 4 + 4 <= p.N) {
                                uint4 w = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                                *reinterpret_cast<uint4*>(orow + n + g * 4) = w;
                            }
                        }
                    }
                }
            }
            ++acc_it;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn block_encode_fn() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    return reinterpret_cast<EncodeFn>(fn);
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

template <int BN, int STAGES, typename OutT>
cudaError_t launch_block(const SpmmArgs& a, const CUtensorMap& ta, const CUtensorMap& tb, const BlockProblem& p, int sms) {
    using L = BlockLayout<BN, STAGES>;
    auto kern = sspmm_block_kernel<BN, STAGES, OutT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess) return e;
    const int grid = p.total_tiles < sms ? p.total_tiles : sms;
    kern<<<grid, kBlockThreads, L::kDynamic, a.stream>>>(ta, tb, p, static_cast<OutT*>(a.out));
    return cudaGetLastError();
}

}  // namespace

size_t sspmm_block_scratch_bytes(const SpmmArgs& a) {
    return (size_t)a.K * (size_t)a.m_vec * a.V * sizeof(__half);
}

// `scratch` holds K * m_vec*V halfs (the transposed dense copy of A), owned by the caller.
cudaError_t launch_sspmm_block(const SpmmArgs& a, void* scratch) {
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
    cudaError_t e = cudaMemsetAsync(at, 0, sspmm_block_scratch_bytes(a), a.stream);
    if (e != cudaSuccess) return e;
    {
        // enough blocks per vector row to cover up to K vectors, a few thousand blocks at most
        int bx = (a.K + 255) / 256;
        if (bx > 32) bx = 32;
        const int by = a.m_vec < 32768 ? a.m_vec : 32768;
        const dim3 grid(bx, by);
        if (a.V == 16)
            expand_transposed_kernel<16><<<grid, 256, 0, a.stream>>>(a.m_vec, a.K, a.row_offsets, a.column_indices, a.values, at);
        else
            expand_transposed_kernel<8><<<grid, 256, 0, a.stream>>>(a.m_vec, a.K, a.row_offsets, a.column_indices, a.values, at);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) return cudaErrorNoDevice;

    const int m_tiles = (Mp + kBM - 1) / kBM;
    const int64_t tiles256 = (int64_t)m_tiles * ((a.N + 255) / 256) * a.batch;
    const bool wide = tiles256 >= sms;          // enough 128x256 tiles to fill the machine
    const int BN = wide ? 256 : 128;
    BlockProblem p;
    p.Mp = Mp; p.N = a.N; p.K = a.K;
    p.m_tiles = m_tiles; p.n_tiles = (a.N + BN - 1) / BN;
    const int64_t total = (int64_t)p.m_tiles * p.n_tiles * a.batch;
    if (total > 0x7fffffffLL || (int64_t)a.K * a.batch > 0x7fffffffLL) {
        set_error("problem too large for 32-bit tile ids");
        return cudaErrorInvalidValue;
    }
    p.total_tiles = (int)total;
    p.out_stride = a.out_stride;
    CUtensorMap ta, tb;
    if (!encode_2d(enc, &ta, at, (uint64_t)Mp, (uint64_t)a.K, 64, 64) ||
        !encode_2d(enc, &tb, a.rhs, (uint64_t)a.N, (uint64_t)a.K * a.batch, 64, 64)) {
        set_error("cuTensorMapEncodeTiled failed (Mp=%d N=%d K=%d)", Mp, a.N, a.K);
        return cudaErrorInvalidValue;
    }
    if (wide)
        return a.out_f16 ? launch_block<256, 4, __half>(a, ta, tb, p, sms) : launch_block<256, 4, float>(a, ta, tb, p, sms);
    return a.out_f16 ? launch_block<128, 6, __half>(a, ta, tb, p, sms) : launch_block<128, 6, float>(a, ta, tb, p, sms);
}

}  // namespace sspmm_b200
