// Row reordering before compression (extension; parity unpinned).
//
// The reference's README runs `row_merge_reorder.py` after `row_merge.py` (README.md:36) and its
// driver reads the reordered data sets (SSpMM/sspmm_test.cpp:313-319), but reorder.py and
// row_merge_reorder.py are not part of the reference checkout, so there is nothing to be
// bit-identical to.  This file implements the idea stated for that stage -- put rows that share
// columns into the same V-row group so that fewer V x 1 vectors are non-zero -- as a greedy
// grouping inside windows of 256 consecutive rows:
//   * every row gets a bit signature of its column set (exact bitmap when K <= 2048, else columns
//     hashed into 2048 bits), kept word-major in shared memory;
//   * a group starts with the first unassigned row of the window; V-1 times, all threads score one
//     candidate row each by the number of signature bits it would ADD to the group's union
//     (popc(cand & ~group)), a block reduction picks the smallest (ties: lowest row), and the
//     group's union is updated.
// Output: perm[M], the new row order (row perm[r] of A becomes row r).  Windows are multiples of V
// rows, so groups never straddle windows.  CPU restatement: oracle/reorder_oracle.py.
#include <cuda_runtime.h>

#include "../../include/sspmm_b200.h"
#include "launch.h"

namespace sspmm_b200 {
namespace {

constexpr int kWindow = 256;
constexpr int kSigBits = 2048;
constexpr int kSigWords = kSigBits / 32;

__device__ __forceinline__ unsigned sig_bit(int c, int K) {
    if (K <= kSigBits) return (unsigned)c;
    return ((unsigned)c * 2654435761u) >> (32 - 11);        // 11 bits = 2048 buckets
}

__global__ void __launch_bounds__(kWindow)
svc_reorder_kernel(int M, int K, int V, const int* __restrict__ row_ptr, const int* __restrict__ col, int* __restrict__ perm) {
    extern __shared__ unsigned int sm[];
    unsigned int* sig = sm;                                   // [kSigWords][kWindow]
    unsigned int* group = sm + kSigWords * kWindow;           // [kSigWords]
    unsigned long long* red = reinterpret_cast<unsigned long long*>(group + kSigWords);   // [8]
    int* assigned = reinterpret_cast<int*>(red + 8);          // [kWindow]
    __shared__ int s_best;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int w0 = blockIdx.x * kWindow;
    const int wn = min(kWindow, M - w0);

    for (int i = t; i < kSigWords * kWindow; i += kWindow) sig[i] = 0u;
    assigned[t] = (t < wn) ? 0 : 1;
    __syncthreads();
    for (int r = warp; r < wn; r += kWindow / 32) {
        const int e0 = row_ptr[w0 + r], e1 = row_ptr[w0 + r + 1];
        for (int e = e0 + lane; e < e1; e += 32) {
            const int c = col[e];
            if ((unsigned)c < (unsigned)K) {
                const unsigned b = sig_bit(c, K);
                atomicOr(&sig[(b >> 5) * kWindow + r], 1u << (b & 31));
            }
        }
    }
    __syncthreads();

    int pos = 0;
    while (pos < wn) {
        // seed: first unassigned row
        unsigned long long key = assigned[t] ? ~0ull : (unsigned long long)t;
        for (int o = 16; o > 0; o >>= 1) { const unsigned long long x = __shfl_xor_sync(0xffffffffu, key, o); key = x < key ? x : key; }
        if (lane == 0) red[warp] = key;
        __syncthreads();
        if (t == 0) {
            unsigned long long b = red[0];
            for (int w = 1; w < kWindow / 32; ++w) b = red[w] < b ? red[w] : b;
            s_best = (int)b;
        }
        __syncthreads();
        int best = s_best;
        if (t < kSigWords) group[t] = sig[t * kWindow + best];
        if (t == 0) { assigned[best] = 1; perm[w0 + pos] = w0 + best; }
        ++pos;
        __syncthreads();
        for (int k = 1; k < V && pos < wn; ++k) {
            unsigned long long sc = ~0ull;
            if (!assigned[t]) {
                int growth = 0;
#pragma unroll 8
                for (int w = 0; w < kSigWords; ++w) growth += __popc(sig[w * kWindow + t] & ~group[w]);
                sc = ((unsigned long long)growth << 32) | (unsigned)t;
            }
            for (int o = 16; o > 0; o >>= 1) { const unsigned long long x = __shfl_xor_sync(0xffffffffu, sc, o); sc = x < sc ? x : sc; }
            if (lane == 0) red[warp] = sc;
            __syncthreads();
            if (t == 0) {
                unsigned long long b = red[0];
                for (int w = 1; w < kWindow / 32; ++w) b = red[w] < b ? red[w] : b;
                s_best = (int)(b & 0xffffffffu);
            }
            __syncthreads();
            best = s_best;
            if (t < kSigWords) group[t] |= sig[t * kWindow + best];
            if (t == 0) { assigned[best] = 1; perm[w0 + pos] = w0 + best; }
            ++pos;
            __syncthreads();
        }
    }
}

}  // namespace
}  // namespace sspmm_b200

extern "C" int svc_reorder(int M, int K, int vec_length, const int* d_csr_row_ptr, const int* d_csr_col_idx, int* d_perm,
                           void* stream) {
    using namespace sspmm_b200;
    set_error("%s", "");
    if (vec_length != 8 && vec_length != 16) {
        set_error("vec_length must be 8 or 16 (got %d)", vec_length);
        return (int)cudaErrorInvalidValue;
    }
    if (M < 0 || K < 0 || (M > 0 && (!d_csr_row_ptr || !d_perm))) {
        set_error("bad argument");
        return (int)cudaErrorInvalidValue;
    }
    if (M == 0) return 0;
    const size_t smem = (size_t)(kSigWords * kWindow + kSigWords) * 4 + 8 * 8 + kWindow * 4;
    static DeviceOnce once;
    if (!once.done()) {
        cudaError_t e = cudaFuncSetAttribute(svc_reorder_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { set_error("reorder set-up: %s", cudaGetErrorString(e)); return (int)e; }
        once.mark();
    }
    svc_reorder_kernel<<<(M + kWindow - 1) / kWindow, kWindow, smem, static_cast<cudaStream_t>(stream)>>>(
        M, K, vec_length, d_csr_row_ptr, d_csr_col_idx, d_perm);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("reorder launch: %s", cudaGetErrorString(e)); return (int)e; }
    return 0;
}
