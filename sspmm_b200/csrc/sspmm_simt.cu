// CUDA-core variant of the vector-sparse SpMM for operands the tensor-core path
// cannot take: N not a multiple of 8, or pointers that are not 16-byte aligned.
// Same contract as the reference entry (SSpMM/src/sspmm.cu:626-649); fp32
// accumulation in the order of the column list.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "launch.h"

namespace sspmm_b200 {
namespace {

template <int V, typename OutT>
__global__ void __launch_bounds__(128)
sspmm_simt_kernel(int m_vec, int N, const int* __restrict__ row_indices, const int* __restrict__ row_offsets,
                  const int* __restrict__ col, const __half* __restrict__ values, const __half* __restrict__ rhs,
                  OutT* __restrict__ out, int64_t values_stride, int64_t rhs_stride, int64_t out_stride) {
    const int sched = blockIdx.x;
    const int i = row_indices ? row_indices[sched] : sched;
    if ((unsigned)i >= (unsigned)m_vec) return;
    const int n = blockIdx.y * 128 + threadIdx.x;
    const int b = blockIdx.z;
    values += b * values_stride;
    rhs += b * rhs_stride;
    out += b * out_stride;
    const int j0 = row_offsets[i], j1 = row_offsets[i + 1];
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    if (n < N) {
        for (int j = j0; j < j1; ++j) {
            const float bv = __half2float(rhs[(int64_t)col[j] * N + n]);
            const __half* a = values + (int64_t)j * V;
#pragma unroll
            for (int v = 0; v < V; ++v) acc[v] = fmaf(__half2float(a[v]), bv, acc[v]);
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int64_t o = ((int64_t)i * V + v) * N + n;
            if constexpr (sizeof(OutT) == 2) out[o] = __float2half_rn(acc[v]);
            else out[o] = acc[v];
        }
    }
}

template <int V, typename OutT>
cudaError_t run(const SpmmArgs& a) {
    dim3 grid(a.m_vec, (a.N + 127) / 128, a.batch);
    sspmm_simt_kernel<V, OutT><<<grid, 128, 0, a.stream>>>(a.m_vec, a.N, a.row_indices, a.row_offsets, a.column_indices,
                                                           a.values, a.rhs, static_cast<OutT*>(a.out), a.values_stride,
                                                           a.rhs_stride, a.out_stride);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_sspmm_simt(const SpmmArgs& a) {
    if (a.N > 128 * 65535 || a.batch > 65535) {
        set_error("N or batch too large for the CUDA-core path");
        return cudaErrorInvalidValue;
    }
    if (a.V == 16) return a.out_f16 ? run<16, __half>(a) : run<16, float>(a);
    return a.out_f16 ? run<8, __half>(a) : run<8, float>(a);
}

}  // namespace sspmm_b200
