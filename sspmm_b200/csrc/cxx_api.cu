// namespace spmm overloads declared in include/sspmm.cuh, forwarding to the C ABI.
#include <cstdio>

#include "../../include/sspmm.cuh"
#include "../../include/sspmm_b200.h"

namespace spmm {

namespace {
// Unsupported vector length: the reference prints and launches nothing
// (SSpMM/src/sspmm.cu:582-586); an invalid-argument status is reported the same way.
inline cudaError_t finish(int rc, int vec_length) {
    if (rc != 0 && vec_length != 8 && vec_length != 16) {
        std::printf("Unsupported Vector Length!\n");
        return cudaGetLastError();
    }
    return static_cast<cudaError_t>(rc);
}
}  // namespace

cudaError_t SSpMM(int m_vec, int vec_length, int N, int K, const int* __restrict__ row_indices,
                  const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                  const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                  float* __restrict__ output_matrix) {
    return finish(sspmm_f16_f32(m_vec, vec_length, N, K, row_indices, row_offsets, column_indices, values, rhs_matrix,
                                output_matrix, nullptr), vec_length);
}

cudaError_t SSpMM(int m_vec, int vec_length, int N, int K, const int* __restrict__ row_indices,
                  const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                  const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                  half* __restrict__ output_matrix) {
    return finish(sspmm_f16_f16(m_vec, vec_length, N, K, row_indices, row_offsets, column_indices, values, rhs_matrix,
                                output_matrix, nullptr), vec_length);
}

cudaError_t SSpMM(int, int, int, int, const int* __restrict__, const int* __restrict__, const int* __restrict__,
                  const float* __restrict__, const float* __restrict__, float* __restrict__) {
    std::printf("wmmaSpmm doesn't support float input.\n");
    return cudaSuccess;
}

cudaError_t SpMM(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                 const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                 const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                 float* __restrict__ output_matrix) {
    return SSpMM(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix, output_matrix);
}

cudaError_t SpMM(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                 const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                 const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                 half* __restrict__ output_matrix) {
    return SSpMM(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix, output_matrix);
}

cudaError_t SpMM(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                 const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                 const float* __restrict__ values, const float* __restrict__ rhs_matrix,
                 float* __restrict__ output_matrix) {
    return SSpMM(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, values, rhs_matrix, output_matrix);
}

}  // namespace spmm
