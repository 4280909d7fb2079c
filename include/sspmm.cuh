// C++ link-level drop-in for the reference kernel library: a driver written
// against SSpMM/include/sspmm.cuh (e.g. SSpMM/sspmm_test.cpp:141,189) compiles
// and links against libsspmm_b200.so unchanged.  Every overload forwards to the
// C ABI in sspmm_b200.h on the legacy default stream and returns its status as
// a cudaError_t.  Unlike the reference's kernel these calls may take scratch from
// the stream-ordered allocator and synchronise once per new row_offsets pointer;
// sspmm_b200.h ("What the regular entry points do behind the call") has the details.
//
// The driver passes (m_vec, vec_length, N, K) to BOTH families below
// (SSpMM/sspmm_test.cpp:141 and :189), whatever the parameter names say, so
// both take the dense operand's column count third and its row count fourth.
#pragma once
#ifndef SSPMM_H
#define SSPMM_H
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace spmm {

#define SSPMM_B200_OPERANDS(VT)                                                   \
    const int* __restrict__ row_indices, const int* __restrict__ row_offsets,     \
    const int* __restrict__ column_indices, const VT* __restrict__ values,        \
    const VT* __restrict__ rhs_matrix

// Replaces SSpMM/src/sspmm.cu:626-649 (fp32 and fp16 output).
cudaError_t SSpMM(int m_vec, int vec_length, int N, int K, SSPMM_B200_OPERANDS(half), float* __restrict__ output_matrix);
cudaError_t SSpMM(int m_vec, int vec_length, int N, int K, SSPMM_B200_OPERANDS(half), half* __restrict__ output_matrix);
// Replaces SSpMM/src/sspmm.cu:651-661: prints that fp32 input is unsupported, returns cudaSuccess.
cudaError_t SSpMM(int m_vec, int vec_length, int N, int K, SSPMM_B200_OPERANDS(float), float* __restrict__ output_matrix);

// The reference's older m8n8k4 family (SSpMM/src/sspmm.cu:504-546) computes the
// same product; here it is an alias of the same kernels.
cudaError_t SpMM(int m_vec, int vec_length, int k, int n, SSPMM_B200_OPERANDS(half), float* __restrict__ output_matrix);
cudaError_t SpMM(int m_vec, int vec_length, int k, int n, SSPMM_B200_OPERANDS(half), half* __restrict__ output_matrix);
cudaError_t SpMM(int m_vec, int vec_length, int k, int n, SSPMM_B200_OPERANDS(float), float* __restrict__ output_matrix);

#undef SSPMM_B200_OPERANDS

}  // namespace spmm
#endif  // SSPMM_H
