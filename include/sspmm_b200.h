/*
 * sspmm_b200 -- C ABI of the B200 (sm_100a) implementation of sparse vector
 * compression (SVC) and of the vector-sparse SpMM  C = A_vs * B.
 *
 * Plain pointers and sizes only.  All pointers named d_* and all SpMM operand
 * pointers are DEVICE pointers on the current CUDA device; `stream` is a
 * cudaStream_t passed as void* (NULL = legacy default stream).  Every function
 * returns 0 on success, otherwise a cudaError_t value (1 = invalid argument);
 * sspmm_last_error_string() describes the last failure on the calling thread.
 * No function prints, traps, or falls back to the CPU.
 *
 * Compressed format (the reference's "CVSE", RowMerge/sparse_matrix_format.py:94-175,
 * read back by SSpMM/sspmm_test.cpp:28-64):
 *   m_vec                     = ceil(M / V) vector rows, V in {8, 16}
 *   row_offsets[m_vec + 1]    first vector of each vector row; nvec = row_offsets[m_vec]
 *   column_indices[nvec]      column shared by the V entries of a vector
 *   values[nvec * V]  (fp16)  values[j*V + v] = A[i*V + v][column_indices[j]] for j in row i
 */
#ifndef SSPMM_B200_H
#define SSPMM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ SpMM --- */

/*
 * out[m_vec*V][N] (row-major, fully overwritten) = A_vs * rhs[K][N], fp16
 * operands, fp32 accumulation, fp32 output.
 * Replaces spmm::SSpMM(..., float* output_matrix), SSpMM/src/sspmm.cu:626-636
 * (declared SSpMM/include/sspmm.cuh:31-37); called at SSpMM/sspmm_test.cpp:189.
 * row_indices (may be NULL) is a permutation of 0..m_vec-1 giving the order in
 * which vector rows are scheduled (the reference's row swizzle,
 * SSpMM/include/bm_test_utils.h:206-225); it never changes the result.
 * Asynchronous on `stream`; allocates nothing; keeps no state.
 */
int sspmm_f16_f32(int m_vec, int vec_length, int N, int K, const int* row_indices, const int* row_offsets,
                  const int* column_indices, const void* values_f16, const void* rhs_f16, float* out_f32,
                  void* stream);

/* Same with fp16 output (round to nearest even of the fp32 accumulator).
 * Replaces spmm::SSpMM(..., half* output_matrix), SSpMM/src/sspmm.cu:638-649. */
int sspmm_f16_f16(int m_vec, int vec_length, int N, int K, const int* row_indices, const int* row_offsets,
                  const int* column_indices, const void* values_f16, const void* rhs_f16, void* out_f16, void* stream);

/*
 * Batched form: `batch` products sharing row_offsets / column_indices, operand b
 * at values + b*values_stride, rhs + b*rhs_stride, out + b*out_stride (strides in
 * elements; values_stride 0 shares one value array).  fp16 output.
 * Replaces batched_spmm_cuda, end2end/sspmm_e2e/src/cuda/spmm_kernel.cu:516-586
 * (batch in grid.z, strides at :527-529); batch = 1 replaces spmm_cuda, :460-514.
 */
int sspmm_f16_f16_batched(int m_vec, int vec_length, int N, int K, int batch, const int* row_indices,
                          const int* row_offsets, const int* column_indices, const void* values_f16,
                          int64_t values_stride, const void* rhs_f16, int64_t rhs_stride, void* out_f16,
                          int64_t out_stride, void* stream);

/*
 * Same product as sspmm_f16_f16, for callers that must not allocate device memory when they call:
 * a server that gave all device memory to its own arena at start-up, or a latency-critical loop
 * in which an allocation could fail or stall other streams.  No counterpart in the reference (its
 * kernels need no scratch).  Always runs the block kernel; its scratch (a dense transposed copy of
 * A) lives in a fixed array inside the library image, so
 *   - K * m_vec * vec_length * 2 must not exceed SSPMM_NOALLOC_MAX_SCRATCH_BYTES, K > 0,
 *     N % 8 == 0, values / rhs / out 16-byte aligned; anything else is rejected with an error;
 *   - every GPU that loads the library holds that array until the process exits;
 *   - all calls on a device share it: two calls whose GPU work overlaps (different streams) race.
 *     Calls on one stream are safe, and nothing a call leaves in the array is read by the next;
 *   - the first call on each device looks up the array's device address; make that first call
 *     before starting any stream capture.
 * Calls no cudaMalloc / cudaFree / allocating library routine.
 */
#define SSPMM_NOALLOC_MAX_SCRATCH_BYTES (8u << 20)
int sspmm_f16_f16_noalloc(int m_vec, int vec_length, int N, int K, const int* row_indices, const int* row_offsets,
                          const int* column_indices, const void* values_f16, const void* rhs_f16, void* out_f16,
                          void* stream);

/* Kernel selection for the calls above: 0 = automatic (default), 1 = tensor-core
 * row-gather kernel fed by TMA gather requests (error if the operands do not qualify),
 * 2 = CUDA-core kernel only, 3 = tensor-core block kernel only, 4 = tensor-core
 * row-gather kernel fed by load instructions, 5 = block kernel only and without its
 * CTA-pair variant (one CTA per tile).  Process-wide; for tests and profiling. */
int sspmm_set_kernel(int which);

/* Reads (and clears) the device-side status word of the current device:
 * 0 = healthy, otherwise the code of the first bounded wait that gave up
 * inside a kernel.  Synchronises the device. */
int sspmm_device_status(int* status);

/*
 * Self test of the bounded device-side waits.  Every wait on an mbarrier inside the kernels gives
 * up after a cycle budget (about two seconds), records a status code and lets the kernel return
 * instead of spinning.  This call shortens the budget to `limit_cycles` for one launch of a
 * one-thread kernel that waits on a barrier nobody arrives at, restores the budget, and reports
 * whether the wait gave up (*gave_up = 1).  Afterwards sspmm_device_status() returns 6 once.
 * Synchronises the device before and after; nothing traps, faults or spins without bound.
 * No counterpart in the reference (its kernels have no waits).
 */
int sspmm_selftest_wait_expiry(long long limit_cycles, int* gave_up);

/* ------------------------------------------------------------------- SVC --- */

typedef struct svc_job svc_job;

/*
 * Sparse vector compression of a CSR matrix (M x K, int32 row pointers and
 * column ids, optional fp16 values) into vector rows of V consecutive matrix
 * rows.  Replaces CVSE.__init__, RowMerge/sparse_matrix_format.py:94-123 (called
 * from generate_CVSE_file :224 and generate_suitesparse_CVSE_file,
 * RowMerge/suit_sparse_matrix.py:211); column order inside a vector row is
 * bit-identical to that code run under CPython 3.12.
 *
 * Two phases because nvec is data dependent:
 *   svc_begin   counts, scans, returns nvec (synchronises `stream`);
 *   svc_finish  writes d_vec_row_ptr[m_vec+1], d_vec_col[nvec] and, when both
 *               d_csr_values and d_vec_values are non-NULL, d_vec_values[nvec*V]
 *               (fp16, zero-filled where A has no entry).  Asynchronous.
 *   svc_free    releases the job (after svc_finish's work has been enqueued).
 * Scratch is taken from the stream-ordered allocator of the current device.
 */
int svc_begin(int M, int K, int vec_length, const int* d_csr_row_ptr, const int* d_csr_col_idx,
              const void* d_csr_values_f16, void* stream, svc_job** job, int64_t* nvec);
int svc_finish(svc_job* job, int* d_vec_row_ptr, int* d_vec_col, void* d_vec_values_f16, void* stream);
int svc_free(svc_job* job);

/* Number of vector rows whose column order needed the hash-order replay (the
 * others are ascending); diagnostic, valid after svc_begin. */
int svc_replayed_rows(svc_job* job, int64_t* rows);

/*
 * Row swizzle: vector rows by decreasing length, ties by increasing row id.
 * Replaces SortedRowSwizzle, SSpMM/include/bm_test_utils.h:210-225 (std::sort
 * there leaves the order of ties unspecified).  d_row_indices[m_vec].
 */
int sspmm_sorted_row_swizzle(int m_vec, const int* d_row_offsets, int* d_row_indices, void* stream);

/*
 * Row reordering before compression: d_perm[M] = new order of the rows of A (row d_perm[r]
 * becomes row r), grouping rows that share columns inside windows of 256 rows so that fewer V x 1
 * vectors are non-zero.  Stands where the reference runs row_merge_reorder.py (README.md:36; data
 * sets read at SSpMM/sspmm_test.cpp:313-319); that script is absent from the reference checkout, so
 * this is an extension with its own definition (csrc/reorder.cu), not a bit-exact replacement.
 */
int svc_reorder(int M, int K, int vec_length, const int* d_csr_row_ptr, const int* d_csr_col_idx, int* d_perm,
                void* stream);

/* ------------------------------------------------------------- .smtx files --- */

/*
 * The three-line text format between the two stages: "rows, cols, nnz" / row pointers / column
 * ids.  HOST pointers.  smtx_write replaces CVSE_out, RowMerge/sparse_matrix_format.py:152-175
 * (byte-identical output); smtx_read_header + smtx_read replace the parsers at
 * SSpMM/sspmm_test.cpp:28-64 and RowMerge/sparse_matrix_format.py:8-25.  For a compressed file
 * rows = m_vec and nnz = the ORIGINAL non-zero count (the vector count is row_ptr[m_vec]).
 */
int smtx_read_header(const char* path, int* rows, int* cols, int* nnz, int64_t* n_row_ptr, int64_t* n_col_idx);
int smtx_read(const char* path, int* row_ptr, int64_t n_row_ptr, int* col_idx, int64_t n_col_idx);
int smtx_write(const char* path, int rows, int cols, int nnz, const int* row_ptr, int64_t n_row_ptr,
               const int* col_idx, int64_t n_col_idx);

/* ------------------------------------------------------------------ misc --- */

const char* sspmm_last_error_string(void);
/* "sspmm_b200 <version> sm_100a" */
const char* sspmm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SSPMM_B200_H */
