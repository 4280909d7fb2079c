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
 * Asynchronous on `stream` except for the first call with a given row_offsets pointer; see
 * "What the regular entry points do behind the call" below for allocation and remembered state.
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
 * kernel needs no scratch).  Always runs the block kernel; its scratch (a dense transposed copy of
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

/*
 * What the regular entry points (sspmm_f16_f32, sspmm_f16_f16, sspmm_f16_f16_batched) do behind the
 * call.  The reference's kernel needs no scratch and its driver owns every buffer
 * (SSpMM/sspmm_test.cpp:108-127, 256-262); these entry points keep that signature but not that
 * property:
 *   - the choice between the row-gather kernel and the block kernel needs nvec = row_offsets[m_vec]
 *     on the host.  It is read with a device-to-host copy and a synchronisation of `stream` the
 *     first time a (row_offsets pointer, m_vec, device) triple is seen and remembered in a table of
 *     64 entries keyed by that triple.  A freed and re-used pointer therefore gets the previous
 *     matrix's nvec: the result is still right (every kernel accepts every operand), only the
 *     choice of kernel may be the slower one.  While `stream` is being captured nothing is read
 *     and the row-gather kernel is used;
 *   - the block kernel takes K * m_vec*V * 2 bytes (a dense transposed copy of A), plus fp32
 *     partial tiles when it splits K, from cudaMallocAsync on `stream` and returns them with
 *     cudaFreeAsync; the row-gather kernel does the same for the partial tiles of split long rows;
 *   - once per device the release threshold of the device's default memory pool is raised to 1 GiB
 *     so that this scratch is not returned to the system at every synchronisation.
 * Callers that must not allocate or synchronise at call time use a plan (below), or
 * sspmm_f16_f16_noalloc.
 */

/*
 * The same product as sspmm_f16_f16 for a caller that owns every buffer, as the reference's driver
 * does (SSpMM/sspmm_test.cpp:108-127, 256-262): the vector count nvec = row_offsets[m_vec] is passed
 * in (the compression returns it) and the scratch is the caller's, so the call reads nothing back,
 * allocates nothing, remembers nothing and never synchronises.  sspmm_workspace_bytes reports what
 * the kernel chosen for these sizes would like (0 for most sparse operands).  With less, long
 * vector rows are not split (slower, same result); the dense-ish (block) kernel needs at least
 * K * m_vec*V * 2 bytes and rejects less.  The workspace must stay untouched until the call's work
 * on `stream` has finished; 256-byte alignment.
 */
int sspmm_workspace_bytes(int m_vec, int vec_length, int N, int K, int64_t nvec, int out_is_f16, int64_t* bytes);
int sspmm_f16_f16_ws(int m_vec, int vec_length, int N, int K, const int* row_indices, const int* row_offsets,
                     const int* column_indices, const void* values_f16, const void* rhs_f16, void* out_f16, int64_t nvec,
                     void* workspace, int64_t workspace_bytes, void* stream);

/* --------------------------------------------- plans and groups (one launch) --- */

/*
 * The entry points above follow the reference's calling convention, which has no place for anything
 * computed ahead of time: they must work for whatever arrays they are handed, so for dense-ish
 * matrices they expand A into scratch from the stream-ordered allocator and launch two or three
 * kernels (see "What the regular entry points do behind the call" at the end of this header).
 * A PLAN is the ahead-of-time part: built once per weight STRUCTURE (row_offsets and
 * column_indices, which must stay alive and unchanged while the plan is used; the VALUES may
 * change between calls), it lets the product run as ONE kernel launch straight from the compressed
 * operand, with no scratch, no allocation and no host synchronisation at call time.
 * The reference has no counterpart (its kernel, SSpMM/src/sspmm.cu:548-649, needs none: one launch,
 * no scratch); a maintainer of SSpMM/sspmm_test.cpp would create the plan after the cudaMemcpy calls
 * at :120-127 and call sspmm_planned in the timed loop at :189.
 *
 * sspmm_plan_create reads nvec, allocates the plan's device metadata (16 bytes per vector row and 64
 * columns, plus 4 bytes per vector when some row's column list is not ascending) and synchronises
 * `stream` twice.  Structures that are too sparse for dense tiles (fewer than 1/16 of the
 * (vector row, column) slots filled), or irregular (a column listed twice in a vector row, a column
 * id outside [0, K)), get a plan without metadata: sspmm_planned then forwards to
 * sspmm_f16_f16 / sspmm_f16_f32, and such a plan cannot join a group.
 */
typedef struct sspmm_plan sspmm_plan;
int sspmm_plan_create(int m_vec, int vec_length, int K, const int* d_row_offsets, const int* d_column_indices,
                      void* stream, sspmm_plan** plan);
int sspmm_plan_destroy(sspmm_plan* plan);
/* Any output pointer may be NULL.  one_launch = 1 when the plan carries metadata. */
int sspmm_plan_info(const sspmm_plan* plan, int64_t* nvec, int* one_launch, int* ascending, int64_t* device_bytes);

/* out[m_vec*V][N] = A_vs * rhs[K][N] with the plan's structure: one launch on `stream`, nothing
 * allocated, no host synchronisation (N % 8 == 0; values, rhs, out 16-byte aligned; out fp16 when
 * out_is_f16 != 0, else fp32). */
int sspmm_planned(const sspmm_plan* plan, const void* values_f16, const void* rhs_f16, void* out, int N, int out_is_f16,
                  void* stream);

/*
 * A GROUP binds several products (the layers of a model step, the members of a batch) to their
 * operands and runs all of them as one persistent tensor-core launch: the tiles of all products
 * form one work list, longest first, taken by the CTAs from a shared queue, so that small products
 * fill the SMs a large one leaves idle; tiles with a long K range are cut into parts whose fp32
 * partial tiles are added, in part order, by whichever part finishes last.
 * Every mode is ONE launch per run.
 * mode 1 (compressed): the A tiles are built inside the kernel from the compressed operand, in
 *     registers, by eight loader warps per CTA; no scratch for A;
 * mode 2 (expanded): the loader warps of all CTAs first write dense transposed copies of the A
 *     operands (K * m_vec*V * 2 bytes per product, owned by the group), block by block and in the
 *     order the products are multiplied, while the other warps already multiply; the tensor-core
 *     warps fetch their A tiles from the copies by TMA once a product's copy is complete.  About a
 *     quarter less time per K step, which pays off once every SM has a few dozen K steps of work;
 * mode 3 (expanded, CTA pairs): as mode 2 with tiles of 256 rows x 256 columns computed by two
 *     CTAs of a cluster (tcgen05 cta_group::2, each CTA fetching its own 128 rows of A and half of
 *     the B tile).  Measured no faster than mode 2 on the conv workload (products with fewer than
 *     256 rows pay for the padding), so never chosen automatically;
 * mode 0: 1 or 2, chosen from the amount of work per SM.
 * Products of one group that multiply the same dense operand (same rhs pointer, N and K) are
 * scheduled panel by panel, so that a column panel of B is fetched from HBM once for all of them.
 * sspmm_group_create allocates the descriptors and the scratch once (and synchronises);
 * sspmm_group_run allocates nothing and does not synchronise.  Operand pointers are fixed at
 * creation; the contents of every operand, the values included, may change between runs.  A group
 * must not run twice at the same time (its queue and scratch serve one run at a time), and the
 * current device must be the one it was created on.
 */
typedef struct sspmm_group sspmm_group;
typedef struct sspmm_group_item {
    const sspmm_plan* plan;
    const void* values_f16;
    const void* rhs_f16;   /* [K][N] */
    void* out;             /* [m_vec*V][N] */
    int N;
} sspmm_group_item;
int sspmm_group_create(const sspmm_group_item* items, int count, int out_is_f16, int mode, sspmm_group** group);
int sspmm_group_run(sspmm_group* group, void* stream);
/* Any output pointer may be NULL.  launches = kernels per run (always 1). */
int sspmm_group_info(const sspmm_group* group, int* tile_columns, int* work_items, int* ctas, int* launches,
                     int64_t* scratch_bytes);
int sspmm_group_destroy(sspmm_group* group);

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

/*
 * The same compression for a BATCH of independent matrices in one pass (a sweep over many
 * matrices, RowMerge/sparse_matrix_format.py:199-237 and RowMerge/suit_sparse_matrix.py:199-216
 * loop over them one by one).  HOST arrays of `count` sizes and of `count` DEVICE pointers;
 * d_csr_values_f16 may be NULL (structure only, as the reference).  The matrices are stacked on the
 * device and compressed together; svc_batch_begin returns each matrix's vector count in nvec[count]
 * (synchronises `stream`), svc_batch_finish writes the results of all matrices one after another:
 *   d_vec_row_ptr   sum(m_vec_i + 1) ints, matrix i's pointers starting again at 0
 *   d_vec_col       sum(nvec_i) ints          d_vec_values   sum(nvec_i) * V fp16 (or NULL)
 * so matrix i's pieces start at the running sums of (m_vec + 1), nvec and nvec * V.  Column order
 * inside every vector row is the reference's, as in svc_begin.
 */
typedef struct svc_batch_job svc_batch_job;
int svc_batch_begin(int count, int vec_length, const int* M, const int* K, const int* nnz,
                    const int* const* d_csr_row_ptr, const int* const* d_csr_col_idx, const void* const* d_csr_values_f16,
                    void* stream, svc_batch_job** job, int64_t* nvec);
int svc_batch_finish(svc_batch_job* job, int* d_vec_row_ptr, int* d_vec_col, void* d_vec_values_f16, void* stream);
int svc_batch_free(svc_batch_job* job);
/* Vector rows of the whole batch that needed the hash-order replay; valid after svc_batch_begin. */
int svc_batch_replayed_rows(svc_batch_job* job, int64_t* rows);

/* Number of vector rows whose column order needed the hash-order replay (the
 * others are ascending); diagnostic, valid after svc_begin. */
int svc_replayed_rows(svc_job* job, int64_t* rows);

/*
 * Row swizzle: vector rows by decreasing length, ties by increasing row id.
 * Replaces SortedRowSwizzle, SSpMM/include/bm_test_utils.h:210-225 (std::sort
 * there leaves the order of ties unspecified).  d_row_indices[m_vec].
 * Asynchronous on stream.  Above 8192 vector rows the rows are sorted, with
 * 8 bytes of scratch per row (next power of two) from the stream-ordered pool.
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
