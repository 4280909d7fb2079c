// Sparse vector compression (SVC) on the GPU: internal interface.
//
// Computes what the reference's CVSE.__init__ computes on the CPU
// (RowMerge/sparse_matrix_format.py:94-123): vector row i covers matrix rows
// V*i .. V*i+V-1; its column list is the union of those rows' column ids, in
// the order CPython's  list(set(previous + row))  leaves them after V rebuilds.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sspmm_b200 {

// Largest K the bitmap kernels accept (bitmap of K bits + a 32-bit prefix per
// word must fit one CTA's shared memory).
constexpr int kSvcMaxK = 262144;

struct SvcProblem {
    int M, K, V, m_vec;
    const int* row_ptr;   // [M+1]
    const int* col_idx;   // [nnz]
    const __half* vals;   // [nnz] or null
};

// Scratch owned by one compression.  Sizes in elements.
struct SvcScratch {
    int* vec_ptr;         // [m_vec+1]  counts, then exclusive scan = vector row pointers
    int* mode;            // [m_vec]    0 = ascending order is exact, 1 = replay the hash table
    int* tbl_len;         // [m_vec]    final table length of replayed groups (0 otherwise; -1: ascending and large)
    long long* tbl_off;   // [m_vec+1]  exclusive scan of per-group table scratch
    long long* totals;    // [kSvcTotals] {nvec, scratch ints, groups per list segment (kSvcSegs; [0] = ascending order), bad-column flag}
    int* tables;          // [totals[1]] replay scratch, allocated after the counting pass
    int* class_list;      // [m_vec]    replayed groups, class by class (written by the scan)
    int* queue;           // [8]        work counters of the replay classes
    long long* block_sums;  // [svc_scan_blocks(m_vec) * kSvcScanFields] partial sums of the scans
};

// Number of blocks the scan kernels cut m_vec groups into.
inline long long svc_scan_blocks(long long m_vec) { return m_vec > 0 ? (m_vec + 4095) / 4096 : 1; }

constexpr int kSvcClasses = 7;                 // ascending order, and six size classes of replayed groups
constexpr int kSvcSegs = 18;                   // segments of the list of replayed groups (classes, some cut by size)
constexpr int kSvcTotals = 3 + kSvcSegs;
constexpr int kSvcScanFields = 2 + kSvcSegs;   // numbers per block of the scans

// Pass 1: per-group distinct counts, mode decision, scans.  Asynchronous on `stream`.
cudaError_t svc_count_and_scan(const SvcProblem& p, const SvcScratch& s, bool with_values, cudaStream_t stream);
// Pass 2: emits column lists (and value vectors when out_vals != null; out_vals must be zero-filled).
// seg_groups = totals[2..2+kSvcSegs) read back by the host (launches are skipped for empty classes).
cudaError_t svc_emit(const SvcProblem& p, const SvcScratch& s, const long long* seg_groups, int* out_col,
                     __half* out_vals, cudaStream_t stream);

// ---- batches: several independent matrices compressed as one stacked matrix ----------------
// Vector rows are independent of one another and their column order does not depend on K, so a batch
// is stacked into one tall CSR (each matrix padded with empty rows to a multiple of V rows, so that
// no vector row straddles two matrices) and compressed in one pass.
struct SvcBatchEntry {
    const int* row_ptr;
    const int* col_idx;
    const __half* vals;
    long long row_base;      // first stacked row (a multiple of V)
    long long nnz_base;      // first stacked entry
    long long vec_row_base;  // first stacked vector row
    int M, nnz;
};
// tab has count + 1 entries (the last one carries the totals).  Builds the stacked CSR.
cudaError_t svc_stack(const SvcBatchEntry* tab, int count, long long rows, long long entries, int V, int* row_ptr,
                      int* col_idx, __half* vals, cudaStream_t stream);
// cuts[m] = vec_ptr[first vector row of matrix m] for m in 0..count.
cudaError_t svc_batch_cuts(const SvcBatchEntry* tab, int count, const int* vec_ptr, long long* cuts, cudaStream_t stream);
// out: for every matrix its m_vec + 1 row pointers, rebased to 0, matrices one after another.
cudaError_t svc_batch_row_ptrs(const SvcBatchEntry* tab, int count, long long vec_rows, const int* vec_ptr,
                               const long long* cuts, int* out, cudaStream_t stream);

// Device flag set when a column id outside [0, K) was met (such entries are skipped).
cudaError_t svc_read_and_clear_bad_column_flag(int* flag, cudaStream_t stream);

}  // namespace sspmm_b200
