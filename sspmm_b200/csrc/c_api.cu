// extern "C" entry points declared in include/sspmm_b200.h.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/sspmm_b200.h"
#include "launch.h"
#include "ptx.cuh"
#include "svc.cuh"

namespace sspmm_b200 {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

static std::atomic<int> g_kernel_choice{0};

static int fail(cudaError_t e, const char* what) {
    if (g_err[0] == 0) set_error("%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}

// The stream-ordered allocator returns memory to the OS at every synchronisation unless told to
// keep some; scratch is requested per call, so let the pool keep up to 1 GiB (once per device).
static void keep_pool_memory() {
    static DeviceOnce once;
    if (once.done()) return;
    int dev = 0;
    cudaMemPool_t pool;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
        unsigned long long cur = 0, want = 1ull << 30;
        if (cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &cur) == cudaSuccess && cur < want)
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &want);
    }
    once.mark();
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// nvec = row_offsets[m_vec] lives in device memory; the kernel choice needs it on
// the host.  It is read once per (pointer, m_vec, device) and remembered: weights
// are static across calls.  A stale entry can only make the choice of kernel
// suboptimal, never the result wrong (both kernels accept any operand).
struct NvecEntry { const int* ptr; int m_vec; int dev; long long nvec; };
static std::mutex g_nvec_mu;
static NvecEntry g_nvec_cache[64];
static int g_nvec_next = 0;

static long long lookup_nvec(const int* row_offsets, int m_vec, cudaStream_t st) {
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lk(g_nvec_mu);
        for (const NvecEntry& e : g_nvec_cache)
            if (e.ptr == row_offsets && e.m_vec == m_vec && e.dev == dev) return e.nvec;
    }
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return -1;
    int h = 0;
    if (cudaMemcpyAsync(&h, row_offsets + m_vec, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
    std::lock_guard<std::mutex> lk(g_nvec_mu);
    g_nvec_cache[g_nvec_next] = NvecEntry{row_offsets, m_vec, dev, h};
    g_nvec_next = (g_nvec_next + 1) % 64;
    return h;
}

// Modelled times (seconds) of the two tensor-core kernels; constants from measurements on B200.
// Gather kernel: one work item per (vector row, 128 output columns); an item costs about 1 us plus
// 0.9 us per 64 gathered rows while items are few (latency of the gather chain), and the whole kernel
// never beats 4 TB/s of gathered bytes.  Block kernel: expansion + dense GEMM, about 9 us of fixed cost
// (two or three dependent launches).
static bool block_kernel_is_faster(long long nvec, const SpmmArgs& a) {
    const double n = (double)a.N * a.batch;
    const double mp = (double)a.m_vec * a.V;
    const int sms = current_device_sm_count() > 0 ? current_device_sm_count() : 148;
    const double items = (double)a.m_vec * ((a.N + 127) / 128) * a.batch;
    const double waves = (items + sms - 1) / sms >= 1.0 ? (double)(long long)((items + sms - 1) / sms) : 1.0;
    const double steps = (double)nvec / (a.m_vec > 0 ? a.m_vec : 1) / 64.0;
    const double t_chain = waves * (1.0e-6 + steps * 0.9e-6);
    const double t_stream = 2.0 * (double)nvec * n / 4.0e12;
    const double t_gather = 3e-6 + (t_chain > t_stream ? t_chain : t_stream);
    const double t_block = 2.0 * mp * a.K * n / 6.0e14 + 4.0 * mp * a.K / 3e12 + 9e-6;
    return t_block < t_gather;
}

// Length-sorted scheduling order: rank by (length descending, row id ascending).
__global__ void __launch_bounds__(256)
row_swizzle_kernel(int m_vec, const int* __restrict__ row_offsets, int* __restrict__ row_indices) {
    __shared__ int tile_len[256];
    const int i = blockIdx.x * 256 + threadIdx.x;
    const int my = (i < m_vec) ? row_offsets[i + 1] - row_offsets[i] : 0;
    int rank = 0;
    for (int base = 0; base < m_vec; base += 256) {
        const int k = base + threadIdx.x;
        tile_len[threadIdx.x] = (k < m_vec) ? row_offsets[k + 1] - row_offsets[k] : -1;
        __syncthreads();
        const int lim = min(256, m_vec - base);
        for (int t = 0; t < lim; ++t) {
            const int l = tile_len[t];
            rank += (l > my || (l == my && base + t < i)) ? 1 : 0;
        }
        __syncthreads();
    }
    if (i < m_vec) row_indices[rank] = i;
}

// The same order for many rows: the rank loop above compares every row with every other (7e10 comparisons at
// 262 144 rows), so beyond a few thousand rows the rows are sorted instead.  Key = (2^32 - 1 - length) in the high
// word, row id in the low word: all keys differ, ascending keys are the wanted order.  Bitonic network over the next
// power of two of keys in global memory (padding keys are all ones and end up last).
constexpr int kSwizzleRankLimit = 8192;
__global__ void __launch_bounds__(256)
swizzle_keys_kernel(int m_vec, long long padded, const int* __restrict__ row_offsets, unsigned long long* __restrict__ keys) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= padded) return;
    unsigned long long k = ~0ull;
    if (i < m_vec) {
        const unsigned len = (unsigned)max(0, row_offsets[i + 1] - row_offsets[i]);
        k = ((unsigned long long)(0xffffffffu - len) << 32) | (unsigned)i;
    }
    keys[i] = k;
}
__global__ void __launch_bounds__(256)
swizzle_bitonic_kernel(long long padded, long long j, long long k, unsigned long long* __restrict__ keys) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= padded) return;
    const long long partner = i ^ j;
    if (partner <= i) return;
    const unsigned long long a = keys[i], b = keys[partner];
    const bool ascending = (i & k) == 0;
    if ((a > b) == ascending) { keys[i] = b; keys[partner] = a; }
}
__global__ void __launch_bounds__(256)
swizzle_write_kernel(int m_vec, const unsigned long long* __restrict__ keys, int* __restrict__ row_indices) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < m_vec) row_indices[i] = (int)(keys[i] & 0xffffffffull);
}

// Wait-expiry self test: one thread waits on an mbarrier that nobody arrives at.  The bounded wait
// must give up after g_wait_cycle_limit cycles, record kStatusWaitSelfTest and let the kernel return.
__global__ void wait_expiry_selftest_kernel(int* gave_up) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
        const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, kStatusWaitSelfTest);
        *gave_up = ok ? 0 : 1;
    }
}

// Caller-provided knowledge and room: with nvec >= 0 nothing is read back from the device, with a workspace nothing
// is allocated.  query != null: only report the workspace size the chosen kernel wants, launch nothing.
struct SpmmExtra {
    long long nvec = -1;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    bool caller_workspace = false;
    size_t* query = nullptr;
};

static int spmm_entry(int m_vec, int V, int N, int K, int batch, const int* row_indices, const int* row_offsets,
                      const int* column_indices, const void* values, int64_t values_stride, const void* rhs,
                      int64_t rhs_stride, void* out, int64_t out_stride, bool out_f16, void* stream,
                      const SpmmExtra& ex = SpmmExtra()) {
    g_err[0] = 0;
    if (V != 8 && V != 16) {
        set_error("vec_length must be 8 or 16 (got %d)", V);
        return (int)cudaErrorInvalidValue;
    }
    if (m_vec < 0 || N < 0 || K < 0 || batch < 0) {
        set_error("negative dimension (m_vec=%d N=%d K=%d batch=%d)", m_vec, N, K, batch);
        return (int)cudaErrorInvalidValue;
    }
    if (ex.query) *ex.query = 0;
    if (m_vec == 0 || N == 0 || batch == 0) return 0;
    if (!ex.query && (!row_offsets || !out || (K > 0 && (!column_indices || !values || !rhs)))) {
        set_error("null operand pointer");
        return (int)cudaErrorInvalidValue;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    SpmmArgs a;
    a.m_vec = m_vec; a.V = V; a.N = N; a.K = K;
    a.row_indices = row_indices; a.row_offsets = row_offsets; a.column_indices = column_indices;
    a.values = static_cast<const __half*>(values); a.rhs = static_cast<const __half*>(rhs);
    a.out = out; a.out_f16 = out_f16; a.batch = batch;
    a.values_stride = values_stride; a.rhs_stride = rhs_stride; a.out_stride = out_stride;
    a.stream = st;

    const int choice = g_kernel_choice.load();
    const bool tc_ok = K > 0 && (N % 8 == 0) && aligned16(rhs) && aligned16(values) &&
                       (values_stride * 2) % 16 == 0 && (batch == 1 || rhs_stride == (int64_t)K * N);
    if (choice == 1 && !tc_ok) {
        set_error("tensor-core kernel needs N %% 8 == 0, 16-byte aligned values/rhs and contiguous batches");
        return (int)cudaErrorInvalidValue;
    }
    cudaError_t e;
    if (K == 0 || choice == 2 || !tc_ok) {
        if (ex.query) return 0;
        e = launch_sspmm_simt(a);
        return e == cudaSuccess ? 0 : fail(e, "SpMM launch");
    }
    const int64_t oes = out_f16 ? 2 : 4;
    const bool block_ok = (batch == 1 || (values_stride == 0 && (rhs_stride * 2) % 16 == 0 && (out_stride * oes) % 16 == 0)) &&
                          aligned16(out) && ((int64_t)N * oes) % 16 == 0 &&
                          sspmm_block_scratch_bytes(a) <= ((size_t)2 << 30);
    if (choice == 3 && !block_ok) {
        set_error("block kernel needs 16-byte aligned output, a shared value array for batches and <= 2 GiB of scratch");
        return (int)cudaErrorInvalidValue;
    }
    if (choice == 1) {                                     // TMA row-gather producers
        if (ex.query) return 0;
        e = launch_sspmm_gather(a);
        return e == cudaSuccess ? 0 : fail(e, "SpMM launch");
    }
    bool use_block = choice == 3;
    long long nvec = ex.nvec;
    if (nvec < 0 && !ex.query && (choice == 0 || choice == 4)) nvec = lookup_nvec(row_offsets, m_vec, st);
    if (choice == 0 && block_ok) use_block = nvec >= 0 && block_kernel_is_faster(nvec, a);
    if (!use_block) {                                      // gather kernel with load-instruction producers
        int chunk = 0, cap = 0;
        size_t bytes = 0;
        sspmm_gather_lsu_plan(a, nvec, &chunk, &cap, &bytes);
        if (ex.query) { *ex.query = bytes; return 0; }
        void* scratch = nullptr;
        if (ex.caller_workspace) {
            if (bytes > ex.workspace_bytes) {          // too small: long rows are not split (slower, same result)
                chunk = 0; cap = 0;
                bytes = (ex.workspace && ex.workspace_bytes >= 16) ? 16 : 0;     // the work counter alone still fits
            }
            if (bytes) scratch = ex.workspace;
        } else if (bytes) {
            keep_pool_memory();
            e = cudaMallocAsync(&scratch, bytes, st);
            if (e != cudaSuccess) return fail(e, "scratch allocation for split rows");
        }
        e = launch_sspmm_gather_lsu(a, chunk, cap, bytes ? scratch : nullptr);
        if (scratch && !ex.caller_workspace) cudaFreeAsync(scratch, st);
        return e == cudaSuccess ? 0 : fail(e, "SpMM launch");
    }
    const size_t want = sspmm_block_scratch_bytes(a);
    if (ex.query) { *ex.query = want; return 0; }
    if (ex.caller_workspace) {
        const size_t need = (size_t)K * m_vec * V * sizeof(__half);
        if (ex.workspace_bytes < need || !ex.workspace) {
            set_error("workspace of %zu bytes is too small: the block kernel needs at least %zu (sspmm_workspace_bytes reports %zu)",
                      ex.workspace_bytes, need, want);
            return (int)cudaErrorInvalidValue;
        }
        e = launch_sspmm_block(a, ex.workspace, ex.workspace_bytes);
        return e == cudaSuccess ? 0 : fail(e, "SpMM launch");
    }
    void* scratch = nullptr;
    keep_pool_memory();
    e = cudaMallocAsync(&scratch, want, st);
    if (e != cudaSuccess) return fail(e, "scratch allocation for the block kernel");
    e = launch_sspmm_block(a, scratch, want);
    cudaFreeAsync(scratch, st);
    return e == cudaSuccess ? 0 : fail(e, "SpMM launch");
}

}  // namespace sspmm_b200

using namespace sspmm_b200;

struct svc_job {
    SvcProblem p;
    SvcScratch s;
    bool with_values;
    long long nvec;
    long long table_ints;
    long long class_groups[kSvcSegs];      // groups per list segment; [0] = groups whose ascending order is exact
    int device;
    cudaStream_t stream;
};

struct svc_batch_job {
    int count, V;
    long long rows, entries, vec_rows;
    bool with_values;
    svc_job* inner;              // the compression of the stacked matrix
    void* block;                 // table, cuts and the stacked CSR
    SvcBatchEntry* d_tab;
    long long* d_cuts;
    cudaStream_t stream;
};

extern "C" {

int sspmm_f16_f32(int m_vec, int vec_length, int N, int K, const int* row_indices, const int* row_offsets,
                  const int* column_indices, const void* values_f16, const void* rhs_f16, float* out_f32,
                  void* stream) {
    return spmm_entry(m_vec, vec_length, N, K, 1, row_indices, row_offsets, column_indices, values_f16, 0, rhs_f16, 0,
                      out_f32, 0, false, stream);
}

int sspmm_f16_f16(int m_vec, int vec_length, int N, int K, const int* row_indices, const int* row_offsets,
                  const int* column_indices, const void* values_f16, const void* rhs_f16, void* out_f16, void* stream) {
    return spmm_entry(m_vec, vec_length, N, K, 1, row_indices, row_offsets, column_indices, values_f16, 0, rhs_f16, 0,
                      out_f16, 0, true, stream);
}

int sspmm_f16_f16_batched(int m_vec, int vec_length, int N, int K, int batch, const int* row_indices,
                          const int* row_offsets, const int* column_indices, const void* values_f16,
                          int64_t values_stride, const void* rhs_f16, int64_t rhs_stride, void* out_f16,
                          int64_t out_stride, void* stream) {
    return spmm_entry(m_vec, vec_length, N, K, batch, row_indices, row_offsets, column_indices, values_f16,
                      values_stride, rhs_f16, rhs_stride, out_f16, out_stride, true, stream);
}

int sspmm_workspace_bytes(int m_vec, int vec_length, int N, int K, int64_t nvec, int out_is_f16, int64_t* bytes) {
    if (!bytes || nvec < 0) { g_err[0] = 0; set_error("bytes must be non-null and nvec >= 0"); return (int)cudaErrorInvalidValue; }
    SpmmExtra ex;
    size_t q = 0;
    ex.nvec = nvec; ex.query = &q;
    // aligned dummy operands: only sizes and alignment enter the choice of kernel
    void* dummy = reinterpret_cast<void*>(uintptr_t(256));
    const int rc = spmm_entry(m_vec, vec_length, N, K, 1, nullptr, nullptr, nullptr, dummy, 0, dummy, 0, dummy, 0, out_is_f16 != 0,
                              nullptr, ex);
    *bytes = (int64_t)q;
    return rc;
}

int sspmm_f16_f16_ws(int m_vec, int vec_length, int N, int K, const int* row_indices, const int* row_offsets,
                     const int* column_indices, const void* values_f16, const void* rhs_f16, void* out_f16, int64_t nvec,
                     void* workspace, int64_t workspace_bytes, void* stream) {
    if (nvec < 0 || workspace_bytes < 0) { g_err[0] = 0; set_error("nvec and workspace_bytes must be >= 0"); return (int)cudaErrorInvalidValue; }
    SpmmExtra ex;
    ex.nvec = nvec; ex.workspace = workspace; ex.workspace_bytes = (size_t)workspace_bytes; ex.caller_workspace = true;
    return spmm_entry(m_vec, vec_length, N, K, 1, row_indices, row_offsets, column_indices, values_f16, 0, rhs_f16, 0, out_f16, 0,
                      true, stream, ex);
}

int sspmm_set_kernel(int which) {
    if (which < 0 || which > 5) {
        set_error("kernel selector must be 0..5");
        return (int)cudaErrorInvalidValue;
    }
    sspmm_block_allow_pairs(which != 5);
    g_kernel_choice.store(which == 5 ? 3 : which);
    return 0;
}

int sspmm_device_status(int* status) {
    g_err[0] = 0;
    if (!status) return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(e, "device synchronize");
    e = cudaMemcpyFromSymbol(status, g_device_status, sizeof(int));
    if (e != cudaSuccess) return fail(e, "status read");
    if (*status != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
        if (e != cudaSuccess) return fail(e, "status clear");
    }
    return 0;
}

int sspmm_selftest_wait_expiry(long long limit_cycles, int* gave_up) {
    g_err[0] = 0;
    if (!gave_up || limit_cycles <= 0 || limit_cycles > kDefaultWaitCycleLimit) {
        set_error("limit_cycles must be in (0, %lld] and gave_up non-null", kDefaultWaitCycleLimit);
        return (int)cudaErrorInvalidValue;
    }
    *gave_up = -1;
    int* d_flag = nullptr;
    cudaError_t e = cudaDeviceSynchronize();                       // no other kernel of ours sees the short limit
    if (e == cudaSuccess) e = cudaMalloc(&d_flag, sizeof(int));
    if (e != cudaSuccess) return fail(e, "self test set-up");
    e = cudaMemcpyToSymbol(g_wait_cycle_limit, &limit_cycles, sizeof(long long));
    if (e == cudaSuccess) {
        wait_expiry_selftest_kernel<<<1, 32>>>(d_flag);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        const long long back = kDefaultWaitCycleLimit;
        const cudaError_t e2 = cudaMemcpyToSymbol(g_wait_cycle_limit, &back, sizeof(long long));
        if (e == cudaSuccess) e = e2;
    }
    if (e == cudaSuccess) e = cudaMemcpy(gave_up, d_flag, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(d_flag);
    return e == cudaSuccess ? 0 : fail(e, "wait-expiry self test");
}

int svc_begin(int M, int K, int vec_length, const int* d_csr_row_ptr, const int* d_csr_col_idx,
              const void* d_csr_values_f16, void* stream, svc_job** job, int64_t* nvec) {
    g_err[0] = 0;
    if (!job || !nvec) { set_error("null output pointer"); return (int)cudaErrorInvalidValue; }
    *job = nullptr;
    if (vec_length != 8 && vec_length != 16) {
        set_error("vec_length must be 8 or 16 (got %d)", vec_length);
        return (int)cudaErrorInvalidValue;
    }
    if (M < 0 || K < 0) { set_error("negative dimension"); return (int)cudaErrorInvalidValue; }
    if (K > kSvcMaxK) {
        set_error("K = %d exceeds the supported maximum of %d columns", K, kSvcMaxK);
        return (int)cudaErrorInvalidValue;
    }
    // d_csr_col_idx may be NULL when the matrix has no entries (it is then never read)
    if (!d_csr_row_ptr) { set_error("null CSR row pointer"); return (int)cudaErrorInvalidValue; }
    svc_job* j = new (std::nothrow) svc_job();
    if (!j) return (int)cudaErrorMemoryAllocation;
    memset(j, 0, sizeof *j);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    j->stream = st;
    cudaGetDevice(&j->device);
    j->p.M = M; j->p.K = K; j->p.V = vec_length; j->p.m_vec = (M + vec_length - 1) / vec_length;
    j->p.row_ptr = d_csr_row_ptr; j->p.col_idx = d_csr_col_idx;
    j->p.vals = static_cast<const __half*>(d_csr_values_f16);
    j->with_values = d_csr_values_f16 != nullptr;
    const size_t mv = (size_t)j->p.m_vec;
    // one allocation: vec_ptr[mv+1] | mode[mv] | tbl_len[mv] | class_list[mv] | queue[8] | pad | tbl_off[mv+1] | totals
    const size_t ints = (mv + 1) + mv + mv + mv + 8;
    const size_t ints_padded = (ints + 3) & ~(size_t)3;
    const size_t scan_blocks = (size_t)svc_scan_blocks((long long)mv);
    const size_t bytes = ints_padded * 4 + (mv + 1 + kSvcTotals + scan_blocks * kSvcScanFields) * 8;
    void* base = nullptr;
    keep_pool_memory();
    cudaError_t e = cudaMallocAsync(&base, bytes, st);
    if (e != cudaSuccess) { delete j; return fail(e, "scratch allocation"); }
    j->s.vec_ptr = static_cast<int*>(base);
    j->s.mode = j->s.vec_ptr + mv + 1;
    j->s.tbl_len = j->s.mode + mv;
    j->s.class_list = j->s.tbl_len + mv;
    j->s.queue = j->s.class_list + mv;
    j->s.tbl_off = reinterpret_cast<long long*>(static_cast<int*>(base) + ints_padded);
    j->s.totals = j->s.tbl_off + mv + 1;
    j->s.block_sums = j->s.totals + kSvcTotals;
    j->s.tables = nullptr;
    e = svc_count_and_scan(j->p, j->s, j->with_values, st);
    long long totals[kSvcTotals] = {0};
    if (e == cudaSuccess) e = cudaMemcpyAsync(totals, j->s.totals, sizeof totals, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    const int bad = (int)totals[2 + kSvcSegs];
    if (e != cudaSuccess || bad || totals[0] > 0x7fffffffLL) {
        cudaFreeAsync(base, st);
        delete j;
        if (e != cudaSuccess) return fail(e, "SVC counting pass");
        if (bad) set_error("CSR column id outside [0, K)");
        else set_error("more than 2^31-1 vectors");
        return (int)cudaErrorInvalidValue;
    }
    j->nvec = totals[0];
    j->table_ints = totals[1];
    for (int c = 0; c < kSvcSegs; ++c) j->class_groups[c] = totals[2 + c];
    *nvec = totals[0];
    *job = j;
    return 0;
}

int svc_finish(svc_job* j, int* d_vec_row_ptr, int* d_vec_col, void* d_vec_values_f16, void* stream) {
    g_err[0] = 0;
    if (!j || !d_vec_row_ptr || (j->nvec > 0 && !d_vec_col)) { set_error("null pointer"); return (int)cudaErrorInvalidValue; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(d_vec_row_ptr, j->s.vec_ptr, ((size_t)j->p.m_vec + 1) * 4, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return fail(e, "row pointer copy");
    if (j->nvec == 0) return 0;
    __half* ov = j->with_values ? static_cast<__half*>(d_vec_values_f16) : nullptr;
    if (ov) {
        e = cudaMemsetAsync(ov, 0, (size_t)j->nvec * j->p.V * sizeof(__half), st);
        if (e != cudaSuccess) return fail(e, "value clear");
    }
    if (j->table_ints > 0 && !j->s.tables) {
        e = cudaMallocAsync(reinterpret_cast<void**>(&j->s.tables), (size_t)j->table_ints * 4, st);
        if (e != cudaSuccess) return fail(e, "table scratch allocation");
    }
    e = svc_emit(j->p, j->s, j->class_groups, d_vec_col, ov, st);
    if (e != cudaSuccess) return fail(e, "SVC emit");
    j->stream = st;
    return 0;
}

int svc_free(svc_job* j) {
    if (!j) return 0;
    if (j->s.tables) cudaFreeAsync(j->s.tables, j->stream);
    if (j->s.vec_ptr) cudaFreeAsync(j->s.vec_ptr, j->stream);
    delete j;
    return 0;
}

int svc_batch_begin(int count, int vec_length, const int* M, const int* K, const int* nnz,
                    const int* const* d_csr_row_ptr, const int* const* d_csr_col_idx, const void* const* d_csr_values_f16,
                    void* stream, svc_batch_job** job, int64_t* nvec) {
    g_err[0] = 0;
    if (!job || !nvec) { set_error("null output pointer"); return (int)cudaErrorInvalidValue; }
    *job = nullptr;
    if (count <= 0 || !M || !K || !nnz || !d_csr_row_ptr || !d_csr_col_idx) {
        set_error("a batch needs at least one matrix and its size arrays");
        return (int)cudaErrorInvalidValue;
    }
    if (vec_length != 8 && vec_length != 16) {
        set_error("vec_length must be 8 or 16 (got %d)", vec_length);
        return (int)cudaErrorInvalidValue;
    }
    const int V = vec_length;
    std::vector<SvcBatchEntry> tab((size_t)count + 1);
    long long rows = 0, entries = 0, vec_rows = 0;
    int k_max = 0;
    bool with_values = d_csr_values_f16 != nullptr;
    for (int i = 0; i < count; ++i) {
        if (M[i] < 0 || K[i] < 0 || nnz[i] < 0 || !d_csr_row_ptr[i] || (nnz[i] > 0 && !d_csr_col_idx[i])) {
            set_error("matrix %d: bad size or null array", i);
            return (int)cudaErrorInvalidValue;
        }
        if (with_values && nnz[i] > 0 && !d_csr_values_f16[i]) with_values = false;
        const long long mv = (M[i] + V - 1) / V;
        tab[i] = SvcBatchEntry{d_csr_row_ptr[i], d_csr_col_idx[i], with_values ? static_cast<const __half*>(d_csr_values_f16[i]) : nullptr,
                               rows, entries, vec_rows, M[i], nnz[i]};
        rows += mv * V; entries += nnz[i]; vec_rows += mv;
        if (K[i] > k_max) k_max = K[i];
    }
    tab[count] = SvcBatchEntry{nullptr, nullptr, nullptr, rows, entries, vec_rows, 0, 0};
    if (rows >= 0x7fffffffLL || entries >= 0x7fffffffLL) {
        set_error("stacked batch does not fit 32-bit indices (%lld rows, %lld entries)", rows, entries);
        return (int)cudaErrorInvalidValue;
    }
    if (k_max > kSvcMaxK) {
        set_error("K = %d exceeds the supported maximum of %d columns", k_max, kSvcMaxK);
        return (int)cudaErrorInvalidValue;
    }
    svc_batch_job* b = new (std::nothrow) svc_batch_job();
    if (!b) return (int)cudaErrorMemoryAllocation;
    b->count = count; b->V = V; b->rows = rows; b->entries = entries; b->vec_rows = vec_rows; b->with_values = with_values;
    b->inner = nullptr; b->block = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // one allocation: table | cuts[count+1] (int64) | stacked row_ptr | stacked col | stacked values
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const size_t off_cuts = up(tab.size() * sizeof(SvcBatchEntry));
    const size_t off_ptr = off_cuts + up(((size_t)count + 1) * 8);
    const size_t off_col = off_ptr + up(((size_t)rows + 1) * 4);
    const size_t off_val = off_col + up((size_t)entries * 4);
    const size_t total = off_val + (with_values ? up((size_t)entries * 2) : 0);
    keep_pool_memory();
    cudaError_t e = cudaMallocAsync(&b->block, total, st);
    if (e != cudaSuccess) { delete b; return fail(e, "batch scratch allocation"); }
    uint8_t* base = static_cast<uint8_t*>(b->block);
    b->d_tab = reinterpret_cast<SvcBatchEntry*>(base);
    b->d_cuts = reinterpret_cast<long long*>(base + off_cuts);
    int* s_ptr = reinterpret_cast<int*>(base + off_ptr);
    int* s_col = reinterpret_cast<int*>(base + off_col);
    __half* s_val = with_values ? reinterpret_cast<__half*>(base + off_val) : nullptr;
    e = cudaMemcpyAsync(b->d_tab, tab.data(), tab.size() * sizeof(SvcBatchEntry), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);          // `tab` is pageable host memory about to go out of scope
    if (e == cudaSuccess) e = svc_stack(b->d_tab, count, rows, entries, V, s_ptr, s_col, s_val, st);
    int64_t total_nvec = 0;
    int rc = 0;
    if (e == cudaSuccess) {
        rc = svc_begin((int)rows, k_max, V, s_ptr, s_col, s_val, stream, &b->inner, &total_nvec);
        if (rc == 0) {
            e = svc_batch_cuts(b->d_tab, count, b->inner->s.vec_ptr, b->d_cuts, st);
            std::vector<long long> cuts((size_t)count + 1);
            if (e == cudaSuccess) e = cudaMemcpyAsync(cuts.data(), b->d_cuts, cuts.size() * 8, cudaMemcpyDeviceToHost, st);
            if (e == cudaSuccess) e = cudaStreamSynchronize(st);
            if (e == cudaSuccess)
                for (int i = 0; i < count; ++i) nvec[i] = cuts[i + 1] - cuts[i];
        }
    }
    if (e != cudaSuccess || rc != 0) {
        if (b->inner) svc_free(b->inner);
        cudaFreeAsync(b->block, st);
        delete b;
        return rc != 0 ? rc : fail(e, "batch stacking");
    }
    b->stream = st;
    *job = b;
    return 0;
}

int svc_batch_finish(svc_batch_job* b, int* d_vec_row_ptr, int* d_vec_col, void* d_vec_values_f16, void* stream) {
    g_err[0] = 0;
    if (!b || !d_vec_row_ptr) { set_error("null pointer"); return (int)cudaErrorInvalidValue; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    svc_job* j = b->inner;
    // vector row pointers of each matrix, rebased to start at 0, one after another
    cudaError_t e = svc_batch_row_ptrs(b->d_tab, b->count, b->vec_rows, j->s.vec_ptr, b->d_cuts, d_vec_row_ptr, st);
    if (e != cudaSuccess) return fail(e, "row pointer rebase");
    if (j->nvec == 0) return 0;
    if (!d_vec_col) { set_error("null pointer"); return (int)cudaErrorInvalidValue; }
    __half* ov = j->with_values ? static_cast<__half*>(d_vec_values_f16) : nullptr;
    if (ov) {
        e = cudaMemsetAsync(ov, 0, (size_t)j->nvec * j->p.V * sizeof(__half), st);
        if (e != cudaSuccess) return fail(e, "value clear");
    }
    if (j->table_ints > 0 && !j->s.tables) {
        e = cudaMallocAsync(reinterpret_cast<void**>(&j->s.tables), (size_t)j->table_ints * 4, st);
        if (e != cudaSuccess) return fail(e, "table scratch allocation");
    }
    e = svc_emit(j->p, j->s, j->class_groups, d_vec_col, ov, st);
    if (e != cudaSuccess) return fail(e, "SVC emit");
    j->stream = st;
    b->stream = st;
    return 0;
}

int svc_batch_replayed_rows(svc_batch_job* b, int64_t* rows) {
    if (!b || !b->inner) return (int)cudaErrorInvalidValue;
    return svc_replayed_rows(b->inner, rows);
}

int svc_batch_free(svc_batch_job* b) {
    if (!b) return 0;
    if (b->inner) svc_free(b->inner);
    if (b->block) cudaFreeAsync(b->block, b->stream);
    delete b;
    return 0;
}

int svc_replayed_rows(svc_job* j, int64_t* rows) {
    g_err[0] = 0;
    if (!j || !rows) return (int)cudaErrorInvalidValue;
    *rows = 0;
    for (int c = 1; c < kSvcSegs; ++c) *rows += j->class_groups[c];       // every class but "ascending"
    return 0;
}

int sspmm_sorted_row_swizzle(int m_vec, const int* d_row_offsets, int* d_row_indices, void* stream) {
    g_err[0] = 0;
    if (m_vec < 0 || (m_vec > 0 && (!d_row_offsets || !d_row_indices))) {
        set_error("bad argument");
        return (int)cudaErrorInvalidValue;
    }
    if (m_vec == 0) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (m_vec <= kSwizzleRankLimit) {
        row_swizzle_kernel<<<(m_vec + 255) / 256, 256, 0, st>>>(m_vec, d_row_offsets, d_row_indices);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? 0 : fail(e, "row swizzle launch");
    }
    long long padded = 1;
    while (padded < m_vec) padded <<= 1;
    unsigned long long* keys = nullptr;
    keep_pool_memory();
    cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&keys), (size_t)padded * sizeof(unsigned long long), st);
    if (e != cudaSuccess) return fail(e, "scratch allocation for the row order");
    const unsigned blocks = (unsigned)((padded + 255) / 256);
    swizzle_keys_kernel<<<blocks, 256, 0, st>>>(m_vec, padded, d_row_offsets, keys);
    for (long long k = 2; k <= padded; k <<= 1)
        for (long long j = k >> 1; j > 0; j >>= 1) swizzle_bitonic_kernel<<<blocks, 256, 0, st>>>(padded, j, k, keys);
    swizzle_write_kernel<<<(m_vec + 255) / 256, 256, 0, st>>>(m_vec, keys, d_row_indices);
    e = cudaGetLastError();
    cudaFreeAsync(keys, st);
    return e == cudaSuccess ? 0 : fail(e, "row swizzle launch");
}

const char* sspmm_last_error_string(void) { return g_err; }
const char* sspmm_version(void) { return "sspmm_b200 0.1 sm_100a"; }

}  // extern "C"
