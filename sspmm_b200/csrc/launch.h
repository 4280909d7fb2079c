// Internal launcher interface shared by the kernel translation units and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <atomic>

namespace sspmm_b200 {

struct SpmmArgs {
    int m_vec;                 // vector rows
    int V;                     // rows per vector (8 or 16)
    int N;                     // columns of the dense operand / of the output
    int K;                     // rows of the dense operand
    const int* row_indices;    // optional scheduling order of vector rows (may be null)
    const int* row_offsets;    // [m_vec + 1]
    const int* column_indices; // [nvec]
    const __half* values;      // [nvec * V]
    const __half* rhs;         // [K * N] row-major
    void* out;                 // [m_vec * V * N] row-major, fp32 or fp16
    bool out_f16;
    // batching (one launch, grid z-less: tiles enumerate the batch too)
    int batch;                 // >= 1
    int64_t values_stride;     // elements between batches (0 = shared)
    int64_t rhs_stride;
    int64_t out_stride;
    cudaStream_t stream;
};

// tcgen05 row-gather kernel.  Requires N % 8 == 0, 16-byte aligned rhs/values.
cudaError_t launch_sspmm_gather(const SpmmArgs& a);
// tcgen05 row-gather kernel with load-instruction producers and splitting of long rows.
// sspmm_gather_lsu_plan sizes the optional scratch from the vector count (chunk = cap = 0: no splitting).
void sspmm_gather_lsu_plan(const SpmmArgs& a, long long nvec, int* chunk, int* cap, size_t* scratch_bytes);
cudaError_t launch_sspmm_gather_lsu(const SpmmArgs& a, int chunk, int cap, void* scratch);
// tcgen05 block kernel on a dense transposed copy of A held in `scratch` (caller-owned, stream-ordered).
// sspmm_block_scratch_bytes(a) is what the kernel would like (copy of A + split-K partial tiles); with less
// (at least K * m_vec*V halfs) it runs without split-K.
size_t sspmm_block_scratch_bytes(const SpmmArgs& a);
cudaError_t launch_sspmm_block(const SpmmArgs& a, void* scratch, size_t scratch_bytes);
// Allows (default) or forbids the CTA-pair variant of the block kernel.  Process-wide.
void sspmm_block_allow_pairs(bool allow);
// CUDA-core kernel without alignment requirements.
cudaError_t launch_sspmm_simt(const SpmmArgs& a);

// Per-device "already done" flags for one-time, per-device set-up (function
// attributes are per device).  Supports device ordinals 0..63.
class DeviceOnce {
public:
    bool done() const {
        int d = 0;
        cudaGetDevice(&d);
        return d >= 0 && d < 64 && (mask_.load(std::memory_order_acquire) >> d) & 1ull;
    }
    void mark() {
        int d = 0;
        cudaGetDevice(&d);
        if (d >= 0 && d < 64) mask_.fetch_or(1ull << d, std::memory_order_release);
    }
private:
    std::atomic<unsigned long long> mask_{0};
};

// Multiprocessor count of the current device (cached per device ordinal).
int current_device_sm_count();

// Records a message retrievable through sspmm_last_error_string().
void set_error(const char* fmt, ...);

}  // namespace sspmm_b200
