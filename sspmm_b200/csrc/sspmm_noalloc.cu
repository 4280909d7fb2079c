// SpMM entry point that never allocates device memory.
//
// The block kernel needs a dense, transposed copy of the compressed operand (K x m_vec*V halfs).
// The regular entry points take that room from the stream-ordered allocator on every call.  Some
// callers must not allocate at call time: an inference server that handed all device memory to its
// own arena at start-up, or a latency-critical loop in which an allocation could fail, or stall
// other streams.  For them the same kernels run here on a fixed scratch array that is part of the
// library image: every GPU that loads the library holds kNoAllocScratchBytes of it until exit.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/sspmm_b200.h"
#include "launch.h"

namespace sspmm_b200 {
namespace {

constexpr size_t kNoAllocScratchBytes = (size_t)SSPMM_NOALLOC_MAX_SCRATCH_BYTES;

// Device code of this file could name the array directly; host code cannot: on the host the name
// is only a handle, and its device address has to be asked for (below).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of the array on the current device, resolved on the first call per device.
cudaError_t noalloc_scratch_address(void** out) {
    static void* cache[64] = {nullptr};
    static DeviceOnce resolved;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!resolved.done()) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) return e;
        cache[dev] = p;
        resolved.mark();
    }
    *out = cache[dev];
    return cudaSuccess;
}

}  // namespace
}  // namespace sspmm_b200

extern "C" int sspmm_f16_f16_noalloc(int m_vec, int vec_length, int N, int K, const int* row_indices,
                                     const int* row_offsets, const int* column_indices, const void* values_f16,
                                     const void* rhs_f16, void* out_f16, void* stream) {
    using namespace sspmm_b200;
    set_error("%s", "");
    if (vec_length != 8 && vec_length != 16) {
        set_error("vec_length must be 8 or 16 (got %d)", vec_length);
        return (int)cudaErrorInvalidValue;
    }
    if (m_vec < 0 || N < 0 || K < 0) {
        set_error("negative dimension (m_vec=%d N=%d K=%d)", m_vec, N, K);
        return (int)cudaErrorInvalidValue;
    }
    if (m_vec == 0 || N == 0) return 0;
    const unsigned long long need = 2ull * (unsigned long long)K * (unsigned long long)m_vec * (unsigned long long)vec_length;
    if (need > kNoAllocScratchBytes) {
        set_error("K * m_vec * vec_length * 2 = %llu bytes exceeds the fixed scratch of %llu bytes of the "
                  "no-allocation entry point; use sspmm_f16_f16",
                  need, (unsigned long long)kNoAllocScratchBytes);
        return (int)cudaErrorInvalidValue;
    }
    if (!row_offsets || !out_f16 || !column_indices || !values_f16 || !rhs_f16) {
        set_error("null operand pointer");
        return (int)cudaErrorInvalidValue;
    }
    auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (K == 0 || N % 8 != 0 || misaligned(values_f16) || misaligned(rhs_f16) || misaligned(out_f16)) {
        set_error("the no-allocation entry point needs K > 0, N %% 8 == 0 and 16-byte aligned values, rhs and output");
        return (int)cudaErrorInvalidValue;
    }
    void* scratch = nullptr;
    cudaError_t e = noalloc_scratch_address(&scratch);
    if (e != cudaSuccess) {
        set_error("cudaGetSymbolAddress for the fixed scratch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    SpmmArgs a;
    a.m_vec = m_vec; a.V = vec_length; a.N = N; a.K = K;
    a.row_indices = row_indices; a.row_offsets = row_offsets; a.column_indices = column_indices;
    a.values = static_cast<const __half*>(values_f16); a.rhs = static_cast<const __half*>(rhs_f16);
    a.out = out_f16; a.out_f16 = true; a.batch = 1;
    a.values_stride = 0; a.rhs_stride = 0; a.out_stride = 0;
    a.stream = static_cast<cudaStream_t>(stream);
    // The expansion kernel writes every element of the K x m_vec*V region it uses (zeros included),
    // so nothing left in the array by an earlier call can leak into this one.
    e = launch_sspmm_block(a, scratch, kNoAllocScratchBytes);
    if (e != cudaSuccess) {
        set_error("SpMM launch: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
