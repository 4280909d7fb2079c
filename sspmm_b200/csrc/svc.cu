// Sparse vector compression kernels.
//
// Reference behaviour (RowMerge/sparse_matrix_format.py:100-123): for vector row i,
//     cols = []
//     for j in 0..V-1 (rows below M only):  cols = list(set(cols + row[V*i+j]))
// and the vector row pointer is the running sum of len(cols).  The order of `cols`
// is CPython's set order, which for small non-negative ints is decided by an
// open-addressing table (hash(x) = x; probe nine neighbours when the window fits,
// else jump to (5*i + 1 + perturb) & mask; the table grows to the power of two
// above 4*used -- 2*used beyond 50 000 -- once 5*fill >= 3*mask, re-inserting in
// slot order; iteration is in slot order).
//
// Kernels, one warp per vector row (the V rows of a group are one contiguous
// CSR range):
//   svc_count_kernel   marks the group's columns in a shared-memory bitmap with
//                      atomicOr, counts first-time bits by ballot-free popc of
//                      the returned words, and decides per group whether
//                      ascending order is already the exact answer: it is when
//                      the largest column id is below the final table length,
//                      because then every key sits in its home slot.
//   svc_scan_kernel    exclusive scans (vector row pointers, scratch offsets).
//   svc_emit_sorted    rebuilds the bitmap, turns it into the ascending column
//                      list with a popc prefix scan across the warp, and places
//                      value vectors with prefix[word] + popc(lower bits).
//   svc_emit_replay    replays the V set rebuilds in a scratch table, exactly.
#include "svc.cuh"

#include "launch.h"

namespace sspmm_b200 {

__device__ int g_svc_bad_column = 0;

namespace {

constexpr int kMinTable = 8;
constexpr int kLinearProbes = 9;
constexpr int kPerturbShift = 5;

// Table length after `distinct` different keys were added to an empty set.
__host__ __device__ inline int final_table_len(int distinct) {
    long long size = kMinTable;
    for (;;) {
        const long long mask = size - 1;
        const long long trig = (3 * mask + 4) / 5;       // smallest fill with 5*fill >= 3*mask
        if (distinct < trig) return (int)size;
        const long long minused = trig > 50000 ? trig * 2 : trig * 4;
        long long ns = kMinTable;
        while (ns <= minused) ns <<= 1;
        size = ns;
        if (size > (1ll << 30)) return (int)size;
    }
}

__host__ __device__ inline long long group_table_ints(int tbl_len, bool with_values) {
    if (tbl_len == 0) return 0;
    const long long small = tbl_len / 4 > kMinTable ? tbl_len / 4 : kMinTable;
    return (long long)tbl_len + small + (with_values ? tbl_len : 0);
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_max(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

// ---------------------------------------------------------------- pass 1: count
__global__ void __launch_bounds__(256)
svc_count_kernel(SvcProblem p, int words, int* __restrict__ counts, int* __restrict__ mode, int* __restrict__ tbl_len) {
    extern __shared__ unsigned int sm_words[];
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned int* bm = sm_words + (size_t)warp * words;
    for (int i = blockIdx.x * warps + warp; i < p.m_vec; i += gridDim.x * warps) {
        const int r0 = min(i * p.V, p.M), r1 = min(i * p.V + p.V, p.M);
        const int e0 = p.row_ptr[r0], e1 = p.row_ptr[r1];
        if (e1 - e0 < words) {
            for (int e = e0 + lane; e < e1; e += 32) {
                const unsigned c = (unsigned)p.col_idx[e];
                if (c < (unsigned)p.K) bm[c >> 5] = 0u;
            }
        } else {
            for (int w = lane; w < words; w += 32) bm[w] = 0u;
        }
        __syncwarp();
        int cnt = 0, mx = -1, bad = 0;
        for (int e = e0 + lane; e < e1; e += 32) {
            const int c = p.col_idx[e];
            if ((unsigned)c < (unsigned)p.K) {
                const unsigned bit = 1u << (c & 31);
                const unsigned old = atomicOr(&bm[c >> 5], bit);
                cnt += (old & bit) ? 0 : 1;
                mx = max(mx, c);
            } else {
                bad = 1;
            }
        }
        cnt = warp_sum(cnt);
        mx = warp_max(mx);
        bad = warp_max(bad);
        if (lane == 0) {
            counts[i] = cnt;
            const int len = final_table_len(cnt);
            const int replay = (mx >= len) ? 1 : 0;
            mode[i] = replay;
            tbl_len[i] = replay ? len : 0;
            if (bad) g_svc_bad_column = 1;
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------- scans (one CTA)
__global__ void __launch_bounds__(1024)
svc_scan_kernel(int m_vec, int* __restrict__ vec_ptr, const int* __restrict__ tbl_len, long long* __restrict__ tbl_off,
                long long* __restrict__ totals, int with_values) {
    __shared__ long long sh_a[32], sh_b[32];
    __shared__ long long carry_a, carry_b;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { carry_a = 0; carry_b = 0; }
    __syncthreads();
    for (int base = 0; base < m_vec; base += 1024) {
        const int i = base + threadIdx.x;
        long long a = 0, b = 0;
        if (i < m_vec) {
            a = vec_ptr[i];
            b = group_table_ints(tbl_len[i], with_values != 0);
        }
        long long ia = a, ib = b;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long ta = __shfl_up_sync(0xffffffffu, ia, o);
            const long long tb = __shfl_up_sync(0xffffffffu, ib, o);
            if (lane >= o) { ia += ta; ib += tb; }
        }
        if (lane == 31) { sh_a[warp] = ia; sh_b[warp] = ib; }
        __syncthreads();
        if (warp == 0) {
            long long wa = sh_a[lane], wb = sh_b[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const long long ta = __shfl_up_sync(0xffffffffu, wa, o);
                const long long tb = __shfl_up_sync(0xffffffffu, wb, o);
                if (lane >= o) { wa += ta; wb += tb; }
            }
            sh_a[lane] = wa; sh_b[lane] = wb;
        }
        __syncthreads();
        const long long off_a = carry_a + (warp ? sh_a[warp - 1] : 0);
        const long long off_b = carry_b + (warp ? sh_b[warp - 1] : 0);
        if (i < m_vec) {
            vec_ptr[i] = (int)(off_a + ia - a);
            tbl_off[i] = off_b + ib - b;
        }
        __syncthreads();
        if (threadIdx.x == 1023) { carry_a = off_a + ia; carry_b = off_b + ib; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        vec_ptr[m_vec] = (int)carry_a;
        tbl_off[m_vec] = carry_b;
        totals[0] = carry_a;
        totals[1] = carry_b;
    }
}

// ---------------------------------------------------------------- pass 2a: ascending order
__global__ void __launch_bounds__(256)
svc_emit_sorted_kernel(SvcProblem p, int words, const int* __restrict__ vec_ptr, const int* __restrict__ mode,
                       int* __restrict__ out_col, __half* __restrict__ out_vals) {
    extern __shared__ unsigned int sm_words[];
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned int* bm = sm_words + (size_t)warp * words * 2;
    unsigned int* pre = bm + words;
    for (int i = blockIdx.x * warps + warp; i < p.m_vec; i += gridDim.x * warps) {
        if (mode[i] != 0) continue;
        const int r0 = min(i * p.V, p.M), r1 = min(i * p.V + p.V, p.M);
        const int e0 = p.row_ptr[r0], e1 = p.row_ptr[r1];
        const int base = vec_ptr[i];
        if (e1 == e0) continue;
        for (int w = lane; w < words; w += 32) bm[w] = 0u;
        __syncwarp();
        for (int e = e0 + lane; e < e1; e += 32) {
            const int c = p.col_idx[e];
            if ((unsigned)c < (unsigned)p.K) atomicOr(&bm[c >> 5], 1u << (c & 31));
        }
        __syncwarp();
        int running = 0;
        for (int w0 = 0; w0 < words; w0 += 32) {
            const int w = w0 + lane;
            unsigned word = (w < words) ? bm[w] : 0u;
            const int pc = __popc(word);
            const int incl = warp_incl_scan(pc, lane);
            int o = running + incl - pc;
            if (w < words) pre[w] = (unsigned)o;
            o += base;
            while (word) {
                const int b = __ffs(word) - 1;
                out_col[o++] = w * 32 + b;
                word &= word - 1;
            }
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (out_vals) {
            __syncwarp();
            for (int r = r0; r < r1; ++r) {
                const int v = r - i * p.V;
                for (int e = p.row_ptr[r] + lane; e < p.row_ptr[r + 1]; e += 32) {
                    const int c = p.col_idx[e];
                    if ((unsigned)c < (unsigned)p.K) {
                        const int pos = (int)pre[c >> 5] + __popc(bm[c >> 5] & ((1u << (c & 31)) - 1u));
                        out_vals[((int64_t)base + pos) * p.V + v] = p.vals[e];
                    }
                }
            }
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------- pass 2b: hash-table replay
// Slot that `key` occupies, or the first free slot on its probe path.
__device__ __forceinline__ int probe_slot(const int* tab, unsigned mask, int key) {
    unsigned perturb = (unsigned)key;
    unsigned i = (unsigned)key & mask;
    for (;;) {
        const unsigned window = (i + kLinearProbes <= mask) ? kLinearProbes : 0;
        for (unsigned s = i; s <= i + window; ++s) {
            const int e = tab[s];
            if (e == -1 || e == key) return (int)s;
        }
        perturb >>= kPerturbShift;
        i = (i * 5u + 1u + perturb) & mask;
    }
}

__global__ void __launch_bounds__(256)
svc_emit_replay_kernel(SvcProblem p, const int* __restrict__ vec_ptr, const int* __restrict__ mode,
                       const int* __restrict__ tbl_len, const long long* __restrict__ tbl_off, int* __restrict__ tables,
                       int* __restrict__ out_col, __half* __restrict__ out_vals) {
    const int warps = blockDim.x >> 5;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = blockIdx.x * warps + warp; i < p.m_vec; i += gridDim.x * warps) {
        if (mode[i] == 0) continue;
        const int r0 = min(i * p.V, p.M), r1 = min(i * p.V + p.V, p.M);
        const int base = vec_ptr[i];
        int* list = out_col + base;                 // current ordered list lives in the output slice
        const int cap = tbl_len[i];
        int* reg0 = tables + tbl_off[i];            // holds the final table
        int* reg1 = reg0 + cap;                     // holds the table one growth step earlier
        const int small = cap / 4 > kMinTable ? cap / 4 : kMinTable;
        int* pos_tab = reg1 + small;                // slot -> position, only with values
        int cur_len = 0;
        int* tab = reg0;
        unsigned mask = kMinTable - 1;
        for (int r = r0; r < r1; ++r) {
            const int rs = p.row_ptr[r], rlen = p.row_ptr[r + 1] - rs;
            const int total = cur_len + rlen;
            // a fresh 8-slot table; regions alternate so that a table of length `cap` lands in reg0
            int size = kMinTable;
            int used = 0;
            mask = kMinTable - 1;
            // parity of the number of growth steps still possible decides the start region
            int steps_to_cap = 0;
            for (int s = kMinTable; s < cap; s <<= 2) ++steps_to_cap;
            tab = (steps_to_cap & 1) ? reg1 : reg0;
            if (lane < kMinTable) tab[lane] = -1;
            __syncwarp();
            int t = 0;
            for (;;) {
                int grow = 0;
                if (lane == 0) {
                    while (t < total) {
                        const int key = (t < cur_len) ? list[t] : p.col_idx[rs + t - cur_len];
                        ++t;
                        if ((unsigned)key >= (unsigned)p.K) continue;
                        const int s = probe_slot(tab, mask, key);
                        if (tab[s] == key) continue;
                        tab[s] = key;
                        ++used;
                        if ((long long)used * 5 >= (long long)mask * 3) { grow = 1; break; }
                    }
                }
                t = __shfl_sync(0xffffffffu, t, 0);
                used = __shfl_sync(0xffffffffu, used, 0);
                grow = __shfl_sync(0xffffffffu, grow, 0);
                if (!grow) break;
                const long long minused = used > 50000 ? (long long)used * 2 : (long long)used * 4;
                int nsize = kMinTable;
                while (nsize <= minused) nsize <<= 1;
                int* ntab = (tab == reg0) ? reg1 : reg0;
                if (nsize > cap) { nsize = cap; }     // cannot happen when counts are consistent
                for (int s = lane; s < nsize; s += 32) ntab[s] = -1;
                __syncwarp();
                if (lane == 0) {
                    const unsigned nmask = (unsigned)nsize - 1u;
                    for (int s = 0; s < size; ++s) {
                        const int key = tab[s];
                        if (key != -1) ntab[probe_slot(ntab, nmask, key)] = key;
                    }
                }
                __syncwarp();
                tab = ntab;
                size = nsize;
                mask = (unsigned)nsize - 1u;
            }
            // ordered extraction into the output slice
            int n = 0;
            for (int s0 = 0; s0 < size; s0 += 32) {
                const int s = s0 + lane;
                const int key = (s < size) ? tab[s] : -1;
                const unsigned bal = __ballot_sync(0xffffffffu, key != -1);
                if (key != -1) list[n + __popc(bal & ((1u << lane) - 1u))] = key;
                n += __popc(bal);
            }
            cur_len = n;
            __syncwarp();
        }
        if (out_vals && cur_len > 0) {
            const int size = (int)mask + 1;
            int n = 0;
            for (int s0 = 0; s0 < size; s0 += 32) {
                const int s = s0 + lane;
                const int key = (s < size) ? tab[s] : -1;
                const unsigned bal = __ballot_sync(0xffffffffu, key != -1);
                if (s < size) pos_tab[s] = n + __popc(bal & ((1u << lane) - 1u));
                n += __popc(bal);
            }
            __syncwarp();
            for (int r = r0; r < r1; ++r) {
                const int v = r - i * p.V;
                for (int e = p.row_ptr[r] + lane; e < p.row_ptr[r + 1]; e += 32) {
                    const int c = p.col_idx[e];
                    if ((unsigned)c < (unsigned)p.K) {
                        const int pos = pos_tab[probe_slot(tab, mask, c)];
                        out_vals[((int64_t)base + pos) * p.V + v] = p.vals[e];
                    }
                }
            }
        }
        __syncwarp();
    }
}

int device_sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
}

}  // namespace

cudaError_t svc_count_and_scan(const SvcProblem& p, const SvcScratch& s, bool with_values, cudaStream_t stream) {
    if (p.m_vec > 0) {
        const int words = (p.K + 31) / 32;
        int warps = 8;
        while (warps > 1 && (size_t)warps * words * 4 > 160 * 1024) warps >>= 1;
        const size_t smem = (size_t)warps * words * 4;
        cudaError_t ea = cudaFuncSetAttribute(svc_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (ea != cudaSuccess) return ea;
        const int sms = device_sm_count();
        int grid = (p.m_vec + warps - 1) / warps;
        const int cap = sms * 8;
        if (grid > cap) grid = cap;
        svc_count_kernel<<<grid, warps * 32, smem, stream>>>(p, words, s.vec_ptr, s.mode, s.tbl_len);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    svc_scan_kernel<<<1, 1024, 0, stream>>>(p.m_vec, s.vec_ptr, s.tbl_len, s.tbl_off, s.totals, with_values ? 1 : 0);
    return cudaGetLastError();
}

cudaError_t svc_emit(const SvcProblem& p, const SvcScratch& s, int* out_col, __half* out_vals, cudaStream_t stream) {
    if (p.m_vec == 0) return cudaSuccess;
    const int sms = device_sm_count();
    {
        const int words = (p.K + 31) / 32;
        int warps = 8;
        while (warps > 1 && (size_t)warps * words * 8 > 200 * 1024) warps >>= 1;
        const size_t smem = (size_t)warps * words * 8;
        cudaError_t ea =
            cudaFuncSetAttribute(svc_emit_sorted_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024);
        if (ea != cudaSuccess) return ea;
        int grid = (p.m_vec + warps - 1) / warps;
        if (grid > sms * 8) grid = sms * 8;
        svc_emit_sorted_kernel<<<grid, warps * 32, smem, stream>>>(p, words, s.vec_ptr, s.mode, out_col, out_vals);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    {
        const int warps = 4;
        int grid = (p.m_vec + warps - 1) / warps;
        if (grid > sms * 16) grid = sms * 16;
        svc_emit_replay_kernel<<<grid, warps * 32, 0, stream>>>(p, s.vec_ptr, s.mode, s.tbl_len, s.tbl_off, s.tables,
                                                                out_col, out_vals);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t svc_read_and_clear_bad_column_flag(int* flag, cudaStream_t stream) {
    cudaError_t e = cudaMemcpyFromSymbolAsync(flag, g_svc_bad_column, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    if (*flag) {
        const int zero = 0;
        e = cudaMemcpyToSymbolAsync(g_svc_bad_column, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    }
    return e;
}

}  // namespace sspmm_b200
