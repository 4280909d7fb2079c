/*
 * TEST INFRASTRUCTURE -- CPU oracle for the vector-sparse SpMM.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may load this
 * file's shared object; the product library never does.
 *
 * Restates the host verification loop of the reference driver
 * (SSpMM/sspmm_test.cpp:75-95): fp16 operands are widened to fp32, products are
 * accumulated in fp32 in the loop order  vector row i -> vector j -> lane v ->
 * column l, and the output is row-major [m_vec*V][N].
 *
 * Value layout (SSpMM/sspmm_test.cpp:84-90): values[j*V+v] multiplies row
 * i*V+v of the output and row column_indices[j] of the dense operand.
 *
 * Compile with -ffp-contract=off so that multiply and add stay two roundings,
 * as in the reference (which is built without FMA contraction on x86-64).
 */
#include <stdint.h>
#include <string.h>

static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

/* One vector row, exactly the reference's inner three loops. */
static void one_vector_row(int i, int V, int N, const int* row_offsets, const int* col_indices,
                           const uint16_t* values, const float* rhs_f32, float* out) {
    for (int j = row_offsets[i]; j < row_offsets[i + 1]; ++j) {
        const float* brow = rhs_f32 + (int64_t)col_indices[j] * N;
        for (int v = 0; v < V; ++v) {
            float a = half_bits_to_float(values[(int64_t)j * V + v]);
            float* orow = out + ((int64_t)i * V + v) * N;
            for (int l = 0; l < N; ++l) orow[l] += a * brow[l];
        }
    }
}

/*
 * out must hold (i_end - i_begin)*V*N floats; row (i - i_begin)*V + v of `out`
 * is output row i*V+v.  rhs_f32 is the dense operand already widened to fp32
 * (widening is exact, so this does not change any rounding).  threads <= 1 runs
 * the scalar loop; otherwise vector rows are split over OpenMP threads (each
 * output row is still produced by one thread in the reference's order).
 */
void oracle_sspmm_rows(int i_begin, int i_end, int V, int N, const int* row_offsets,
                       const int* col_indices, const uint16_t* values, const float* rhs_f32,
                       float* out, int threads) {
    memset(out, 0, (size_t)(i_end - i_begin) * V * N * sizeof(float));
    float* base = out - (int64_t)i_begin * V * N;
#ifdef _OPENMP
    if (threads > 1) {
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
        for (int i = i_begin; i < i_end; ++i)
            one_vector_row(i, V, N, row_offsets, col_indices, values, rhs_f32, base);
        return;
    }
#endif
    (void)threads;
    for (int i = i_begin; i < i_end; ++i)
        one_vector_row(i, V, N, row_offsets, col_indices, values, rhs_f32, base);
}

void oracle_half_to_float(const uint16_t* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; ++i) dst[i] = half_bits_to_float(src[i]);
}
