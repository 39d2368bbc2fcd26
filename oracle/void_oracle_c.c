/* CPU restatement in plain C of the INT8 SpMM of the reference, for tests and for the timed CPU baseline.
 * TEST INFRASTRUCTURE ONLY: nothing under void_b200/ links, loads or calls this file.
 *
 * Follows void_spmm_int8_kernel, void/int_quant.py:435-540 of the reference:
 *   - one int32 accumulator per tile row and output column, acc += A_q[32x32] . B_q[32 x N] over the
 *     row's tiles in row order (:484-516; integer sums, so the order does not matter);
 *   - avg_scale = (sum over the row's tiles of a_scale * b_scale, added in row order in fp32) / count
 *     (:518-526), C = float(acc) * avg_scale (:528-540); empty rows give zeros;
 *   - per-column scales of B (an extension of this repository; the reference result is linear in
 *     b_scale) multiply the result column by column.
 * Rows of B beyond K read as zero (boundary_check, :504-512).
 *
 * Parallel over (tile row, block of 128 output columns) with OpenMP; the hot loop is compiled for several
 * instruction sets and chosen at load time, so the library runs on any x86-64 host.
 */
#include <stdint.h>
#include <string.h>

#define TILE 32
#define NB 128

#if defined(__GNUC__) && defined(__x86_64__)
#define CLONES __attribute__((target_clones("arch=skylake-avx512", "avx2", "default")))
#else
#define CLONES
#endif

/* acc[32][nb] += tile[32][32] . b_rows[kmax][ldb] (first nb columns) */
CLONES static void tile_product(const int8_t* tile, const int8_t* b_rows, int64_t ldb, int kmax, int nb,
                                int32_t (*acc)[NB]) {
  for (int m = 0; m < TILE; ++m) {
    int32_t* row = acc[m];
    for (int k = 0; k < kmax; ++k) {
      const int32_t a = tile[m * TILE + k];
      const int8_t* b = b_rows + (int64_t)k * ldb;
      for (int n = 0; n < nb; ++n) row[n] += a * (int32_t)b[n];
    }
  }
}

/* values [nnz][32][32] int8 in the caller's (Morton) order; block_indices [nnz] = tile-row-major order;
 * row_ptr [nbr + 1]; scales [nnz]; b [K][N] int8 row-major; col_scale [N] or NULL; acc_out [nbr*32][N] or NULL;
 * out [M][N] fp32.  Returns 0. */
int void_oracle_spmm_int8(const int8_t* values, const float* scales, const int32_t* block_cols,
                          const int32_t* row_ptr, const int32_t* block_indices, int32_t nbr, int32_t M, int32_t K,
                          int32_t N, const int8_t* b, float b_scale, const float* col_scale, int32_t* acc_out,
                          float* out) {
  const int n_chunks = (N + NB - 1) / NB;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int r = 0; r < nbr; ++r) {
    for (int c = 0; c < n_chunks; ++c) {
      int32_t acc[TILE][NB];
      memset(acc, 0, sizeof(acc));
      const int n0 = c * NB;
      const int nb = (N - n0) < NB ? (N - n0) : NB;
      const int t0 = row_ptr[r], t1 = row_ptr[r + 1];
      float sum = 0.0f;
      for (int t = t0; t < t1; ++t) {
        const int i = block_indices[t];
        const int k0 = block_cols[i] * TILE;
        int kmax = K - k0;
        if (kmax > TILE) kmax = TILE;
        if (kmax > 0) tile_product(values + (int64_t)i * TILE * TILE, b + (int64_t)k0 * N + n0, N, kmax, nb, acc);
        sum = sum + scales[i] * b_scale;
      }
      const float avg = (t1 > t0) ? sum / (float)(t1 - t0) : 0.0f;
      for (int m = 0; m < TILE; ++m) {
        const int64_t row = (int64_t)r * TILE + m;
        if (acc_out != NULL) memcpy(acc_out + row * N + n0, acc[m], (size_t)nb * sizeof(int32_t));
        if (row < M) {
          float* o = out + row * N + n0;
          for (int n = 0; n < nb; ++n) {
            float v = (float)acc[m][n] * avg;
            if (col_scale != NULL) v = v * col_scale[n0 + n];
            o[n] = v;
          }
        }
      }
    }
  }
  return 0;
}
