/*
 * TEST INFRASTRUCTURE - CPU restatement of the dense projection inside the
 * reference's unfused Ulysses path (F.linear in
 * tests/run_distributed_correctness.py:236-336 and
 * benchmarks/bench_bshd.py:225-494 of the reference tree). Only tests, the
 * smoke check and the bench's CPU-baseline leg may call this; the product
 * never does.
 *
 * Numerics contract being restated (README.md:90-92, 411-418 and
 * mega_up/kernels/peer_write_gemm.py:2533-2539 of the reference): BF16
 * operands, one FP32 accumulator per output element fed in ascending K
 * order, bias added in FP32, one round-to-nearest-even to BF16.
 *
 * Values travel as float32 arrays that hold BF16-representable numbers.
 *
 * Build: gcc -O3 -mavx2 -mfma -fopenmp -shared -fPIC (see oracle/build.py).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float round_to_bf16(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep quiet NaN */
    u = (u | 0x00400000u) & 0xffff0000u;
  } else {
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
  }
  memcpy(&v, &u, 4);
  return v;
}

/* out[m, n] = bf16( sum_k x[m, k] * w[n, k]  (k ascending, FP32) + bias[n] )
 * wt is w transposed to [K, N] so the n loop vectorises while each output
 * keeps its own sequential accumulator. bias may be NULL. */
void oracle_linear_bf16(const float *x, const float *wt, const float *bias, float *out,
                        int64_t M, int64_t N, int64_t K) {
  const int64_t NB = 512;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n0 = 0; n0 < N; n0 += NB) {
      float acc[512];
      const int64_t nb = (N - n0 < NB) ? (N - n0) : NB;
      for (int64_t j = 0; j < nb; ++j) acc[j] = 0.0f;
      const float *xr = x + m * K;
      for (int64_t k = 0; k < K; ++k) {
        const float xv = xr[k];
        const float *wr = wt + k * N + n0;
        for (int64_t j = 0; j < nb; ++j) acc[j] += xv * wr[j];
      }
      float *o = out + m * N + n0;
      if (bias != NULL) {
        for (int64_t j = 0; j < nb; ++j) o[j] = round_to_bf16(acc[j] + bias[n0 + j]);
      } else {
        for (int64_t j = 0; j < nb; ++j) o[j] = round_to_bf16(acc[j]);
      }
    }
  }
}

/* dst row i = src row index[i]; rows of `width` float32. */
void oracle_gather_rows(const float *src, const int64_t *index, float *dst, int64_t rows,
                        int64_t width) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < rows; ++i) {
    memcpy(dst + i * width, src + index[i] * width, (size_t)width * sizeof(float));
  }
}

int oracle_abi_version(void) { return 1; }
