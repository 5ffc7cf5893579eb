/*
 * CPU oracle for the weight-only quantised GEMM path.  TEST INFRASTRUCTURE ONLY:
 * it restates the reference's algorithm in plain C so the CUDA path can be
 * checked against it; nothing in the shipped package links or calls it.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks every function below
 * against golden vectors produced by the reference itself
 * (tests/golden/make_golden.py imports the reference's quantiser and its torch
 * dequantise-then-matmul and stores inputs and outputs).
 *
 * Reference being restated (paths inside the reference project):
 *   python/dexter/quant.py:62-72                 split-half nibble packing
 *   python/dexter/ops/reference/gemm.py:44-48    unpack_int4
 *   python/dexter/ops/reference/gemm.py:51-73    dequantize
 *   python/dexter/ops/reference/gemm.py:76-79    _quantized_matmul
 *
 * The arithmetic itself lives in torch (pyproject.toml:10, torch>=2.6, 2.11.0 in
 * the image that made the golden vectors): every bf16 tensor op computes in
 * fp32 and rounds the result to bf16 (round to nearest even), which is what
 * bf16_rne() below does after each step.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* fp32 -> bf16, round to nearest even; NaN stays NaN. */
static inline uint16_t bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* gemm.py:44-48 -- [K/2, N] packed bytes -> [K, N] values 0..15: low nibbles
 * are rows 0..K/2-1, high nibbles are rows K/2..K-1 (quant.py:62-72). */
void dxo_unpack_int4(const uint8_t* qweight, int64_t k_half, int64_t n, uint8_t* out) {
  for (int64_t i = 0; i < k_half; ++i)
    for (int64_t j = 0; j < n; ++j) {
      uint8_t b = qweight[i * n + j];
      out[i * n + j] = b & 0x0F;
      out[(i + k_half) * n + j] = (b >> 4) & 0x0F;
    }
}

/* gemm.py:51-73 -- w[k,n] = bf16((bf16(q) - zero) * scale), every step rounded
 * to bf16.  `zeros` may be NULL (symmetric: zero = 2^(bits-1)); stored 4-bit
 * zero points carry +128 which is removed first (gemm.py:67-70).
 * qweight is [K/2, N] for bits == 4 and [K, N] for bits == 8; scales and zeros
 * are [K/group, N] bf16 bit patterns; out is [K, N] bf16 bit patterns. */
int dxo_dequantize(const uint8_t* qweight, const uint16_t* scales, const uint16_t* zeros,
                   int64_t k, int64_t n, int64_t group, int bits, uint16_t* out) {
  if ((bits != 4 && bits != 8) || group <= 0 || k % group) return -1;
  if (bits == 4 && (k & 1)) return -1;
  const int64_t half = k / 2;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < k; ++r) {
    const int64_t g = r / group;
    for (int64_t j = 0; j < n; ++j) {
      unsigned q;
      if (bits == 4)
        q = r < half ? (qweight[r * n + j] & 0x0Fu) : ((qweight[(r - half) * n + j] >> 4) & 0x0Fu);
      else
        q = qweight[r * n + j];
      const float qf = bf16_to_f32(bf16_rne((float)q));
      float zero;
      if (zeros)
        zero = bf16_to_f32(bf16_rne(bf16_to_f32(zeros[g * n + j]) - (bits == 4 ? 128.0f : 0.0f)));
      else
        zero = (float)(1 << (bits - 1));
      const float centred = bf16_to_f32(bf16_rne(qf - zero));
      out[r * n + j] = bf16_rne(centred * bf16_to_f32(scales[g * n + j]));
    }
  }
  return 0;
}

/* gemm.py:76-79 -- out = bf16(x @ w) with fp32 accumulation, then, when a bias
 * is given, a second bf16 op out = bf16(out + bias).  x is [M, K] with row
 * stride ldx (elements), w is [K, N], out is [M, N], all bf16 bit patterns. */
void dxo_matmul_bias(const uint16_t* x, int64_t ldx, const uint16_t* w, const uint16_t* bias,
                     int64_t m, int64_t k, int64_t n, uint16_t* out) {
#pragma omp parallel
  {
    float* acc = (float*)malloc((size_t)n * sizeof(float));
    float* wrow = (float*)malloc((size_t)n * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
      for (int64_t j = 0; j < n; ++j) acc[j] = 0.0f;
      for (int64_t r = 0; r < k; ++r) {
        const float xv = bf16_to_f32(x[i * ldx + r]);
        const uint16_t* wr = w + r * n;
        for (int64_t j = 0; j < n; ++j) wrow[j] = bf16_to_f32(wr[j]);
        for (int64_t j = 0; j < n; ++j) acc[j] += xv * wrow[j];
      }
      for (int64_t j = 0; j < n; ++j) {
        uint16_t o = bf16_rne(acc[j]);
        if (bias) o = bf16_rne(bf16_to_f32(o) + bf16_to_f32(bias[j]));
        out[i * n + j] = o;
      }
    }
    free(acc);
    free(wrow);
  }
}

/* The whole op as the reference's torch_w4a16 / torch_w8a16 run it
 * (gemm.py:82-89): dequantise the full weight, then matmul (+bias).
 * `scratch_w` is a caller-provided [K, N] bf16 buffer for the dense weight. */
int dxo_wq_gemm(const uint16_t* x, int64_t ldx, const uint8_t* qweight, const uint16_t* scales,
                const uint16_t* zeros, const uint16_t* bias, int64_t m, int64_t k, int64_t n,
                int64_t group, int bits, uint16_t* scratch_w, uint16_t* out) {
  int rc = dxo_dequantize(qweight, scales, zeros, k, n, group, bits, scratch_w);
  if (rc) return rc;
  dxo_matmul_bias(x, ldx, scratch_w, bias, m, k, n, out);
  return 0;
}
