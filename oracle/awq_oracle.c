/* Plain-C restatement of the AWQ W4A16 linear arithmetic.  TEST INFRASTRUCTURE
 * ONLY: it checks the CUDA kernels and is timed as the CPU baseline; nothing
 * in the shipped package links or calls it.
 *
 * Parity status: pinned through oracle/awq_oracle.py, which is checked against
 * vectors made by the reference's packer and kernels; tests/test_oracle_c.py
 * requires this file to agree with that module bit for bit (unpack, dequant)
 * and to 1e-5 (fp32 GEMM).
 *
 * Reference sites followed (nanoquantization/layers/gemm.py):
 *   shift table            gemm.py:64-69, 245-249, 301-302
 *   (q - z) * s            gemm.py:112, 303-304
 *   bias add               gemm.py:565-566
 */
#include <stdint.h>
#include <string.h>

static const int AWQ_SHIFT[8] = {0, 16, 4, 20, 8, 24, 12, 28};

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f;
}
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
static inline float f16_to_f32(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
static inline uint16_t f32_to_f16_rne(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

/* out[r, 8*i + e] = (word[r, i] >> shift[e]) & 0xF */
void awq_oracle_unpack_int4(const uint32_t* words, uint8_t* out, int64_t rows, int64_t cols_packed) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t i = 0; i < cols_packed; ++i) {
      uint32_t w = words[r * cols_packed + i];
      for (int e = 0; e < 8; ++e) out[(r * cols_packed + i) * 8 + e] = (uint8_t)((w >> AWQ_SHIFT[e]) & 0xF);
    }
}

/* dtype: 0 = fp16, 1 = bf16.  scales/out are raw 16-bit patterns.
 * The product of an integer |d| <= 15 and a 16-bit float is exact in fp32, so
 * one conversion back gives the single rounding the reference performs. */
void awq_oracle_dequant(const uint32_t* qweight, const uint16_t* scales, const uint32_t* qzeros,
                        uint16_t* out, int64_t K, int64_t N, int64_t group, int dtype) {
  int64_t NW = N / 8;
  for (int64_t k = 0; k < K; ++k) {
    int64_t gi = k / group;
    for (int64_t i = 0; i < NW; ++i) {
      uint32_t w = qweight[k * NW + i], z = qzeros[gi * NW + i];
      for (int e = 0; e < 8; ++e) {
        int d = (int)((w >> AWQ_SHIFT[e]) & 0xF) - (int)((z >> AWQ_SHIFT[e]) & 0xF);
        uint16_t sb = scales[gi * N + i * 8 + e];
        float s = dtype ? bf16_to_f32(sb) : f16_to_f32(sb);
        float p = (float)d * s;
        out[k * N + i * 8 + e] = dtype ? f32_to_bf16_rne(p) : f32_to_f16_rne(p);
      }
    }
  }
}

/* y[M, N] (fp32) = x.float() @ float(dequant) (+ bias).  bias_dtype as dtype; bias may be NULL. */
void awq_oracle_gemm_f32(const uint16_t* x, const uint32_t* qweight, const uint16_t* scales,
                         const uint32_t* qzeros, const uint16_t* bias, int bias_dtype, float* y,
                         int64_t M, int64_t N, int64_t K, int64_t group, int dtype,
                         uint16_t* w_scratch /* K*N */) {
  awq_oracle_dequant(qweight, scales, qzeros, w_scratch, K, N, group, dtype);
  for (int64_t m = 0; m < M; ++m) {
    float* yr = y + m * N;
    for (int64_t n = 0; n < N; ++n) yr[n] = 0.f;
    for (int64_t k = 0; k < K; ++k) {
      uint16_t xb = x[m * K + k];
      float xv = dtype ? bf16_to_f32(xb) : f16_to_f32(xb);
      const uint16_t* wr = w_scratch + k * N;
      if (dtype) for (int64_t n = 0; n < N; ++n) yr[n] += xv * bf16_to_f32(wr[n]);
      else       for (int64_t n = 0; n < N; ++n) yr[n] += xv * f16_to_f32(wr[n]);
    }
    if (bias) for (int64_t n = 0; n < N; ++n) yr[n] += bias_dtype ? bf16_to_f32(bias[n]) : f16_to_f32(bias[n]);
  }
}
