/*
 * CPU oracle for the FP8 grouped-GEMM hot path (TEST INFRASTRUCTURE, not product code).
 *
 * Plain-C restatement of the arithmetic the reference performs on the GPU.  Only the test-suite,
 * the smoke check and the CPU-baseline leg of the benchmark may load this library; the product
 * path never falls back to it.
 *
 * Each function cites the reference source it restates (paths relative to the reference project):
 *   - quantise          csrc/multi_pointwise.cu:75-80, csrc/multi_pad_fusion.cu:230-237
 *                       (`OType(scale * fp32(x))`, OType = __nv_fp8_e4m3 / __nv_fp8_e5m2, i.e.
 *                       round-to-nearest-even with saturation to the largest finite value)
 *   - amax              csrc/multi_pointwise.cu:78,93-96, csrc/utils.cuh:151-185
 *   - padded transpose  csrc/multi_pad_fusion.cu:46-153 (fp8 -> fp8), :155-292 (cast + transpose)
 *   - dgelu             csrc/multi_pad_fusion.cu:38-44,378
 *   - scale_mul         csrc/multi_pointwise.cu:138
 *   - grouped matmul    fp8_gmm/test.py:209-214 (per-group loop), csrc/fp8_gmm.h:7-11 (layouts),
 *                       fp8_gmm/grouped_linear.py:154-182 (dgrad / wgrad operands)
 *
 * The float -> fp8 converter is an independent implementation of the published OCP FP8 formats
 * (E4M3: bias 7, no infinities, max 448; E5M2: bias 15, max finite 57344).  It is pinned against the
 * CUDA toolkit's own host converter (the one the reference calls) by tests/test_oracle_pins.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define FP8_E4M3 0
#define FP8_E5M2 1

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* fp32 -> bf16, round to nearest even (what `bf16(float)` does in the reference kernels). */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF; /* canonical NaN, as __float2bfloat16_rn */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7FFFu + lsb;
  return (uint16_t)(u >> 16);
}

/*
 * fp32 -> fp8 byte, round-to-nearest-even, saturate-to-finite.
 * man_bits = 3 (E4M3) or 2 (E5M2).  NaN maps to 0x7F in both formats (sign dropped), matching the
 * canonical-NaN step of the toolkit's __nv_cvt_float_to_fp8.
 */
uint8_t fp8_oracle_cvt(float x, int format) {
  const int man_bits = (format == FP8_E4M3) ? 3 : 2;
  const int bias = (format == FP8_E4M3) ? 7 : 15;
  const uint8_t max_byte = (format == FP8_E4M3) ? 0x7E : 0x7B;
  const float max_val = (format == FP8_E4M3) ? 448.0f : 57344.0f;
  uint32_t u;
  memcpy(&u, &x, 4);
  const uint8_t sign = (uint8_t)((u >> 31) << 7);
  const uint32_t absu = u & 0x7FFFFFFFu;
  if (absu > 0x7F800000u) return 0x7F;
  float ax;
  memcpy(&ax, &absu, 4);
  /* Everything above max + half an ulp saturates; everything up to it rounds (RNE) to <= max. */
  const float half_ulp_at_max = (format == FP8_E4M3) ? 16.0f : 4096.0f;
  if (ax > max_val + half_ulp_at_max) return (uint8_t)(sign | max_byte);
  if (ax == max_val + half_ulp_at_max) return (uint8_t)(sign | max_byte); /* tie: would round to even = overflow -> saturate */
  const int min_norm_exp = 1 - bias; /* exponent of the smallest normal */
  int e;
  (void)frexpf(ax, &e); /* ax = m * 2^e, m in [0.5, 1) -> unbiased exponent is e-1 */
  int ue = e - 1;
  if (ax == 0.0f) return sign;
  if (ue < min_norm_exp) ue = min_norm_exp; /* subnormal range: fixed quantum */
  /* quantum = 2^(ue - man_bits); q = ax / quantum is exactly representable in double */
  const double q = ldexp((double)ax, -(ue - man_bits));
  double r = nearbyint(q); /* default rounding mode: nearest even */
  /* r is in [0, 2^(man_bits+1)] */
  uint32_t ri = (uint32_t)r;
  uint32_t byte;
  if (ue == min_norm_exp && ri < (1u << man_bits)) {
    byte = ri; /* subnormal (or zero) */
  } else {
    if (ri == (2u << man_bits)) { /* mantissa overflowed into the next binade */
      ri >>= 1;
      ue += 1;
    }
    byte = ((uint32_t)(ue + bias) << man_bits) | (ri & ((1u << man_bits) - 1u));
  }
  if (byte > max_byte) byte = max_byte;
  return (uint8_t)(sign | byte);
}

void fp8_oracle_cvt_array(const float* x, uint8_t* out, int64_t n, int format) {
  for (int64_t i = 0; i < n; ++i) out[i] = fp8_oracle_cvt(x[i], format);
}

float fp8_oracle_to_f32(uint8_t b, int format) {
  const int man_bits = (format == FP8_E4M3) ? 3 : 2;
  const int bias = (format == FP8_E4M3) ? 7 : 15;
  const int exp_bits = 7 - man_bits;
  const uint32_t man = b & ((1u << man_bits) - 1u);
  const uint32_t ex = (b >> man_bits) & ((1u << exp_bits) - 1u);
  float v;
  if (format == FP8_E4M3) {
    if ((b & 0x7F) == 0x7F) return NAN;
  } else {
    if (ex == 31) return man ? NAN : ((b & 0x80) ? -INFINITY : INFINITY);
  }
  if (ex == 0)
    v = ldexpf((float)man, 1 - bias - man_bits);
  else
    v = ldexpf((float)(man | (1u << man_bits)), (int)ex - bias - man_bits);
  return (b & 0x80) ? -v : v;
}

/* Flat quantise + amax.  amax is max-merged into *amax (which the caller may have pre-loaded). */
void fp8_oracle_quantize(const uint16_t* in_bf16, uint8_t* out, int64_t n, float scale, int format, float* amax) {
  float m = amax ? *amax : 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    const float v = bf16_to_f32(in_bf16[i]);
    const float a = fabsf(v);
    if (a > m) m = a; /* NaN never wins, like fmaxf */
    out[i] = fp8_oracle_cvt(v * scale, format);
  }
  if (amax) *amax = m;
}

/* Tanh-approximated GELU derivative, same expression and constants as the reference. */
static inline float dgelu_f32(float x) {
  const float t = tanhf(0.79788456f * x * (1.f + 0.044715f * x * x));
  return 0.5f * x * ((1.f - t * t) * (0.79788456f + 0.1070322243f * x * x)) + 0.5f * (1.f + t);
}

/*
 * bf16 (rows x cols) -> fp8 same shape (out, may be NULL) and fp8 transposed (cols x padded_rows,
 * out_t, may be NULL).  Rows >= rows of the transposed output hold cvt(scale * 0).
 * gelu_in != NULL selects the dGELU variant: x = in * dgelu(gelu_in).
 */
void fp8_oracle_pad_cast_transpose(const uint16_t* in_bf16, const uint16_t* gelu_in, uint8_t* out, uint8_t* out_t,
                                   int64_t rows, int64_t cols, int64_t padded_rows, float scale, int format,
                                   float* amax) {
  float m = amax ? *amax : 0.0f;
  const uint8_t pad = fp8_oracle_cvt(scale * 0.0f, format);
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < cols; ++c) {
      float v = bf16_to_f32(in_bf16[r * cols + c]);
      if (gelu_in) v = v * dgelu_f32(bf16_to_f32(gelu_in[r * cols + c]));
      const float a = fabsf(v);
      if (a > m) m = a;
      const uint8_t q = fp8_oracle_cvt(scale * v, format);
      if (out) out[r * cols + c] = q;
      if (out_t) out_t[c * padded_rows + r] = q;
    }
  }
  if (out_t)
    for (int64_t c = 0; c < cols; ++c)
      for (int64_t r = rows; r < padded_rows; ++r) out_t[c * padded_rows + r] = pad;
  if (amax) *amax = m;
}

/* fp8 (rows x cols) -> fp8 (cols x padded_rows), zero bytes in the padding. */
void fp8_oracle_pad_transpose(const uint8_t* in, uint8_t* out_t, int64_t rows, int64_t cols, int64_t padded_rows) {
  for (int64_t c = 0; c < cols; ++c) {
    for (int64_t r = 0; r < rows; ++r) out_t[c * padded_rows + r] = in[r * cols + c];
    for (int64_t r = rows; r < padded_rows; ++r) out_t[c * padded_rows + r] = 0;
  }
}

/* In-place x = bf16(fp32(x) * s1 * s2). */
void fp8_oracle_scale_mul(uint16_t* x_bf16, int64_t n, float s1, float s2) {
  for (int64_t i = 0; i < n; ++i) x_bf16[i] = f32_to_bf16(bf16_to_f32(x_bf16[i]) * s1 * s2);
}

/*
 * One group's GEMM on fp8 operands, both K-major: C (m x n) = A (m x k) * B (n x k)^T, fp32
 * accumulation of the dequantised values, one final rounding bf16(acc * alpha) with
 * alpha = a_scale_inv * b_scale_inv (the single-rounding fused epilogue).
 */
void fp8_oracle_gemm_nt(const uint8_t* a, int a_format, const uint8_t* b, int b_format, uint16_t* c_bf16, int64_t m,
                        int64_t n, int64_t k, float alpha) {
  float lut_a[256], lut_b[256];
  for (int i = 0; i < 256; ++i) {
    lut_a[i] = fp8_oracle_to_f32((uint8_t)i, a_format);
    lut_b[i] = fp8_oracle_to_f32((uint8_t)i, b_format);
  }
  float* arow = (float*)malloc(sizeof(float) * (size_t)k);
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t p = 0; p < k; ++p) arow[p] = lut_a[a[i * k + p]];
    for (int64_t j = 0; j < n; ++j) {
      const uint8_t* brow = b + j * k;
      float acc = 0.f;
      for (int64_t p = 0; p < k; ++p) acc += arow[p] * lut_b[brow[p]];
      c_bf16[i * n + j] = f32_to_bf16(acc * alpha);
    }
  }
  free(arow);
}
