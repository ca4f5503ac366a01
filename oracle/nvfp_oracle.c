/*
 * CPU restatement (plain C, OpenMP) of the NVFP4 / MXFP4 quantize -> block-scaled GEMM path.
 *
 * TEST INFRASTRUCTURE ONLY: used by the tests, the smoke test and the CPU-baseline leg of
 * the benchmark as the checker.  The product library never links or loads it.
 *
 * Follows the reference (huweim/nvfp_kernel):
 *   quantizer arithmetic ....... kernel/nvfp4_utils.cuh:166-242 (fast-math build: fp32
 *                                multiplies flush denormals, setup.py:45)
 *   nibble order ............... kernel/nvfp4_utils.cuh:70-109
 *   swizzled scale offset ...... kernel/nvfp4_utils.cuh:126-153
 *   GEMM contract .............. kernel/nvfp4_scaled_mm_sm120_kernels.cu:151-164
 *   dequantize ................. nvfp/pseudo_quant.py:166-180
 * It agrees bit for bit with oracle/nvfp_oracle.py (checked by the CPU tests), which in
 * turn is pinned against outputs of the reference itself (tests/golden/).
 * MXFP4: the reference has no reachable MXFP4 path; its disabled e8m0 branch (kernel/nvfp4_utils.cuh:196-202) pins the
 * `floor` scale rounding of the numpy oracle's quantizer (tests/golden/ref_kernel_ue8m0_sm100.npz); this file holds
 * the MXFP4 GEMM only.
 *
 * The hardware reciprocal rcp.approx.ftz.f32 is modelled either by the correctly rounded
 * 1/x or by a caller-supplied table of (input, output) bit patterns captured on a GPU.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bits_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float ftz(float x) {
  uint32_t u = f_bits(x);
  if ((u & 0x7f800000u) == 0) u &= 0x80000000u;
  return bits_f(u);
}
static inline float mul_ftz(float a, float b) { volatile float p = ftz(a) * ftz(b); return ftz(p); }

typedef struct { const uint32_t* in; const uint32_t* out; int n; } rcp_table;

static float rcp_model(float x, const rcp_table* t) {
  if (t && t->n > 0) {
    uint32_t u = f_bits(x);
    for (int i = 0; i < t->n; ++i) if (t->in[i] == u) return bits_f(t->out[i]);
  }
  x = ftz(x);
  volatile float r = (float)(1.0 / (double)x);
  return ftz(r);
}

static inline float bf16_to_f(uint16_t h) { return bits_f((uint32_t)h << 16); }
static float f16_to_f(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ff;
  if (e == 0) { float v = ldexpf((float)m, -24); return s ? -v : v; }
  if (e == 31) return bits_f(s | 0x7f800000u | (m << 13));
  return bits_f(s | ((e + 112) << 23) | (m << 13));
}

/* cvt.rn.satfinite.e4m3 of a non-negative fp32 */
static uint8_t e4m3_encode(float s) {
  if (s != s) return 0x7f;
  double v = s > 448.0f ? 448.0 : (double)s;
  if (v <= 0) return 0;
  int e; frexp(v, &e); e -= 1;               /* v = 1.xxx * 2^e */
  if (e < -6) e = -6;
  double step = ldexp(1.0, e - 3);
  double q = nearbyint(v / step) * step;     /* default rounding mode: half to even */
  if (q > 448.0) q = 448.0;
  if (q < ldexp(1.0, -6)) return (uint8_t)(q * 512.0);
  int e2; frexp(q, &e2); e2 -= 1;
  int mant = (int)(q / ldexp(1.0, e2) * 8.0 - 8.0);
  return (uint8_t)(((e2 + 7) << 3) | mant);
}
static float e4m3_decode(uint8_t b) {
  int e = (b >> 3) & 0xf, m = b & 7;
  if ((b & 0x7f) == 0x7f) return NAN;
  float v = e == 0 ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
  return (b & 0x80) ? -v : v;
}
static double e8m0_decode(uint8_t b) { return b == 255 ? NAN : ldexp(1.0, (int)b - 127); }

/* cvt.rn.satfinite.e2m1 */
static uint8_t e2m1_encode(float y) {
  if (y != y) return 0x7;
  double a = fabs((double)y);
  uint8_t c = 0;
  if (a > 0.25) c = 1;
  if (a >= 0.75) c = 2;
  if (a > 1.25) c = 3;
  if (a >= 1.75) c = 4;
  if (a > 2.5) c = 5;
  if (a >= 3.5) c = 6;
  if (a > 5.0) c = 7;
  return (uint8_t)(c | (signbit(y) ? 8 : 0));
}
static const float kE2M1[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
static inline float e2m1_decode(uint8_t n) { float v = kE2M1[n & 7]; return (n & 8) ? -v : v; }

static inline int64_t sf_offset(int64_t m, int64_t kb, int64_t k_tiles) {
  return (m / 128) * (k_tiles * 512) + (kb / 4) * 512 + (m % 32) * 16 + ((m % 128) / 32) * 4 + (kb % 4);
}

/* out_sf must hold round_up(m,128) * round_up(n/16,4) bytes; it is zero-filled here. */
void nvfp_oracle_quantize_nvfp4(const uint16_t* x, int is_bf16, int64_t m, int64_t n, int64_t stride,
                                float gs, const uint32_t* rcp_in, const uint32_t* rcp_out, int rcp_count,
                                uint8_t* out_fp4, uint8_t* out_sf) {
  rcp_table t = {rcp_in, rcp_out, rcp_count};
  const int64_t kb_count = n / 16, k_tiles = (kb_count + 3) / 4;
  memset(out_sf, 0, (size_t)(((m + 127) / 128) * 128 * k_tiles * 4));
  const float r6 = rcp_model(6.0f, &t), rg = rcp_model(gs, &t);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    for (int64_t kb = 0; kb < kb_count; ++kb) {
      float v[16], amax = NAN;   /* fmaxf skips a NaN operand, as __hmax2 does: NaN only if every element is */
      for (int i = 0; i < 16; ++i) {
        uint16_t h = x[r * stride + kb * 16 + i];
        v[i] = is_bf16 ? bf16_to_f(h) : f16_to_f(h);
        float a = fabsf(v[i]);
        amax = fmaxf(amax, a);                 /* NaN inputs are ignored, like __hmax2 */
      }
      float sfv = mul_ftz(gs, mul_ftz(amax, r6));
      uint8_t sb = e4m3_encode(sfv);
      float sq = e4m3_decode(sb);
      float o = sq != 0.f ? rcp_model(mul_ftz(sq, rg), &t) : 0.f;
      out_sf[sf_offset(r, kb, k_tiles)] = sb;
      for (int i = 0; i < 16; i += 2) {
        uint8_t lo = e2m1_encode(mul_ftz(v[i], o)), hi = e2m1_encode(mul_ftz(v[i + 1], o));
        out_fp4[r * (n / 2) + kb * 8 + i / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
}

/* rounding: 0 = exponent rounded up, 1 = truncated.  32-element blocks, ue8m0 scales. */
void nvfp_oracle_quantize_mxfp4(const uint16_t* x, int is_bf16, int64_t m, int64_t n, int64_t stride,
                                int rounding, uint8_t* out_fp4, uint8_t* out_sf) {
  const int64_t kb_count = n / 32, k_tiles = (kb_count + 3) / 4;
  memset(out_sf, 0, (size_t)(((m + 127) / 128) * 128 * k_tiles * 4));
  const float r6 = bits_f(0x3E2AAAABu);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    for (int64_t kb = 0; kb < kb_count; ++kb) {
      float v[32], amax = NAN;   /* fmaxf skips a NaN operand, as __hmax2 does: NaN only if every element is */
      for (int i = 0; i < 32; ++i) {
        uint16_t h = x[r * stride + kb * 32 + i];
        v[i] = is_bf16 ? bf16_to_f(h) : f16_to_f(h);
        float a = fabsf(v[i]);
        amax = fmaxf(amax, a);
      }
      float sfv = mul_ftz(amax, r6);
      uint32_t bits = f_bits(sfv), e = (bits >> 23) & 0xff;
      if (rounding == 0 && (bits & 0x7fffffu) != 0 && e < 254) e += 1;
      if (e > 254 && rounding == 0) e = 254;   /* infinite block: rceil keeps 254, floor the raw exponent 255 (the reference's branch) */
      if (sfv != sfv) e = 255;
      float o = (e > 0 && e < 254) ? bits_f((254u - e) << 23) : 0.f;
      out_sf[sf_offset(r, kb, k_tiles)] = (uint8_t)e;
      for (int i = 0; i < 32; i += 2) {
        uint8_t lo = e2m1_encode(mul_ftz(v[i], o)), hi = e2m1_encode(mul_ftz(v[i + 1], o));
        out_fp4[r * (n / 2) + kb * 16 + i / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
}

/* value * block scale (no global scale) as fp32: exact, both factors have few bits */
static void dequant_rows(const uint8_t* q, const uint8_t* sf, int64_t rows, int64_t k, int block, int ue8m0,
                         float* out) {
  const int64_t k_tiles = (k / block + 3) / 4;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t c = 0; c < k; ++c) {
      uint8_t byte = q[r * (k / 2) + c / 2];
      uint8_t nib = (c & 1) ? (byte >> 4) : (byte & 0xf);
      uint8_t sb = sf[sf_offset(r, c / block, k_tiles)];
      double s = ue8m0 ? e8m0_decode(sb) : (double)e4m3_decode(sb);
      out[r * k + c] = (float)((double)e2m1_decode(nib) * s);
    }
}

/* d[m,n] (double, unrounded) = alpha * dequant(a) . dequant(b)^T with fp64 accumulation */
int nvfp_oracle_scaled_mm(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb,
                          float alpha, int64_t m, int64_t n, int64_t k, int block, int ue8m0, double* d) {
  float* fa = (float*)malloc(sizeof(float) * (size_t)(m * k));
  float* fb = (float*)malloc(sizeof(float) * (size_t)(n * k));
  if (!fa || !fb) { free(fa); free(fb); return 1; }
  dequant_rows(a, sfa, m, k, block, ue8m0, fa);
  dequant_rows(b, sfb, n, k, block, ue8m0, fb);
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      const float* pa = fa + i * k;
      const float* pb = fb + j * k;
      double acc = 0.0;
      for (int64_t c = 0; c < k; ++c) acc += (double)pa[c] * (double)pb[c];
      d[i * n + j] = (double)alpha * acc;
    }
  free(fa); free(fb);
  return 0;
}

/* max |x| as fp32 (exact in the input type) */
float nvfp_oracle_amax(const uint16_t* x, int is_bf16, int64_t m, int64_t n, int64_t stride) {
  float amax = 0.f;   /* torch.abs(x).max(): a NaN anywhere makes the result NaN */
  int nan_seen = 0;
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < n; ++c) {
      uint16_t h = x[r * stride + c];
      float a = fabsf(is_bf16 ? bf16_to_f(h) : f16_to_f(h));
      if (a != a) nan_seen = 1;
      amax = fmaxf(amax, a);
    }
  return nan_seen ? NAN : amax;
}
