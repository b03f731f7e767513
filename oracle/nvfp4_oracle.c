/*
 * CPU restatement of the reference's NVFP4 fake-quantizer, extended to emit the packed
 * representation the reference never materialises.  TEST INFRASTRUCTURE ONLY: the product
 * never links or calls this file; tests, the smoke check and the CPU-baseline leg of the
 * benchmark do.
 *
 * Follows decisivemoments/fp4-post, file src/Metis/Metis/quant.py:
 *   block scale      s = amax(|x|, 16)/6 + 1e-9                          quant.py:19
 *   tensor unit      unit = max(s)/448                                   quant.py:21-22
 *   stored scale     e4m3fn(s/unit), decoded d = fp32(e4m3)*unit         quant.py:23-24
 *   code             q = |x|/(s/2); q -= relu(q-4)/2 + relu(q-8)/4;
 *                    r = round_half_even(q)  (the e2m1 magnitude code)   quant.py:26-31
 *   value            ((expand(r)*sign(x))/2)*d                           quant.py:32-35
 * and, for the mean-centred variant, bitlinear.py:330-332 (x - me quantized, me added back).
 * The float8_e4m3fn conversion is PyTorch's (round to nearest even, subnormals down to 2^-9,
 * NaN above 464); it is restated here from the format's definition.
 *
 * Parity is pinned by tests/golden: vectors produced by importing the reference itself.
 *
 * Build: see oracle/Makefile (plain gcc, -ffp-contract=off so that no multiply-add is fused).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <string.h>

static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* float -> float8_e4m3fn byte, round to nearest even. */
uint8_t oracle_f32_to_e4m3fn(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  const uint8_t sign = (uint8_t)((bits >> 31) << 7);
  const float a = fabsf(f);
  if (isnan(a)) return (uint8_t)(sign | 0x7f);
  if (a < 0.015625f) { /* below 2^-6: multiples of 2^-9; 8 lands on the smallest normal */
    const int n = (int)rintf(a * 512.0f);
    return (uint8_t)(sign | n);
  }
  int e;
  const float m = frexpf(a, &e); /* a = m * 2^e, m in [0.5, 1) */
  int E = e - 1;
  int mant = (int)rintf((2.0f * m - 1.0f) * 8.0f);
  if (mant == 8) { mant = 0; E += 1; }
  if (E > 8 || (E == 8 && mant == 7)) return (uint8_t)(sign | 0x7f);
  return (uint8_t)(sign | ((E + 7) << 3) | mant);
}

float oracle_e4m3fn_to_f32(uint8_t b) {
  const int exp = (b >> 3) & 15, mant = b & 7;
  float v;
  if (exp == 15 && mant == 7) v = NAN;
  else if (exp == 0) v = (float)mant * 0.001953125f; /* 2^-9 */
  else v = ldexpf(1.0f + (float)mant * 0.125f, exp - 7);
  return (b & 0x80) ? -v : v;
}

static inline float relu(float v) { return v > 0.0f ? v : 0.0f; }

/* e2m1 magnitude code of one element given the block's s/2 (quant.py:26-31). */
static inline uint32_t magnitude_code(float ax, float half_s) {
  float q = ax / half_s;
  const float t1 = relu(q - 4.0f) / 2.0f;
  const float t2 = relu(q - 8.0f) / 4.0f;
  q = q - (t1 + t2);
  q = rintf(q);
  if (q > 7.0f) q = 7.0f;
  return (uint32_t)q;
}

/* Pass 1 over rows [r0, r1): codes, un-rounded block scales s, and the largest s seen. */
static float quantize_rows_pass1(const float* x, int64_t r0, int64_t r1, int64_t cols,
                                 const float* col_mean, uint8_t* codes, float* block_scale) {
  const int64_t nb = cols / 16;
  float smax = 0.0f;
  for (int64_t r = r0; r < r1; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      float v[16];
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        float e = x[r * cols + b * 16 + i];
        if (col_mean) e = e - col_mean[b * 16 + i];
        v[i] = e;
        const float a = fabsf(e);
        if (a > amax) amax = a;
      }
      const float s = amax / 6.0f + 1e-9f;
      block_scale[r * nb + b] = s;
      if (s > smax) smax = s;
      const float half_s = s / 2.0f;
      for (int i = 0; i < 16; i += 2) {
        const uint32_t lo = magnitude_code(fabsf(v[i]), half_s) | (v[i] < 0.0f ? 8u : 0u);
        const uint32_t hi = magnitude_code(fabsf(v[i + 1]), half_s) | (v[i + 1] < 0.0f ? 8u : 0u);
        codes[r * (cols / 2) + b * 8 + i / 2] = (uint8_t)(lo | (hi << 4));
      }
    }
  }
  return smax;
}

/* Pass 2 over rows [r0, r1): block scales relative to the tensor unit, as e4m3fn bytes. */
static void quantize_rows_pass2(const float* block_scale, int64_t r0, int64_t r1, int64_t nb,
                                float unit, uint8_t* scales) {
  for (int64_t i = r0 * nb; i < r1 * nb; ++i) scales[i] = oracle_f32_to_e4m3fn(block_scale[i] / unit);
}

typedef struct {
  const float* x; int64_t r0, r1, cols; const float* col_mean;
  uint8_t* codes; float* block_scale; uint8_t* scales; float unit; float smax;
} quant_job;

static void* job_pass1(void* arg) {
  quant_job* j = (quant_job*)arg;
  j->smax = quantize_rows_pass1(j->x, j->r0, j->r1, j->cols, j->col_mean, j->codes, j->block_scale);
  return 0;
}
static void* job_pass2(void* arg) {
  quant_job* j = (quant_job*)arg;
  quantize_rows_pass2(j->block_scale, j->r0, j->r1, j->cols / 16, j->unit, j->scales);
  return 0;
}

/*
 * x [rows, cols] fp32 row-major (ld == cols); col_mean optional [cols].
 * codes       [rows, cols/2]  low nibble = even element, nibble = sign<<3 | magnitude code
 * scales      [rows, cols/16] float8_e4m3fn bytes, row-major
 * block_scale [rows, cols/16] the un-rounded fp32 s (required: it is also the scratch)
 * threads     rows are split over this many pthreads (<= 1: run in the caller)
 * Returns 0, or -1 if 16 does not divide cols (quant.py:400-403 raises there).
 */
int oracle_nvfp4_quantize(const float* x, int64_t rows, int64_t cols, const float* col_mean,
                          uint8_t* codes, uint8_t* scales, float* unit, float* block_scale,
                          int threads) {
  if (cols % 16 != 0 || rows <= 0 || cols <= 0) return -1;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  if (threads > rows) threads = (int)rows;
  quant_job jobs[256];
  pthread_t tid[256];
  for (int t = 0; t < threads; ++t) {
    quant_job j = {x, rows * t / threads, rows * (t + 1) / threads, cols, col_mean,
                   codes, block_scale, scales, 0.0f, 0.0f};
    jobs[t] = j;
  }
  for (int t = 1; t < threads; ++t) pthread_create(&tid[t], 0, job_pass1, &jobs[t]);
  job_pass1(&jobs[0]);
  for (int t = 1; t < threads; ++t) pthread_join(tid[t], 0);
  float smax = 0.0f;
  for (int t = 0; t < threads; ++t) if (jobs[t].smax > smax) smax = jobs[t].smax;
  const float u = smax / 448.0f;
  *unit = u;
  for (int t = 0; t < threads; ++t) jobs[t].unit = u;
  for (int t = 1; t < threads; ++t) pthread_create(&tid[t], 0, job_pass2, &jobs[t]);
  job_pass2(&jobs[0]);
  for (int t = 1; t < threads; ++t) pthread_join(tid[t], 0);
  return 0;
}

/* out = e2m1(code) * (e4m3(scale) * unit) (+ col_mean), the reference's dequantized value. */
int oracle_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, float unit, int64_t rows,
                            int64_t cols, const float* col_mean, float* out) {
  if (cols % 16 != 0 || rows <= 0 || cols <= 0) return -1;
  const int64_t nb = cols / 16;
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t b = 0; b < nb; ++b) {
      const float d = oracle_e4m3fn_to_f32(scales[r * nb + b]) * unit;
      for (int i = 0; i < 16; ++i) {
        const uint8_t byte = codes[r * (cols / 2) + b * 8 + i / 2];
        const uint32_t nib = (i & 1) ? (byte >> 4) : (byte & 15);
        float val = kE2M1[nib & 7];
        if (nib & 8) val = -val;
        val = val * d;
        if (col_mean) val = col_mean[b * 16 + i] + val;
        out[r * cols + b * 16 + i] = val;
      }
    }
  }
  return 0;
}

/* Scale bytes row-major [R, C/16] -> the 128x4 tile order used by block-scaled tensor-core
 * instructions: tile (R/128, k/4), byte (r%32)*16 + (r/32%4)*4 + k%4; rows of tiles padded to a
 * multiple of 4 tiles, padding zero. out must hold ceil(R/128)*4*ceil(C/256)*512 bytes. */
void oracle_scales_to_mma_layout(const uint8_t* rowmajor, int64_t R, int64_t C, uint8_t* out) {
  const int64_t nb = C / 16;
  const int64_t tiles = ((C + 255) / 256) * 4;
  const int64_t rblocks = (R + 127) / 128;
  memset(out, 0, (size_t)(rblocks * tiles * 512));
  for (int64_t r = 0; r < R; ++r)
    for (int64_t k = 0; k < nb; ++k)
      out[((r >> 7) * tiles + (k >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (k & 3)] =
          rowmajor[r * nb + k];
}

/* ---- cross-check of the conversion-based rounding the CUDA kernels use --------------------------------
 * The kernels take the code from a round-to-nearest-even conversion of v = x/s onto the e2m1 grid
 * {0, .5, 1, 1.5, 2, 3, 4, 6}, where the reference (quant.py:26-31) rounds the folded index
 * q - (relu(q-4)/2 + relu(q-8)/4), q = 2v, twice.  This walks every fp32 v whose bit pattern lies in
 * [lo_bits, hi_bits] and counts where the reference's code differs from (a) the plain conversion and
 * (b) the conversion applied to (v + t) - t with t = 2 on [2, 4), 4 on [4, 8), 0 or 2^-126 below 2
 * (t = bits(v) & 0xC0800000), which drops the last bit of v the way the reference's addition does. */
static inline uint32_t e2m1_round_nearest_even(float a) {
  if (a >= 6.0f) return 7;
  int lo = 0;
  for (int i = 0; i < 8; ++i) if (kE2M1[i] <= a) lo = i;
  const float dl = a - kE2M1[lo], dh = kE2M1[lo + 1] - a; /* exact: neighbours within a factor of two */
  if (dl < dh) return (uint32_t)lo;
  if (dl > dh) return (uint32_t)lo + 1;
  return (uint32_t)((lo & 1) ? lo + 1 : lo);
}

void oracle_compare_conversion_rounding(uint32_t lo_bits, uint32_t hi_bits, uint64_t* plain_differs,
                                        uint64_t* fixed_differs, uint32_t* first_plain_bits) {
  uint64_t plain = 0, fixed = 0;
  int n_first = 0;
  for (uint32_t b = lo_bits;; ++b) {
    float v;
    memcpy(&v, &b, 4);
    const float half_s = 0.5f;                       /* q = v / 0.5 = 2v exactly */
    const uint32_t want = magnitude_code(v, half_s);
    if (e2m1_round_nearest_even(v) != want) {
      ++plain;
      if (n_first < 8 && first_plain_bits) first_plain_bits[n_first++] = b;
    }
    const uint32_t tb = b & 0xC0800000u;
    float t;
    memcpy(&t, &tb, 4);
    volatile float w = v + t;
    const float v2 = w - t;
    if (e2m1_round_nearest_even(v2) != want) ++fixed;
    if (b == hi_bits) break;
  }
  *plain_differs = plain;
  *fixed_differs = fixed;
}
