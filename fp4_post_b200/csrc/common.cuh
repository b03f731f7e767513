// Shared host/device helpers of the Metis NVFP4 library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/metis_nvfp4.h"

namespace metis {

// ---- host-side status plumbing ---------------------------------------------------------

// Records a formatted message for metis_last_error_string() and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...);

#define METIS_CUDA_OK(expr)                                                          \
  do {                                                                               \
    cudaError_t e__ = (expr);                                                        \
    if (e__ != cudaSuccess)                                                          \
      return ::metis::fail(METIS_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- quantizer scratch ------------------------------------------------------------------------

constexpr int kWorkspaceHeaderBytes = 256;  // [0,4): bits of the global amax; then block maxima
struct WorkspaceView {
  unsigned int* gmax;  // bits of the largest block amax (a non-negative float orders like a uint)
  float* amax;         // [R, C/16]
};
static inline WorkspaceView view_workspace(void* ws) {
  return {reinterpret_cast<unsigned int*>(ws),
          reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWorkspaceHeaderBytes)};
}
// Shared by the stand-alone and the RMSNorm-fused quantizers (defined in quantize.cu).
int32_t launch_finalize(const WorkspaceView& ws, int64_t R, int64_t C, int32_t sf_layout,
                        uint8_t* scales, float* unit, cudaStream_t st);
int32_t check_quant_outputs(int64_t R, int64_t C, int32_t sf_layout, const void* codes,
                            const void* scales, const void* unit, const void* workspace,
                            int64_t workspace_bytes);
int device_sm_count();

// ---- scale-factor addressing ---------------------------------------------------------------

// Number of 512-byte tiles along the scale columns of a row of tiles: a tile holds 4 scale
// columns (64 elements); rows of tiles are padded to a multiple of 4 tiles (256 elements)
// so that one GEMM pipeline stage always reads 4 whole tiles.
__host__ __device__ static inline int64_t sf_tiles_per_row(int64_t C) { return ((C + 255) / 256) * 4; }

// Byte offset of the scale of row r, scale column k (= element column / 16) in METIS_SF_MMA.
__host__ __device__ static inline int64_t sf_mma_offset(int64_t r, int64_t k, int64_t tiles_per_row) {
  const int64_t tile = (r >> 7) * tiles_per_row + (k >> 2);
  return tile * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (k & 3);
}

// ---- number formats --------------------------------------------------------------------------

#ifdef __CUDACC__

// e2m1 magnitude code (0..7) -> value.
__device__ __forceinline__ float e2m1_value(uint32_t mag) {
  // {0, .5, 1, 1.5, 2, 3, 4, 6}
  const float lo = 0.5f * (float)mag;                      // codes 0..4
  const float hi = (float)(1u << (((mag >> 1) - 1u) & 3u)) * ((mag & 1u) ? 1.5f : 1.0f);  // codes >= 4
  return mag < 4u ? lo : hi;
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}

__device__ __forceinline__ uint8_t float_to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// Block scale from the block's absolute maximum: amax/6 + 1e-9 with two fp32 roundings
// (quant.py:19).
__device__ __forceinline__ float block_scale_from_amax(float amax) {
  return __fadd_rn(__fdiv_rn(amax, 6.0f), 1e-9f);
}

// Exact reference code of one magnitude: |x| / (s/2), folded onto 0..7, round half to even
// (quant.py:26-31).  relu(q-4)/2 == max(fma(q, .5, -2), 0) because scaling by a power of
// two commutes with rounding; likewise relu(q-8)/4.
__device__ __forceinline__ uint32_t e2m1_code_exact(float ax, float half_s) {
  const float q = __fdiv_rn(ax, half_s);
  const float a = fmaxf(__fmaf_rn(q, 0.5f, -2.0f), 0.0f);
  const float b = fmaxf(__fmaf_rn(q, 0.25f, -2.0f), 0.0f);
  const float q2 = __fsub_rn(q, __fadd_rn(a, b));
  const float r = fminf(rintf(q2), 7.0f);
  return (uint32_t)r;
}

// Two fp32 -> one byte of two e2m1 nibbles, round-to-nearest-even, saturating.
// `hi` lands in bits 7..4 and `lo` in bits 3..0.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float hi, float lo) {
  uint16_t out;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }"
      : "=h"(out) : "f"(hi), "f"(lo));
  return (uint32_t)out;
}

// Relative half-width of the band around a rounding boundary inside which the fast
// reciprocal path is not trusted and the exact division is used instead.
#define METIS_AMBIG_DELTA 1.9073486328125e-06f /* 2^-19 */

// Round-to-nearest codes of 8 consecutive values that share the block scale `s`.
// Returns 4 bytes (element 0 in the low nibble of byte 0).  Fast path: multiply by
// (1/s)(1 -+ delta) and convert both with the hardware e2m1 conversion; if the two results
// agree no rounding boundary lies in between, and because the reference's own boundary sits
// within a few ulps of the ideal one the result equals the reference's.  Otherwise every
// element is redone with the exact division sequence.
__device__ __forceinline__ uint32_t quantize8_rn(const float (&x)[8], float s) {
  const float r = __frcp_rn(s);
  const float rlo = r * (1.0f - METIS_AMBIG_DELTA);
  const float rhi = r * (1.0f + METIS_AMBIG_DELTA);
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // fma with +0 turns an input of -0.0 into +0.0 (the reference's sign(x) is 0 there)
    // while keeping the sign of every non-zero input, however small.
    lo |= cvt_e2m1x2(__fmaf_rn(x[2 * i + 1], rlo, 0.0f), __fmaf_rn(x[2 * i], rlo, 0.0f)) << (8 * i);
    hi |= cvt_e2m1x2(__fmaf_rn(x[2 * i + 1], rhi, 0.0f), __fmaf_rn(x[2 * i], rhi, 0.0f)) << (8 * i);
  }
  if (lo != hi) {
    const float half_s = 0.5f * s;
    lo = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t mag = e2m1_code_exact(fabsf(x[i]), half_s);
      const uint32_t nib = mag | (x[i] < 0.0f ? 8u : 0u);
      lo |= nib << (4 * i);
    }
  }
  return lo;
}

// ---- Philox4x32-10 ---------------------------------------------------------------------------------

struct Philox {
  uint32_t k0, k1;
  __device__ __forceinline__ Philox(uint64_t seed) : k0((uint32_t)seed), k1((uint32_t)(seed >> 32)) {}
  __device__ __forceinline__ uint4 operator()(uint64_t ctr_lo, uint64_t ctr_hi) const {
    uint32_t c0 = (uint32_t)ctr_lo, c1 = (uint32_t)(ctr_lo >> 32);
    uint32_t c2 = (uint32_t)ctr_hi, c3 = (uint32_t)(ctr_hi >> 32);
    uint32_t a = k0, b = k1;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
      const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
      const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
      c0 = h1 ^ c1 ^ a;  c1 = l1;  c2 = h0 ^ c3 ^ b;  c3 = l0;
      a += 0x9E3779B9u;  b += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
  }
};

// Stochastic-rounding codes of 8 values sharing scale s: fold |x|/(s/2) onto the index
// axis, add u in (-0.5, 0.5) built from 16 random bits, round (quant.py:139-147).
__device__ __forceinline__ uint32_t quantize8_sr(const float (&x)[8], float s, uint4 rnd) {
  const float inv_half = __fdividef(2.0f, s);
  const uint32_t rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float q = fabsf(x[i]) * inv_half;
    const float a = fmaxf(__fmaf_rn(q, 0.5f, -2.0f), 0.0f);
    const float b = fmaxf(__fmaf_rn(q, 0.25f, -2.0f), 0.0f);
    float q2 = q - (a + b);
    const uint32_t bits = (rw[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
    const float u = ((float)bits + 0.5f) * (1.0f / 65536.0f) - 0.5f;
    q2 = fminf(fmaxf(rintf(q2 + u), 0.0f), 7.0f);
    const uint32_t nib = (uint32_t)q2 | (x[i] < 0.0f ? 8u : 0u);
    out |= nib << (4 * i);
  }
  return out;
}

// ---- loads ------------------------------------------------------------------------------------------------

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// 8 consecutive elements starting at p (16-byte aligned for bf16, 32-byte for fp32).
template <typename T> struct Load8;
template <> struct Load8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(p));
    v[0] = bf16_lo(w.x); v[1] = bf16_hi(w.x); v[2] = bf16_lo(w.y); v[3] = bf16_hi(w.y);
    v[4] = bf16_lo(w.z); v[5] = bf16_hi(w.z); v[6] = bf16_lo(w.w); v[7] = bf16_hi(w.w);
  }
};
template <> struct Load8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

#endif  // __CUDACC__

}  // namespace metis
