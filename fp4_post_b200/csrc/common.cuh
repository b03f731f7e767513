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
                        uint8_t* scales, float* unit, cudaStream_t st, uint64_t* offset_ctr = nullptr);
int32_t check_quant_outputs(int64_t R, int64_t C, int32_t sf_layout, const void* codes,
                            const void* scales, const void* unit, const void* workspace,
                            int64_t workspace_bytes);
int device_sm_count();
int gemm_sm_budget(int32_t limit);   // device_sm_count(), capped by a positive per-call limit

// ---- overlapped launches ------------------------------------------------------------------------
// Every kernel of the library is launched with programmatic stream serialization: its CTAs may become
// resident (and run their shared-memory prologue) while the previous kernel of the stream drains,
// instead of after its last store has been flushed.  The contract that keeps this correct: a kernel
// calls grid_dependency_wait() on every thread, before its first global access and before any early
// return (the wait returns when the whole previous grid, and through it every earlier one, has
// completed and flushed).  grid_launch_dependents() lets the successor's CTAs in once every CTA of this
// grid has called it: the GEMMs call it when their last loads are issued and the split-K reduction at
// its top, so that the prologue of the next GEMM (barriers, tensor memory) hides behind the tail of
// this one; every other kernel leaves it to the implicit trigger at CTA exit.  Measured on the two-stream
// training step: successors let in earlier than that sit on the thread slots that the second stream's
// kernels run in beside a GEMM (0.91 ms per step against 0.865).  After a
// predecessor that is not a kernel, or for a class of kernels whose bit is cleared in METIS_LAUNCH_OVERLAP
// (environment; a mask of LaunchClass), the launch is an ordinary one and both calls are no-ops.
enum LaunchClass { kLaunchShort = 1, kLaunchGemm = 2, kLaunchStream = 4 };
bool launch_overlap_enabled(int launch_class);
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_overlapped(int launch_class, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                            cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_overlap_enabled(launch_class) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

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
// (quant.py:19).  The division is the correctly rounded one: q0 = a*r, e = fma(-6, q0, a),
// q = fma(e, r, q0) with r = RN(1/6) equals RN(a/6) for every finite a >= 2^-125 (checked
// exhaustively against IEEE division); below that the quotient is < 2^-127 and the sum with
// 1e-9 is 1e-9 either way.
__device__ __forceinline__ float block_scale_from_amax(float amax) {
  const float r6 = 0x1.555556p-3f;
  const float q0 = __fmul_rn(amax, r6);
  const float q = __fmaf_rn(__fmaf_rn(-6.0f, q0, amax), r6, q0);
  return __fadd_rn(q, 1e-9f);
}

__device__ __forceinline__ float rcp_approx(float v) {
  float r;
  asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 1.0f if v < 0 else 0.0f, on the multiply pipe: v * -inf is +inf, -inf or (for +-0) NaN, and the
// saturating multiply maps those to 1, 0 and 0.  This is the reference's sign(x) < 0, for which
// -0.0 counts as zero.
__device__ __forceinline__ float is_negative(float v) {
  float d;
  asm("mul.sat.f32 %0, %1, 0fFF800000;" : "=f"(d) : "f"(v));
  return d;
}

#define METIS_ROUND_MAGIC 12582912.0f          /* 1.5 * 2^23: adding it leaves rint(v) in the low mantissa bits */

// Index on the folded axis of the reference (quant.py:27-29): q = |x|/(s/2) in [0,12] is mapped
// to [0,7] by halving the slope above 4 and quartering it above 8, i.e. the pointwise minimum of
// the three lines q, q/2 + 2, q/4 + 4.  rint of it is the e2m1 magnitude code.
//
// With one rounding per line this reproduces the reference's op-by-op sequence
//   q - (relu(q-4)/2 + relu(q-8)/4)
// after rint for every q in [0, 12]: up to 4 both are q; on (4, 8] relu(q-4)/2 is exact, so the
// reference's q - a is the single rounding of q/2 + 2; on (8, 32/3) both relu terms and their sum
// are exact, so the result is the single rounding of q/4 + 4; from 32/3 on the sum may carry one
// extra rounding of 2^-22, but there the index is at least 6.66 and rounds to 7 either way.
__device__ __forceinline__ float folded_index(float q) {
  return min3(q, __fmaf_rn(q, 0.5f, 2.0f), __fmaf_rn(q, 0.25f, 4.0f));
}

// Correctly rounded a / h for |a| <= 12.1 h from a refined reciprocal r of h: one
// multiplication, the exact remainder and one correction (Markstein).  A remainder that
// underflows only occurs for quotients far below the first rounding boundary.
__device__ __forceinline__ float refine_reciprocal(float h) {
  const float r = rcp_approx(h);
  return __fmaf_rn(__fmaf_rn(-h, r, 1.0f), r, r);
}
__device__ __forceinline__ float divide_exact(float a, float h, float r) {
  const float q0 = __fmul_rn(a, r);
  return __fmaf_rn(__fmaf_rn(-h, q0, a), r, q0);
}

// 8 values -> 8 e2m1 nibbles, element 0 in the low nibble: round to nearest, ties to the even code,
// saturating, sign bit included (-0.0 and negative values that round to zero keep theirs).
__device__ __forceinline__ uint32_t pack_e2m1x8(const float (&v)[8]) {
  uint32_t out;
  asm("{ .reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3}; }"
      : "=r"(out)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return out;
}

// The reference rounds twice (quant.py:27-30): the folded index q/2 + 2 (or q/4 + 4) is rounded to
// fp32 before it is rounded to an integer, which drops the last bit of v = x/s for |v| >= 2.  The
// conversion to e2m1 rounds v itself, once.  Over all fp32 v in [0, 6.5] the two differ at exactly three
// values, the fp32 neighbours nextafter(2.5), prev(3.5) and nextafter(5) of a tie, which the reference
// sends to the tie's even code.  Dropping that bit the same way first, (v + t) - t with t = 2 on [2, 4)
// and 4 on [4, 8) (round to nearest even in the binade of the sum, as the reference's addition does),
// makes them agree everywhere.  t comes from the exponent bits of v: 0x40000000 is 2.0, 0x40800000 is
// 4.0; below 2, bit 30 is clear and what is left (0 or 2^-126) changes nothing; the sign is kept.
__device__ __forceinline__ float round_like_folded(float v) {
  const float t = __uint_as_float(__float_as_uint(v) & 0xC0800000u);
  return __fsub_rn(__fadd_rn(v, t), t);
}

// Round-to-nearest codes of kGroups*8 consecutive values sharing the block scale `s`
// (kGroups = 1: half a block, 2: a whole block); out[g] holds elements 8g..8g+7, element 0 in
// the low nibble.  Every element goes through the reference's own arithmetic: the correctly
// rounded quotient x/s (half the reference's |x|/(s/2), exactly), its second rounding, and round
// half to even onto the e2m1 grid by the hardware conversion, which packs two codes with their
// sign bits per instruction.  (The conversion runs on the special-function unit at about 26 cycles
// per warp; sending half of every block down an FMA/ALU-only path of the folded index, magic-number
// rounding and shifted adds instead was measured slower: 4 more instructions per element cost more
// than the relieved unit gives back.)  There is no approximate fast path because with bf16
// inputs exact ties (an element equal to amax/8, 5/24 amax, ...) are common.  The division is
// signed: -0.0 comes out as +0.0 (the remainder +0 wins the final sum), any negative x keeps its
// sign down to -0.0, which is the reference's sign bit (x < 0).
template <int kGroups>
__device__ __forceinline__ void quantize_rn(const float (&x)[8 * kGroups], float s, uint32_t (&out)[kGroups]) {
  const float r = refine_reciprocal(s);
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = round_like_folded(divide_exact(x[8 * g + i], s, r));
    out[g] = pack_e2m1x8(v);
  }
}

__device__ __forceinline__ uint32_t quantize8_rn(const float (&x)[8], float s) {
  uint32_t out[1];
  quantize_rn<1>(x, s, out);
  return out[0];
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

// Stochastic-rounding codes of one block (16 values sharing scale s): floor(folded index + U) with
// U uniform on [0, 1) in steps of 2^-16, which rounds up with probability frac(index) (quant.py:139-147:
// the reference adds rand - 0.5 and rounds to nearest).  No exact division here: the quotient only
// enters in distribution.  One Philox call (128 bits) serves the 16 elements: element 4w + j takes bytes
// j and j+1 (mod 4) of word w.  Each 16-bit window is exactly uniform; neighbours share one byte, the
// low byte of one being the high byte of the next, which moves the other's rounding probability by
// less than 2^-8.  Per element: one byte permute builds the float 2^23 + window (window in the low
// mantissa bits under the exponent of 2^23); index + window * 2^-16 + 128 is one multiply-add (the
// window's 16 bits survive exactly in [128, 256)); + 8 for x < 0; an addition of 2^23 rounding down
// leaves floor(index + U) + 8 [x < 0] + 128 in the low mantissa bits, and the integers are summed
// into nibbles with shifted adds (the constant bits are subtracted once at the end).
__device__ __forceinline__ void quantize16_sr(const float (&x)[16], float s, uint4 rnd, uint32_t (&out)[2]) {
  const float two_over_s = 2.0f * rcp_approx(s);
  const uint32_t rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
  const uint32_t magic_sum = 0x4B000080u * 0x11111111u;                  // (2^23 + 128) << 4i summed, mod 2^32
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = 8 * g + i;
      const float m = folded_index(fabsf(x[e]) * two_over_s);
      constexpr uint32_t kWindow[4] = {0x7610u, 0x7621u, 0x7632u, 0x7603u};     // bytes (j, j+1 mod 4) below 0x4B00
      const float rf = __uint_as_float(__byte_perm(rw[e >> 2], 0x4B000000u, kWindow[e & 3]));
      const float s1 = __fmaf_rn(rf, 0x1p-16f, m);                       // index + 128 + U
      const float s2 = __fmaf_rn(is_negative(x[e]), 8.0f, s1);
      const float t = __fadd_rd(s2, 8388608.0f);                         // floor
      acc += __float_as_uint(t) << (4 * i);
    }
    out[g] = acc - magic_sum;
  }
}

// The same rounding by the hardware conversion cvt.rs.satfinite.e2m1x4.f32: four elements and 32 random bits
// per instruction, 8 bits per element, up with probability floor(256 frac) / 256 where frac is the element's
// position between its two e2m1 neighbours (measured on every probe value and byte of the random word; which
// byte serves which element does not matter, all are uniform).  One Philox word per four elements, no other
// arithmetic than the multiplication by 1/s.  Operand order: the last of the four lands in the lowest nibble.
__device__ __forceinline__ uint32_t cvt_rs_e2m1x4(float e0, float e1, float e2, float e3, uint32_t rbits) {
  uint16_t r;
  asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;" : "=h"(r) : "f"(e3), "f"(e2), "f"(e1), "f"(e0), "r"(rbits));
  return r;
}
__device__ __forceinline__ void quantize16_sr_hw(const float (&x)[16], float s, uint4 rnd, uint32_t (&out)[2]) {
  const float inv = rcp_approx(s);
  const uint32_t rw[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
  uint32_t h[4];
#pragma unroll
  for (int w = 0; w < 4; ++w)
    h[w] = cvt_rs_e2m1x4(x[4 * w] * inv, x[4 * w + 1] * inv, x[4 * w + 2] * inv, x[4 * w + 3] * inv, rw[w]);
  out[0] = h[0] | (h[1] << 16);
  out[1] = h[2] | (h[3] << 16);
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

// Largest magnitude of a 16-element block (three-input maxima: 8 instructions).
__device__ __forceinline__ float abs_max16(const float (&v)[16]) {
  float a = fmaxf(fabsf(v[0]), fabsf(v[1]));
#pragma unroll
  for (int i = 2; i < 16; i += 2) a = max3(a, fabsf(v[i]), fabsf(v[i + 1]));
  return a;
}

// 16 consecutive elements (one quantization block) starting at p, 16-byte aligned.
template <typename T> struct Load16;
template <> struct Load16<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[16]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[2 * i] = bf16_lo(w[i]); v[2 * i + 1] = bf16_hi(w[i]); }
  }
};
template <> struct Load16<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p) + i);
      v[4 * i] = a.x; v[4 * i + 1] = a.y; v[4 * i + 2] = a.z; v[4 * i + 3] = a.w;
    }
  }
};

// The same block kept as loaded (8 or 16 registers) so that the next block's loads can be in
// flight while the current one is worked on.
template <typename T> struct RawBlock;
template <> struct RawBlock<__nv_bfloat16> {
  uint4 a, b;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    a = __ldg(reinterpret_cast<const uint4*>(p));
    b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  }
  __device__ __forceinline__ void unpack(float (&v)[16]) const {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[2 * i] = bf16_lo(w[i]); v[2 * i + 1] = bf16_hi(w[i]); }
  }
};
template <> struct RawBlock<float> {
  float4 q[4];
  __device__ __forceinline__ void load(const float* p) {
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = __ldg(reinterpret_cast<const float4*>(p) + i);
  }
  __device__ __forceinline__ void unpack(float (&v)[16]) const {
#pragma unroll
    for (int i = 0; i < 4; ++i) { v[4 * i] = q[i].x; v[4 * i + 1] = q[i].y; v[4 * i + 2] = q[i].z; v[4 * i + 3] = q[i].w; }
  }
};

// ---- one-cluster kernels for small tensors ------------------------------------------------------
// The tensor-wide maximum of a kernel that runs as ONE thread-block cluster: warp shuffle, shared
// memory of the CTA, then every CTA reads its peers' maxima through distributed shared memory between
// two hardware cluster barriers.  All threads of all CTAs call cluster_fmax() once, and
// cluster_leave() before they exit (no CTA may go while a peer can still read its shared memory).
struct ClusterMaxSmem {
  float warp[32];
  float cta;
  float all;
};
__device__ __forceinline__ uint32_t cluster_cta_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_cta_count() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ float cluster_fmax(float v, ClusterMaxSmem& sm) {
  const uint32_t tid = threadIdx.y * blockDim.x + threadIdx.x;
  const uint32_t warps = (blockDim.x * blockDim.y + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((tid & 31u) == 0) sm.warp[tid >> 5] = v;
  __syncthreads();
  if (tid < 32) {
    float m = tid < warps ? sm.warp[tid] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (tid == 0) sm.cta = m;
  }
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (tid < 32) {
    float m = 0.0f;
    if (tid < cluster_cta_count()) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(&sm.cta)), "r"(tid));
      asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(m) : "r"(remote) : "memory");
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (tid == 0) sm.all = m;
  }
  __syncthreads();
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");     // this CTA has read its peers
  return sm.all;
}
__device__ __forceinline__ void cluster_leave() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// METIS_SF_MMA pads rows to a multiple of 128 and scale columns to whole tiles of 4: thread t of
// `stride` clears those bytes (padded_words = 32-bit words of the whole scale array).  The walk is over
// the 16-byte pieces of the layout: piece p holds rows l, l+32, l+64, l+96 (l = p % 32) of one tile, so
// a piece whose first row is past the end is padding as a whole.
__device__ __forceinline__ void zero_scale_padding(uint8_t* scales, int rows, int blocks_per_row, int tiles,
                                                   int padded_words, int t, int stride) {
  const int pieces = padded_words >> 2;
  for (int p = t; p < pieces; p += stride) {
    const int l = p & 31, tu = p >> 5;
    const int rb = tu / tiles, u = tu - rb * tiles;
    uint8_t* piece = scales + (int64_t)p * 16;
    const int r0 = rb * 128 + l;
    if (u * 4 >= blocks_per_row || r0 >= rows) {
      *reinterpret_cast<uint4*>(piece) = make_uint4(0u, 0u, 0u, 0u);
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (r0 + 32 * c >= rows) {
          *reinterpret_cast<uint32_t*>(piece + 4 * c) = 0u;
        } else {
          for (int k = 1; k < 4; ++k) if (u * 4 + k >= blocks_per_row) piece[4 * c + k] = 0;
        }
      }
    }
  }
}

// Limits of the one-cluster kernels (shared by the stand-alone and the RMSNorm-fused quantizer).
constexpr int kSmallCtas = 8;                      // portable cluster size
// Sum of the 16 signed codes of one block, in half units.  prmt looks four codes up at once in the
// 8-entry magnitude table {0,1,2,3,4,6,8,12}; a selector nibble with bit 3 set yields the sign
// replica of the table byte, i.e. zero, so the first look-up keeps the positive codes and the second
// (sign bits flipped) the negative ones.  Byte sums stay below 256, one dp4a adds the four bytes.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ int block_code_sum(uint2 w) {
  constexpr uint32_t kLo = 0x03020100u, kHi = 0x0C080604u;
  const uint32_t nx = w.x ^ 0x88888888u, ny = w.y ^ 0x88888888u;
  const uint32_t pos = prmt(kLo, kHi, w.x) + prmt(kLo, kHi, w.x >> 16) + prmt(kLo, kHi, w.y) + prmt(kLo, kHi, w.y >> 16);
  const uint32_t neg = prmt(kLo, kHi, nx) + prmt(kLo, kHi, nx >> 16) + prmt(kLo, kHi, ny) + prmt(kLo, kHi, ny >> 16);
  return __dp4a(pos, 0x01010101u, 0u) - __dp4a(neg, 0x01010101u, 0u);
}

constexpr int64_t kSmallMaxPaddedWords = 16384;    // words of the tiled scale array, zero-filled padding included

#endif  // __CUDACC__

}  // namespace metis
