// NVFP4 -> dense conversion and the quantized matrix x vector product.
#include "common.cuh"

#include <cuda_fp16.h>

namespace metis {

__device__ __forceinline__ float scale_at(const uint8_t* scales, int32_t sf_layout, int64_t r,
                                          int64_t k, int64_t sf_cols, int64_t tiles) {
  const int64_t off = (sf_layout == METIS_SF_MMA) ? sf_mma_offset(r, k, tiles) : r * sf_cols + k;
  return e4m3_to_float(__ldg(scales + off));
}

// One thread per 8 elements (4 code bytes).
template <typename TO>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                  const float* __restrict__ unit_ptr, int32_t sf_layout, int64_t R, int64_t C,
                  const float* __restrict__ add_row_vec, TO* __restrict__ out, int64_t ld) {
  grid_dependency_wait();
  const float unit = __ldg(unit_ptr);
  const int64_t chunks_per_row = C >> 3;
  const int64_t total = R * chunks_per_row;
  const int64_t sf_cols = C >> 4;
  const int64_t tiles = sf_tiles_per_row(C);
  for (int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x; c < total; c += (int64_t)gridDim.x * 256) {
    const int64_t r = c / chunks_per_row;
    const int64_t ch = c - r * chunks_per_row;
    const uint32_t w = __ldg(codes + c);
    // value = e2m1 * (e4m3 * unit): the same two roundings as quant.py:23-35
    const float d = __fmul_rn(scale_at(scales, sf_layout, r, ch >> 1, sf_cols, tiles), unit);
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t nib = (w >> (4 * i)) & 15u;
      float val = __fmul_rn(e2m1_value(nib & 7u), d);
      if (nib & 8u) val = -val;
      y[i] = val;
    }
    if (add_row_vec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = __fadd_rn(__ldg(add_row_vec + ch * 8 + i), y[i]);
    }
    TO* dst = out + r * ld + ch * 8;
    if constexpr (sizeof(TO) == 2) {
      __nv_bfloat162 o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(o);
    } else {
      reinterpret_cast<float4*>(dst)[0] = make_float4(y[0], y[1], y[2], y[3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(y[4], y[5], y[6], y[7]);
    }
  }
}

// out[r] = sum_c v[c] * value(Q[r][c]).  One warp per row; per step a lane takes one block (16
// elements: one 64-bit load of codes, one scale byte), so a warp reads 512 consecutive elements and
// the matching stretch of v with 128-bit loads.  Twice the e2m1 magnitude comes from a nibble table
// held in one 32-bit constant; a block's partial sum is formed in integers (v == NULL) or with one
// multiply-add per element, then scaled once.
__device__ __forceinline__ int twice_e2m1(uint32_t nib) {
  const int mag = (int)((0xC8643210u >> ((nib & 7u) * 4u)) & 15u);     // {0,1,2,3,4,6,8,12}
  return (nib & 8u) ? -mag : mag;
}

template <bool kHasV>
__global__ void __launch_bounds__(256)
gemv_kernel(const uint2* __restrict__ codes, const uint8_t* __restrict__ scales,
            const float* __restrict__ unit_ptr, int32_t sf_layout, int64_t R, int64_t C,
            const float* __restrict__ v, float* __restrict__ out) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= R) return;
  const int64_t sf_cols = C >> 4;               // blocks per row
  const int64_t tiles = sf_tiles_per_row(C);
  const uint2* row_codes = codes + row * sf_cols;
  float acc = 0.0f;
  if (!kHasV && sf_layout == METIS_SF_MMA && (sf_cols & 3) == 0) {
    // row sums: four blocks per lane and trip (two 16-byte loads of codes, the four scale bytes
    // are one aligned word of the tile layout)
#pragma unroll 2
    for (int64_t g = lane; g < (sf_cols >> 2); g += 32) {
      const uint4 a = __ldg(reinterpret_cast<const uint4*>(row_codes + 4 * g));
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(row_codes + 4 * g) + 1);
      const uint32_t s4 = __ldg(reinterpret_cast<const uint32_t*>(scales + sf_mma_offset(row, 4 * g, tiles)));
      acc = fmaf((float)block_code_sum(make_uint2(a.x, a.y)), e4m3_to_float(s4 & 0xFFu), acc);
      acc = fmaf((float)block_code_sum(make_uint2(a.z, a.w)), e4m3_to_float((s4 >> 8) & 0xFFu), acc);
      acc = fmaf((float)block_code_sum(make_uint2(b.x, b.y)), e4m3_to_float((s4 >> 16) & 0xFFu), acc);
      acc = fmaf((float)block_code_sum(make_uint2(b.z, b.w)), e4m3_to_float(s4 >> 24), acc);
    }
  } else
#pragma unroll 4
  for (int64_t k = lane; k < sf_cols; k += 32) {
    const uint2 w2 = __ldg(row_codes + k);
    const int64_t off = (sf_layout == METIS_SF_MMA) ? sf_mma_offset(row, k, tiles) : row * sf_cols + k;
    const float sc = e4m3_to_float(__ldg(scales + off));
    const uint32_t w[2] = {w2.x, w2.y};
    float part;
    if (kHasV) {
      part = 0.0f;
      const float4* v4 = reinterpret_cast<const float4*>(v + k * 16);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 f = __ldg(v4 + j);
        const uint32_t n4 = w[j >> 1] >> (16 * (j & 1));
        part = fmaf((float)twice_e2m1(n4), f.x, part);
        part = fmaf((float)twice_e2m1(n4 >> 4), f.y, part);
        part = fmaf((float)twice_e2m1(n4 >> 8), f.z, part);
        part = fmaf((float)twice_e2m1(n4 >> 12), f.w, part);
      }
    } else {
      part = (float)block_code_sum(w2);
    }
    acc = fmaf(part, sc, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[row] = acc * (0.5f * __ldg(unit_ptr));
}

// The same product for a tall matrix (12288 rows and more: the wide MLP projections at rollout, where
// this pass over the whole weight sits on the critical path of a step).  Two e2m1 codes become two
// halves with one cvt (exact), and the 16 floats of v for a lane's block stay in registers across the
// 4 rows of the warp (v otherwise costs 8 times the bytes of the codes in L1 traffic).  Shorter
// matrices keep gemv_kernel: with four rows per warp they would not fill the SMs.
__device__ __forceinline__ float2 e2m1x2_to_float2(uint32_t byte) {
  uint32_t h2;
  asm("{ .reg .b8 lo, hi; mov.b16 {lo, hi}, %1; cvt.rn.f16x2.e2m1x2 %0, lo; }" : "=r"(h2) : "h"((unsigned short)byte));
  return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}

constexpr int kGemvTallRows = 4;          // rows per warp
constexpr int64_t kGemvTallMinRows = 12288;

__global__ void __launch_bounds__(256)
gemv_tall_kernel(const uint2* __restrict__ codes, const uint8_t* __restrict__ scales,
                 const float* __restrict__ unit_ptr, int32_t sf_layout, int64_t R, int64_t C,
                 const float* __restrict__ v, float* __restrict__ out) {
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * kGemvTallRows;
  if (row0 >= R) return;
  const int64_t sf_cols = C >> 4;                          // blocks per row
  const int64_t tiles = sf_tiles_per_row(C);
  float acc[kGemvTallRows];
#pragma unroll
  for (int j = 0; j < kGemvTallRows; ++j) acc[j] = 0.0f;
  for (int64_t k = lane; k < sf_cols; k += 32) {
    float f[16];
    const float4* v4 = reinterpret_cast<const float4*>(v + k * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 q = __ldg(v4 + i);
      f[4 * i] = q.x; f[4 * i + 1] = q.y; f[4 * i + 2] = q.z; f[4 * i + 3] = q.w;
    }
#pragma unroll
    for (int j = 0; j < kGemvTallRows; ++j) {
      const int64_t row = row0 + j;
      if (row >= R) break;                                 // uniform over the warp
      const uint2 w2 = __ldg(codes + row * sf_cols + k);
      const int64_t off = (sf_layout == METIS_SF_MMA) ? sf_mma_offset(row, k, tiles) : row * sf_cols + k;
      const float sc = e4m3_to_float(__ldg(scales + off));
      const uint32_t w[2] = {w2.x, w2.y};
      float part = 0.0f;
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const float2 c = e2m1x2_to_float2((w[b >> 2] >> (8 * (b & 3))) & 0xFFu);
        part = fmaf(c.x, f[2 * b], part);
        part = fmaf(c.y, f[2 * b + 1], part);
      }
      acc[j] = fmaf(part, sc, acc[j]);
    }
  }
  const float unit = __ldg(unit_ptr);
#pragma unroll
  for (int j = 0; j < kGemvTallRows; ++j) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    if (lane == 0 && row0 + j < R) out[row0 + j] = acc[j] * unit;
  }
}

// The same product with the vector staged in shared memory once per CTA and shared by all its rows: a CTA
// takes 8 * kRowsPerWarp consecutive rows and the whole of C, a warp kRowsPerWarp of them, a lane the blocks
// lane, lane + 32, ...  From global memory a block then costs its 8 bytes of codes and its scale byte; the 64
// bytes of v come from shared memory (stored chunk-major, so the lanes' 16-byte reads are conflict free) and are
// used for every row of the warp.  gemv_kernel reads v through L1 once per row: 8 times the bytes of the
// codes, which is what bounds it on wide matrices (3584 x 18944: 50 us; here 10).  Codes become floats by the
// hardware conversion, two per instruction.
constexpr int64_t kGemvStagedMaxCols = 40960;           // 160 KiB of v
constexpr int64_t kGemvStagedMinCols = 2048;
template <int kRowsPerWarp>
__global__ void __launch_bounds__(256)
gemv_staged_kernel(const uint2* __restrict__ codes, const uint8_t* __restrict__ scales,
                   const float* __restrict__ unit_ptr, int32_t sf_layout, int64_t R, int64_t C,
                   const float* __restrict__ v, float* __restrict__ out) {
  extern __shared__ float4 s_v[];                          // [4][sf_cols]: chunk j of block k at j * sf_cols + k
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sf_cols = (int)(C >> 4);                       // blocks per row
  const int64_t tiles = sf_tiles_per_row(C);
  for (int i = threadIdx.x; i < sf_cols * 4; i += 256)     // coalesced read of v, scattered 16-byte writes
    s_v[(i & 3) * sf_cols + (i >> 2)] = __ldg(reinterpret_cast<const float4*>(v) + i);
  __syncthreads();
  const int64_t row0 = ((int64_t)blockIdx.x * 8 + warp) * kRowsPerWarp;
  if (row0 >= R) return;
  float acc[kRowsPerWarp];
#pragma unroll
  for (int j = 0; j < kRowsPerWarp; ++j) acc[j] = 0.0f;
#pragma unroll(kRowsPerWarp == 1 ? 4 : 2)
  for (int k = lane; k < sf_cols; k += 32) {
    uint2 w2[kRowsPerWarp];
    uint32_t sb[kRowsPerWarp];
#pragma unroll
    for (int j = 0; j < kRowsPerWarp; ++j) {               // every global load of the trip before the arithmetic
      const int64_t row = row0 + j < R ? row0 + j : R - 1;
      w2[j] = __ldg(codes + row * sf_cols + k);
      const int64_t off = (sf_layout == METIS_SF_MMA) ? sf_mma_offset(row, k, tiles) : row * sf_cols + k;
      sb[j] = __ldg(scales + off);
    }
    float f[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 q = s_v[i * sf_cols + k];
      f[4 * i] = q.x; f[4 * i + 1] = q.y; f[4 * i + 2] = q.z; f[4 * i + 3] = q.w;
    }
#pragma unroll
    for (int j = 0; j < kRowsPerWarp; ++j) {
      const uint32_t w[2] = {w2[j].x, w2[j].y};
      float part = 0.0f;
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const float2 c = e2m1x2_to_float2((w[b >> 2] >> (8 * (b & 3))) & 0xFFu);
        part = fmaf(c.x, f[2 * b], part);
        part = fmaf(c.y, f[2 * b + 1], part);
      }
      acc[j] = fmaf(part, e4m3_to_float((uint8_t)sb[j]), acc[j]);
    }
  }
  const float unit = __ldg(unit_ptr);
#pragma unroll
  for (int j = 0; j < kRowsPerWarp; ++j) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    if (lane == 0 && row0 + j < R) out[row0 + j] = acc[j] * unit;
  }
}

// Few, wide rows (the rank-r factor V against a wide activation mean): one row per CTA, its blocks dealt round
// robin to all 256 threads, the eight warps' sums added in warp order.
__global__ void __launch_bounds__(256)
gemv_row_kernel(const uint2* __restrict__ codes, const uint8_t* __restrict__ scales,
                const float* __restrict__ unit_ptr, int32_t sf_layout, int64_t R, int64_t C,
                const float* __restrict__ v, float* __restrict__ out) {
  __shared__ float s_part[8];
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x;
  const int sf_cols = (int)(C >> 4);
  const int64_t tiles = sf_tiles_per_row(C);
  float acc = 0.0f;
#pragma unroll 2
  for (int k = threadIdx.x; k < sf_cols; k += 256) {
    const uint2 w2 = __ldg(codes + row * sf_cols + k);
    const int64_t off = (sf_layout == METIS_SF_MMA) ? sf_mma_offset(row, k, tiles) : row * sf_cols + k;
    const uint32_t sb = __ldg(scales + off);
    const float4* v4 = reinterpret_cast<const float4*>(v) + 4 * (int64_t)k;
    float f[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 q = __ldg(v4 + i);
      f[4 * i] = q.x; f[4 * i + 1] = q.y; f[4 * i + 2] = q.z; f[4 * i + 3] = q.w;
    }
    const uint32_t w[2] = {w2.x, w2.y};
    float part = 0.0f;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const float2 c = e2m1x2_to_float2((w[b >> 2] >> (8 * (b & 3))) & 0xFFu);
      part = fmaf(c.x, f[2 * b], part);
      part = fmaf(c.y, f[2 * b + 1], part);
    }
    acc = fmaf(part, e4m3_to_float((uint8_t)sb), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = 0.0f;
#pragma unroll
    for (int w8 = 0; w8 < 8; ++w8) sum += s_part[w8];
    out[row] = sum * __ldg(unit_ptr);
  }
}

template <int kRowsPerWarp>
static cudaError_t launch_gemv_staged(const uint2* codes, const uint8_t* scales, const float* unit, int32_t sf_layout,
                                      int64_t R, int64_t C, const float* v, float* out, cudaStream_t st) {
  auto kern = gemv_staged_kernel<kRowsPerWarp>;
  const size_t smem = (size_t)C * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  return launch_overlapped(kLaunchShort, kern, dim3((unsigned)ceil_div(R, 8 * kRowsPerWarp)), dim3(256), smem, st,
                           codes, scales, unit, sf_layout, R, C, v, out);
}

// t = bf16( float(bf16(yv * s)) / (unit_a * unit_b) ), 8 elements per thread
template <typename TS>
__global__ void __launch_bounds__(256)
lowrank_scale_kernel(const __nv_bfloat16* __restrict__ yv, int64_t M, int64_t r, int64_t ld,
                     const TS* __restrict__ s, const float* __restrict__ unit_a,
                     const float* __restrict__ unit_b, __nv_bfloat16* __restrict__ t) {
  grid_dependency_wait();
  const int64_t groups_per_row = r >> 3;
  const float div = __fmul_rn(__ldg(unit_a), __ldg(unit_b));
  const bool small = M * groups_per_row < ((int64_t)1 << 31);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M * groups_per_row;
       i += (int64_t)gridDim.x * blockDim.x) {
    // 32-bit index arithmetic where it fits (a 64-bit division is a subroutine of ~100 instructions)
    const int64_t m = small ? (int64_t)((uint32_t)i / (uint32_t)groups_per_row) : i / groups_per_row;
    const int64_t j0 = (i - m * groups_per_row) * 8;
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(yv + m * ld + j0));
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    uint32_t out[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      __nv_bfloat162 s2;
      if constexpr (sizeof(TS) == 2) s2 = *reinterpret_cast<const __nv_bfloat162*>(s + j0 + 2 * k);
      else s2 = __floats2bfloat162_rn(__ldg(s + j0 + 2 * k), __ldg(s + j0 + 2 * k + 1));
      const __nv_bfloat162 ts = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&ww[k]), s2);   // one rounding: the product is exact in fp32
      const uint32_t tw = *reinterpret_cast<const uint32_t*>(&ts);
      const __nv_bfloat162 o = __floats2bfloat162_rn(__fdiv_rn(bf16_lo(tw), div), __fdiv_rn(bf16_hi(tw), div));
      out[k] = *reinterpret_cast<const uint32_t*>(&o);
    }
    *reinterpret_cast<uint4*>(t + m * r + j0) = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

}  // namespace metis

using namespace metis;

extern "C" int32_t metis_lowrank_scale(const void* yv, int64_t M, int64_t r, int64_t ld, const void* s,
                                       int32_t s_dtype, const float* unit_a, const float* unit_b, void* t,
                                       void* stream) {
  if (!yv || !s || !unit_a || !unit_b || !t) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer");
  if (M <= 0 || r <= 0 || r % 8 != 0) return fail(METIS_ERR_BAD_SHAPE, "bad shape [%lld, %lld]: r must be a positive multiple of 8", (long long)M, (long long)r);
  if (s_dtype != METIS_DTYPE_BF16 && s_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown s_dtype %d", s_dtype);
  if (ld < r || ld % 8 != 0 || !aligned16(yv) || !aligned16(t) || (reinterpret_cast<uintptr_t>(s) & 3u))
    return fail(METIS_ERR_BAD_ALIGNMENT, "yv and t must be 16-byte aligned, ld a multiple of 8 and >= r");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int64_t blocks = ceil_div(M * (r >> 3), 256);
  const int64_t cap = (int64_t)device_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(yv);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(t);
  if (s_dtype == METIS_DTYPE_BF16)
    launch_overlapped(kLaunchShort, lowrank_scale_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, st, y, M, r, ld, static_cast<const __nv_bfloat16*>(s), unit_a, unit_b, o);
  else
    launch_overlapped(kLaunchShort, lowrank_scale_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, st, y, M, r, ld, static_cast<const float*>(s), unit_a, unit_b, o);
  METIS_CUDA_OK(cudaGetLastError());
  return METIS_OK;
}

extern "C" int32_t metis_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, const float* unit,
                                          int32_t sf_layout, int64_t R, int64_t C,
                                          const float* add_row_vec, void* out, int32_t out_dtype,
                                          int64_t ld, void* stream) {
  if (!codes || !scales || !unit || !out) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer");
  if (R <= 0 || C <= 0 || C % 16 != 0) return fail(METIS_ERR_BAD_SHAPE, "bad shape [%lld, %lld]", (long long)R, (long long)C);
  if (sf_layout != METIS_SF_ROWMAJOR && sf_layout != METIS_SF_MMA) return fail(METIS_ERR_BAD_ARGUMENT, "unknown sf_layout %d", sf_layout);
  if (out_dtype != METIS_DTYPE_BF16 && out_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown out_dtype %d", out_dtype);
  if (ld < C || ld % 8 != 0 || !aligned16(out) || !aligned16(codes))
    return fail(METIS_ERR_BAD_ALIGNMENT, "out and codes must be 16-byte aligned, ld a multiple of 8 and >= C");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t total = R * (C >> 3);
  int64_t blocks = ceil_div(total, 256);
  const int64_t cap = (int64_t)device_sm_count() * 32;
  if (blocks > cap) blocks = cap;
  const uint32_t* c32 = reinterpret_cast<const uint32_t*>(codes);
  if (out_dtype == METIS_DTYPE_BF16)
    launch_overlapped(kLaunchShort, dequantize_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, st, c32, scales, unit, sf_layout, R, C, add_row_vec, static_cast<__nv_bfloat16*>(out), ld);
  else
    launch_overlapped(kLaunchShort, dequantize_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, st, c32, scales, unit, sf_layout, R, C, add_row_vec, static_cast<float*>(out), ld);
  METIS_CUDA_OK(cudaGetLastError());
  return METIS_OK;
}

extern "C" int32_t metis_nvfp4_gemv(const uint8_t* codes, const uint8_t* scales, const float* unit,
                                    int32_t sf_layout, int64_t R, int64_t C, const float* v, float* out,
                                    void* stream) {
  if (!codes || !scales || !unit || !out) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer");
  if (R <= 0 || C <= 0 || C % 16 != 0) return fail(METIS_ERR_BAD_SHAPE, "bad shape [%lld, %lld]", (long long)R, (long long)C);
  if (sf_layout != METIS_SF_ROWMAJOR && sf_layout != METIS_SF_MMA) return fail(METIS_ERR_BAD_ARGUMENT, "unknown sf_layout %d", sf_layout);
  if (!aligned16(codes)) return fail(METIS_ERR_BAD_ALIGNMENT, "codes must be 16-byte aligned");
  if (v && !aligned16(v)) return fail(METIS_ERR_BAD_ALIGNMENT, "v must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const uint2* c4 = reinterpret_cast<const uint2*>(codes);
  // rows of 2048 elements and more: the kernel that stages v in shared memory; too few rows for it: a CTA per
  // row.  Every CTA stages the whole of v, so with very wide rows fewer CTAs of more rows win although they
  // fill the SMs less evenly (3584 x 18944: 16 rows per CTA 19.6 us, 8 rows 28.2).
  if (v && C >= kGemvStagedMinCols && C <= kGemvStagedMaxCols) {
    const int64_t sms = device_sm_count();
    const bool wide = C >= 8192;
    const int64_t want = wide ? sms : 3 * sms;               // CTAs a launch should at least have
    if (ceil_div(R, 32) >= want) METIS_CUDA_OK(launch_gemv_staged<4>(c4, scales, unit, sf_layout, R, C, v, out, st));
    else if (ceil_div(R, 16) >= want) METIS_CUDA_OK(launch_gemv_staged<2>(c4, scales, unit, sf_layout, R, C, v, out, st));
    else if (R >= (wide ? 4 * sms : want)) METIS_CUDA_OK(launch_gemv_staged<1>(c4, scales, unit, sf_layout, R, C, v, out, st));
    else METIS_CUDA_OK(launch_overlapped(kLaunchShort, gemv_row_kernel, dim3((unsigned)R), dim3(256), 0, st, c4, scales, unit, sf_layout, R, C, v, out));
  } else if (v && R >= kGemvTallMinRows) launch_overlapped(kLaunchShort, gemv_tall_kernel, dim3((unsigned)ceil_div(R, 8 * kGemvTallRows)), dim3(256), 0, st, c4, scales, unit, sf_layout, R, C, v, out);
  else if (v) launch_overlapped(kLaunchShort, gemv_kernel<true>, dim3((unsigned)ceil_div(R, 8)), dim3(256), 0, st, c4, scales, unit, sf_layout, R, C, v, out);
  else   launch_overlapped(kLaunchShort, gemv_kernel<false>, dim3((unsigned)ceil_div(R, 8)), dim3(256), 0, st, c4, scales, unit, sf_layout, R, C, v, out);
  METIS_CUDA_OK(cudaGetLastError());
  return METIS_OK;
}
