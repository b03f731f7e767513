// Fused RMSNorm -> NVFP4 quantizer: every activation row is read from HBM exactly once.
//
// A CTA of 256 threads owns one row at a time (persistent loop over rows).  Each thread keeps
// up to kChunks groups of 8 elements in registers, the CTA reduces the sum of squares, and
// the normalised, gamma-scaled row is quantized straight from registers: two neighbouring
// lanes form a 16-element block exactly as in the stand-alone quantizer.  The E4M3 scale
// bytes are produced by the shared finalisation pass (they need the tensor-wide maximum).
#include "common.cuh"

namespace metis {

constexpr int kNormThreads = 256;

// Rounds two floats to bf16 and back (one packed conversion).
__device__ __forceinline__ void round_bf16x2(float& a, float& b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
  a = bf16_lo(w);
  b = bf16_hi(w);
}

// A CTA is bx x by threads: bx threads (a power of two, or a multiple of 32) share a row, each owning kBlocks
// 16-element blocks tx, tx + bx, ...; by rows are in flight per CTA.  Row sums of squares are
// reduced with shuffles inside a warp and through shared memory across the warps of a row.
template <typename TX, typename TG, int kBlocks, bool kWriteNorm>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_quantize_kernel(const TX* __restrict__ x, int rows, int blocks_per_row, int64_t ld,
                        const TG* __restrict__ gamma, float eps, uint2* __restrict__ codes,
                        float* __restrict__ amax_out, unsigned int* __restrict__ gmax,
                        void* __restrict__ norm_out) {
  grid_dependency_wait();
  // The product normalised(x) * gamma has the promoted dtype: bf16 only if both are bf16.
  constexpr bool kProductBf16 = (sizeof(TX) == 2) && (sizeof(TG) == 2);
  __shared__ float s_red[kNormThreads / 32];
  __shared__ float s_rs[kNormThreads / 32];        // reciprocal RMS of each row in flight (rows span >= 1 warp here)
  const int bx = blockDim.x, by = blockDim.y;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int tid = ty * bx + tx;
  const int lane = tid & 31, warp = tid >> 5;
  const int seg = bx < 32 ? bx : 32;                 // lanes of one row inside a warp
  const int warps_per_row = bx >> 5;                 // 0 when a warp holds several rows
  const float n_cols = (float)(blocks_per_row * 16);
  float running = 0.0f;

  // The row after the current one is already on its way from HBM while the current one is reduced,
  // normalised and quantized: its blocks wait in registers as loaded.
  RawBlock<TX> raw[kBlocks];
  auto fetch = [&](int r_first) {
    const int r = r_first + ty;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (r < rows && bc < blocks_per_row) raw[j].load(x + (int64_t)r * ld + (int64_t)bc * 16);
    }
  };
  fetch(blockIdx.x * by);

  for (int r0 = blockIdx.x * by; r0 < rows; r0 += gridDim.x * by) {
    const int r = r0 + ty;
    const bool row_live = r < rows;
    float v[kBlocks][16];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (row_live && bc < blocks_per_row) {
        raw[j].unpack(v[j]);
#pragma unroll
        for (int i = 0; i < 16; ++i) ss = __fmaf_rn(v[j][i], v[j][i], ss);
      }
    }
    fetch(r0 + gridDim.x * by);
    for (int o = seg >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    // x * rsqrt(mean(x^2) + eps) with the IEEE operations the CPU reference uses: correctly
    // rounded division, square root and reciprocal (llama.py:23-24).  The sequence is some 50
    // instructions, so one thread per row runs it and the others pick the result up.
    float rs;
    if (warps_per_row > 1) {                           // uniform over the CTA
      if (lane == 0) s_red[warp] = ss;
      __syncthreads();
      if (tx == 0) {
        float tot = 0.0f;
        for (int w = 0; w < warps_per_row; ++w) tot += s_red[ty * warps_per_row + w];
        s_rs[ty] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, n_cols), eps)));
      }
      __syncthreads();                                 // also: s_red may be rewritten by the next row
      rs = s_rs[ty];
    } else {
      rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, n_cols), eps)));   // every lane of the row holds the sum
    }

#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (!(row_live && bc < blocks_per_row)) continue;
      float y[16];
      float a;
      if constexpr (kProductBf16) {
        // both roundings of the reference in packed bf16: n = bf16(x * rs) (llama.py:28), then
        // n * gamma as one bf16x2 multiply: the product of two bf16 is exact in fp32, so rounding
        // it once to bf16 is what the fp32 multiply followed by the conversion gives (llama.py:31)
        RawBlock<__nv_bfloat16> graw;
        graw.load(reinterpret_cast<const __nv_bfloat16*>(gamma) + (int64_t)bc * 16);
        const uint32_t gw[8] = {graw.a.x, graw.a.y, graw.a.z, graw.a.w, graw.b.x, graw.b.y, graw.b.z, graw.b.w};
        __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __nv_bfloat162 n2 = __floats2bfloat162_rn(__fmul_rn(v[j][2 * i], rs), __fmul_rn(v[j][2 * i + 1], rs));
          const __nv_bfloat162 p2 = __hmul2(n2, *reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
          amax2 = __hmax2(amax2, __habs2(p2));
          const uint32_t w = *reinterpret_cast<const uint32_t*>(&p2);
          y[2 * i] = bf16_lo(w);
          y[2 * i + 1] = bf16_hi(w);
        }
        const uint32_t aw = *reinterpret_cast<const uint32_t*>(&amax2);
        a = fmaxf(bf16_lo(aw), bf16_hi(aw));
      } else {
        float g[16];
        Load16<TG>::load(gamma + (int64_t)bc * 16, g);
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float n0 = __fmul_rn(v[j][i], rs), n1 = __fmul_rn(v[j][i + 1], rs);
          if (sizeof(TX) == 2) round_bf16x2(n0, n1);                      // .type_as(x), llama.py:28
          y[i] = __fmul_rn(n0, g[i]);                                     // * weight, llama.py:31
          y[i + 1] = __fmul_rn(n1, g[i + 1]);
        }
        a = abs_max16(y);
      }
      uint32_t packed[2];
      quantize_rn<2>(y, block_scale_from_amax(a), packed);
      const int64_t b = (int64_t)r * blocks_per_row + bc;
      codes[b] = make_uint2(packed[0], packed[1]);
      amax_out[b] = a;
      running = fmaxf(running, a);
      if (kWriteNorm) {
        if (kProductBf16) {
          __nv_bfloat162 o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);   // exact: already bf16 values
          uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(norm_out) + b * 16);
          dst[0] = reinterpret_cast<uint4*>(o)[0];
          dst[1] = reinterpret_cast<uint4*>(o)[1];
        } else {
          float4* dst = reinterpret_cast<float4*>(static_cast<float*>(norm_out) + b * 16);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) running = fmaxf(running, __shfl_xor_sync(0xffffffffu, running, o));
  if (lane == 0 && running > 0.0f) atomicMax(gmax, __float_as_uint(running));
}

// ---- decode-sized inputs: one launch ---------------------------------------------------------------
// The same row arithmetic for a handful of rows, run as ONE thread-block cluster of up to 8 CTAs: a CTA
// of bx x by = 512 threads takes up to kNormSmallPasses groups of `by` rows, every block maximum stays in a
// register, the tensor-wide maximum crosses the cluster through shared memory, and the threads write
// their own E4M3 bytes: no zero-fill node, no scale pass, no scratch in global memory.

// normalised(x) * gamma for one 16-element block, with the reference's roundings (llama.py:28, 31);
// returns the block maximum.
template <typename TX, typename TG>
__device__ __forceinline__ float norm_block(const float (&v)[16], float rs, const TG* __restrict__ gamma16, float (&y)[16]) {
  constexpr bool kProductBf16 = (sizeof(TX) == 2) && (sizeof(TG) == 2);
  if constexpr (kProductBf16) {
    RawBlock<__nv_bfloat16> graw;
    graw.load(reinterpret_cast<const __nv_bfloat16*>(gamma16));
    const uint32_t gw[8] = {graw.a.x, graw.a.y, graw.a.z, graw.a.w, graw.b.x, graw.b.y, graw.b.z, graw.b.w};
    __nv_bfloat162 amax2 = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_bfloat162 n2 = __floats2bfloat162_rn(__fmul_rn(v[2 * i], rs), __fmul_rn(v[2 * i + 1], rs));
      const __nv_bfloat162 p2 = __hmul2(n2, *reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
      amax2 = __hmax2(amax2, __habs2(p2));
      const uint32_t w = *reinterpret_cast<const uint32_t*>(&p2);
      y[2 * i] = bf16_lo(w);
      y[2 * i + 1] = bf16_hi(w);
    }
    const uint32_t aw = *reinterpret_cast<const uint32_t*>(&amax2);
    return fmaxf(bf16_lo(aw), bf16_hi(aw));
  } else {
    float g[16];
    Load16<TG>::load(gamma16, g);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      float n0 = __fmul_rn(v[i], rs), n1 = __fmul_rn(v[i + 1], rs);
      if (sizeof(TX) == 2) round_bf16x2(n0, n1);
      y[i] = __fmul_rn(n0, g[i]);
      y[i + 1] = __fmul_rn(n1, g[i + 1]);
    }
    return abs_max16(y);
  }
}

constexpr int kNormSmallPasses = 2;
constexpr int kNormSmallThreads = 512;             // twice the rows per CTA of the streaming kernel: 16 rows of 4096 in one pass
constexpr int kNormSmallBlocks = 2;                // blocks per thread and row: rows of up to 8192 elements

template <typename TX, typename TG, int kBlocks, bool kWriteNorm>
__global__ void __launch_bounds__(kNormSmallThreads)
rmsnorm_quantize_small_kernel(const TX* __restrict__ x, int rows, int blocks_per_row, int64_t ld,
                              const TG* __restrict__ gamma, float eps, uint2* __restrict__ codes, int32_t sf_layout,
                              int tiles, int padded_words, uint8_t* __restrict__ scales, float* __restrict__ unit_out,
                              void* __restrict__ norm_out) {
  constexpr bool kProductBf16 = (sizeof(TX) == 2) && (sizeof(TG) == 2);
  __shared__ ClusterMaxSmem s_max;
  __shared__ float s_red[kNormSmallPasses][kNormSmallThreads / 32];
  __shared__ float s_rs[kNormSmallPasses][kNormSmallThreads / 32];
  grid_dependency_wait();
  const int bx = blockDim.x, by = blockDim.y;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int tid = ty * bx + tx;
  const int lane = tid & 31, warp = tid >> 5;
  const int seg = bx < 32 ? bx : 32;                 // lanes of one row inside a warp
  const int warps_per_row = bx >> 5;                 // 0 when a warp holds several rows
  const float n_cols = (float)(blocks_per_row * 16);
  const int ncta = (int)cluster_cta_count(), rank = (int)cluster_cta_rank();
  if (sf_layout == METIS_SF_MMA)
    zero_scale_padding(scales, rows, blocks_per_row, tiles, padded_words, rank * bx * by + tid, ncta * bx * by);

  // every row of this thread is on its way before the first one is worked on
  RawBlock<TX> raw[kNormSmallPasses][kBlocks];
#pragma unroll
  for (int p = 0; p < kNormSmallPasses; ++p) {
    const int r = (p * ncta + rank) * by + ty;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (r < rows && bc < blocks_per_row) raw[p][j].load(x + (int64_t)r * ld + (int64_t)bc * 16);
    }
  }
  // sums of squares of all passes, then one round through shared memory for all of them
  float ss[kNormSmallPasses];
#pragma unroll
  for (int p = 0; p < kNormSmallPasses; ++p) {
    const int r = (p * ncta + rank) * by + ty;
    ss[p] = 0.0f;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (r < rows && bc < blocks_per_row) {
        float v[16];
        raw[p][j].unpack(v);
#pragma unroll
        for (int i = 0; i < 16; ++i) ss[p] = __fmaf_rn(v[i], v[i], ss[p]);
      }
    }
    for (int o = seg >> 1; o > 0; o >>= 1) ss[p] += __shfl_xor_sync(0xffffffffu, ss[p], o);
    if (warps_per_row > 1 && lane == 0) s_red[p][warp] = ss[p];
  }
  float rs[kNormSmallPasses];
  if (warps_per_row > 1) {                             // uniform over the CTA
    __syncthreads();
    if (tx == 0) {
#pragma unroll
      for (int p = 0; p < kNormSmallPasses; ++p) {
        if ((p * ncta + rank) * by + ty >= rows) continue;
        float tot = 0.0f;
        for (int w = 0; w < warps_per_row; ++w) tot += s_red[p][ty * warps_per_row + w];
        s_rs[p][ty] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, n_cols), eps)));   // llama.py:23-24
      }
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < kNormSmallPasses; ++p) rs[p] = s_rs[p][ty];
  } else {
#pragma unroll
    for (int p = 0; p < kNormSmallPasses; ++p) rs[p] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss[p], n_cols), eps)));
  }

  float amax[kNormSmallPasses][kBlocks];
  float running = 0.0f;
#pragma unroll
  for (int p = 0; p < kNormSmallPasses; ++p) {
    const int r = (p * ncta + rank) * by + ty;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      amax[p][j] = 0.0f;
      if (!(r < rows && bc < blocks_per_row)) continue;
      float v[16], y[16];
      raw[p][j].unpack(v);
      const float a = norm_block<TX, TG>(v, rs[p], gamma + (int64_t)bc * 16, y);
      uint32_t packed[2];
      quantize_rn<2>(y, block_scale_from_amax(a), packed);
      const int64_t b = (int64_t)r * blocks_per_row + bc;
      codes[b] = make_uint2(packed[0], packed[1]);
      amax[p][j] = a;
      running = fmaxf(running, a);
      if (kWriteNorm) {
        if (kProductBf16) {
          __nv_bfloat162 o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);   // exact: already bf16 values
          uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(norm_out) + b * 16);
          dst[0] = reinterpret_cast<uint4*>(o)[0];
          dst[1] = reinterpret_cast<uint4*>(o)[1];
        } else {
          float4* dst = reinterpret_cast<float4*>(static_cast<float*>(norm_out) + b * 16);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
        }
      }
    }
  }

  const float unit = __fdiv_rn(block_scale_from_amax(cluster_fmax(running, s_max)), 448.0f);   // quant.py:21-22
  if (rank == 0 && tid == 0) *unit_out = unit;
#pragma unroll
  for (int p = 0; p < kNormSmallPasses; ++p) {
    const int r = (p * ncta + rank) * by + ty;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (!(r < rows && bc < blocks_per_row)) continue;
      const float ratio = __fdiv_rn(block_scale_from_amax(amax[p][j]), unit);                 // quant.py:23
      const int64_t off = (sf_layout == METIS_SF_MMA) ? sf_mma_offset(r, bc, tiles) : (int64_t)r * blocks_per_row + bc;
      scales[off] = float_to_e4m3(ratio);
    }
  }
  cluster_leave();
}

// Launches the one-cluster kernel if [rows, cols] fits it; *taken says whether it did.
template <typename TX, typename TG>
static int32_t try_small(const TX* x, int64_t rows, int64_t cols, int64_t ld, const TG* gamma, float eps, uint8_t* codes,
                         int32_t sf_layout, uint8_t* scales, float* unit, void* norm_out, cudaStream_t st, bool* taken) {
  *taken = false;
  const int bpr = (int)(cols >> 4);
  int bx = 1;
  if (bpr >= 32) {
    bx = ((bpr + 31) / 32) * 32;
    if (bx > kNormThreads) bx = kNormThreads;
  } else {
    while (bx < bpr) bx <<= 1;
  }
  const int by = kNormSmallThreads / bx;
  const int per_thread = (bpr + bx - 1) / bx;
  const int64_t tiles = sf_tiles_per_row(cols);
  const int64_t padded_words = sf_layout == METIS_SF_MMA ? ceil_div(rows, 128) * 128 * tiles : 0;
  if (per_thread > kNormSmallBlocks || rows > (int64_t)kSmallCtas * kNormSmallPasses * by ||
      padded_words > kSmallMaxPaddedWords || !aligned16(scales))
    return METIS_OK;
  int64_t ctas = ceil_div(rows, by);
  const int64_t for_padding = ceil_div(padded_words / 4, kNormSmallThreads);     // CTAs without rows still clear padding
  if (ctas < for_padding) ctas = for_padding;
  if (ctas > kSmallCtas) ctas = kSmallCtas;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3((unsigned)bx, (unsigned)by);
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ctas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_overlap_enabled(kLaunchShort) ? 2 : 1;
  uint2* c2 = reinterpret_cast<uint2*>(codes);
#define METIS_NORM_SMALL(KB, WN)                                                                                       \
  METIS_CUDA_OK(cudaLaunchKernelEx(&cfg, rmsnorm_quantize_small_kernel<TX, TG, KB, WN>, x, (int)rows, bpr, ld, gamma, eps, c2, \
                                   sf_layout, (int)tiles, (int)padded_words, scales, unit, norm_out))
  if (per_thread <= 1) { if (norm_out) METIS_NORM_SMALL(1, true); else METIS_NORM_SMALL(1, false); }
  else                 { if (norm_out) METIS_NORM_SMALL(2, true); else METIS_NORM_SMALL(2, false); }
#undef METIS_NORM_SMALL
  *taken = true;
  return METIS_OK;
}

template <typename TX, typename TG, int kBlocks>
static void launch_norm(const TX* x, int64_t rows, int bpr, int bx, int64_t ld, const TG* gamma, float eps,
                        uint32_t* codes, const WorkspaceView& ws, void* norm_out, int sms, cudaStream_t st) {
  const int by = kNormThreads / bx;
  // persistent CTAs: exactly as many as are resident at once, so that all of them finish together
  int per_sm = 0;
  if (norm_out) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rmsnorm_quantize_kernel<TX, TG, kBlocks, true>, bx * by, 0);
  else          cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rmsnorm_quantize_kernel<TX, TG, kBlocks, false>, bx * by, 0);
  if (per_sm < 1) per_sm = 1;
  int64_t blocks = (int64_t)sms * per_sm;
  const int64_t need = ceil_div(rows, by);
  if (blocks > need) blocks = need;
  const dim3 b((unsigned)bx, (unsigned)by);
  uint2* c2 = reinterpret_cast<uint2*>(codes);
  if (norm_out)
    launch_overlapped(kLaunchStream, rmsnorm_quantize_kernel<TX, TG, kBlocks, true>, dim3((unsigned)blocks), b, 0, st,
                      x, (int)rows, bpr, ld, gamma, eps, c2, ws.amax, ws.gmax, norm_out);
  else
    launch_overlapped(kLaunchStream, rmsnorm_quantize_kernel<TX, TG, kBlocks, false>, dim3((unsigned)blocks), b, 0, st,
                      x, (int)rows, bpr, ld, gamma, eps, c2, ws.amax, ws.gmax, norm_out);
}

template <typename TX, typename TG>
static int32_t dispatch_chunks(const TX* x, int64_t rows, int64_t cols, int64_t ld, const TG* gamma,
                               float eps, uint32_t* codes, const WorkspaceView& ws, void* norm_out,
                               int sms, cudaStream_t st) {
  const int bpr = (int)(cols >> 4);
  // threads along the row: whole warps, as many as the row has 32-block groups (hidden 1536 runs
  // with 96 threads per row and two rows per CTA instead of 128 with a quarter of them idle);
  // rows shorter than a warp take the next power of two
  int bx = 1;
  if (bpr >= 32) {
    bx = ((bpr + 31) / 32) * 32;
    if (bx > kNormThreads) bx = kNormThreads;
  } else {
    while (bx < bpr) bx <<= 1;
  }
  const int per_thread = (bpr + bx - 1) / bx;
  if (per_thread <= 1) launch_norm<TX, TG, 1>(x, rows, bpr, bx, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 2) launch_norm<TX, TG, 2>(x, rows, bpr, bx, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 3) launch_norm<TX, TG, 3>(x, rows, bpr, bx, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 5) launch_norm<TX, TG, 5>(x, rows, bpr, bx, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 8) launch_norm<TX, TG, 8>(x, rows, bpr, bx, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else return fail(METIS_ERR_TOO_LARGE, "rmsnorm rows longer than %d elements are not supported", 8 * kNormThreads * 16);
  return METIS_OK;
}

// ---- RMSNorm with the column sums of its output (the mean-centred path) ------------------------------------
// The mean-centred quantizer (bitlinear.py:326-332) needs the column mean of the NORMALISED activation before
// it can quantize anything, so normalisation and quantization cannot share one pass.  This kernel is the first
// of the two: it reads x once, writes y = norm(x) * gamma (the reference's roundings, llama.py:23-31), the
// reciprocal RMS of every row (what a backward pass needs) and, per resident row slot, the sums of the y it
// produced for every column; col_mean_finish_kernel adds those in a fixed order.  The quantizer then reads y
// once for both orientations.  Same thread layout as rmsnorm_quantize_kernel: a thread keeps its column blocks
// for all the rows it sees, so the sums stay in registers.
template <typename TX, typename TG, int kBlocks>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_colsum_kernel(const TX* __restrict__ x, int rows, int blocks_per_row, int64_t ld, const TG* __restrict__ gamma,
                      float eps, void* __restrict__ norm_out, float* __restrict__ rstd_out, float* __restrict__ partial) {
  grid_dependency_wait();
  constexpr bool kProductBf16 = (sizeof(TX) == 2) && (sizeof(TG) == 2);
  __shared__ float s_red[kNormThreads / 32];
  __shared__ float s_rs[kNormThreads / 32];
  const int bx = blockDim.x, by = blockDim.y;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int tid = ty * bx + tx;
  const int lane = tid & 31, warp = tid >> 5;
  const int seg = bx < 32 ? bx : 32;
  const int warps_per_row = bx >> 5;
  const float n_cols = (float)(blocks_per_row * 16);
  float csum[kBlocks][16];
#pragma unroll
  for (int j = 0; j < kBlocks; ++j)
#pragma unroll
    for (int i = 0; i < 16; ++i) csum[j][i] = 0.0f;

  RawBlock<TX> raw[kBlocks];
  auto fetch = [&](int r_first) {
    const int r = r_first + ty;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (r < rows && bc < blocks_per_row) raw[j].load(x + (int64_t)r * ld + (int64_t)bc * 16);
    }
  };
  fetch(blockIdx.x * by);
  for (int r0 = blockIdx.x * by; r0 < rows; r0 += gridDim.x * by) {
    const int r = r0 + ty;
    const bool row_live = r < rows;
    float v[kBlocks][16];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (row_live && bc < blocks_per_row) {
        raw[j].unpack(v[j]);
#pragma unroll
        for (int i = 0; i < 16; ++i) ss = __fmaf_rn(v[j][i], v[j][i], ss);
      }
    }
    fetch(r0 + gridDim.x * by);
    for (int o = seg >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    float rs;
    if (warps_per_row > 1) {
      if (lane == 0) s_red[warp] = ss;
      __syncthreads();
      if (tx == 0) {
        float tot = 0.0f;
        for (int w = 0; w < warps_per_row; ++w) tot += s_red[ty * warps_per_row + w];
        s_rs[ty] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, n_cols), eps)));
      }
      __syncthreads();
      rs = s_rs[ty];
    } else {
      rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, n_cols), eps)));
    }
    if (row_live && tx == 0 && rstd_out) rstd_out[r] = rs;
#pragma unroll
    for (int j = 0; j < kBlocks; ++j) {
      const int bc = tx + j * bx;
      if (!(row_live && bc < blocks_per_row)) continue;
      float y[16];
      norm_block<TX, TG>(v[j], rs, gamma + (int64_t)bc * 16, y);
#pragma unroll
      for (int i = 0; i < 16; ++i) csum[j][i] += y[i];
      const int64_t b = (int64_t)r * blocks_per_row + bc;
      if (kProductBf16) {
        __nv_bfloat162 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);   // exact: already bf16 values
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(norm_out) + b * 16);
        dst[0] = reinterpret_cast<uint4*>(o)[0];
        dst[1] = reinterpret_cast<uint4*>(o)[1];
      } else {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(norm_out) + b * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_float4(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
      }
    }
  }
  // this row slot's sums: partial[slot][cols], slot = blockIdx.x * by + ty
  float* dst = partial + ((int64_t)blockIdx.x * by + ty) * (int64_t)blocks_per_row * 16;
#pragma unroll
  for (int j = 0; j < kBlocks; ++j) {
    const int bc = tx + j * bx;
    if (bc >= blocks_per_row) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reinterpret_cast<float4*>(dst + (int64_t)bc * 16)[i] = make_float4(csum[j][4 * i], csum[j][4 * i + 1], csum[j][4 * i + 2], csum[j][4 * i + 3]);
  }
}

__global__ void rmsnorm_mean_finish_kernel(const float* __restrict__ partial, int64_t slots, int64_t rows, int64_t cols,
                                           float* __restrict__ mean) {
  grid_dependency_wait();
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float sum = 0.0f;
  for (int64_t s = 0; s < slots; ++s) sum += partial[s * cols + c];        // fixed order
  mean[c] = __fdiv_rn(sum, (float)rows);
}

struct NormShape { int bx, by, per_thread; };
static NormShape norm_shape(int bpr) {
  int bx = 1;
  if (bpr >= 32) {
    bx = ((bpr + 31) / 32) * 32;
    if (bx > kNormThreads) bx = kNormThreads;
  } else {
    while (bx < bpr) bx <<= 1;
  }
  return {bx, kNormThreads / bx, (bpr + bx - 1) / bx};
}
// row slots (CTAs x rows in flight per CTA) the kernel above runs with: two CTAs per SM
static int64_t colsum_ctas(int64_t rows, int by) {
  int64_t blocks = (int64_t)device_sm_count() * 2;
  const int64_t need = ceil_div(rows, by);
  return blocks > need ? need : blocks;
}

template <typename TX, typename TG>
static int32_t launch_colsum(const TX* x, int64_t rows, int64_t cols, int64_t ld, const TG* gamma, float eps, void* norm_out,
                             float* rstd, float* partial, cudaStream_t st) {
  const int bpr = (int)(cols >> 4);
  const NormShape sh = norm_shape(bpr);
  const dim3 g((unsigned)colsum_ctas(rows, sh.by)), b((unsigned)sh.bx, (unsigned)sh.by);
#define METIS_COLSUM(KB) METIS_CUDA_OK(launch_overlapped(kLaunchStream, rmsnorm_colsum_kernel<TX, TG, KB>, g, b, 0, st, x, (int)rows, bpr, ld, gamma, eps, norm_out, rstd, partial))
  if (sh.per_thread <= 1) METIS_COLSUM(1);
  else if (sh.per_thread <= 2) METIS_COLSUM(2);
  else if (sh.per_thread <= 3) METIS_COLSUM(3);
  else if (sh.per_thread <= 5) METIS_COLSUM(5);
  else return fail(METIS_ERR_TOO_LARGE, "rmsnorm rows longer than %d elements are not supported here", 5 * kNormThreads * 16);
#undef METIS_COLSUM
  return METIS_OK;
}

}  // namespace metis

using namespace metis;

extern "C" int32_t metis_rmsnorm_nvfp4_quantize(const void* x, int32_t x_dtype, int64_t rows, int64_t cols,
                                                int64_t ld, const void* gamma, int32_t gamma_dtype,
                                                float eps, int32_t sf_layout, uint8_t* codes,
                                                uint8_t* scales, float* unit, void* norm_out,
                                                void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x || !gamma) return fail(METIS_ERR_BAD_ARGUMENT, "x or gamma is null");
  if ((x_dtype != METIS_DTYPE_BF16 && x_dtype != METIS_DTYPE_F32) ||
      (gamma_dtype != METIS_DTYPE_BF16 && gamma_dtype != METIS_DTYPE_F32))
    return fail(METIS_ERR_BAD_ARGUMENT, "unknown dtype");
  if (rows <= 0 || cols <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty tensor [%lld, %lld]", (long long)rows, (long long)cols);
  if (ld < cols) return fail(METIS_ERR_BAD_ARGUMENT, "ld %lld < cols %lld", (long long)ld, (long long)cols);
  if (int32_t rc = check_quant_outputs(rows, cols, sf_layout, codes, scales, unit, workspace, workspace_bytes)) return rc;
  if (ld % 8 != 0 || !aligned16(x) || !aligned16(gamma) || (norm_out && !aligned16(norm_out)))
    return fail(METIS_ERR_BAD_ALIGNMENT, "x, gamma and norm_out must be 16-byte aligned and ld a multiple of 8");

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int32_t rc;
  bool taken = false;
  if (x_dtype == METIS_DTYPE_BF16 && gamma_dtype == METIS_DTYPE_BF16)
    rc = try_small(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, static_cast<const __nv_bfloat16*>(gamma), eps, codes, sf_layout, scales, unit, norm_out, st, &taken);
  else if (x_dtype == METIS_DTYPE_BF16)
    rc = try_small(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, static_cast<const float*>(gamma), eps, codes, sf_layout, scales, unit, norm_out, st, &taken);
  else if (gamma_dtype == METIS_DTYPE_BF16)
    rc = try_small(static_cast<const float*>(x), rows, cols, ld, static_cast<const __nv_bfloat16*>(gamma), eps, codes, sf_layout, scales, unit, norm_out, st, &taken);
  else
    rc = try_small(static_cast<const float*>(x), rows, cols, ld, static_cast<const float*>(gamma), eps, codes, sf_layout, scales, unit, norm_out, st, &taken);
  if (rc || taken) return rc;
  const WorkspaceView ws = view_workspace(workspace);
  METIS_CUDA_OK(cudaMemsetAsync(ws.gmax, 0, 2 * sizeof(unsigned int), st));   // running maximum and error word
  const int sms = device_sm_count();
  uint32_t* c32 = reinterpret_cast<uint32_t*>(codes);
  if (x_dtype == METIS_DTYPE_BF16 && gamma_dtype == METIS_DTYPE_BF16)
    rc = dispatch_chunks(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, static_cast<const __nv_bfloat16*>(gamma), eps, c32, ws, norm_out, sms, st);
  else if (x_dtype == METIS_DTYPE_BF16)
    rc = dispatch_chunks(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, static_cast<const float*>(gamma), eps, c32, ws, norm_out, sms, st);
  else if (gamma_dtype == METIS_DTYPE_BF16)
    rc = dispatch_chunks(static_cast<const float*>(x), rows, cols, ld, static_cast<const __nv_bfloat16*>(gamma), eps, c32, ws, norm_out, sms, st);
  else
    rc = dispatch_chunks(static_cast<const float*>(x), rows, cols, ld, static_cast<const float*>(gamma), eps, c32, ws, norm_out, sms, st);
  if (rc) return rc;
  METIS_CUDA_OK(cudaGetLastError());
  return launch_finalize(ws, rows, cols, sf_layout, scales, unit, st);
}


extern "C" int64_t metis_rmsnorm_mean_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0 || cols % 16 != 0) return 0;
  const NormShape sh = norm_shape((int)(cols >> 4));
  return colsum_ctas(rows, sh.by) * sh.by * cols * (int64_t)sizeof(float);
}

extern "C" int32_t metis_rmsnorm_mean(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                      const void* gamma, int32_t gamma_dtype, float eps, void* norm_out, float* rstd,
                                      float* mean, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x || !gamma || !norm_out || !mean || !workspace) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer");
  if ((x_dtype != METIS_DTYPE_BF16 && x_dtype != METIS_DTYPE_F32) || (gamma_dtype != METIS_DTYPE_BF16 && gamma_dtype != METIS_DTYPE_F32))
    return fail(METIS_ERR_BAD_ARGUMENT, "unknown dtype");
  if (rows <= 0 || cols <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty tensor [%lld, %lld]", (long long)rows, (long long)cols);
  if (cols % 16 != 0) return fail(METIS_ERR_BAD_SHAPE, "NVFP4 block shape (1, 16) does not divide tensor shape (%lld, %lld)", (long long)rows, (long long)cols);
  if (ld < cols || ld % 8 != 0 || !aligned16(x) || !aligned16(gamma) || !aligned16(norm_out) || !aligned16(workspace))
    return fail(METIS_ERR_BAD_ALIGNMENT, "x, gamma, norm_out and workspace must be 16-byte aligned and ld a multiple of 8");
  if (workspace_bytes < metis_rmsnorm_mean_workspace_bytes(rows, cols)) return fail(METIS_ERR_WORKSPACE, "workspace too small");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
  int32_t rc;
  if (x_dtype == METIS_DTYPE_BF16 && gamma_dtype == METIS_DTYPE_BF16)
    rc = launch_colsum(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, static_cast<const __nv_bfloat16*>(gamma), eps, norm_out, rstd, partial, st);
  else if (x_dtype == METIS_DTYPE_BF16)
    rc = launch_colsum(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, static_cast<const float*>(gamma), eps, norm_out, rstd, partial, st);
  else if (gamma_dtype == METIS_DTYPE_BF16)
    rc = launch_colsum(static_cast<const float*>(x), rows, cols, ld, static_cast<const __nv_bfloat16*>(gamma), eps, norm_out, rstd, partial, st);
  else
    rc = launch_colsum(static_cast<const float*>(x), rows, cols, ld, static_cast<const float*>(gamma), eps, norm_out, rstd, partial, st);
  if (rc) return rc;
  const NormShape sh = norm_shape((int)(cols >> 4));
  const int64_t slots = colsum_ctas(rows, sh.by) * sh.by;
  METIS_CUDA_OK(launch_overlapped(kLaunchShort, rmsnorm_mean_finish_kernel, dim3((unsigned)ceil_div(cols, 256)), dim3(256), 0, st,
                                  (const float*)partial, slots, rows, cols, mean));
  return METIS_OK;
}
