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

template <typename TX, typename TG, int kChunks, bool kWriteNorm>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_quantize_kernel(const TX* __restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                        const TG* __restrict__ gamma, float eps, uint32_t* __restrict__ codes,
                        float* __restrict__ amax_out, unsigned int* __restrict__ gmax,
                        void* __restrict__ norm_out) {
  // The product normalised(x) * gamma has the promoted dtype: bf16 only if both are bf16.
  constexpr bool kProductBf16 = (sizeof(TX) == 2) && (sizeof(TG) == 2);
  __shared__ float s_red[kNormThreads / 32];
  const int chunks_per_row = (int)(cols >> 3);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float inv_cols_den = (float)cols;

  // gamma is the same for every row: keep it in registers
  float g[kChunks][8];
#pragma unroll
  for (int j = 0; j < kChunks; ++j) {
    const int ch = threadIdx.x + j * kNormThreads;
    if (ch < chunks_per_row) Load8<TG>::load(gamma + (int64_t)ch * 8, g[j]);
  }

  float running = 0.0f;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float v[kChunks][8];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const int ch = threadIdx.x + j * kNormThreads;
      if (ch < chunks_per_row) {
        Load8<TX>::load(x + r * ld + (int64_t)ch * 8, v[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = __fmaf_rn(v[j][i], v[j][i], ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) tot += s_red[w];
    __syncthreads();   // s_red is rewritten by the next row
    // x * rsqrt(mean(x^2) + eps) with the IEEE operations the CPU reference uses:
    // correctly rounded division, square root and reciprocal (llama.py:23-24).
    const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, inv_cols_den), eps)));

#pragma unroll
    for (int j = 0; j < kChunks; ++j) {
      const int ch = threadIdx.x + j * kNormThreads;
      const bool live = ch < chunks_per_row;   // uniform over a lane pair (chunks_per_row is even)
      float y[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float n = live ? __fmul_rn(v[j][i], rs) : 0.0f;
        if (sizeof(TX) == 2) n = __bfloat162float(__float2bfloat16_rn(n));   // .type_as(x), llama.py:28
        float p = __fmul_rn(n, live ? g[j][i] : 0.0f);                       // * weight, llama.py:31
        if (kProductBf16) p = __bfloat162float(__float2bfloat16_rn(p));
        y[i] = p;
      }
      float a = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) a = fmaxf(a, fabsf(y[i]));
      a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
      const uint32_t packed = quantize8_rn(y, block_scale_from_amax(a));
      if (live) {
        const int64_t c = r * chunks_per_row + ch;
        codes[c] = packed;
        if ((ch & 1) == 0) amax_out[c >> 1] = a;
        if (kWriteNorm) {
          if (kProductBf16) {
            __nv_bfloat162 o[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(norm_out) + c * 8) = *reinterpret_cast<uint4*>(o);
          } else {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(norm_out) + c * 8);
            dst[0] = make_float4(y[0], y[1], y[2], y[3]);
            dst[1] = make_float4(y[4], y[5], y[6], y[7]);
          }
        }
        running = fmaxf(running, a);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) running = fmaxf(running, __shfl_xor_sync(0xffffffffu, running, o));
  if (lane == 0 && running > 0.0f) atomicMax(gmax, __float_as_uint(running));
}

template <typename TX, typename TG, int kChunks>
static void launch_norm(const TX* x, int64_t rows, int64_t cols, int64_t ld, const TG* gamma, float eps,
                        uint32_t* codes, const WorkspaceView& ws, void* norm_out, int sms, cudaStream_t st) {
  int64_t blocks = (int64_t)sms * (kChunks <= 2 ? 8 : (kChunks <= 4 ? 4 : 2));
  if (blocks > rows) blocks = rows;
  if (norm_out)
    rmsnorm_quantize_kernel<TX, TG, kChunks, true><<<(unsigned)blocks, kNormThreads, 0, st>>>(
        x, rows, cols, ld, gamma, eps, codes, ws.amax, ws.gmax, norm_out);
  else
    rmsnorm_quantize_kernel<TX, TG, kChunks, false><<<(unsigned)blocks, kNormThreads, 0, st>>>(
        x, rows, cols, ld, gamma, eps, codes, ws.amax, ws.gmax, norm_out);
}

template <typename TX, typename TG>
static int32_t dispatch_chunks(const TX* x, int64_t rows, int64_t cols, int64_t ld, const TG* gamma,
                               float eps, uint32_t* codes, const WorkspaceView& ws, void* norm_out,
                               int sms, cudaStream_t st) {
  const int64_t per_thread = ceil_div(cols >> 3, kNormThreads);
  if (per_thread <= 1) launch_norm<TX, TG, 1>(x, rows, cols, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 2) launch_norm<TX, TG, 2>(x, rows, cols, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 4) launch_norm<TX, TG, 4>(x, rows, cols, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 8) launch_norm<TX, TG, 8>(x, rows, cols, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else if (per_thread <= 12) launch_norm<TX, TG, 12>(x, rows, cols, ld, gamma, eps, codes, ws, norm_out, sms, st);
  else return fail(METIS_ERR_TOO_LARGE, "rmsnorm rows longer than %d elements are not supported", 12 * kNormThreads * 8);
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
  const WorkspaceView ws = view_workspace(workspace);
  METIS_CUDA_OK(cudaMemsetAsync(ws.gmax, 0, sizeof(unsigned int), st));
  const int sms = device_sm_count();
  uint32_t* c32 = reinterpret_cast<uint32_t*>(codes);
  int32_t rc;
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
