// Backward of the unquantized low-rank branch  y_u = (s . y_v) U^T  on the tensor core (sm_100a).
//
// The reference leaves these products to autograd: ulinear is a plain nn.Linear and the scaling by s a
// torch.mul (src/Metis/Metis/bitlinear.py:752-760, 872-879), so with G = grad_output [M, N] in bf16
//     d_ts = G U            [M, r]   contraction over N
//     dU   = G^T (s . y_v)  [N, r]   contraction over the tokens M
//     ds   = sum_m d_ts . y_v,   d_yv = d_ts . s
// Both products are skinny (r <= 256) and bound by the one read of G each needs.  One kernel serves
// both: a bf16 tcgen05 GEMM  D[Mg, Ng] = A [Mg, Kg] B [Ng, Kg]^T  whose operands may be stored either way
// round:
//     K-major   memory [rows = Mg or Ng, Kg contiguous]   (G for d_ts: Kg = N)
//     MN-major  memory [Kg rows, Mg or Ng contiguous]     (U [N, r] for d_ts; G and s . y_v for dU: Kg = M)
// so no operand is ever transposed in memory.  TMA boxes are 64 elements (128 bytes) wide, 128-byte
// swizzled; an MN-major operand tile is made of 64-element column boxes placed side by side (leading
// byte offset = one box), its 8-row groups 1024 bytes apart exactly like a K-major tile.
//
// One CTA per work item (128 rows of D, one K split): warp 0 TMA producer, warp 1 MMA issuer, warps 2-5
// epilogue (raw fp32 partial sums to scratch).  The small finish kernels add the splits in a fixed order
// and apply what autograd would: the bf16 roundings, the product with s, the reduction for ds.
// Every wait is bounded and reports through the status word.
#include "gemm_common.cuh"

namespace metis {

constexpr int kPanelThreads = 192;          // producer, issuer, 4 epilogue warps
constexpr int kPanelKStage = 64;            // elements of the contraction per pipeline stage
constexpr int kPanelABytes = 128 * 128;     // 128 rows of D x 64 bf16
constexpr int kPanelBoxBytes = 64 * 128;    // one MN-major box: 64 contraction rows x 64 elements

struct PanelParams {
  int64_t Mg, Ng, Kg;
  int32_t bn;                 // Ng rounded up to a multiple of 64: the MMA's N
  int32_t stages;
  int32_t splits, k_per_split;      // K stages per split
  float* partial;  int64_t ldp;     // [splits, Mg, ldp] fp32
  int32_t* status;
  // fused finish of d_ts = G U (one split only): d_yv, and the column sums of bf16(d_ts * y_v) for ds
  const __nv_bfloat16* yv;  int64_t ldyv;
  const void* s;  int32_t s_is_f32;
  __nv_bfloat16* d_yv;  int64_t ldd;
  float* block_sums;  unsigned int* ticket;  float* ds;
  int32_t r;
};

static inline int panel_stage_bytes(int bn) { return kPanelABytes + bn * 128; }
static inline int panel_smem_bytes(int bn, int stages) { return stages * panel_stage_bytes(bn) + 1024 + 256 + 4 * 256 * 4; }

// Column sums of a 32 x 32 block held one row per lane: after five exchange-and-add steps lane l holds
// the sum of column l (31 shuffles instead of 160).
__device__ __forceinline__ float column_sums32(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int j = 0; j < off; ++j) {
      const float send = upper ? v[j] : v[j + off];
      const float keep = upper ? v[j + off] : v[j];
      v[j] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0];
}

template <bool kAMn, bool kBMn, bool kDts>
__global__ void __launch_bounds__(kPanelThreads, 1)
bf16_panel_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const PanelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int stage_bytes = kPanelABytes + p.bn * 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* full = bars;                       // [stages]
  uint64_t* empty = bars + p.stages;           // [stages]
  uint64_t* acc_full = bars + 2 * p.stages;
  uint64_t* drain = bars + 2 * p.stages + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * p.stages + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_colsum = reinterpret_cast<float*>(smem + p.stages * stage_bytes + 256);     // [4][256], fused finish only

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t tile_m = blockIdx.x / p.splits;
  const int split = (int)(blockIdx.x - tile_m * p.splits);
  const int k_iters_all = (int)((p.Kg + kPanelKStage - 1) / kPanelKStage);
  const int it0 = split * p.k_per_split;
  const int iters = (k_iters_all - it0 < p.k_per_split) ? k_iters_all - it0 : p.k_per_split;
  const uint32_t tmem_cols = p.bn <= 64 ? 64u : (p.bn <= 128 ? 128u : 256u);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();

  if (warp == 0) {
    // ===== TMA producer =====
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full_base = smem_u32(full);
    const int32_t m0 = (int32_t)(tile_m * 128);
    const int b_boxes = p.bn / 64;
    for (int it = 0; it < iters && ok; ++it) {
      ok = __all_sync(0xffffffffu, mbar_wait(&empty[stage], phase ^ 1u, abort_flag));
      if (!ok) {
        if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_MMA);
        break;
      }
      const uint32_t sa = smem_base + stage * stage_bytes;
      const uint32_t sb = sa + kPanelABytes;
      const uint32_t bar = full_base + stage * 8;
      const int32_t k0 = (it0 + it) * kPanelKStage;
      if (elect_one()) {
        mbar_expect_tx_addr(bar, (uint32_t)stage_bytes);
        if (kAMn) {
          tma_load_2d_addr(sa, &map_a, m0, k0, bar);                       // [64 k rows, 64 columns of D's rows]
          tma_load_2d_addr(sa + kPanelBoxBytes, &map_a, m0 + 64, k0, bar);
        } else {
          tma_load_2d_addr(sa, &map_a, k0, m0, bar);                       // [128 rows, 64 k]
        }
        if (kBMn) {
          for (int h = 0; h < b_boxes; ++h) tma_load_2d_addr(sb + h * kPanelBoxBytes, &map_b, h * 64, k0, bar);
        } else {
          tma_load_2d_addr(sb, &map_b, k0, 0, bar);                        // [bn rows, 64 k]
        }
      }
      if (++stage == p.stages) { stage = 0; phase ^= 1u; }
    }
    grid_launch_dependents();
  } else if (warp == 1) {
    // ===== tensor-core issuer =====
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true, issued = false;
    const uint32_t empty_base = smem_u32(empty);
    // descriptor low words: address, and for an MN-major tile the distance between its 64-element
    // column boxes as the leading byte offset
    const uint32_t a_lead = kAMn ? (uint32_t)(kPanelBoxBytes >> 4) : 1u;
    const uint32_t b_lead = kBMn ? (uint32_t)(kPanelBoxBytes >> 4) : 1u;
    // one MMA takes 16 elements of the contraction: 32 bytes along a K-major row, 16 rows of an MN-major tile
    const uint32_t a_step = kAMn ? (16u * 128u) >> 4 : 2u;
    const uint32_t b_step = kBMn ? (16u * 128u) >> 4 : 2u;
    const uint32_t idesc = idesc_bf16(p.bn) | (kAMn ? (1u << 15) : 0u) | (kBMn ? (1u << 16) : 0u);
    for (int it = 0; it < iters; ++it) {
      ok = __all_sync(0xffffffffu, mbar_wait(&full[stage], phase, abort_flag));
      if (!ok) {
        if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_TMA);
        break;
      }
      tc_fence_after();
      const uint32_t sa = smem_u32(smem) + stage * stage_bytes;
      const uint32_t a_lo = ((sa & 0x3FFFFu) >> 4) | (a_lead << 16);
      const uint32_t b_lo = (((sa + kPanelABytes) & 0x3FFFFu) >> 4) | (b_lead << 16);
      if (elect_one()) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          tc_mma_bf16(tmem_base, a_lo + a_step * j, b_lo + b_step * j, kOperandDescHi, idesc, (it > 0 || j > 0) ? 1u : 0u);
        tc_commit_addr(empty_base + stage * 8);
        if (it == iters - 1) tc_commit(acc_full);
      }
      issued = true;
      if (++stage == p.stages) { stage = 0; phase ^= 1u; }
    }
    if (!ok && issued && elect_one()) {
      tc_commit(drain);
      const uint64_t t0 = global_ns();
      while (!mbar_try(drain, 0) && global_ns() - t0 < kWaitLimitNs) {}
    }
    __syncwarp();
  } else {
    // ===== epilogue: warps 2..5 own tensor-memory lanes 32*(warp%4) .. +31 =====
    const int q = warp & 3;
    const int64_t row = tile_m * 128 + q * 32 + lane;
    if (iters > 0) {
      if (!mbar_wait(acc_full, 0, abort_flag)) {
        if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_MMA);
      } else {
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16);
        if constexpr (kDts) {
          // autograd's bf16 steps on this CTA's 128 rows of d_ts, straight from the accumulator
          const bool live = row < p.Mg;
          for (int ch = 0; ch * 32 < p.r; ++ch) {
            uint32_t acc[32];
            tc_load32(t_row + ch * 32, acc);
            uint32_t yw[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) yw[i] = 0u;
            if (live) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if (ch * 32 + 8 * i < p.r) {
                  const uint4 w = __ldg(reinterpret_cast<const uint4*>(p.yv + row * p.ldyv + ch * 32) + i);
                  yw[4 * i] = w.x; yw[4 * i + 1] = w.y; yw[4 * i + 2] = w.z; yw[4 * i + 3] = w.w;
                }
              }
            }
            tc_wait_ld(acc);
            float prod[32];
            uint32_t ow[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int c = ch * 32 + i;
              float s0 = 0.0f, s1 = 0.0f;
              if (c < p.r) {
                if (p.s_is_f32) { s0 = static_cast<const float*>(p.s)[c]; s1 = static_cast<const float*>(p.s)[c + 1]; }
                else { const uint32_t sw = *reinterpret_cast<const uint32_t*>(static_cast<const __nv_bfloat16*>(p.s) + c); s0 = bf16_lo(sw); s1 = bf16_hi(sw); }
              }
              const __nv_bfloat162 s2 = __floats2bfloat162_rn(s0, s1);                             // s.to(bf16)
              const __nv_bfloat162 d2 = __floats2bfloat162_rn(__uint_as_float(acc[i]), __uint_as_float(acc[i + 1]));   // the product's bf16 output
              const __nv_bfloat162 o2 = __hmul2(d2, s2);                                             // d_ts * s, one rounding
              const __nv_bfloat162 p2 = __hmul2(d2, *reinterpret_cast<const __nv_bfloat162*>(&yw[i >> 1]));   // d_ts * y_v
              ow[i >> 1] = *reinterpret_cast<const uint32_t*>(&o2);
              const uint32_t pw = *reinterpret_cast<const uint32_t*>(&p2);
              prod[i] = live ? bf16_lo(pw) : 0.0f;
              prod[i + 1] = live ? bf16_hi(pw) : 0.0f;
            }
            if (live) {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (ch * 32 + 8 * i < p.r)
                  reinterpret_cast<uint4*>(p.d_yv + row * p.ldd + ch * 32)[i] = make_uint4(ow[4 * i], ow[4 * i + 1], ow[4 * i + 2], ow[4 * i + 3]);
            }
            s_colsum[q * 256 + ch * 32 + lane] = column_sums32(prod, lane);
          }
        } else {
          float* dst = p.partial + ((int64_t)split * p.Mg + row) * p.ldp;
          for (int ch = 0; ch < p.bn / 32; ++ch) {
            uint32_t r[32];
            tc_load32(t_row + ch * 32, r);
            tc_wait_ld(r);
            if (row < p.Mg && ch * 32 < p.ldp) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(dst + ch * 32)[i] =
                    make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
            }
          }
        }
        tc_fence_before();
      }
    } else if (row < p.Mg) {
      // a split without iterations contributes zeros
      float* dst = p.partial + ((int64_t)split * p.Mg + row) * p.ldp;
      for (int64_t c = 0; c < p.ldp; ++c) dst[c] = 0.0f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
  if constexpr (kDts) {
    // this CTA's column sums (its four 32-row groups in a fixed order), then the last CTA to arrive adds all
    // CTAs' sums in CTA order: ds does not depend on timing
    for (int c = threadIdx.x; c < p.r; c += kPanelThreads)
      p.block_sums[(int64_t)blockIdx.x * p.r + c] = (s_colsum[c] + s_colsum[256 + c]) + (s_colsum[512 + c] + s_colsum[768 + c]);
    __threadfence();
    __syncthreads();
    __shared__ unsigned int s_last;
    if (threadIdx.x == 0) s_last = (atomicAdd(p.ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int c = threadIdx.x; c < p.r; c += kPanelThreads) {
        float total = 0.0f;
        for (unsigned b = 0; b < gridDim.x; ++b) total += __ldcg(p.block_sums + (int64_t)b * p.r + c);
        p.ds[c] = total;
      }
      if (threadIdx.x == 0) *p.ticket = 0u;
    }
  }
}

// ---- finish kernels -------------------------------------------------------------------------------------------

// d_ts = bf16(sum over splits); d_yv = bf16(d_ts * bf16(s)); per-CTA column sums of bf16(d_ts * y_v)
// go to block_sums [gridDim.x, r]; the last CTA to finish adds them in block order into ds.
constexpr int kFinishThreads = 256;
__global__ void __launch_bounds__(kFinishThreads)
lowrank_dts_finish_kernel(const float* __restrict__ partial, int splits, int64_t M, int r, int64_t ldp,
                          const __nv_bfloat16* __restrict__ yv, int64_t ldyv, const void* __restrict__ s, int s_is_f32,
                          __nv_bfloat16* __restrict__ d_yv, int64_t ldd, float* __restrict__ block_sums,
                          unsigned int* __restrict__ ticket, float* __restrict__ ds) {
  grid_dependency_wait();
  // thread (cx, ry): columns cx, cx + 64, ... ; rows ry, ry + 4, ... of this CTA's row range
  const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;
  const int64_t rows_per_cta = (M + gridDim.x - 1) / gridDim.x;
  const int64_t r_begin = (int64_t)blockIdx.x * rows_per_cta;
  const int64_t r_end = r_begin + rows_per_cta < M ? r_begin + rows_per_cta : M;
  __shared__ float s_sum[4][256];
  for (int c = cx; c < r; c += 64) {
    const float sc = s_is_f32 ? __bfloat162float(__float2bfloat16_rn(static_cast<const float*>(s)[c]))
                              : __bfloat162float(static_cast<const __nv_bfloat16*>(s)[c]);
    float acc = 0.0f;
    for (int64_t row = r_begin + ry; row < r_end; row += 4) {
      float v = 0.0f;
      for (int sp = 0; sp < splits; ++sp) v += partial[((int64_t)sp * M + row) * ldp + c];
      const float dts = __bfloat162float(__float2bfloat16_rn(v));                   // the product's bf16 output
      d_yv[row * ldd + c] = __float2bfloat16_rn(dts * sc);
      acc += __bfloat162float(__float2bfloat16_rn(dts * __bfloat162float(yv[row * ldyv + c])));
    }
    s_sum[ry][c] = acc;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < r; c += kFinishThreads)
    block_sums[(int64_t)blockIdx.x * r + c] = (s_sum[0][c] + s_sum[1][c]) + (s_sum[2][c] + s_sum[3][c]);
  // the last CTA adds the block sums in block order: the result does not depend on timing
  __threadfence();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    __threadfence();
    for (int c = threadIdx.x; c < r; c += kFinishThreads) {
      float total = 0.0f;
      for (unsigned b = 0; b < gridDim.x; ++b) total += __ldcg(block_sums + (int64_t)b * r + c);
      ds[c] = total;
    }
    if (threadIdx.x == 0) *ticket = 0u;                // ready for the next call
  }
}

template <typename TU>
__global__ void __launch_bounds__(kFinishThreads)
lowrank_du_finish_kernel(const float* __restrict__ partial, int splits, int64_t N, int r, int64_t ldp,
                         TU* __restrict__ grad_u, int64_t ldu) {
  grid_dependency_wait();
  const int64_t total = N * r;
  for (int64_t i = (int64_t)blockIdx.x * kFinishThreads + threadIdx.x; i < total; i += (int64_t)gridDim.x * kFinishThreads) {
    const int64_t n = i / r;
    const int c = (int)(i - n * r);
    float v = 0.0f;
    for (int sp = 0; sp < splits; ++sp) v += partial[((int64_t)sp * N + n) * ldp + c];
    if constexpr (sizeof(TU) == 2) grad_u[n * ldu + c] = __float2bfloat16_rn(v);
    else grad_u[n * ldu + c] = v;
  }
}

// ---- host side ----------------------------------------------------------------------------------------------

struct PanelPlan {
  int bn, stages, splits, k_per_split;
  int64_t ldp, tiles_m, partial_bytes;
};

static PanelPlan plan_panel(int64_t Mg, int64_t Ng, int64_t Kg) {
  PanelPlan pl;
  pl.bn = (int)(ceil_div(Ng, 64) * 64);
  pl.stages = pl.bn <= 128 ? 6 : 4;
  pl.tiles_m = ceil_div(Mg, 128);
  const int64_t k_iters = ceil_div(Kg, kPanelKStage);
  // enough work items to fill the SMs once, never fewer than 8 K stages per split
  int64_t s = device_sm_count() / pl.tiles_m;
  if (s > k_iters / 8) s = k_iters / 8;
  if (s > 16) s = 16;
  if (s < 1) s = 1;
  pl.k_per_split = (int)ceil_div(k_iters, s);
  pl.splits = (int)ceil_div(k_iters, pl.k_per_split);
  pl.ldp = pl.bn;
  pl.partial_bytes = (int64_t)pl.splits * Mg * pl.ldp * (int64_t)sizeof(float);
  return pl;
}

// D partial sums [splits, Mg, ldp]; a: [Mg, Kg] (K-major) or [Kg, Mg] (MN-major), b likewise with Ng
static int32_t launch_panel(const void* a, bool a_mn, int64_t lda, const void* b, bool b_mn, int64_t ldb, int64_t Mg, int64_t Ng,
                            int64_t Kg, const PanelPlan& pl, float* partial, int32_t* status, cudaStream_t st,
                            const PanelParams* dts = nullptr) {
  CUtensorMap ma, mb;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (a_mn) { if (int32_t rc = make_map(&ma, dt, 2, a, Mg, Kg, lda * 2, 64, kPanelKStage, "A (MN-major)")) return rc; }
  else      { if (int32_t rc = make_map(&ma, dt, 2, a, Kg, Mg, lda * 2, 64, 128, "A (K-major)")) return rc; }
  if (b_mn) { if (int32_t rc = make_map(&mb, dt, 2, b, Ng, Kg, ldb * 2, 64, kPanelKStage, "B (MN-major)")) return rc; }
  else      { if (int32_t rc = make_map(&mb, dt, 2, b, Kg, Ng, ldb * 2, 64, pl.bn, "B (K-major)")) return rc; }
  PanelParams p = {};
  if (dts) p = *dts;
  p.Mg = Mg; p.Ng = Ng; p.Kg = Kg; p.bn = pl.bn; p.stages = pl.stages; p.splits = pl.splits; p.k_per_split = pl.k_per_split;
  p.partial = partial; p.ldp = pl.ldp; p.status = status;
  const int smem = panel_smem_bytes(pl.bn, pl.stages);
  const dim3 grid((unsigned)(pl.tiles_m * pl.splits)), block(kPanelThreads);
#define METIS_LAUNCH_PANEL(AMN, BMN)                                                                         \
  do {                                                                                                       \
    auto kern = bf16_panel_gemm_kernel<AMN, BMN, false>;                                                     \
    METIS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));            \
    METIS_CUDA_OK(launch_overlapped(kLaunchGemm, kern, grid, block, (size_t)smem, st, ma, mb, p));           \
  } while (0)
  if (dts) {                                   // d_ts = G U with the fused finish: K-major G, U read as it lies
    auto kern = bf16_panel_gemm_kernel<false, true, true>;
    METIS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    METIS_CUDA_OK(launch_overlapped(kLaunchGemm, kern, grid, block, (size_t)smem, st, ma, mb, p));
    return METIS_OK;
  }
  if (a_mn) { if (b_mn) METIS_LAUNCH_PANEL(true, true); else METIS_LAUNCH_PANEL(true, false); }
  else      { if (b_mn) METIS_LAUNCH_PANEL(false, true); else METIS_LAUNCH_PANEL(false, false); }
#undef METIS_LAUNCH_PANEL
  return METIS_OK;
}

static int32_t check_bf16_matrix(const void* p, int64_t ld, int64_t cols, const char* what) {
  if (!p) return fail(METIS_ERR_BAD_ARGUMENT, "%s is null", what);
  if (!aligned16(p) || ld < cols || ld % 8 != 0) return fail(METIS_ERR_BAD_ALIGNMENT, "%s must be 16-byte aligned with a leading dimension that is a multiple of 8", what);
  return METIS_OK;
}

constexpr int kDtsFinishCtas = 256;
// ticket word + per-CTA column sums: the finish kernel's CTAs, or one per 128 rows when the finish is fused
static int64_t dts_tail_bytes(int64_t M, int64_t r) {
  const int64_t ctas = ceil_div(M, 128) > kDtsFinishCtas ? ceil_div(M, 128) : kDtsFinishCtas;
  return 256 + ctas * r * (int64_t)sizeof(float);
}

}  // namespace metis

using namespace metis;

extern "C" int64_t metis_bf16_panel_gemm_workspace_bytes(int64_t Mg, int64_t Ng, int64_t Kg) {
  if (Mg <= 0 || Ng <= 0 || Kg <= 0) return 0;
  return plan_panel(Mg, Ng, Kg).partial_bytes;
}

extern "C" int32_t metis_bf16_panel_gemm(const void* a, int32_t a_mn_major, int64_t lda, const void* b, int32_t b_mn_major, int64_t ldb,
                                         int64_t Mg, int64_t Ng, int64_t Kg, float* d, int64_t ldd, void* workspace,
                                         int64_t workspace_bytes, int32_t* status, void* stream) {
  if (Mg <= 0 || Ng <= 0 || Kg <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty product %lld x %lld x %lld", (long long)Mg, (long long)Ng, (long long)Kg);
  if (Ng > 256) return fail(METIS_ERR_BAD_SHAPE, "Ng = %lld: the panel product takes up to 256 columns", (long long)Ng);
  if (int32_t rc = check_bf16_matrix(a, lda, a_mn_major ? Mg : Kg, "a")) return rc;
  if (int32_t rc = check_bf16_matrix(b, ldb, b_mn_major ? Ng : Kg, "b")) return rc;
  if (!d || !workspace || ldd < Ng) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer or ldd < Ng");
  if (!aligned16(workspace) || workspace_bytes < metis_bf16_panel_gemm_workspace_bytes(Mg, Ng, Kg)) return fail(METIS_ERR_WORKSPACE, "workspace too small or misaligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PanelPlan pl = plan_panel(Mg, Ng, Kg);
  float* partial = static_cast<float*>(workspace);
  if (int32_t rc = launch_panel(a, a_mn_major != 0, lda, b, b_mn_major != 0, ldb, Mg, Ng, Kg, pl, partial, status, st)) return rc;
  int64_t blocks = ceil_div(Mg * Ng, kFinishThreads);
  if (blocks > (int64_t)device_sm_count() * 8) blocks = (int64_t)device_sm_count() * 8;
  METIS_CUDA_OK(launch_overlapped(kLaunchShort, lowrank_du_finish_kernel<float>, dim3((unsigned)blocks), dim3(kFinishThreads), 0, st,
                                  (const float*)partial, pl.splits, Mg, (int)Ng, pl.ldp, d, ldd));
  return METIS_OK;
}

extern "C" int64_t metis_lowrank_dts_workspace_bytes(int64_t M, int64_t N, int64_t r) {
  if (M <= 0 || N <= 0 || r <= 0) return 0;
  return plan_panel(M, r, N).partial_bytes + dts_tail_bytes(M, r);
}

extern "C" int32_t metis_lowrank_dts(const void* g, int64_t ldg, int64_t M, int64_t N, const void* u, int64_t ldu, int64_t r,
                                     const void* yv, int64_t ldyv, const void* s, int32_t s_dtype, void* d_yv, int64_t ldd,
                                     float* ds, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream) {
  if (M <= 0 || N <= 0 || r <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty product %lld x %lld x %lld", (long long)M, (long long)N, (long long)r);
  if (r > 256 || r % 8 != 0 || N % 8 != 0) return fail(METIS_ERR_BAD_SHAPE, "rank %lld must be a multiple of 8 up to 256 and N = %lld a multiple of 8", (long long)r, (long long)N);
  if (int32_t rc = check_bf16_matrix(g, ldg, N, "g")) return rc;
  if (int32_t rc = check_bf16_matrix(u, ldu, r, "u")) return rc;
  if (int32_t rc = check_bf16_matrix(yv, ldyv, r, "yv")) return rc;
  if (int32_t rc = check_bf16_matrix(d_yv, ldd, r, "d_yv")) return rc;
  if (!s || !ds || !workspace) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer");
  if (s_dtype != METIS_DTYPE_BF16 && s_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown s_dtype %d", s_dtype);
  if (!aligned16(workspace) || workspace_bytes < metis_lowrank_dts_workspace_bytes(M, N, r)) return fail(METIS_ERR_WORKSPACE, "workspace too small or misaligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PanelPlan pl = plan_panel(M, r, N);
  float* partial = static_cast<float*>(workspace);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(static_cast<char*>(workspace) + pl.partial_bytes);
  float* block_sums = reinterpret_cast<float*>(static_cast<char*>(workspace) + pl.partial_bytes + 256);
  METIS_CUDA_OK(cudaMemsetAsync(ticket, 0, sizeof(unsigned int), st));
  // d_ts = G U: G [M, N] is K-major (contraction over its columns), U [N, r] holds the contraction in its rows
  if (pl.splits == 1) {
    // one split (many tokens): d_yv and ds come straight from the accumulator, no partial sums in memory
    PanelParams f = {};
    f.yv = static_cast<const __nv_bfloat16*>(yv); f.ldyv = ldyv; f.s = s; f.s_is_f32 = (s_dtype == METIS_DTYPE_F32);
    f.d_yv = static_cast<__nv_bfloat16*>(d_yv); f.ldd = ldd; f.block_sums = block_sums; f.ticket = ticket; f.ds = ds; f.r = (int32_t)r;
    return launch_panel(g, false, ldg, u, true, ldu, M, r, N, pl, partial, status, st, &f);
  }
  if (int32_t rc = launch_panel(g, false, ldg, u, true, ldu, M, r, N, pl, partial, status, st)) return rc;
  int64_t ctas = ceil_div(M, 64);
  if (ctas > kDtsFinishCtas) ctas = kDtsFinishCtas;
  METIS_CUDA_OK(launch_overlapped(kLaunchShort, lowrank_dts_finish_kernel, dim3((unsigned)ctas), dim3(kFinishThreads), 0, st,
                                  (const float*)partial, pl.splits, M, (int)r, pl.ldp, static_cast<const __nv_bfloat16*>(yv), ldyv, s,
                                  (int)(s_dtype == METIS_DTYPE_F32), static_cast<__nv_bfloat16*>(d_yv), ldd, block_sums, ticket, ds));
  return METIS_OK;
}

extern "C" int64_t metis_lowrank_du_workspace_bytes(int64_t M, int64_t N, int64_t r) {
  if (M <= 0 || N <= 0 || r <= 0) return 0;
  return plan_panel(N, r, M).partial_bytes;
}

extern "C" int32_t metis_lowrank_du(const void* g, int64_t ldg, int64_t M, int64_t N, const void* ts, int64_t ldts, int64_t r,
                                    void* grad_u, int32_t u_dtype, int64_t ldgu, void* workspace, int64_t workspace_bytes,
                                    int32_t* status, void* stream) {
  if (M <= 0 || N <= 0 || r <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty product %lld x %lld x %lld", (long long)M, (long long)N, (long long)r);
  if (r > 256 || r % 8 != 0 || N % 8 != 0) return fail(METIS_ERR_BAD_SHAPE, "rank %lld must be a multiple of 8 up to 256 and N = %lld a multiple of 8", (long long)r, (long long)N);
  if (int32_t rc = check_bf16_matrix(g, ldg, N, "g")) return rc;
  if (int32_t rc = check_bf16_matrix(ts, ldts, r, "ts")) return rc;
  if (!grad_u || !workspace) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer");
  if (u_dtype != METIS_DTYPE_BF16 && u_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown u_dtype %d", u_dtype);
  if (ldgu < r) return fail(METIS_ERR_BAD_ARGUMENT, "ldgu %lld < r %lld", (long long)ldgu, (long long)r);
  if (!aligned16(workspace) || workspace_bytes < metis_lowrank_du_workspace_bytes(M, N, r)) return fail(METIS_ERR_WORKSPACE, "workspace too small or misaligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const PanelPlan pl = plan_panel(N, r, M);
  float* partial = static_cast<float*>(workspace);
  // dU = G^T ts: both operands hold the contraction (the tokens) in their rows
  if (int32_t rc = launch_panel(g, true, ldg, ts, true, ldts, N, r, M, pl, partial, status, st)) return rc;
  int64_t blocks = ceil_div(N * r, kFinishThreads);
  if (blocks > (int64_t)device_sm_count() * 8) blocks = (int64_t)device_sm_count() * 8;
  if (u_dtype == METIS_DTYPE_BF16)
    METIS_CUDA_OK(launch_overlapped(kLaunchShort, lowrank_du_finish_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(kFinishThreads), 0, st,
                                    (const float*)partial, pl.splits, N, (int)r, pl.ldp, static_cast<__nv_bfloat16*>(grad_u), ldgu));
  else
    METIS_CUDA_OK(launch_overlapped(kLaunchShort, lowrank_du_finish_kernel<float>, dim3((unsigned)blocks), dim3(kFinishThreads), 0, st,
                                    (const float*)partial, pl.splits, N, (int)r, pl.ldp, static_cast<float*>(grad_u), ldgu));
  return METIS_OK;
}
