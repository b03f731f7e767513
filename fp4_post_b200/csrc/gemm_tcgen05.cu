// NVFP4 block-scaled GEMM with a fused bf16 rank-r side product, for sm_100a: the single-CTA kernel
// (one row block of A, or N <= 128; larger products run on CTA pairs, gemm_tcgen05_pair.cu) and the
// C entry point that chooses between the two.
//
//   D[M,N] = g * ( sum_k A[m,k] B[n,k] + sum_j T[m,j] U[n,j] ) + rank-1 terms (+ C)
//
// One persistent CTA per SM, 320 threads in four roles:
//   warp 0     TMA producer: per pipeline stage one 128 x 128-byte box of A codes, one
//              BN x 128-byte box of B codes (both 128-byte swizzled) and the matching E4M3
//              scale tiles (plain bulk copies: the scale layout makes them contiguous).
//   warp 1     tensor-core issuer: four K=64 tcgen05.mma.kind::mxf4nvf4.block_scale per stage
//              into the fp32 accumulator in tensor memory; the rank-r product runs as extra
//              pipeline iterations whose stages hold 64-column bf16 panels of T and U and are
//              consumed by tcgen05.mma.kind::f16 into the same accumulator.
//   warps 2-5  epilogue: tcgen05.ld the accumulator (each warp its own 32 lanes), apply the
//              scalar, the rank-1 terms and the optional addend, store bf16 or fp32.
//   warps 6-9  scale movers: carry each stage's E4M3 scale tiles shared memory -> registers ->
//              tensor memory (tcgen05.st, each warp its own 32 lanes: the four copies the
//              block-scale layout wants) beside the MMAs; a tcgen05.cp issued by warp 1 does the
//              same inside the MMA pipe, where three copies cost more than half an MMA.
// Decode-sized products split their K loop over idle SMs: a work item is (tile, K split), partial
// sums go to caller scratch and splitk_finish_kernel adds them up and applies the epilogue terms.
// Hand-offs are mbarriers; every wait is bounded and reports through the status word.
#include "gemm_common.cuh"

namespace metis {

// ---- the kernel ---------------------------------------------------------------------------------------

template <int BN, typename TD>
__global__ void __launch_bounds__(kGemmThreads, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_t, const __grid_constant__ CUtensorMap map_u,
                  const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStages = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::kStagingBytes);
  uint64_t* full = bars;                                   // [kStages]  TMA bytes landed
  uint64_t* empty = bars + kStages;                        // [kStages]  MMAs finished reading the stage
  uint64_t* acc_full = bars + 2 * kStages;                 // accumulator of the current tile complete
  uint64_t* acc_release = bars + 2 * kStages + 1;          // columns the next tile needs are drained
  uint64_t* drain = bars + 2 * kStages + 2;                // error path only
  uint64_t* sf_ready = bars + 2 * kStages + 3;             // [2] scale buffer written by the four movers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int64_t tiles_m = (p.M + kBM - 1) / kBM;
  const int64_t tiles_n = (p.N + BN - 1) / BN;
  const int64_t num_tiles = tiles_m * tiles_n;
  const int k_iters_all = (int)((p.K + 255) / 256);
  const int r_iters = (p.rank + 63) / 64;
  // Split-K: a work item is (tile, split); split s owns the K iterations [s k_per, (s+1) k_per) and,
  // if it is split 0, the rank-r iterations after them.  With more than one split the epilogue
  // stores raw fp32 partial sums and a second kernel adds them up and applies the epilogue terms.
  const int splits = p.splits;
  const int64_t num_work = num_tiles * splits;
#define METIS_WORK_ITEM(w)                                                                        \
  const int64_t tile = (w) / splits;                                                              \
  const int split = (int)((w) - tile * splits);                                                   \
  const int it0 = split * p.k_per_split;                                                          \
  const int k_iters = (k_iters_all - it0 < p.k_per_split) ? k_iters_all - it0 : p.k_per_split;    \
  const int iters = k_iters + (split == 0 ? r_iters : 0);                                         \
  (void)it0
  const int64_t sf_tiles_a = sf_tiles_per_row(p.K);        // per 128-row block (A and B share K)
  const int64_t b_row_blocks = (p.N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_release, 4);
    for (int b = 0; b < 2; ++b) mbar_init(&sf_ready[b], 4);
    mbar_init(drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();                                  // everything above touches shared and tensor memory only

  if (warp == 0) {
    // ===== TMA producer: the whole warp walks the pipeline, one elected lane issues the copies =====
    int stage = 0;
    uint32_t phase = 0;
    bool first = true;
    bool ok = true;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full_base = smem_u32(full);
    for (int64_t w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
      METIS_WORK_ITEM(w);
      int64_t tm, tn;
      tile_coords(tile, tiles_m, tiles_n, 16, tm, tn);
      const int32_t m0 = (int32_t)(tm * kBM), n0 = (int32_t)(tn * BN);
      // scale tiles: 4 per stage (2 KiB) and per 128 rows, contiguous along K; those of B exist
      // only for whole 128-row blocks of N
      const uint8_t* sfa_src = p.a_scales + ((int64_t)m0 >> 7) * sf_tiles_a * 512;
      const int64_t rb0 = (int64_t)n0 >> 7;
      const uint8_t* sfb_src = p.b_scales + rb0 * sf_tiles_a * 512;
      const bool sfb_second = (BN == 256) && (rb0 + 1 < b_row_blocks);
      const uint32_t k_bytes = Cfg::kABytes + Cfg::kBBytes + Cfg::kSfaBytes + 2048 + (sfb_second ? 2048 : 0);
      for (int it = 0; it < iters; ++it) {
        ok = __all_sync(0xffffffffu, mbar_wait(&empty[stage], phase ^ 1u, abort_flag));
        if (!ok) {
          if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_MMA);
          break;
        }
        const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
        const uint32_t sb = sa + Cfg::kABytes;
        const uint32_t ssfa = sb + Cfg::kBBytes;
        const uint32_t ssfb = ssfa + Cfg::kSfaBytes;
        const uint32_t bar = full_base + stage * 8;
        if (elect_one()) {
          if (p.debug & kDebugNoLoad) {
            mbar_arrive_addr(bar);
          } else if (it < k_iters) {
            mbar_expect_tx_addr(bar, k_bytes);
            const int kit = it0 + it;
            tma_load_2d_addr(sa, &map_a, kit * kBKBytes, m0, bar);
            tma_load_2d_addr(sb, &map_b, kit * kBKBytes, n0, bar);
            const bool drop = first && (p.debug & kDebugDropFirstSfa);
            if (!drop) bulk_load_addr(ssfa, sfa_src + (int64_t)kit * 2048, 2048, bar);
            bulk_load_addr(ssfb, sfb_src + (int64_t)kit * 2048, 2048, bar);
            if (sfb_second) bulk_load_addr(ssfb + 2048, sfb_src + (sf_tiles_a + (int64_t)kit * 4) * 512, 2048, bar);
          } else {
            const int j = it - k_iters;   // 64-column panel of the rank-r factors
            mbar_expect_tx_addr(bar, Cfg::kABytes + Cfg::kBBytes);
            tma_load_2d_addr(sa, &map_t, j * 64, m0, bar);
            tma_load_2d_addr(sb, &map_u, j * 64, n0, bar);
          }
        }
        first = false;
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    grid_launch_dependents();                                // the last loads of this CTA are on their way: let the next kernel's CTAs in
  } else if (warp == 1) {
    // ===== tensor-core issuer: the whole warp walks the pipeline, one elected lane issues =====
    // Keeping the loop warp-uniform lets the descriptors and addresses live in uniform registers;
    // a single diverged lane pays a register move per operand of every MMA and copy.
    int stage = 0;
    uint32_t phase = 0;
    uint32_t local_tile = 0;
    bool ok = true;
    bool issued = false;
    const uint32_t stage0_lo = operand_desc_lo(smem_u32(smem));
    const uint32_t empty_base = smem_u32(empty);
    uint32_t stage_lo = stage0_lo;
    uint32_t sf_buf = 0, sf_phase = 0;
    const bool no_mma = (p.debug & kDebugNoMma) != 0;
    for (int64_t w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++local_tile) {
      METIS_WORK_ITEM(w);
      // Tile j may start once the epilogue of tile j-1 has drained the columns the two
      // accumulators share (release number j-1, i.e. phase parity (j-1)&1).  That also covers
      // tile j-2, whose accumulator this one reuses: the epilogue finished it before it began j-1.
      if (local_tile > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(acc_release, (local_tile - 1u) & 1u, abort_flag));
        if (!ok) {
          if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_EPI);
          break;
        }
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (local_tile & 1u) * Cfg::kAccStride;
      for (int it = 0; it < iters; ++it) {
        const bool scaled = it < k_iters;
        // A scaled iteration waits for the movers only: they pass the stage's TMA barrier before
        // they copy, so their arrival also says that the code tiles have landed.
        uint64_t* wait_bar = (scaled && !no_mma) ? &sf_ready[sf_buf] : &full[stage];
        const uint32_t wait_parity = (scaled && !no_mma) ? sf_phase : phase;
        ok = __all_sync(0xffffffffu, mbar_wait(wait_bar, wait_parity, abort_flag));
        if (!ok) {
          if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_TMA);
          break;
        }
        tc_fence_after();
        // descriptor address fields (16-byte units) of this stage's A and B tiles
        const uint32_t a_lo = stage_lo;
        const uint32_t b_lo = stage_lo + (Cfg::kABytes >> 4);
        const uint32_t t_sfa = tmem_base + kSfCol + sf_buf * kSfBufCols, t_sfb = t_sfa + 16;
        if (elect_one()) {
          if (no_mma) {
          } else if (scaled) {
            // the movers have put this iteration's scales into buffer sf_buf: 4 columns per MMA
            // and 128 rows for A, then for B
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // 64 elements of K = 32 bytes (2 units) inside the 128-byte swizzled row
              tc_mma_fp4(d_tmem, a_lo + 2 * j, b_lo + 2 * j, kOperandDescHi, idesc_fp4(BN), t_sfa + 4 * j,
                         t_sfb + (BN / 128) * 4 * j, (it > 0 || j > 0) ? 1u : 0u);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // 16 bf16 of the rank dimension = 32 bytes
              tc_mma_bf16(d_tmem, a_lo + 2 * j, b_lo + 2 * j, kOperandDescHi, idesc_bf16(BN), (it > 0 || j > 0) ? 1u : 0u);
            }
          }
          // frees the stage (for the producer) and, two iterations on, its scale buffer (for the
          // movers) once these MMAs have read them
          tc_commit_addr(empty_base + stage * 8);
          if (it == iters - 1) tc_commit(acc_full);   // accumulator complete
        }
        issued = true;
        if (scaled && (sf_buf ^= 1u) == 0) sf_phase ^= 1u;
        stage_lo += Cfg::kStageBytes >> 4;
        if (++stage == kStages) { stage = 0; phase ^= 1u; stage_lo = stage0_lo; }
      }
    }
    if (!ok && issued && elect_one()) {
      // error path: let the tensor core finish what was issued before tensor memory is freed
      tc_commit(drain);
      const uint64_t t0 = global_ns();
      while (!mbar_try(drain, 0) && global_ns() - t0 < kWaitLimitNs) {}
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ===== scale movers: warps 6..9 own tensor-memory lanes 32*(warp%4) .. +31 =====
    // Lane l of every mover reads bytes [16 l, 16 l + 16) of a 512-byte scale tile: the scales of
    // rows l, l+32, l+64, l+96 for 4 scale columns, i.e. exactly the 4 tensor-memory columns that
    // lane l holds for that tile.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    int stage = 0;
    uint32_t phase = 0, sf_buf = 0;
    uint32_t slot = 0;                       // pipeline iterations so far, of either kind
    bool ok = true;
    for (int64_t w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
      METIS_WORK_ITEM(w);
      for (int it = 0; it < iters; ++it, ++slot) {
        if (it < k_iters && !(p.debug & kDebugNoMma)) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          const uint4* sf = reinterpret_cast<const uint4*>(smem + stage * Cfg::kStageBytes + Cfg::kABytes + Cfg::kBBytes) + lane;
          uint32_t ra[16], rb[(BN / 128) * 16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 w = sf[j * 32];                                  // tile j of A: 512 bytes = 32 uint4
            ra[4 * j] = w.x; ra[4 * j + 1] = w.y; ra[4 * j + 2] = w.z; ra[4 * j + 3] = w.w;
#pragma unroll
            for (int b = 0; b < BN / 128; ++b) {                         // tile j of each 128-row block of B
              const uint4 u = sf[(4 + b * 4 + j) * 32];
              uint32_t* dst = rb + ((BN / 128) * 4 * j + 4 * b);
              dst[0] = u.x; dst[1] = u.y; dst[2] = u.z; dst[3] = u.w;
            }
          }
          // The scale buffer was last read by the MMAs of an iteration at least two pipeline slots
          // back; the commit of slot - 2 (which frees that slot's stage) covers every MMA before it.
          if (slot >= 2) {
            const int s2 = stage >= 2 ? stage - 2 : stage - 2 + kStages;
            const uint32_t par2 = stage >= 2 ? phase : phase ^ 1u;
            if (!mbar_wait(&empty[s2], par2, abort_flag)) { ok = false; break; }
          }
          tc_fence_after();
          const uint32_t t_sfa = tmem_base + lane_base + kSfCol + sf_buf * kSfBufCols;
          tc_store16(t_sfa, ra);
#pragma unroll
          for (int h = 0; h < BN / 128; ++h) {
            const uint32_t (&half)[16] = *reinterpret_cast<const uint32_t (*)[16]>(rb + 16 * h);
            tc_store16(t_sfa + 16 + 16 * h, half);
          }
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sf_ready[sf_buf]);
          sf_buf ^= 1u;
        }
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (!ok && lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_TMA);
  } else {
    // ===== epilogue: warps 2..5 own tensor-memory lanes 32*(warp%4) .. +31 =====
    const int q = warp & 3;
    EpilogueCtx<TD> ctx;
    ctx.g = p.alpha * __ldg(p.a_unit) * __ldg(p.b_unit);
    ctx.p = &p;
    ctx.staging = staging + q * 2048;
    uint32_t local_tile = 0;
    for (int64_t w = blockIdx.x; w < num_work; w += gridDim.x, ++local_tile) {
      METIS_WORK_ITEM(w);
      int64_t tm, tn;
      tile_coords(tile, tiles_m, tiles_n, 16, tm, tn);
      const int64_t row = tm * kBM + q * 32 + lane;
      const int64_t n0 = tn * BN;
      ctx.row0 = tm * kBM + q * 32;
      ctx.partial = splits > 1 ? p.partial + (int64_t)split * p.M * p.ldp : nullptr;
      ctx.ldp = p.ldp;
      ctx.c0 = p.rvec0 ? (p.cvec0 ? (row < p.M ? __ldg(p.cvec0 + row) : 0.f) : 1.0f) : 0.0f;
      ctx.c1 = p.rvec1 ? (p.cvec1 ? (row < p.M ? __ldg(p.cvec1 + row) : 0.f) : 1.0f) : 0.0f;
      if (!mbar_wait(acc_full, local_tile & 1u, abort_flag)) {
        if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_MMA);
        break;
      }
      tc_fence_after();
      const uint32_t odd = local_tile & 1u;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + odd * Cfg::kAccStride;
      // chunk order: the columns shared with the other accumulator first.  For the even
      // accumulator [0,256) they are its last chunks, for the odd one [160,416) its first ones.
      constexpr int kChunks = BN / 32;
      constexpr int kShared = Cfg::kSharedChunks;
      const int first_chunk = (kShared > 0 && !odd) ? kChunks - kShared : 0;
      if constexpr (kShared > 0) {
        // pull every shared column into registers, hand the columns to the next tile's MMAs,
        // and only then do the arithmetic and the stores
        uint32_t rs[kShared][32];
#pragma unroll
        for (int s = 0; s < kShared; ++s) tc_load32(t_row + (first_chunk + s) * 32, rs[s]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_release);
#pragma unroll
        for (int s = 0; s < kShared; ++s) emit_chunk<TD>(ctx, rs[s], n0 + (first_chunk + s) * 32);
      } else {
        // separate accumulators: the next tile never touches this one
        if (lane == 0) mbar_arrive(acc_release);
      }
#pragma unroll 1
      for (int step = kShared; step < kChunks; ++step) {
        int ch = first_chunk + step;
        if (ch >= kChunks) ch -= kChunks;
        uint32_t r[32];
        tc_load32(t_row + ch * 32, r);
        tc_wait_ld();
        emit_chunk<TD>(ctx, r, n0 + ch * 32);
      }
      // the accumulator is free again only when every lane has read it
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- split-K: sum of the partial products + the epilogue terms -----------------------------------------

template <typename TD>
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const GemmParams p) {
  grid_dependency_wait();
  grid_launch_dependents();
  const int64_t groups_per_row = (p.N + 3) / 4;
  const float g = p.alpha * __ldg(p.a_unit) * __ldg(p.b_unit);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.M * groups_per_row; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / groups_per_row, col = (i - row * groups_per_row) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < p.splits; ++s) {            // fixed order: the result does not depend on timing
      const float4 v = *reinterpret_cast<const float4*>(p.partial + ((int64_t)s * p.M + row) * p.ldp + col);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float o[4] = {acc.x * g, acc.y * g, acc.z * g, acc.w * g};
    const float c0 = p.rvec0 ? (p.cvec0 ? __ldg(p.cvec0 + row) : 1.0f) : 0.0f;
    const float c1 = p.rvec1 ? (p.cvec1 ? __ldg(p.cvec1 + row) : 1.0f) : 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (col + j >= p.N) break;
      if (p.rvec0) o[j] = fmaf(c0, __ldg(p.rvec0 + col + j), o[j]);
      if (p.rvec1) o[j] = fmaf(c1, __ldg(p.rvec1 + col + j), o[j]);
      if (p.c) {
        if constexpr (sizeof(TD) == 2) o[j] += __bfloat162float(static_cast<const __nv_bfloat16*>(p.c)[row * p.ldc + col + j]);
        else o[j] += static_cast<const float*>(p.c)[row * p.ldc + col + j];
      }
      if constexpr (sizeof(TD) == 2) static_cast<__nv_bfloat16*>(p.d)[row * p.ldd + col + j] = __float2bfloat16_rn(o[j]);
      else static_cast<float*>(p.d)[row * p.ldd + col + j] = o[j];
    }
  }
}

// Splits the library would use for this shape: only products with a single row block of A (decode-
// sized M) whose tiles leave most SMs idle, and never fewer than 2 K iterations per split.
static int choose_splits(int64_t M, int64_t N, int64_t K, int bn, int sms) {
  if (M > 128) return 1;
  const int64_t tiles = ceil_div(N, bn);
  const int64_t k_iters = ceil_div(K, 256);
  int64_t s = sms / tiles;
  if (s > k_iters / 2) s = k_iters / 2;
  if (s > 8) s = 8;
  return s < 2 ? 1 : (int)s;
}
static int tile_width(int64_t M, int64_t N, int sms) {
  int bn = (N > 128) ? 256 : 128;
  // one row block of A and few column tiles (the weight gradient of a rank-r factor, decode):
  // narrower tiles put twice as many SMs to work, which matters more than the MMA shape there
  if (bn == 256 && M <= 128 && ceil_div(N, 256) * 2 <= sms) bn = 128;
  return bn;
}

// ---- host side ----------------------------------------------------------------------------------------------

template <int BN, typename TD>
static int32_t launch_gemm(const metis_gemm_args* a, const CUtensorMap& ma, const CUtensorMap& mb,
                           const CUtensorMap& mt, const CUtensorMap& mu, const GemmParams& p) {
  using Cfg = GemmCfg<BN>;
  auto kern = nvfp4_gemm_kernel<BN, TD>;
  // per device and cheap, so it is simply repeated on every launch
  METIS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
  const int64_t work = ceil_div(a->M, kBM) * ceil_div(a->N, BN) * p.splits;
  int64_t grid = gemm_sm_budget(a->sm_limit);
  if (grid > work) grid = work;
  grid = ceil_div(work, ceil_div(work, grid));        // the fewest CTAs that still finish in the same number of rounds
  cudaStream_t st = reinterpret_cast<cudaStream_t>(a->stream);
  METIS_CUDA_OK(launch_overlapped(kLaunchGemm, kern, dim3((unsigned)grid), dim3(kGemmThreads), Cfg::kSmemBytes, st, ma, mb, mt, mu, p));
  if (p.splits > 1) {
    const int64_t threads = a->M * ceil_div(a->N, 4);
    int64_t blocks = ceil_div(threads, 256);
    if (blocks > (int64_t)device_sm_count() * 8) blocks = (int64_t)device_sm_count() * 8;
    METIS_CUDA_OK(launch_overlapped(kLaunchGemm, splitk_finish_kernel<TD>, dim3((unsigned)blocks), dim3(256), 0, st, p));
  }
  return METIS_OK;
}

int32_t launch_gemm_pair(const metis_gemm_args* a, const CUtensorMap& ma, const CUtensorMap& mb,
                         const CUtensorMap& mt, const CUtensorMap& mu, const GemmParams& p);   // gemm_tcgen05_pair.cu

}  // namespace metis

using namespace metis;

extern "C" int64_t metis_nvfp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
  if (M <= 0 || N <= 0 || K <= 0 || M > 128) return 0;
  const int sms = device_sm_count();
  const int splits = choose_splits(M, N, K, tile_width(M, N, sms), sms);
  return splits > 1 ? (int64_t)splits * M * (ceil_div(N, 32) * 32) * (int64_t)sizeof(float) : 0;
}

extern "C" int32_t metis_nvfp4_gemm(const metis_gemm_args* a) {
  if (!a) return fail(METIS_ERR_BAD_ARGUMENT, "args is null");
  if (a->M <= 0 || a->N <= 0 || a->K <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty GEMM %lld x %lld x %lld", (long long)a->M, (long long)a->N, (long long)a->K);
  if (a->K % 32 != 0) return fail(METIS_ERR_BAD_SHAPE, "K = %lld must be a multiple of 32 (16-byte rows of packed codes)", (long long)a->K);
  if (a->M >= ((int64_t)1 << 31) || a->N >= ((int64_t)1 << 31) || a->K >= ((int64_t)1 << 31)) return fail(METIS_ERR_TOO_LARGE, "dimension too large");
  if (!a->a_codes || !a->a_scales || !a->a_unit || !a->b_codes || !a->b_scales || !a->b_unit || !a->d)
    return fail(METIS_ERR_BAD_ARGUMENT, "null operand pointer");
  if (!aligned16(a->a_codes) || !aligned16(a->b_codes) || !aligned16(a->a_scales) || !aligned16(a->b_scales) || !aligned16(a->d))
    return fail(METIS_ERR_BAD_ALIGNMENT, "codes, scales and d must be 16-byte aligned");
  if (a->d_dtype != METIS_DTYPE_BF16 && a->d_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown d_dtype %d", a->d_dtype);
  const int64_t dsz = a->d_dtype == METIS_DTYPE_BF16 ? 2 : 4;
  if (a->ldd < a->N || (a->ldd * dsz) % 16 != 0) return fail(METIS_ERR_BAD_ALIGNMENT, "ldd must be >= N and give 16-byte aligned rows");
  if (a->c && (a->ldc < a->N || (a->ldc * dsz) % 16 != 0 || !aligned16(a->c))) return fail(METIS_ERR_BAD_ALIGNMENT, "c must be 16-byte aligned with 16-byte aligned rows");
  if (a->rank < 0 || a->rank > 256 || a->rank % 8 != 0) return fail(METIS_ERR_BAD_SHAPE, "rank %d must be a multiple of 8 in [0, 256]", a->rank);
  if (a->rank > 0) {
    if (!a->lr_t || !a->lr_u) return fail(METIS_ERR_BAD_ARGUMENT, "rank > 0 needs lr_t and lr_u");
    if (!aligned16(a->lr_t) || !aligned16(a->lr_u) || a->ldt < a->rank || a->ldu < a->rank || a->ldt % 8 != 0 || a->ldu % 8 != 0)
      return fail(METIS_ERR_BAD_ALIGNMENT, "lr_t and lr_u must be 16-byte aligned with leading dimensions that are multiples of 8");
  }
  if ((a->cvec0 && !a->rvec0) || (a->cvec1 && !a->rvec1)) return fail(METIS_ERR_BAD_ARGUMENT, "a cvec needs its rvec");
  if (a->reserved & ~kDebugMask) return fail(METIS_ERR_BAD_ARGUMENT, "reserved must be 0");
  if (a->sm_limit < 0 || a->reserved2 != 0) return fail(METIS_ERR_BAD_ARGUMENT, "sm_limit must not be negative and reserved2 must be 0");

  const int sms = device_sm_count();
  const int bn = tile_width(a->M, a->N, sms);
  // CTA pairs (256 x 256 tiles) whenever there is more than one 128-row block of each operand
  const bool pair = bn == 256 && a->M > 128 && !(a->reserved & kDebugSingleCta);
  const int b_box = pair ? 128 : bn;       // rows of B (and U) one CTA loads per stage
  CUtensorMap ma, mb, mt, mu;
  if (int32_t rc = make_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->a_codes, a->K / 2, a->M, a->K / 2, kBKBytes, kBM, "A")) return rc;
  if (int32_t rc = make_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->b_codes, a->K / 2, a->N, a->K / 2, kBKBytes, b_box, "B")) return rc;
  if (a->rank > 0) {
    if (int32_t rc = make_map(&mt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->lr_t, a->rank, a->M, a->ldt * 2, 64, kBM, "T")) return rc;
    if (int32_t rc = make_map(&mu, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->lr_u, a->rank, a->N, a->ldu * 2, 64, b_box, "U")) return rc;
  } else {
    mt = ma;
    mu = mb;
  }
  GemmParams p;
  p.M = a->M; p.N = a->N; p.K = a->K; p.rank = a->rank; p.debug = a->reserved;
  p.a_scales = a->a_scales; p.b_scales = a->b_scales; p.a_unit = a->a_unit; p.b_unit = a->b_unit;
  p.alpha = a->alpha;
  p.cvec0 = a->cvec0; p.rvec0 = a->rvec0; p.cvec1 = a->cvec1; p.rvec1 = a->rvec1;
  p.c = a->c; p.ldc = a->ldc; p.d = a->d; p.ldd = a->ldd; p.status = a->status;
  // split-K needs the caller's scratch; without it (or with too little) the product runs unsplit
  const int splits = pair ? 1 : choose_splits(a->M, a->N, a->K, bn, sms);
  if (splits > 1 && a->workspace && a->workspace_bytes >= metis_nvfp4_gemm_workspace_bytes(a->M, a->N, a->K) &&
      aligned16(a->workspace) && !(a->reserved & (kDebugNoMma | kDebugNoLoad | kDebugDropFirstSfa))) {
    const int64_t k_iters = ceil_div(a->K, 256);
    p.k_per_split = (int32_t)ceil_div(k_iters, splits);
    p.splits = (int32_t)ceil_div(k_iters, p.k_per_split);       // no split is left without iterations
    p.partial = static_cast<float*>(a->workspace);
    p.ldp = ceil_div(a->N, 32) * 32;
  }
  if (pair) return launch_gemm_pair(a, ma, mb, mt, mu, p);
  if (bn == 256) {
    if (a->d_dtype == METIS_DTYPE_BF16) return launch_gemm<256, __nv_bfloat16>(a, ma, mb, mt, mu, p);
    return launch_gemm<256, float>(a, ma, mb, mt, mu, p);
  }
  if (a->d_dtype == METIS_DTYPE_BF16) return launch_gemm<128, __nv_bfloat16>(a, ma, mb, mt, mu, p);
  return launch_gemm<128, float>(a, ma, mb, mt, mu, p);
}
