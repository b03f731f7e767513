// NVFP4 block-scaled GEMM on CTA pairs (tcgen05 cta_group::2), for sm_100a.
//
// Two CTAs of one cluster compute a 256 x 256 output tile with M256 x N256 x K64 MMAs issued by the
// pair's leader.  CTA r of the pair holds rows [128 r, 128 r + 128) of the A tile, the same rows of
// the accumulator in its own tensor memory, and rows [128 r, 128 r + 128) of the B tile; the tensor
// core reads the other half of B from the peer's shared memory.  Per stage and SM that is 38 KiB
// instead of the 54 KiB of the single-CTA kernel, for the same 512 tensor-pipe cycles: the operand
// feed (L2 -> shared memory, and shared memory -> tensor core) is what bounds the single-CTA kernel.
//
// Roles per CTA (320 threads): warp 0 TMA producer, warp 1 tensor-core issuer (leader only),
// warps 2-9 epilogue (two warps per 32-lane quarter of tensor memory, alternate column chunks).  The scale tiles travel shared memory -> tensor memory by tcgen05.cp issued
// by the leader in front of each stage's MMAs: one instruction copies in both CTAs, in pipe order
// with the MMAs, so no cross-SM handshake sits inside the pipeline loop (a handshake through the
// peer costs a cluster round trip of more than a thousand cycles per two stages).
//   full[s]      leader's: all bytes of stage s of BOTH CTAs (the peer's TMA loads signal it remotely)
//   empty[s]     local: stage s consumed (commit multicast by the leader to both CTAs)
//   acc_full     local: accumulator complete (commit multicast)
//   acc_release  leader's: 16 epilogue warps (8 remote arrivals) have drained the shared accumulator columns
// No copy is multicast.  Every wait is bounded; both CTAs meet at a cluster barrier before they
// free tensor memory, so neither exits while the other can still signal or read it.
#include "gemm_common.cuh"

namespace metis {

struct PairCfg {
  static constexpr int BN = 256;
  static constexpr int kStages = 5;
  static constexpr int kAccStride = 160;
  static constexpr int kSharedChunks = 3;
  static constexpr int kABytes = kBM * kBKBytes;          // 16 KiB: this CTA's 128 rows of A
  static constexpr int kBBytes = 128 * kBKBytes;          // 16 KiB: this CTA's 128 rows of B
  static constexpr int kSfaBytes = 4 * 512;               // scales of this CTA's rows of A
  static constexpr int kSfbBytes = 2 * 4 * 512;           // scales of all 256 rows of B
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;   // 38 KiB
  static constexpr int kStagingBytes = 8 * 4096;           // epilogue: two buffers of 32 rows x 64 bytes for each of 8 warps
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 + 256;
  static constexpr int kThreads = 320;
};

// ---- cluster plumbing ------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Non-blocking test: a suspended try_wait is not woken early by an arrival that comes from the
// other SM, it sleeps out its whole time hint, so waits with remote arrivals poll instead.
__device__ __forceinline__ bool mbar_test_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// bounded wait on a local barrier whose arrivals may come from the peer CTA
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test_cluster(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_test_cluster(bar, parity)) return true;
    if ((i & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > kWaitLimitNs) return false;
    }
  }
}
// TMA tile load of this CTA whose completion bytes are counted by a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
// arrives on the barrier at this offset in both CTAs once every MMA issued so far has completed
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// One 512-byte scale tile (32 rows of 16 bytes, not swizzled; groups of 8 rows 128 bytes apart)
// from shared to tensor memory, replicated to the four 32-lane quarters, in both CTAs.
constexpr uint32_t kScaleDescHi = (128u >> 4) | (1u << 14);
__device__ __forceinline__ uint32_t scale_desc_lo(uint32_t saddr) { return (saddr & 0x3FFFFu) >> 4; }
__device__ __forceinline__ void tc_copy_scales_pair(uint32_t taddr, uint32_t desc_lo) {
  asm volatile("{ .reg .b64 d; mov.b64 d, {%1, %2}; tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d; }"
               ::"r"(taddr), "r"(desc_lo), "r"(kScaleDescHi) : "memory");
}
__device__ __forceinline__ void tc_mma_fp4_pair(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                                uint32_t sfa, uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %7, 0; mov.b64 da, {%1, %3}; mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %4, [%5], [%6], p; }"
      ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                                 uint32_t acc) {
  asm volatile(
      "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %5, 0; mov.b64 da, {%1, %3}; mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p; }"
      ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(acc) : "memory");
}

// ---- the kernel ---------------------------------------------------------------------------------------

template <typename TD>
__global__ void __launch_bounds__(PairCfg::kThreads, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_sfa, const __grid_constant__ CUtensorMap map_sfb,
                       const __grid_constant__ CUtensorMap map_t, const __grid_constant__ CUtensorMap map_u,
                       const __grid_constant__ CUtensorMap map_d, const GemmParams p) {
  using Cfg = PairCfg;
  constexpr int kStages = Cfg::kStages;
  constexpr int BN = Cfg::BN;

  extern __shared__ uint8_t smem_raw[];
  // the dynamic window starts at the same offset in both CTAs, so this rounding gives both the
  // same layout: descriptors and barrier offsets are valid across the pair
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* staging = smem + kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + Cfg::kStagingBytes);
  uint64_t* full = bars;                                   // [kStages]
  uint64_t* empty = bars + kStages;                        // [kStages]
  uint64_t* acc_full = bars + 2 * kStages;
  uint64_t* acc_release = bars + 2 * kStages + 1;
  uint64_t* drain = bars + 2 * kStages + 2;                // error path only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();                  // 0 = leader
  const int64_t pair = blockIdx.x >> 1;
  const int64_t num_pairs = gridDim.x >> 1;

  const int64_t tiles_m = (p.M + 2 * kBM - 1) / (2 * kBM);
  const int64_t tiles_n = (p.N + BN - 1) / BN;
  const int64_t num_tiles = tiles_m * tiles_n;
  const int k_iters = (int)((p.K + 255) / 256);
  const int r_iters = (p.rank + 63) / 64;
  const int iters = k_iters + r_iters;
  const int64_t sf_tiles_k = sf_tiles_per_row(p.K);        // scale tiles per 128-row block
  const int64_t a_row_blocks = (p.M + 127) / 128;
  const int64_t b_row_blocks = (p.N + 127) / 128;
  const int band = (p.debug & kDebugGroupMask) ? ((p.debug & kDebugGroupMask) >> 8) : 8;   // row tiles per band of the tile order

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_release, 16);
    mbar_init(drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();                                  // everything above touches shared and tensor memory only

  if (warp == 0) {
    // ===== TMA producer (both CTAs): every copy reports to the leader's barrier =====
    int stage = 0;
    uint32_t phase = 0;
    bool first = true;
    bool ok = true;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full_local = smem_u32(full);
    const uint32_t full_leader = map_to_cta(full_local, 0);
    for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      int64_t tm, tn;
      tile_coords(tile, tiles_m, tiles_n, band, tm, tn);
      const int32_t m0 = (int32_t)(tm * 2 * kBM + cta * kBM);         // this CTA's rows of A
      const int32_t n0 = (int32_t)(tn * BN);
      const int32_t nb0 = n0 + (int32_t)cta * 128;                    // this CTA's rows of B
      // a row block past the end of A (ragged M) has no scale tiles: read block 0 instead, its
      // rows are never stored
      const int64_t arb = ((int64_t)m0 >> 7) < a_row_blocks ? ((int64_t)m0 >> 7) : 0;
      const int32_t sfa_tile0 = (int32_t)(arb * sf_tiles_k);           // index of 512-byte scale tiles
      const int64_t rb0 = (int64_t)n0 >> 7;
      const int32_t sfb_tile0 = (int32_t)(rb0 * sf_tiles_k);
      const bool sfb_second = rb0 + 1 < b_row_blocks;
      const uint32_t k_bytes = 2 * (Cfg::kABytes + Cfg::kBBytes + Cfg::kSfaBytes + 2048 + (sfb_second ? 2048 : 0));
      for (int it = 0; it < iters; ++it) {
        ok = __all_sync(0xffffffffu, mbar_wait_cluster(&empty[stage], phase ^ 1u, abort_flag));
        if (!ok) {
          if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_MMA);
          break;
        }
        const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
        const uint32_t sb = sa + Cfg::kABytes;
        const uint32_t ssfa = sb + Cfg::kBBytes;
        const uint32_t ssfb = ssfa + Cfg::kSfaBytes;
        const uint32_t bar = full_leader + stage * 8;
        if (elect_one()) {
          if (p.debug & kDebugNoLoad) {
            if (cta == 0) mbar_arrive_addr(full_local + stage * 8);
          } else if (it < k_iters) {
            // the leader arms its barrier for the bytes of both CTAs
            const bool drop = first && (p.debug & kDebugDropFirstSfa);
            if (cta == 0) mbar_expect_tx_addr(full_local + stage * 8, k_bytes);
            tma_load_2d_pair(sa, &map_a, it * kBKBytes, m0, bar);
            tma_load_2d_pair(sb, &map_b, it * kBKBytes, nb0, bar);
            if (!drop) tma_load_2d_pair(ssfa, &map_sfa, 0, sfa_tile0 + it * 4, bar);
            tma_load_2d_pair(ssfb, &map_sfb, 0, sfb_tile0 + it * 4, bar);
            if (sfb_second) tma_load_2d_pair(ssfb + 2048, &map_sfb, 0, sfb_tile0 + (int32_t)sf_tiles_k + it * 4, bar);
          } else {
            const int j = it - k_iters;   // 64-column panel of the rank-r factors
            if (cta == 0) mbar_expect_tx_addr(full_local + stage * 8, 2 * (Cfg::kABytes + Cfg::kBBytes));
            tma_load_2d_pair(sa, &map_t, j * 64, m0, bar);
            tma_load_2d_pair(sb, &map_u, j * 64, nb0, bar);
          }
        }
        first = false;
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    grid_launch_dependents();                                // the last loads of this CTA are on their way: let the next kernel's CTAs in
  } else if (warp == 1) {
    // ===== tensor-core issuer (leader only) =====
    if (cta == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      bool issued = false;
      const uint32_t stage0_lo = operand_desc_lo(smem_u32(smem));
      const uint32_t empty_base = smem_u32(empty);
      uint32_t stage_lo = stage0_lo;
      uint32_t sf_buf = 0;
      const bool no_mma = (p.debug & kDebugNoMma) != 0;
#ifdef METIS_TIMING_KNOBS
      long long prof_full = 0, prof_release = 0, prof_t;
      const long long prof_start = clock64();
      const uint64_t prof_ns0 = global_ns();
#define METIS_PROF_BEGIN() prof_t = clock64()
#define METIS_PROF_END(acc) acc += clock64() - prof_t
#else
#define METIS_PROF_BEGIN()
#define METIS_PROF_END(acc)
#endif
      for (int64_t tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
        if (local_tile > 0) {
          METIS_PROF_BEGIN();
          ok = __all_sync(0xffffffffu, mbar_wait_cluster(acc_release, (local_tile - 1u) & 1u, abort_flag));
          METIS_PROF_END(prof_release);
          if (!ok) {
            if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_EPI);
            break;
          }
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (local_tile & 1u) * Cfg::kAccStride;
        for (int it = 0; it < iters; ++it) {
          const bool scaled = it < k_iters;
          METIS_PROF_BEGIN();
          ok = __all_sync(0xffffffffu, mbar_wait_cluster(&full[stage], phase, abort_flag));
          METIS_PROF_END(prof_full);
          if (!ok) {
            if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_TMA);
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = stage_lo;
          const uint32_t b_lo = stage_lo + (Cfg::kABytes >> 4);
          // scale tiles follow the code tiles in the stage; same low-half encoding (address >> 4)
          // without the leading-offset bit of the operand descriptors
          const uint32_t sf_lo = (stage_lo & 0x3FFFu) + ((Cfg::kABytes + Cfg::kBBytes) >> 4);
          const uint32_t t_sfa = tmem_base + kSfCol + sf_buf * kSfBufCols, t_sfb = t_sfa + 16;
          if (elect_one()) {
            if (no_mma) {
            } else if (scaled) {
              // Scales of this stage into buffer sf_buf (the MMAs that last read it were issued two
              // stages ago; copies and MMAs run in issue order): per MMA one tile of A and two of B.
              // The copies of MMA j+1 are issued behind MMA j, so that they run while it computes;
              // only the first three of a stage wait for nothing.
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (!(p.debug & kDebugNoScaleCopy)) {
                  tc_copy_scales_pair(t_sfa + 4 * j, sf_lo + 32 * j);
                  tc_copy_scales_pair(t_sfb + 8 * j, sf_lo + 128 + 32 * j);
                  tc_copy_scales_pair(t_sfb + 8 * j + 4, sf_lo + 256 + 32 * j);
                }
                tc_mma_fp4_pair(d_tmem, a_lo + 2 * j, b_lo + 2 * j, kOperandDescHi, idesc_fp4(BN, 2 * kBM), t_sfa + 4 * j,
                                t_sfb + 8 * j, (it > 0 || j > 0) ? 1u : 0u);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                tc_mma_bf16_pair(d_tmem, a_lo + 2 * j, b_lo + 2 * j, kOperandDescHi, idesc_bf16(BN, 2 * kBM), (it > 0 || j > 0) ? 1u : 0u);
              }
            }
            tc_commit_pair(empty_base + stage * 8);
            if (it == iters - 1) tc_commit_pair(smem_u32(acc_full));
          }
          issued = true;
          if (scaled) sf_buf ^= 1u;
          stage_lo += Cfg::kStageBytes >> 4;
          if (++stage == kStages) { stage = 0; phase ^= 1u; stage_lo = stage0_lo; }
        }
      }
#ifdef METIS_TIMING_KNOBS
      if ((p.debug & kDebugProfile) && p.status && blockIdx.x == 0 && lane == 0) {
        // drain the tensor pipe so that the total covers the last tile's MMAs
        tc_commit_pair(smem_u32(drain));
        while (!mbar_try(drain, 0) && global_ns() - prof_ns0 < kWaitLimitNs) {}
        p.status[2] = (int32_t)(clock64() - prof_start);
        p.status[3] = (int32_t)(global_ns() - prof_ns0);
        p.status[4] = (int32_t)prof_full;
        p.status[5] = (int32_t)prof_release;
        p.status[6] = (int32_t)local_tile;
      }
#endif
      if (!ok && issued && elect_one()) {
        // error path: let the tensor core finish what was issued before tensor memory is freed
        tc_commit_pair(smem_u32(drain));
        const uint64_t t0 = global_ns();
        while (!mbar_try(drain, 0) && global_ns() - t0 < kWaitLimitNs) {}
      }
      __syncwarp();
    }
  } else {
    // ===== epilogue (both CTAs): warps 2..9; warp w owns tensor-memory lanes 32*(w%4) .. +31 and,
    // of the 8 column chunks taken in drain order, those with index (w-2)/4, +2, +4, +6 =====
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t release_leader = map_to_cta(smem_u32(acc_release), 0);
    EpilogueCtx<TD> ctx;
    ctx.g = p.alpha * __ldg(p.a_unit) * __ldg(p.b_unit);
    ctx.p = &p;
    ctx.staging = staging + (warp - 2) * 4096;
    ctx.dmap = (p.debug & kDebugLsuStore) ? nullptr : &map_d;
    uint32_t local_tile = 0;
    for (int64_t tile = pair; tile < num_tiles; tile += num_pairs, ++local_tile) {
      int64_t tm, tn;
      tile_coords(tile, tiles_m, tiles_n, band, tm, tn);
      const int64_t row0 = tm * 2 * kBM + cta * kBM + q * 32;
      const int64_t row = row0 + lane;
      const int64_t n0 = tn * BN;
      ctx.row0 = row0;
      ctx.c0 = p.rvec0 ? (p.cvec0 ? (row < p.M ? __ldg(p.cvec0 + row) : 0.f) : 1.0f) : 0.0f;
      ctx.c1 = p.rvec1 ? (p.cvec1 ? (row < p.M ? __ldg(p.cvec1 + row) : 0.f) : 1.0f) : 0.0f;
      if (!mbar_wait_cluster(acc_full, local_tile & 1u, abort_flag)) {
        if (lane == 0) report(p.status, abort_flag, METIS_DEV_TIMEOUT_MMA);
        break;
      }
      tc_fence_after();
      const uint32_t odd = local_tile & 1u;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + odd * Cfg::kAccStride;
      // drain order: the 3 chunks shared with the other accumulator first.  For the even
      // accumulator [0,256) they are its last chunks, for the odd one [160,416) its first ones.
      constexpr int kChunks = BN / 32;
      const int first_chunk = !odd ? kChunks - Cfg::kSharedChunks : 0;
      int ch[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) ch[k] = (first_chunk + half + 2 * k) & (kChunks - 1);
      // this warp's first two chunks cover its part of the shared columns (drain index 0 and 2,
      // or 1): pull them into registers and hand the columns to the next tile's MMAs at once
      uint32_t ra[32], rb[32];
      tc_load32(t_row + ch[0] * 32, ra);
      tc_load32(t_row + ch[1] * 32, rb);
      tc_wait_ld(ra);
      tc_wait_ld(rb);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(release_leader);
      // the other two loads fly while the first two chunks are scaled and stored
      emit_chunk<TD>(ctx, ra, n0 + ch[0] * 32);
      tc_load32(t_row + ch[2] * 32, ra);
      emit_chunk<TD>(ctx, rb, n0 + ch[1] * 32);
      tc_load32(t_row + ch[3] * 32, rb);
      tc_wait_ld(ra);
      tc_wait_ld(rb);
      emit_chunk<TD>(ctx, ra, n0 + ch[2] * 32);
      emit_chunk<TD>(ctx, rb, n0 + ch[3] * 32);
      tc_fence_before();
    }
    if (lane == 0) bulk_store_wait_all();                    // shared memory stays until the TMA unit has read it
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // nobody signals or reads the peer after this
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- host side ----------------------------------------------------------------------------------------------

template <typename TD>
static int32_t launch_pair_t(const metis_gemm_args* a, const CUtensorMap* maps, const GemmParams& p) {
  auto kern = nvfp4_gemm_pair_kernel<TD>;
  METIS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairCfg::kSmemBytes));
  const int64_t tiles = ceil_div(a->M, 2 * kBM) * ceil_div(a->N, PairCfg::BN);
  int64_t pairs = gemm_sm_budget(a->sm_limit) / 2;
  if (pairs > tiles) pairs = tiles;
  // the fewest pairs that still finish in the same number of rounds: 256 tiles take 4 rounds on 74 pairs
  // and on 64, and the SMs left over are free for whatever runs beside this product
  pairs = ceil_div(tiles, ceil_div(tiles, pairs));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(PairCfg::kThreads, 1, 1);
  cfg.dynamicSmemBytes = PairCfg::kSmemBytes;
  cfg.stream = reinterpret_cast<cudaStream_t>(a->stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.numAttrs = launch_overlap_enabled(kLaunchGemm) ? 2 : 1;
  METIS_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], maps[6], p));
  return METIS_OK;
}

// Called by metis_nvfp4_gemm for M > 128 and N > 128.  ma and mt have 128-row boxes (this CTA's rows
// of A and T), mb and mu too (this CTA's half of the 256 rows of B and U).
int32_t launch_gemm_pair(const metis_gemm_args* a, const CUtensorMap& ma, const CUtensorMap& mb,
                         const CUtensorMap& mt, const CUtensorMap& mu, const GemmParams& p) {
  // the scale arrays as [tiles, 512 bytes]: one box = the 4 tiles (2 KiB) of one stage and row block
  const int64_t sf_tiles_k = sf_tiles_per_row(a->K);
  CUtensorMap maps[7] = {ma, mb, {}, {}, mt, mu, {}};
  if (int32_t rc = make_map(&maps[2], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a->a_scales, 128, ceil_div(a->M, 128) * sf_tiles_k, 512,
                            128, 4, "scales of A", 0)) return rc;
  if (int32_t rc = make_map(&maps[3], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, a->b_scales, 128, ceil_div(a->N, 128) * sf_tiles_k, 512,
                            128, 4, "scales of B", 0)) return rc;
  // D in boxes of 32 rows x 64 bytes for the epilogue's TMA stores
  if (a->d_dtype == METIS_DTYPE_BF16) {
    if (int32_t rc = make_map(&maps[6], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->d, a->N, a->M, a->ldd * 2, 32, 32, "D", 64)) return rc;
    return launch_pair_t<__nv_bfloat16>(a, maps, p);
  }
  if (int32_t rc = make_map(&maps[6], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->d, a->N, a->M, a->ldd * 4, 16, 32, "D", 64)) return rc;
  return launch_pair_t<float>(a, maps, p);
}

}  // namespace metis
