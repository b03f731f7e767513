// Pieces shared by the single-CTA and the CTA-pair NVFP4 GEMM kernels: tile constants, the
// parameter block, tcgen05 PTX wrappers, descriptors and the epilogue arithmetic.
#pragma once

#include "common.cuh"
#include "tma.cuh"

namespace metis {


constexpr int kBM = 128;             // rows of A per tile (the MMA M)
constexpr int kBKBytes = 128;        // bytes of packed codes per row per stage = 256 elements
constexpr int kGemmThreads = 320;     // producer, issuer, 4 epilogue warps, 4 scale-mover warps
constexpr int kTmemCols = 512;
// Scale columns in tensor memory: two buffers of 48 columns (16 for A, 32 for B), used by
// alternate pipeline iterations so that the copy for one iteration never has to wait for the
// MMAs of the previous one to finish reading.
constexpr int kSfCol = 416;
constexpr int kSfBufCols = 48;

// debug knob carried in metis_gemm_args.reserved: the producer arms the first stage's barrier
// for the scale bytes of A but never issues that copy, so the consumer's bounded wait expires.
constexpr int kDebugDropFirstSfa = 1;
// timing experiments (results are meaningless): issue no MMAs / request no data.  They exist only in a
// build with -DMETIS_TIMING_KNOBS; the shipped library rejects the bits (they are outside kDebugMask)
// and the code they guard is compiled out.
#ifdef METIS_TIMING_KNOBS
constexpr int kDebugNoMma = 2;
constexpr int kDebugNoLoad = 4;
constexpr int kDebugNoEpilogue = 16;     // accumulator chunks are read and dropped
constexpr int kDebugNoStore = 32;        // everything but the global stores of the epilogue
constexpr int kDebugLsuStore = 64;       // pair kernel: store D with ordinary store instructions instead of TMA
constexpr int kDebugProfile = 128;       // pair kernel: CTA 0's issuer writes its cycle counts to status[2..6]
constexpr int kDebugNoScaleCopy = 0x10000;   // pair kernel: the MMAs read whatever tensor memory holds as scales
constexpr int kDebugGroupMask = 0xFF00;  // pair kernel: row tiles per band of the tile order (0 = the default)
#else
constexpr int kDebugNoMma = 0;
constexpr int kDebugNoLoad = 0;
constexpr int kDebugNoEpilogue = 0;
constexpr int kDebugNoStore = 0;
constexpr int kDebugLsuStore = 0;
constexpr int kDebugProfile = 0;
constexpr int kDebugNoScaleCopy = 0;
constexpr int kDebugGroupMask = 0;
#endif
// run the single-CTA kernel where the CTA-pair kernel would be chosen (tests cover both)
constexpr int kDebugSingleCta = 8;
constexpr int kDebugMask = kDebugDropFirstSfa | kDebugNoMma | kDebugNoLoad | kDebugSingleCta | kDebugNoEpilogue | kDebugNoStore | kDebugLsuStore | kDebugGroupMask | kDebugProfile | kDebugNoScaleCopy;

template <int BN> struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  // Two accumulators.  256 + 256 columns do not fit beside the scale columns, so for BN = 256 the
  // second one starts at column 160: columns [160,256) belong to both.  The epilogue drains those
  // columns first and then lets the next tile's MMAs start while it drains the rest.
  static constexpr int kAccStride = (BN == 256) ? 160 : BN;
  static constexpr int kSharedChunks = (BN == 256) ? 3 : 0;     // 32-column chunks in the overlap
  static constexpr int kABytes = kBM * kBKBytes;                   // 16 KiB
  static constexpr int kBBytes = BN * kBKBytes;                    // 16 or 32 KiB
  static constexpr int kSfaBytes = 4 * 512;                        // 4 scale tiles (256 elements)
  static constexpr int kSfbBytes = (BN / 128) * 4 * 512;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStagingBytes = 4 * 2048;                   // epilogue: 32 rows x 64 bytes per warp
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

struct GemmParams {
  int64_t M, N, K;
  int32_t rank;
  int32_t debug;
  const uint8_t* a_scales;
  const uint8_t* b_scales;
  const float* a_unit;
  const float* b_unit;
  float alpha;
  const float* cvec0;  const float* rvec0;
  const float* cvec1;  const float* rvec1;
  const void* c;  int64_t ldc;
  void* d;        int64_t ldd;
  int32_t* status;
  // split-K (single-CTA kernel only): number of K splits, K iterations per split, partial sums
  // [splits, M, ldp] fp32; splits = 1 means none
  int32_t splits = 1;
  int32_t k_per_split = 1 << 30;
  float* partial = nullptr;
  int64_t ldp = 0;
};

// Tile order: bands of `group` row tiles; inside a band the row tile runs fastest, then the column
// tile.  The CTAs that run at the same time then share a few A row panels and walk the B column
// panels together, so both stay in L2 whatever M, N and K are (row tile fastest over the whole of M
// re-reads all of A from HBM once per column tile as soon as A outgrows L2).
__device__ __forceinline__ void tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int group, int64_t& tm, int64_t& tn) {
  const int64_t per_band = (int64_t)group * tiles_n;
  const int64_t band = tile / per_band, in_band = tile - band * per_band;
  const int64_t first = band * group;
  const int64_t rows = tiles_m - first < group ? tiles_m - first : group;
  tn = in_band / rows;
  tm = first + (in_band - tn * rows);
}

// ---- PTX wrappers ---------------------------------------------------------------------------------

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit_addr(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) { tc_commit_addr(smem_u32(bar)); }
// Operand descriptors are passed as two 32-bit halves: only the low half (the address field)
// changes from stage to stage, so the issuing thread advances it with one 32-bit add.
__device__ __forceinline__ void tc_mma_fp4(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                           uint32_t sfa, uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %7, 0; mov.b64 da, {%1, %3}; mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %4, [%5], [%6], p; }"
      ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                            uint32_t acc) {
  asm volatile(
      "{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %5, 0; mov.b64 da, {%1, %3}; mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p; }"
      ::"r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tc_load32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_store16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Same wait, with the destination registers of an earlier tc_load32 as operands: the compiler then
// cannot move a use of them above the wait, even when other work sits between the load and the wait.
__device__ __forceinline__ void tc_wait_ld(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :: "memory");
}

// Shared-memory matrix descriptors (64-bit): start address >> 4 in [0,14), leading byte offset
// >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48), swizzle
// mode in [61,64) (0 none, 2 = 128-byte).
// K-major operand tile stored as rows of 128 bytes, 128-byte swizzled: groups of 8 rows are
// 1024 bytes apart (stride field 64), leading field 1, version 1, swizzle mode 2.
constexpr uint32_t kOperandDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t operand_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
// Instruction descriptors (32-bit): formats of A [7,10) and B [10,13), N>>3 in [17,23),
// M>>4 in [24,29); both operands K-major.
__host__ __device__ constexpr uint32_t idesc_fp4(int bn, int bm = kBM) {
  // A, B = e2m1 (1); scale format UE4M3 (bit 23 = 0); scale ids 0; K = 64 (bit 31 = 0)
  return (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(bm >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_bf16(int bn, int bm = kBM) {
  // D = f32 (1 in [4,6)); A, B = bf16 (1)
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(bm >> 4) << 24);
}

__device__ __forceinline__ void report(int32_t* status, volatile int* abort_flag, int32_t code) {
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
}

// ---- epilogue arithmetic for one 32-column chunk of one accumulator row -----------------------------

template <typename TD> struct EpilogueCtx {
  const GemmParams* p;
  uint8_t* staging;      // 2 KiB of shared memory owned by this warp
  int64_t row0;          // first of the warp's 32 rows; lane l holds row0 + l
  float g, c0, c1;
  float* partial = nullptr;   // split-K: raw fp32 partial sums [M, ldp] of this split go here instead of D
  int64_t ldp = 0;
  const CUtensorMap* dmap = nullptr;   // D as [M, N] with 32-row x 64-byte boxes, 64-byte swizzle: stores go through the TMA unit
  uint32_t flip = 0;                   //   and `staging` is then two buffers of 2 KiB used in turn
};

// v[i] += c * rvec[col0 + i] for the 32 columns of a chunk (128-bit loads when the chunk is whole
// and the vector 16-byte aligned; every lane reads the same addresses)
__device__ __forceinline__ void add_rank1(float (&v)[32], const float* __restrict__ rvec, float c, int64_t col0,
                                          int64_t N, bool full_chunk) {
  if (!rvec) return;
  if (full_chunk && (reinterpret_cast<uintptr_t>(rvec) & 15u) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(rvec + col0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 f = __ldg(r4 + i);
      v[4 * i] = fmaf(c, f.x, v[4 * i]);
      v[4 * i + 1] = fmaf(c, f.y, v[4 * i + 1]);
      v[4 * i + 2] = fmaf(c, f.z, v[4 * i + 2]);
      v[4 * i + 3] = fmaf(c, f.w, v[4 * i + 3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) if (full_chunk || col0 + i < N) v[i] = fmaf(c, __ldg(rvec + col0 + i), v[i]);
  }
}

// The addend C for the 32 columns of a chunk (src = this lane's row of C at the chunk, or null).
template <typename TD>
__device__ __forceinline__ void add_c(float (&v)[32], const TD* __restrict__ src, int64_t col0, int64_t N, bool full_chunk) {
  if (!src) return;
  if (!full_chunk) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (col0 + i < N) {
        if constexpr (sizeof(TD) == 2) v[i] += __bfloat162float(src[i]); else v[i] += src[i];
      }
    return;
  }
  if constexpr (sizeof(TD) == 2) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(src) + i);
      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) { v[8 * i + 2 * k] += bf16_lo(ww[k]); v[8 * i + 2 * k + 1] += bf16_hi(ww[k]); }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 w = __ldg(reinterpret_cast<const float4*>(src) + i);
      v[4 * i] += w.x; v[4 * i + 1] += w.y; v[4 * i + 2] += w.z; v[4 * i + 3] += w.w;
    }
  }
}

// Lane l arrives with 32 consecutive columns of row row0 + l.  Stored straight from there, one
// 16-byte store instruction would touch 32 different rows; instead the warp turns the chunk
// through shared memory: 64-byte rows, 16-byte pieces XOR-swizzled by the row (the 64-byte swizzle
// pattern of the tensor maps), so that neither side has bank conflicts.
//   with a tensor map of D (ctx.dmap): lane 0 hands each 32 x 64-byte piece to the TMA unit, which
//     clips it at the edges of D.  The warp owns two such buffers and waits, before it refills one,
//     until the store issued from it two pieces ago has read it; the stores never pass through
//     the load/store unit, which the operand feed of the tensor core needs
//   without: every store instruction writes 64 contiguous bytes of 8 rows
template <typename TD>
__device__ __forceinline__ void emit_chunk(EpilogueCtx<TD>& ctx, const uint32_t (&r)[32], int64_t col0) {
  const GemmParams& p = *ctx.p;
  const int lane = threadIdx.x & 31;
  const int64_t row = ctx.row0 + lane;
  if (ctx.row0 >= p.M || col0 >= p.N) return;          // warp-uniform
  if (p.debug & kDebugNoEpilogue) return;
  const bool live = row < p.M;
  if (ctx.partial) {                                   // warp-uniform; ldp is a multiple of 32: the chunk fits
    if (live) {
      float4* dst = reinterpret_cast<float4*>(ctx.partial + row * ctx.ldp + col0);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
    }
    return;
  }
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * ctx.g;
  const bool full_chunk = col0 + 32 <= p.N;
  add_rank1(v, p.rvec0, ctx.c0, col0, p.N, full_chunk);
  add_rank1(v, p.rvec1, ctx.c1, col0, p.N, full_chunk);
  const TD* src = (p.c && live) ? static_cast<const TD*>(p.c) + row * p.ldc + col0 : nullptr;
  const int own_swz = (lane >> 1) & 3;
  if (ctx.dmap) {                                      // warp-uniform
    add_c<TD>(v, src, col0, p.N, full_chunk);
    constexpr int kPieces = sizeof(TD) == 2 ? 1 : 2;   // 64-byte wide pieces per chunk
#pragma unroll
    for (int h = 0; h < kPieces; ++h) {
      uint8_t* buf = ctx.staging + ctx.flip * 2048;
      ctx.flip ^= 1u;
      if (lane == 0) bulk_store_wait_read<1>();
      __syncwarp();
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint4 w;
        if constexpr (sizeof(TD) == 2) {
          __nv_bfloat162 o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(v[8 * k + 2 * e], v[8 * k + 2 * e + 1]);
          w = *reinterpret_cast<uint4*>(o);
        } else {
          w = make_uint4(__float_as_uint(v[16 * h + 4 * k]), __float_as_uint(v[16 * h + 4 * k + 1]),
                         __float_as_uint(v[16 * h + 4 * k + 2]), __float_as_uint(v[16 * h + 4 * k + 3]));
        }
        *reinterpret_cast<uint4*>(buf + lane * 64 + ((k ^ own_swz) << 4)) = w;
      }
      fence_async_shared();
      __syncwarp();
      if (lane == 0 && !(p.debug & kDebugNoStore))
        tma_store_2d(ctx.dmap, smem_u32(buf), (int32_t)col0 + h * 16, (int32_t)ctx.row0);
    }
    return;
  }
  if (full_chunk) {
    add_c<TD>(v, src, col0, p.N, true);
    if constexpr (sizeof(TD) == 2) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        __nv_bfloat162 o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = __floats2bfloat162_rn(v[8 * k + 2 * e], v[8 * k + 2 * e + 1]);
        *reinterpret_cast<uint4*>(ctx.staging + lane * 64 + ((k ^ own_swz) << 4)) = *reinterpret_cast<uint4*>(o);
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int rl = 8 * i + (lane >> 2), j = lane & 3;
        const uint4 w = *reinterpret_cast<const uint4*>(ctx.staging + rl * 64 + ((j ^ ((rl >> 1) & 3)) << 4));
        if (ctx.row0 + rl < p.M && !(p.debug & kDebugNoStore))
          *reinterpret_cast<uint4*>(static_cast<TD*>(p.d) + (ctx.row0 + rl) * p.ldd + col0 + j * 8) = w;
      }
      __syncwarp();
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {                     // 16 columns = 64 bytes per row at a time
#pragma unroll
        for (int k = 0; k < 4; ++k)
          *reinterpret_cast<float4*>(ctx.staging + lane * 64 + ((k ^ own_swz) << 4)) =
              make_float4(v[16 * h + 4 * k], v[16 * h + 4 * k + 1], v[16 * h + 4 * k + 2], v[16 * h + 4 * k + 3]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rl = 8 * i + (lane >> 2), j = lane & 3;
          const float4 w = *reinterpret_cast<const float4*>(ctx.staging + rl * 64 + ((j ^ ((rl >> 1) & 3)) << 4));
          if (ctx.row0 + rl < p.M)
            *reinterpret_cast<float4*>(static_cast<TD*>(p.d) + (ctx.row0 + rl) * p.ldd + col0 + 16 * h + j * 4) = w;
        }
        __syncwarp();
      }
    }
  } else if (live) {
    TD* dst = static_cast<TD*>(p.d) + row * p.ldd + col0;
    for (int i = 0; i < 32 && col0 + i < p.N; ++i) {
      float o = v[i];
      if constexpr (sizeof(TD) == 2) {
        if (src) o += __bfloat162float(src[i]);
        dst[i] = __float2bfloat16_rn(o);
      } else {
        if (src) o += src[i];
        dst[i] = o;
      }
    }
  }
}

}  // namespace metis
