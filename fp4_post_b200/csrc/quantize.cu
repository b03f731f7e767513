// NVFP4 block quantizer kernels (row-major, transposed and both at once, round-to-nearest and stochastic),
// the scale finalisation pass, column means, and the C entry points that launch them.
//
// The work is split in two launches because of one global dependency: the E4M3 block
// scales are expressed relative to the tensor-wide maximum block scale, while the 4-bit
// codes only depend on their own block.  Pass 1 streams x once, writes the packed codes and
// the fp32 block maxima, and folds the global maximum with one atomicMax per warp.  Pass 2
// touches 1/16 of the elements: it turns the block maxima into E4M3 bytes in the layout the
// consumer wants and publishes the per-tensor unit.
#include "common.cuh"
#include "tma.cuh"

#include <mutex>

namespace metis {

constexpr int kQuantThreads = 256;
constexpr int kHeaderBytes = kWorkspaceHeaderBytes;

__device__ __forceinline__ void fold_global_max(unsigned int* gmax, float local) {
  // amax >= 0, so the IEEE bit pattern orders like the value.
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, o));
  const unsigned tid = threadIdx.y * blockDim.x + threadIdx.x;
  if ((tid & 31u) == 0 && local > 0.0f) atomicMax(gmax, __float_as_uint(local));
}

// ---- pass 1, row-major ------------------------------------------------------------------------
// One thread owns one 16-element block (two 128-bit loads for bf16): no cross-lane traffic, one
// 64-bit store of codes and one 32-bit store of the block maximum, both coalesced across the warp.
// Thread (tx, ty) of a bx x by CTA walks the rows ty, ty + by*gridDim.y, ... of its fixed column
// block, so there is no division in the loop and the column means stay in registers.
template <typename T, bool kMean, bool kSR>
__global__ void __launch_bounds__(kQuantThreads)
quantize_rows_kernel(const T* __restrict__ x, int rows, int blocks_per_row, int64_t ld,
                     const float* __restrict__ col_mean, uint64_t seed, uint64_t offset,
                     const uint64_t* __restrict__ offset_ctr, uint2* __restrict__ codes, float* __restrict__ amax_out,
                     unsigned int* __restrict__ gmax, uint32_t sr16) {
  grid_dependency_wait();
  if (kSR && offset_ctr) offset += *offset_ctr;             // per-device call counter (graph-safe stream of offsets)
  const int bc = blockIdx.x * blockDim.x + threadIdx.x;     // column block of this thread
  const int row_step = gridDim.y * blockDim.y;
  float running = 0.0f;
  if (bc < blocks_per_row) {
    float m[16];
    if (kMean) Load16<float>::load(col_mean + (int64_t)bc * 16, m);
    const Philox rng(seed);
    auto quantize_block = [&](float (&v)[16], int r) {
      if (kMean) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __fsub_rn(v[i], m[i]);
      }
      const float a = abs_max16(v);
      const float s = block_scale_from_amax(a);
      const int64_t b = (int64_t)r * blocks_per_row + bc;
      uint32_t packed[2];
      if (kSR) {
        if (sr16) quantize16_sr(v, s, rng((uint64_t)b, offset), packed);      // one counter per block
        else quantize16_sr_hw(v, s, rng((uint64_t)b, offset), packed);
      } else {
        quantize_rn<2>(v, s, packed);
      }
      codes[b] = make_uint2(packed[0], packed[1]);
      amax_out[b] = a;
      running = fmaxf(running, a);
    };
    // the next row's loads are issued before the current block is worked on
    int r = blockIdx.y * blockDim.y + threadIdx.y;
    RawBlock<T> cur, nxt;
    if (r < rows) cur.load(x + (int64_t)r * ld + (int64_t)bc * 16);
    for (; r < rows; r += row_step) {
      const int rn = r + row_step;
      if (rn < rows) nxt.load(x + (int64_t)rn * ld + (int64_t)bc * 16);
      float v[16];
      cur.unpack(v);
      quantize_block(v, r);
      cur = nxt;
    }
  }
  // whole warps reach this point together: a warp never spans the bc bound unevenly in y
  fold_global_max(gmax, running);
}

// ---- pass 1 on shared-memory tiles: the transposed quantization, alone or together with the row-major one ----
// Output Qt = quantize(x^T): blocks of 16 run along the rows of x.  A persistent CTA walks tiles of
// 128 rows x 128 bytes of x (64 bf16 or 32 fp32 columns) that one thread fetches with TMA (128-byte
// swizzle) into a ring of three stages, two tiles ahead of the arithmetic.
//   column phase  lane w of warp rb reads word w of the 16 rows of row block rb: one (fp32) or two (bf16)
//                 columns of x, i.e. whole blocks of Qt, quantized in registers like a row block.  The 8
//                 code bytes per block are parked in shared memory so that global stores are 64-byte
//                 runs along the token dimension.
//   row phase     (kRowsOut: the "dual" mode) the same tile is read once more along its rows, 16 columns
//                 per thread, and the row-major quantization goes straight to global memory.  The tensor
//                 is read from HBM once for both orientations.
// Both phases read shared memory without bank conflicts thanks to the swizzle (16-byte chunk c of row
// r sits at chunk c ^ (r & 7)).  One __syncthreads per tile: staging and the column means are double
// buffered.  A tile load that does not arrive within the wait limit raises the error word of the
// workspace header (the scale pass then publishes NaN as the unit) instead of hanging.
template <typename T> struct TileCfg {
  static constexpr int kRows = 128;
  static constexpr int kCols = 128 / sizeof(T);            // 64 (bf16) or 32 (fp32): 128 bytes per row
  static constexpr int kStages = 3;
  static constexpr int kStageBytes = kRows * 128;          // 16 KiB
  static constexpr int kRowBlocks = kRows / 16;            // 8 = warps per CTA
  static constexpr int kColsPerWord = 4 / sizeof(T);       // columns in one 32-bit word of a row: 2 or 1
  static constexpr int kBlocksPerRow = kCols / 16;         // row-phase blocks per tile row: 4 or 2
  static constexpr int kRowUnits = kRows * kBlocksPerRow / kQuantThreads;   // row-phase blocks per thread: 2 or 1
  // staged codes of Qt: per 32-bit word of a row and per column of that word, 64 bytes (128 tokens) at a
  // pitch of 72; the second column's array starts 16 banks off the first
  static constexpr int kCodePitch = 72;
  static constexpr int kCodeArray = 32 * kCodePitch + 64;
  static constexpr int kStagingBytes = kColsPerWord * kCodeArray + kRowBlocks * kCols * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + 2 * kStagingBytes + 2 * kCols * 4 + 64 + 1024;
};
constexpr int64_t kTileRowsMinElements = 1 << 20;          // row-major tensors from this size on go through the tile kernel
constexpr uint64_t kColumnStream = 1ull << 63;             // Philox counter space of the transposed output in dual mode

// Workspace of the dual quantizer: word 63 = number of CTA records, records from word 64 on (3 words per CTA),
// then the block maxima of Q and of Qt.
constexpr int kDualMaxCtas = 640;
constexpr int kDualHeaderBytes = 256 + ((kDualMaxCtas * 3 * 4 + 255) / 256) * 256;

struct TileOutputs {
  uint8_t* codes_t;  float* amax_t;  unsigned int* gmax_t;        // Qt [cols, rows]
  uint8_t* codes_r;  float* amax_r;  unsigned int* gmax_r;        // Q  [rows, cols] (dual mode)
  unsigned int* error;
  // dual mode: instead of folding into the three header words above (which somebody has to zero first), CTA b
  // leaves {largest maximum of Q, of Qt, error} in records[3b..3b+2] and CTA 0 the number of CTAs in records[-1]
  unsigned int* records;
  uint32_t hadamard;         // bit 16: rotate every 16-row block of Qt first; bits [0, 16): the sign of each row
  uint32_t sr16;             // stochastic rounding in software with 16 random bits per element instead of the hardware conversion's 8
};

// y = H (s . v) for one block of 16 values: the signs flip as the mask says, then the 16-point Walsh-Hadamard
// butterfly in natural (Sylvester) order, fp32 additions in this fixed order (bitlinear.py:75-211: the random
// Hadamard transform of the NVIDIA baseline, x -> (x . signs) H per tile of 16, H unnormalised).
__device__ __forceinline__ void hadamard16(float (&v)[16], uint32_t sign_mask) {
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(__float_as_uint(v[i]) ^ (((sign_mask >> i) & 1u) << 31));
#pragma unroll
  for (int h = 1; h < 16; h <<= 1) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if ((i & h) == 0) {
        const float a = v[i], b = v[i + h];
        v[i] = __fadd_rn(a, b);
        v[i + h] = __fsub_rn(a, b);
      }
    }
  }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

template <typename T, bool kMean, bool kSR, bool kRowsOut, bool kColsOut>
__global__ void __launch_bounds__(kQuantThreads, 3)
quantize_tile_kernel(const __grid_constant__ CUtensorMap map_x, int64_t rows, int64_t cols,
                     const float* __restrict__ col_mean, uint64_t seed, uint64_t offset,
                     const uint64_t* __restrict__ offset_ctr, const TileOutputs out) {
  using TC = TileCfg<T>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* s_staging = smem + TC::kStages * TC::kStageBytes;                    // [2][kStagingBytes]
  float* s_mean = reinterpret_cast<float*>(s_staging + 2 * TC::kStagingBytes);  // [2][kCols]
  uint64_t* full = reinterpret_cast<uint64_t*>(s_mean + 2 * TC::kCols);         // [kStages]
  __shared__ int s_failed;

  grid_dependency_wait();
  if (kSR && offset_ctr) offset += *offset_ctr;
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int64_t row_tiles = (rows + TC::kRows - 1) / TC::kRows;
  const int64_t col_tiles = (cols + TC::kCols - 1) / TC::kCols;
  const int64_t tiles = row_tiles * col_tiles;       // tile id = row tile * col_tiles + column tile
  const int64_t bpr = cols >> 4;                     // blocks per row of Q
  const int64_t bpc = rows >> 4;                     // blocks per row of Qt

  if (tid == 0) {
    for (int s = 0; s < TC::kStages; ++s) mbar_init(&full[s], 1);
    s_failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  auto fill_mean = [&](int64_t tile, int buf) {
    if (kMean && tid < TC::kCols) {
      const int64_t c = (tile % col_tiles) * TC::kCols + tid;
      s_mean[buf * TC::kCols + tid] = c < cols ? __ldg(col_mean + c) : 0.0f;
    }
  };
  if ((int64_t)blockIdx.x < tiles) fill_mean(blockIdx.x, 0);
  __syncthreads();

  auto issue = [&](int64_t tile, int stage) {
    const int64_t rt = tile / col_tiles, ct = tile - rt * col_tiles;
    mbar_expect_tx(&full[stage], TC::kStageBytes);
    tma_load_2d(smem + stage * TC::kStageBytes, &map_x, (int32_t)(ct * TC::kCols), (int32_t)(rt * TC::kRows), &full[stage]);
  };
  if (tid == 0) {
    for (int s = 0; s < TC::kStages; ++s) {
      const int64_t t = (int64_t)blockIdx.x + (int64_t)s * gridDim.x;
      if (t < tiles) issue(t, s);
    }
  }

  const Philox rng(seed);
  float running_t = 0.0f, running_r = 0.0f;
  const uint32_t smem_base = smem_u32(smem);
  // column phase: this lane's word of a row, as chunk and offset inside the chunk
  const uint32_t word_chunk = (uint32_t)lane >> 2, word_in_chunk = ((uint32_t)lane & 3u) * 4u;
  volatile int* failed = &s_failed;
  int stage = 0;
  uint32_t it = 0;
  for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
    const int buf = it & 1;
    if (!mbar_wait(&full[stage], (it / TC::kStages) & 1u, failed)) *failed = 1;
    if (*failed) break;                               // every thread sees the same outcome of the barrier, or the flag

    const int64_t rt = tile / col_tiles, ct = tile - rt * col_tiles;
    const int64_t row0 = rt * TC::kRows, col0 = ct * TC::kCols;
    const uint32_t tile_smem = smem_base + stage * TC::kStageBytes;
    uint8_t* staging = s_staging + buf * TC::kStagingBytes;
    float* s_amax = reinterpret_cast<float*>(staging + TC::kColsPerWord * TC::kCodeArray);   // [kRowBlocks][kCols]
    const float* mean = s_mean + buf * TC::kCols;

    // ---- column phase: warp = row block, lane = 32-bit word of the row ----
    if (kColsOut) {
      const int rb = warp;
      float v[TC::kColsPerWord][16];
      float m[TC::kColsPerWord];
#pragma unroll
      for (int c = 0; c < TC::kColsPerWord; ++c) m[c] = kMean ? mean[lane * TC::kColsPerWord + c] : 0.0f;
      const uint32_t row_base = tile_smem + (uint32_t)(rb * 16) * 128u + word_in_chunk;
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const uint32_t w = lds32(row_base + r * 128 + ((word_chunk ^ (uint32_t)(r & 7)) << 4));
        if constexpr (sizeof(T) == 2) { v[0][r] = bf16_lo(w); v[1][r] = bf16_hi(w); }
        else                          { v[0][r] = __uint_as_float(w); }
        if (kMean) {
#pragma unroll
          for (int c = 0; c < TC::kColsPerWord; ++c) v[c][r] = __fsub_rn(v[c][r], m[c]);
        }
      }
      const bool rows_live = row0 + rb * 16 < rows;
      float amax[TC::kColsPerWord];
#pragma unroll
      for (int c = 0; c < TC::kColsPerWord; ++c) {
        if (out.hadamard) hadamard16(v[c], out.hadamard & 0xFFFFu);           // uniform over the grid
        const int64_t out_row = col0 + lane * TC::kColsPerWord + c;           // row of Qt = column of x
        const float a = abs_max16(v[c]);
        const float s = block_scale_from_amax(a);
        uint32_t packed[2];
        if (kSR) {
          const uint64_t b = (uint64_t)out_row * (uint64_t)bpc + (uint64_t)((row0 >> 4) + rb);
          const uint4 bits = rng(b, kRowsOut ? (offset ^ kColumnStream) : offset);                // alone: the transposed call's own stream
          if (out.sr16) quantize16_sr(v[c], s, bits, packed);
          else quantize16_sr_hw(v[c], s, bits, packed);
        } else {
          quantize_rn<2>(v[c], s, packed);
        }
        *reinterpret_cast<uint2*>(staging + c * TC::kCodeArray + lane * TC::kCodePitch + rb * 8) = make_uint2(packed[0], packed[1]);
        amax[c] = a;
        if (rows_live && out_row < cols) running_t = fmaxf(running_t, a);
      }
      if constexpr (sizeof(T) == 2) *reinterpret_cast<float2*>(s_amax + rb * TC::kCols + 2 * lane) = make_float2(amax[0], amax[1]);
      else                          s_amax[rb * TC::kCols + lane] = amax[0];
    }

    // ---- row phase: a thread owns blocks (row, b) with b fixed, straight to global memory ----
    if (kRowsOut) {
      const int b = tid & (TC::kBlocksPerRow - 1);
      const bool cols_live = col0 + b * 16 < cols;
      float mb[16];
      if (kMean) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 f = *reinterpret_cast<const float4*>(mean + b * 16 + 4 * i);
          mb[4 * i] = f.x; mb[4 * i + 1] = f.y; mb[4 * i + 2] = f.z; mb[4 * i + 3] = f.w;
        }
      }
#pragma unroll
      for (int u = 0; u < TC::kRowUnits; ++u) {
        const int r = (tid + u * kQuantThreads) / TC::kBlocksPerRow;
        const uint32_t row_addr = tile_smem + (uint32_t)r * 128u;
        const uint32_t swz = (uint32_t)(r & 7);
        RawBlock<T> raw;
        if constexpr (sizeof(T) == 2) {
          raw.a = lds128(row_addr + (((uint32_t)(2 * b) ^ swz) << 4));
          raw.b = lds128(row_addr + (((uint32_t)(2 * b + 1) ^ swz) << 4));
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint4 w = lds128(row_addr + (((uint32_t)(4 * b + k) ^ swz) << 4));
            raw.q[k] = make_float4(__uint_as_float(w.x), __uint_as_float(w.y), __uint_as_float(w.z), __uint_as_float(w.w));
          }
        }
        float v[16];
        raw.unpack(v);
        if (kMean) {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __fsub_rn(v[i], mb[i]);
        }
        const float a = abs_max16(v);
        const float s = block_scale_from_amax(a);
        const int64_t blk = (row0 + r) * bpr + (col0 >> 4) + b;
        uint32_t packed[2];
        if (kSR) {
          if (out.sr16) quantize16_sr(v, s, rng((uint64_t)blk, offset), packed);
          else quantize16_sr_hw(v, s, rng((uint64_t)blk, offset), packed);
        }
        else     quantize_rn<2>(v, s, packed);
        if (cols_live && row0 + r < rows) {
          reinterpret_cast<uint2*>(out.codes_r)[blk] = make_uint2(packed[0], packed[1]);
          out.amax_r[blk] = a;
          running_r = fmaxf(running_r, a);
        }
      }
    }

    const int64_t next = tile + gridDim.x;
    if (next < tiles) fill_mean(next, buf ^ 1);        // its last readers passed the previous barrier
    __syncthreads();                                   // staging complete; this tile's stage is free
    if (tid == 0) {
      const int64_t ahead = tile + (int64_t)TC::kStages * gridDim.x;
      if (ahead < tiles) issue(ahead, stage);
    }

    // ---- write-out of Qt: out row j owns 64 contiguous code bytes and 8 maxima of this tile ----
    const int64_t valid_rows = min((int64_t)TC::kRows, rows - row0);            // multiple of 16
#pragma unroll
    for (int k = 0; kColsOut && k < TC::kCols * 8 / kQuantThreads; ++k) {                   // 8-byte pieces: 8 per out row
      const int i = tid + k * kQuantThreads;
      const int j = i >> 3, piece = i & 7;
      const int64_t orow = col0 + j;
      if (orow < cols && piece * 16 < valid_rows)
        *reinterpret_cast<uint2*>(out.codes_t + orow * (rows >> 1) + (row0 >> 1) + piece * 8) =
            *reinterpret_cast<const uint2*>(staging + (j % TC::kColsPerWord) * TC::kCodeArray + (j / TC::kColsPerWord) * TC::kCodePitch + piece * 8);
    }
    if (kColsOut && tid < TC::kCols * 2) {
      const int j = tid & (TC::kCols - 1), h = tid / TC::kCols;                 // half h: row blocks 4h .. 4h+3
      const int64_t orow = col0 + j;
      if (orow < cols) {
        float* dst = out.amax_t + orow * bpc + (row0 >> 4) + 4 * h;
        float a4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) a4[k] = s_amax[(4 * h + k) * TC::kCols + j];
        if (valid_rows == TC::kRows && (bpc & 3) == 0) {
          *reinterpret_cast<float4*>(dst) = make_float4(a4[0], a4[1], a4[2], a4[3]);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) if ((4 * h + k) * 16 < valid_rows) dst[k] = a4[k];
        }
      }
    }
    if (++stage == TC::kStages) stage = 0;
  }
  if (s_failed) {
    // loads of this CTA may still be in flight: give each a bounded chance to land before the CTA leaves
    if (tid == 0) {
      int st = stage;
      for (int64_t t = blockIdx.x + (int64_t)it * gridDim.x, k = 0; t < tiles && k < TC::kStages; t += gridDim.x, ++k) {
        const uint64_t t0 = global_ns();
        while (!mbar_try(&full[st], ((it + k) / TC::kStages) & 1u) && global_ns() - t0 < kWaitLimitNs) {}
        if (++st == TC::kStages) st = 0;
      }
      if (!out.records) *out.error = 1u;               // error word of the workspace header
    }
  }
  if (out.records) {
    // every CTA writes its record, so nothing needs zeroing and no two CTAs touch the same word
    __shared__ float2 s_max[kQuantThreads / 32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      running_r = fmaxf(running_r, __shfl_xor_sync(0xffffffffu, running_r, o));
      running_t = fmaxf(running_t, __shfl_xor_sync(0xffffffffu, running_t, o));
    }
    if (lane == 0) s_max[warp] = make_float2(running_r, running_t);
    __syncthreads();
    if (tid == 0) {
      float2 m = s_max[0];
      for (int w = 1; w < kQuantThreads / 32; ++w) { m.x = fmaxf(m.x, s_max[w].x); m.y = fmaxf(m.y, s_max[w].y); }
      unsigned int* rec = out.records + 3 * (int64_t)blockIdx.x;
      rec[0] = __float_as_uint(m.x);
      rec[1] = __float_as_uint(m.y);
      rec[2] = s_failed ? 1u : 0u;
      if (blockIdx.x == 0) out.records[-1] = gridDim.x;
    }
    return;
  }
  if (kColsOut) fold_global_max(out.gmax_t, running_t);
  if (kRowsOut) fold_global_max(out.gmax_r, running_r);
}

// ---- pass 2: block maxima -> E4M3 bytes + unit ------------------------------------------------------
// One thread per group of 4 scale columns (one 128-bit read of maxima, one 32-bit write).
// For METIS_SF_MMA the loop runs over the padded extent and pads with zero bytes.  blockIdx.y picks
// the job: the dual quantizer finishes both orientations in one launch.
struct FinalizeJob {
  const float* amax;  const unsigned int* gmax;  const unsigned int* error;
  int64_t R, sf_cols;
  int32_t sf_layout;
  uint8_t* scales;  float* unit;
  int32_t bx;                 // threads along a row of groups (a power of two up to the CTA size)
  // optional by-product: row_sums[r] = the sum of the quantized values of row r (unit included), from the
  // codes the first pass wrote.  A weight-gradient product needs these sums of its operands when they
  // were centred; here they cost one extra read of codes that are still in L2 instead of a pass of their own.
  const uint2* codes;  float* row_sums;
  // per-CTA records of the dual quantizer (see TileOutputs) in place of gmax / error: word `which` of each is the maximum
  const unsigned int* records;  int32_t which;
};
struct FinalizeJobs { FinalizeJob job[2]; };

// E4M3 bytes of 4 neighbouring blocks from their maxima (quant.py:23): RN_e4m3(RN_fp32(s / unit)), two packed
// conversions.  The division is replaced by a product with RN(1 / unit), which lies within 3 fp32 steps of the
// correctly rounded quotient; the E4M3 byte of a normal value changes only where the 20 dropped mantissa bits
// pass 0x80000 (the tie), so a product further than that from a tie converts to the same byte.  The others,
// everything in E4M3's subnormal range (other tie positions) and NaN take the division itself.
__device__ __forceinline__ uint32_t scale_bytes4(const float (&a)[4], int live, float unit, float inv_unit) {
  float ratio[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float s = block_scale_from_amax(a[j]);
    float q = __fmul_rn(s, inv_unit);
    const uint32_t low = __float_as_uint(q) & 0xFFFFFu;
    if (low - 0x7FFF8u <= 16u || !(q >= 0.0157f)) q = __fdiv_rn(s, unit);
    ratio[j] = j < live ? q : 0.0f;
  }
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(ratio[0], ratio[1]), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(ratio[2], ratio[3]), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// the four E4M3 bytes of a word as floats (exact)
__device__ __forceinline__ void e4m3x4_to_float(uint32_t packed, float (&f)[4]) {
  const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(packed & 0xFFFFu), __NV_E4M3);
  const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(packed >> 16), __NV_E4M3);
  const float2 l = __half22float2(__half2(lo)), h = __half22float2(__half2(hi));
  f[0] = l.x; f[1] = l.y; f[2] = h.x; f[3] = h.y;
}

// Thread (tx, ty) of a bx x by CTA (bx per job) walks the groups tx, tx + bx, ... of the rows ty,
// ty + by * gridDim.x, ...: no index divisions, and two rows are in flight per thread.
__global__ void __launch_bounds__(kQuantThreads)
finalize_scales_kernel(const FinalizeJob job0, const FinalizeJob job1, uint64_t* __restrict__ offset_ctr) {
  __shared__ float2 s_sum[kQuantThreads / 32];
  grid_dependency_wait();
  const FinalizeJob& J = blockIdx.y == 0 ? job0 : job1;
  const int bx = J.bx, by = kQuantThreads / bx;
  const int tx = threadIdx.x & (bx - 1), ty = threadIdx.x / bx;
  const float* __restrict__ amax = J.amax;
  uint8_t* __restrict__ scales = J.scales;
  const int64_t R = J.R, sf_cols = J.sf_cols;
  const bool tiled = J.sf_layout == METIS_SF_MMA;
  unsigned int top = 0u, bad = 0u;                 // bits of the largest block maximum (>= 0: they order like the value)
  if (J.records) {
    __shared__ unsigned int s_top[2];
    if (threadIdx.x < 32) {                        // one warp reads the few KiB of records (L2) for the CTA
      const int n = (int)J.records[-1];
      for (int i = threadIdx.x; i < n; i += 32) {
        top = max(top, J.records[3 * i + J.which]);
        bad |= J.records[3 * i + 2];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        top = max(top, __shfl_xor_sync(0xffffffffu, top, o));
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
      }
      if (threadIdx.x == 0) { s_top[0] = top; s_top[1] = bad; }
    }
    __syncthreads();
    top = s_top[0];
    bad = s_top[1];
  } else {
    top = *J.gmax;
    bad = *J.error;
  }
  const float smax = block_scale_from_amax(__uint_as_float(top));
  // quant.py:21-22; a pass-1 kernel that gave up on a load raises the error word: publish NaN so that it shows
  const float unit = bad ? __uint_as_float(0x7FC00000u) : __fdiv_rn(smax, 448.0f);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    *J.unit = unit;
    if (offset_ctr && blockIdx.y == 0) *offset_ctr += 1;       // pass 1 of this call has finished: the next call draws fresh bits
  }
  const int64_t tiles = sf_tiles_per_row(sf_cols * 16);
  const int groups_per_row = (int)(tiled ? tiles : (sf_cols + 3) / 4);
  const int64_t R_out = tiled ? ((R + 127) / 128) * 128 : R;
  const bool vec = (sf_cols & 3) == 0;
  const int64_t row_step = (int64_t)gridDim.x * by;
  const bool sums = J.row_sums != nullptr;                       // the host asks for them only when vec holds

  auto load = [&](int64_t r, int g, float (&a)[4]) -> int {       // maxima of group g of row r; returns how many are real
    a[0] = a[1] = a[2] = a[3] = 0.0f;
    const int64_t k0 = (int64_t)g * 4;
    if (r >= R || k0 >= sf_cols) return 0;
    const float* src = amax + r * sf_cols + k0;
    if (vec) {
      const float4 w = *reinterpret_cast<const float4*>(src);
      a[0] = w.x; a[1] = w.y; a[2] = w.z; a[3] = w.w;
      return 4;
    }
    const int live = (int)(sf_cols - k0 < 4 ? sf_cols - k0 : 4);
    for (int j = 0; j < live; ++j) a[j] = src[j];
    return live;
  };
  auto store = [&](int64_t r, int g, uint32_t packed, int live) {
    const int64_t k0 = (int64_t)g * 4;
    if (tiled) {
      *reinterpret_cast<uint32_t*>(scales + sf_mma_offset(r, k0, tiles)) = packed;      // padding bytes are zero
    } else if (vec) {
      *reinterpret_cast<uint32_t*>(scales + r * sf_cols + k0) = packed;
    } else {
      for (int j = 0; j < live; ++j) scales[r * sf_cols + k0 + j] = (uint8_t)(packed >> (8 * j));
    }
  };
  // codes of the 4 blocks of group g of row r, and their sum of code values x scale in half units of `unit`
  auto load_codes = [&](int64_t r, int g, uint4 (&c)[2]) {
    const uint4* src = reinterpret_cast<const uint4*>(J.codes + r * sf_cols + (int64_t)g * 4);
    c[0] = src[0];
    c[1] = src[1];
  };
  auto group_sum = [&](const uint4 (&c)[2], uint32_t packed) -> float {
    float f[4];
    e4m3x4_to_float(packed, f);
    float acc = (float)block_code_sum(make_uint2(c[0].x, c[0].y)) * f[0];
    acc = fmaf((float)block_code_sum(make_uint2(c[0].z, c[0].w)), f[1], acc);
    acc = fmaf((float)block_code_sum(make_uint2(c[1].x, c[1].y)), f[2], acc);
    return fmaf((float)block_code_sum(make_uint2(c[1].z, c[1].w)), f[3], acc);
  };
  const float inv_unit = __fdiv_rn(1.0f, unit);
  // the row loop is uniform over the CTA (the reduction below meets at a barrier)
  for (int64_t r0 = (int64_t)blockIdx.x * by; r0 < R_out; r0 += 2 * row_step) {
    const int64_t r = r0 + ty, r2 = r + row_step;
    float sum_a = 0.0f, sum_b = 0.0f;
    if (r < R_out) {
      const bool second = r2 < R_out;
      for (int g = tx; g < groups_per_row; g += bx) {
        float a[4], b[4];
        uint4 ca[2], cb[2];
        // every load of the two rows is issued before the first use
        const int la = load(r, g, a);
        const int lb = second ? load(r2, g, b) : 0;
        if (sums && la) load_codes(r, g, ca);
        if (sums && lb) load_codes(r2, g, cb);
        const uint32_t pa = scale_bytes4(a, la, unit, inv_unit);
        store(r, g, pa, la);
        if (sums && la) sum_a += group_sum(ca, pa);
        if (second) {
          const uint32_t pb = scale_bytes4(b, lb, unit, inv_unit);
          store(r2, g, pb, lb);
          if (sums && lb) sum_b += group_sum(cb, pb);
        }
      }
    }
    if (sums) {
      // fixed order: lanes of a row by butterfly, then the row's warps one after the other
      for (int o = (bx < 32 ? bx : 32) >> 1; o > 0; o >>= 1) {
        sum_a += __shfl_xor_sync(0xffffffffu, sum_a, o);
        sum_b += __shfl_xor_sync(0xffffffffu, sum_b, o);
      }
      if (bx > 32) {
        const int warp = threadIdx.x >> 5, per_row = bx >> 5;
        if ((threadIdx.x & 31) == 0) s_sum[warp] = make_float2(sum_a, sum_b);
        __syncthreads();
        if (tx == 0) {
          sum_a = sum_b = 0.0f;
          for (int w = 0; w < per_row; ++w) { sum_a += s_sum[ty * per_row + w].x; sum_b += s_sum[ty * per_row + w].y; }
        }
        __syncthreads();
      }
      if (tx == 0) {
        const float half_unit = 0.5f * unit;
        if (r < R) J.row_sums[r] = sum_a * half_unit;
        if (r2 < R) J.row_sums[r2] = sum_b * half_unit;
      }
    }
  }
}

// ---- small tensors (decode-sized activations): one launch --------------------------------------------------
// Up to 16384 blocks (256 Ki elements), round to nearest.  One thread-block cluster of up to 8 CTAs
// holds the whole tensor: a thread quantizes up to 4 blocks and keeps their maxima in registers, the
// tensor-wide maximum goes through the cluster's shared memory (hardware cluster barrier: nothing to
// zero, no spinning, no scratch in global memory), and the same thread then writes its E4M3 bytes.
// Replaces the zero-fill + pass 1 + scale pass of the streaming path where launch latency is all there
// is to save; with more blocks (or more padding words to clear) the 8 SMs of a cluster lose to the
// streaming kernels on 148.  Measured back to back inside a CUDA graph: 16 x 4096 bf16 4.3 us against
// 8.0, 32 x 4096 5.2, 64 x 4096 6.8 against 8.1.
constexpr int kSmallThreads = 512;
constexpr int kSmallBlocks = 4;                    // blocks per thread
constexpr int64_t kSmallMaxBlocks = (int64_t)kSmallCtas * kSmallThreads * kSmallBlocks;

template <typename T, bool kMean>
__global__ void __launch_bounds__(kSmallThreads)
quantize_small_kernel(const T* __restrict__ x, int rows, int blocks_per_row, int64_t ld,
                      const float* __restrict__ col_mean, uint2* __restrict__ codes, int32_t sf_layout,
                      int tiles, int padded_words, uint8_t* __restrict__ scales, float* __restrict__ unit_out) {
  __shared__ ClusterMaxSmem s_max;
  grid_dependency_wait();
  const int t = (int)(cluster_cta_rank() * blockDim.x + threadIdx.x);       // CTAs of 32..512 threads: one block per thread while that fits
  const int stride = (int)(cluster_cta_count() * blockDim.x);
  const int real_blocks = rows * blocks_per_row;
  if (sf_layout == METIS_SF_MMA) zero_scale_padding(scales, rows, blocks_per_row, tiles, padded_words, t, stride);

  float amax[kSmallBlocks];
  float running = 0.0f;
  RawBlock<T> raw[kSmallBlocks];
#pragma unroll
  for (int j = 0; j < kSmallBlocks; ++j) {        // all loads first: one trip to memory
    const int b = t + j * stride;
    if (b < real_blocks) {
      const int r = b / blocks_per_row, c = b - r * blocks_per_row;
      raw[j].load(x + (int64_t)r * ld + (int64_t)c * 16);
    }
  }
#pragma unroll
  for (int j = 0; j < kSmallBlocks; ++j) {
    const int b = t + j * stride;
    amax[j] = 0.0f;
    if (b < real_blocks) {
      float v[16];
      raw[j].unpack(v);
      if (kMean) {
        const int r = b / blocks_per_row, c = b - r * blocks_per_row;
        float m[16];
        Load16<float>::load(col_mean + (int64_t)c * 16, m);
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = __fsub_rn(v[e], m[e]);
      }
      const float a = abs_max16(v);
      uint32_t pk[2];
      quantize_rn<2>(v, block_scale_from_amax(a), pk);
      codes[b] = make_uint2(pk[0], pk[1]);
      amax[j] = a;
      running = fmaxf(running, a);
    }
  }

  const float unit = __fdiv_rn(block_scale_from_amax(cluster_fmax(running, s_max)), 448.0f);       // quant.py:21-22
  if (t == 0) *unit_out = unit;

#pragma unroll
  for (int j = 0; j < kSmallBlocks; ++j) {
    const int b = t + j * stride;
    if (b >= real_blocks) continue;
    const int r = b / blocks_per_row, c = b - r * blocks_per_row;
    const float ratio = __fdiv_rn(block_scale_from_amax(amax[j]), unit);      // quant.py:23
    const int64_t off = (sf_layout == METIS_SF_MMA) ? sf_mma_offset(r, c, tiles) : (int64_t)b;
    scales[off] = float_to_e4m3(ratio);             // 4 neighbouring lanes fill one 32-bit word
  }
  cluster_leave();
}

// Whether the one-launch kernel takes a row-major quantization of [R, C].
static bool small_path(int64_t R, int64_t C, int32_t sf_layout, int64_t* tiles, int64_t* padded_words) {
  *tiles = sf_tiles_per_row(C);
  *padded_words = sf_layout == METIS_SF_MMA ? ceil_div(R, 128) * 128 * *tiles : 0;
  return R * (C / 16) <= kSmallMaxBlocks && *padded_words <= kSmallMaxPaddedWords;
}

template <typename T>
static int32_t launch_small(const T* x, int64_t rows, int64_t cols, int64_t ld, const float* mean, uint8_t* codes,
                            int32_t sf_layout, int64_t tiles, int64_t padded_words, uint8_t* scales,
                            float* unit, cudaStream_t st) {
  const int64_t blocks = rows * (cols / 16);
  const int64_t work = blocks > padded_words / 4 ? blocks : padded_words / 4;   // a block, or a 16-byte piece of padding, per thread
  int64_t ctas = ceil_div(work, 32);
  if (ctas > kSmallCtas) ctas = kSmallCtas;
  int64_t threads = ceil_div(ceil_div(work, ctas), 32) * 32;            // spread thin: latency is what counts here
  if (threads > kSmallThreads) threads = kSmallThreads;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3((unsigned)threads);
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
  if (mean)
    METIS_CUDA_OK(cudaLaunchKernelEx(&cfg, quantize_small_kernel<T, true>, x, (int)rows, (int)(cols / 16), ld, mean, c2, sf_layout,
                                     (int)tiles, (int)padded_words, scales, unit));
  else
    METIS_CUDA_OK(cudaLaunchKernelEx(&cfg, quantize_small_kernel<T, false>, x, (int)rows, (int)(cols / 16), ld, mean, c2, sf_layout,
                                     (int)tiles, (int)padded_words, scales, unit));
  return METIS_OK;
}

// ---- column means -----------------------------------------------------------------------------------------
// Stage 1: CTA (bx, by) sums rows [by*rows_per_split, ...) of 8*32 columns into
// partial[by][col]; stage 2 adds the partials in a fixed order and divides by rows.
constexpr int kMeanThreads = 256;
template <typename T>
__global__ void __launch_bounds__(kMeanThreads)
col_partial_sum_kernel(const T* __restrict__ x, int64_t rows, int64_t cols, int64_t ld,
                       int64_t rows_per_split, float* __restrict__ partial, int64_t mean_of_rows) {
  // mean_of_rows > 0 (a single split): `partial` is the mean itself, sum / mean_of_rows, as stage 2 would write it
  grid_dependency_wait();
  // stage 2 follows in the stream: its few CTAs may take their places now (they wait for this grid to complete)
  if (mean_of_rows == 0) grid_launch_dependents();
  // 32 lanes x 8 columns = 256 columns per CTA; 8 warps stride over the rows.
  __shared__ float s_part[kMeanThreads / 32][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t col = (int64_t)blockIdx.x * 256 + lane * 8;
  const int64_t r_begin = (int64_t)blockIdx.y * rows_per_split;
  const int64_t r_end = min(rows, r_begin + rows_per_split);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < cols) {
    // four rows in flight per warp; the additions keep their order (row after row)
    int64_t r = r_begin + warp;
    for (; r + 3 * (kMeanThreads / 32) < r_end; r += 4 * (kMeanThreads / 32)) {
      float v[4][8];
#pragma unroll
      for (int k = 0; k < 4; ++k) Load8<T>::load(x + (r + k * (kMeanThreads / 32)) * ld + col, v[k]);
#pragma unroll
      for (int k = 0; k < 4; ++k)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += v[k][i];
    }
    for (; r < r_end; r += kMeanThreads / 32) {
      float v[8];
      Load8<T>::load(x + r * ld + col, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) s_part[warp][lane * 8 + i] = acc[i];
  __syncthreads();
  const int c = threadIdx.x;
  float sum = 0.0f;
#pragma unroll
  for (int w = 0; w < kMeanThreads / 32; ++w) sum += s_part[w][c];
  const int64_t oc = (int64_t)blockIdx.x * 256 + c;
  if (oc < cols) partial[(int64_t)blockIdx.y * cols + oc] = mean_of_rows > 0 ? __fdiv_rn(__fadd_rn(0.0f, sum), (float)mean_of_rows) : sum;
}

constexpr int kMeanMaxSplits = 64;
__global__ void __launch_bounds__(256) col_mean_finish_kernel(const float* __restrict__ partial, int64_t splits, int64_t rows,
                                       int64_t cols, float* __restrict__ mean) {
  grid_dependency_wait();
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  // all loads in flight at once (splits <= kMeanMaxSplits), then the additions in their fixed order
  float v[kMeanMaxSplits];
#pragma unroll
  for (int s = 0; s < kMeanMaxSplits; ++s) v[s] = s < splits ? partial[s * cols + c] : 0.0f;
  float sum = 0.0f;
#pragma unroll
  for (int s = 0; s < kMeanMaxSplits; ++s)
    if (s < splits) sum += v[s];
  mean[c] = __fdiv_rn(sum, (float)rows);
}

static int64_t col_mean_splits(int64_t rows) {
  int64_t s = ceil_div(rows, 128);
  return s < 1 ? 1 : (s > kMeanMaxSplits ? kMeanMaxSplits : s);
}

// ---- launch helpers ------------------------------------------------------------------------------------------

int device_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
    return n;
  return 148;
}
static int sm_count() { return device_sm_count(); }

template <typename T>
static void launch_rows(const T* x, int64_t rows, int64_t cols, int64_t ld, const float* mean, bool sr,
                        uint64_t seed, uint64_t offset, const uint64_t* ctr, uint32_t* codes, const WorkspaceView& ws,
                        cudaStream_t st, uint32_t sr16 = 0) {
  const int bpr = (int)(cols >> 4);
  // threads along the row: the power of two that pads the row least (hidden 1536 = 96 blocks runs
  // as 3 x 32, not as 128 with a quarter of the lanes idle); ties go to the wider shape
  int bx = 1;
  while (bx < bpr && bx < kQuantThreads) bx <<= 1;
  for (int cand = bx >> 1; cand >= 32; cand >>= 1)
    if ((bpr + cand - 1) / cand * cand < (bpr + bx - 1) / bx * bx) bx = cand;
  const int by = kQuantThreads / bx;
  const int gx = (bpr + bx - 1) / bx;
  int64_t gy = ceil_div(rows, by);
  // four waves of resident CTAs (grid-stride over the rows): whole waves leave no tail
  int per_sm = 0;
#define METIS_OCC_ROWS(MEAN, SR) cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_rows_kernel<T, MEAN, SR>, kQuantThreads, 0)
  if (mean) { if (sr) METIS_OCC_ROWS(true, true); else METIS_OCC_ROWS(true, false); }
  else      { if (sr) METIS_OCC_ROWS(false, true); else METIS_OCC_ROWS(false, false); }
#undef METIS_OCC_ROWS
  if (per_sm < 1) per_sm = 1;
  int64_t cap = (int64_t)sm_count() * per_sm * 4 / gx;
  if (cap < 1) cap = 1;
  if (gy > cap) gy = cap;
  if (gy > 65535) gy = 65535;
  if (gy < 1) gy = 1;
  const dim3 g((unsigned)gx, (unsigned)gy), b((unsigned)bx, (unsigned)by);
#define METIS_LAUNCH_ROWS(MEAN, SR)                                                              \
  launch_overlapped(kLaunchStream, quantize_rows_kernel<T, MEAN, SR>, g, b, 0, st, x, (int)rows, bpr, ld, mean, seed, offset, ctr, \
                    reinterpret_cast<uint2*>(codes), ws.amax, ws.gmax, sr16)
  if (mean) { if (sr) METIS_LAUNCH_ROWS(true, true); else METIS_LAUNCH_ROWS(true, false); }
  else      { if (sr) METIS_LAUNCH_ROWS(false, true); else METIS_LAUNCH_ROWS(false, false); }
#undef METIS_LAUNCH_ROWS
}

template <typename T>
static int32_t launch_tile(const T* x, int64_t rows, int64_t cols, int64_t ld, const float* mean, bool sr,
                           uint64_t seed, uint64_t offset, const uint64_t* ctr, const TileOutputs& out, cudaStream_t st) {
  using TC = TileCfg<T>;
  CUtensorMap map;
  const CUtensorMapDataType dt = sizeof(T) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (int32_t rc = make_map(&map, dt, sizeof(T), x, cols, rows, ld * (int64_t)sizeof(T), TC::kCols, TC::kRows, "x", 128))
    return rc;
  const int64_t tiles = ceil_div(cols, TC::kCols) * ceil_div(rows, TC::kRows);
  int64_t grid = (int64_t)sm_count() * 3;          // three CTAs of ~63 KiB per SM
  if (grid > tiles) grid = tiles;
  if (out.records && grid > kDualMaxCtas) grid = kDualMaxCtas;
  const bool with_rows = out.codes_r != nullptr, with_cols = out.codes_t != nullptr;
#define METIS_LAUNCH_TILE(MEAN, SR, ROWS, COLS)                                                             \
  do {                                                                                                      \
    auto kern = quantize_tile_kernel<T, MEAN, SR, ROWS, COLS>;                                              \
    METIS_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TC::kSmemBytes)); \
    METIS_CUDA_OK(launch_overlapped(kLaunchStream, kern, dim3((unsigned)grid), dim3(kQuantThreads), TC::kSmemBytes, st, map, rows, cols, \
                                    mean, seed, offset, ctr, out));                                         \
  } while (0)
#define METIS_LAUNCH_TILE_MS(MEAN, SR)                                  \
  do {                                                                  \
    if (with_rows && with_cols) METIS_LAUNCH_TILE(MEAN, SR, true, true); \
    else if (with_cols) METIS_LAUNCH_TILE(MEAN, SR, false, true);       \
    else METIS_LAUNCH_TILE(MEAN, SR, true, false);                      \
  } while (0)
  if (mean) { if (sr) METIS_LAUNCH_TILE_MS(true, true); else METIS_LAUNCH_TILE_MS(true, false); }
  else      { if (sr) METIS_LAUNCH_TILE_MS(false, true); else METIS_LAUNCH_TILE_MS(false, false); }
#undef METIS_LAUNCH_TILE_MS
#undef METIS_LAUNCH_TILE
  return METIS_OK;
}

static int32_t launch_finalize_jobs(FinalizeJobs jobs, int njobs, cudaStream_t st, uint64_t* offset_ctr) {
  int64_t blocks = 1;
  for (int j = 0; j < njobs; ++j) {
    FinalizeJob& J = jobs.job[j];
    const bool tiled = J.sf_layout == METIS_SF_MMA;
    const int64_t groups = tiled ? sf_tiles_per_row(J.sf_cols * 16) : ceil_div(J.sf_cols, 4);
    const int64_t rows = tiled ? ceil_div(J.R, 128) * 128 : J.R;
    int bx = 1;
    while (bx < groups && bx < kQuantThreads) bx <<= 1;
    J.bx = bx;
    const int64_t need = ceil_div(rows, 2 * (kQuantThreads / bx));           // two rows per thread
    if (need > blocks) blocks = need;
  }
  if (njobs == 1) jobs.job[1] = jobs.job[0];
  const int64_t cap = (int64_t)sm_count() * 8 / njobs;
  if (blocks > cap) blocks = ceil_div(blocks, ceil_div(blocks, cap));    // the fewest CTAs that need no more rounds than `cap` would
  METIS_CUDA_OK(launch_overlapped(kLaunchShort, finalize_scales_kernel, dim3((unsigned)blocks, (unsigned)njobs), dim3(kQuantThreads), 0, st,
                                  jobs.job[0], jobs.job[1], offset_ctr));
  return METIS_OK;
}

int32_t launch_finalize(const WorkspaceView& ws, int64_t R, int64_t C, int32_t sf_layout,
                        uint8_t* scales, float* unit, cudaStream_t st, uint64_t* offset_ctr) {
  FinalizeJobs jobs = {};
  jobs.job[0] = {ws.amax, ws.gmax, ws.gmax + 1, R, C / 16, sf_layout, scales, unit, 0, nullptr, nullptr, nullptr, 0};
  return launch_finalize_jobs(jobs, 1, st, offset_ctr);
}

int32_t check_quant_outputs(int64_t R, int64_t C, int32_t sf_layout, const void* codes,
                            const void* scales, const void* unit, const void* workspace,
                            int64_t workspace_bytes) {
  if (R <= 0 || C <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty tensor [%lld, %lld]", (long long)R, (long long)C);
  if (C % 16 != 0)
    return fail(METIS_ERR_BAD_SHAPE, "NVFP4 block shape (1, 16) does not divide tensor shape (%lld, %lld)",
                (long long)R, (long long)C);
  if (sf_layout != METIS_SF_ROWMAJOR && sf_layout != METIS_SF_MMA)
    return fail(METIS_ERR_BAD_ARGUMENT, "unknown sf_layout %d", sf_layout);
  if (!codes || !scales || !unit || !workspace) return fail(METIS_ERR_BAD_ARGUMENT, "null output pointer");
  if (!aligned16(codes) || !aligned16(scales) || !aligned16(workspace))
    return fail(METIS_ERR_BAD_ALIGNMENT, "codes, scales and workspace must be 16-byte aligned");
  if (workspace_bytes < metis_nvfp4_quantize_workspace_bytes(R, C))
    return fail(METIS_ERR_WORKSPACE, "workspace of %lld bytes, need %lld", (long long)workspace_bytes,
                (long long)metis_nvfp4_quantize_workspace_bytes(R, C));
  return METIS_OK;
}

}  // namespace metis

using namespace metis;

extern "C" int64_t metis_nvfp4_sf_bytes(int64_t R, int64_t C, int32_t sf_layout) {
  if (R <= 0 || C <= 0) return 0;
  if (sf_layout == METIS_SF_MMA) return ceil_div(R, 128) * sf_tiles_per_row(C) * 512;
  return R * ceil_div(C, 16);
}

extern "C" int64_t metis_nvfp4_quantize_workspace_bytes(int64_t R, int64_t C) {
  if (R <= 0 || C <= 0) return kHeaderBytes;
  return kHeaderBytes + R * ceil_div(C, 16) * (int64_t)sizeof(float);
}

extern "C" int32_t metis_nvfp4_quantize(const void* x, int32_t x_dtype, int64_t rows, int64_t cols,
                                        int64_t ld, const float* col_mean, uint32_t flags,
                                        uint64_t seed, uint64_t offset, int32_t sf_layout,
                                        uint8_t* codes, uint8_t* scales, float* unit, void* workspace,
                                        int64_t workspace_bytes, void* stream) {
  const bool transpose = flags & METIS_Q_TRANSPOSE;
  const bool sr = flags & METIS_Q_STOCHASTIC;
  // graph-safe random stream: `offset` carries the address of a device counter instead of a value
  uint64_t* ctr = (sr && (flags & METIS_Q_OFFSET_ON_DEVICE)) ? reinterpret_cast<uint64_t*>(static_cast<uintptr_t>(offset)) : nullptr;
  if (ctr) offset = 0;
  if ((flags & METIS_Q_OFFSET_ON_DEVICE) && (!sr || !ctr || (reinterpret_cast<uintptr_t>(ctr) & 7u)))
    return fail(METIS_ERR_BAD_ARGUMENT, "METIS_Q_OFFSET_ON_DEVICE needs METIS_Q_STOCHASTIC and an 8-byte aligned device address in offset");
  if (flags & ~(METIS_Q_TRANSPOSE | METIS_Q_STOCHASTIC | METIS_Q_OFFSET_ON_DEVICE | METIS_Q_HADAMARD | METIS_Q_SIGN_MASK | METIS_Q_SR16)) return fail(METIS_ERR_BAD_ARGUMENT, "unknown flags 0x%x", flags);
  if ((flags & METIS_Q_SR16) && !sr) return fail(METIS_ERR_BAD_ARGUMENT, "METIS_Q_SR16 without METIS_Q_STOCHASTIC");
  const uint32_t sr16 = (flags & METIS_Q_SR16) ? 1u : 0u;
  if ((flags & METIS_Q_HADAMARD) && !transpose) return fail(METIS_ERR_UNSUPPORTED, "METIS_Q_HADAMARD rotates the blocks of the transposed quantization: it needs METIS_Q_TRANSPOSE");
  if ((flags & METIS_Q_SIGN_MASK) && !(flags & METIS_Q_HADAMARD)) return fail(METIS_ERR_BAD_ARGUMENT, "sign bits without METIS_Q_HADAMARD");
  const uint32_t rht = (flags & METIS_Q_HADAMARD) ? ((1u << 16) | (flags >> 16)) : 0u;
  if (!x) return fail(METIS_ERR_BAD_ARGUMENT, "x is null");
  if (x_dtype != METIS_DTYPE_BF16 && x_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown x_dtype %d", x_dtype);
  if (rows <= 0 || cols <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty tensor [%lld, %lld]", (long long)rows, (long long)cols);
  if (ld < cols) return fail(METIS_ERR_BAD_ARGUMENT, "ld %lld < cols %lld", (long long)ld, (long long)cols);
  const int64_t R = transpose ? cols : rows, C = transpose ? rows : cols;
  if (int32_t rc = check_quant_outputs(R, C, sf_layout, codes, scales, unit, workspace, workspace_bytes)) return rc;
  const int64_t esz = x_dtype == METIS_DTYPE_BF16 ? 2 : 4;
  // vector loads: 8 elements per thread row-major, 16 bytes per thread transposed
  const int64_t need = transpose ? 16 / esz : 8;
  if (cols % need != 0 || ld % need != 0 || !aligned16(x))
    return fail(METIS_ERR_BAD_ALIGNMENT, "x must be 16-byte aligned with cols and ld multiples of %lld", (long long)need);
  if (col_mean && !aligned16(col_mean)) return fail(METIS_ERR_BAD_ALIGNMENT, "col_mean must be 16-byte aligned");
  if (rows >= ((int64_t)1 << 31) || cols >= ((int64_t)1 << 31)) return fail(METIS_ERR_TOO_LARGE, "tensor too large");

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int64_t tiles = 0, padded_words = 0;
  if (!transpose && !sr && aligned16(scales) && small_path(R, C, sf_layout, &tiles, &padded_words)) {
    return x_dtype == METIS_DTYPE_BF16
        ? launch_small(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, col_mean, codes, sf_layout, tiles, padded_words, scales, unit, st)
        : launch_small(static_cast<const float*>(x), rows, cols, ld, col_mean, codes, sf_layout, tiles, padded_words, scales, unit, st);
  }
  const WorkspaceView ws = view_workspace(workspace);
  METIS_CUDA_OK(cudaMemsetAsync(ws.gmax, 0, 2 * sizeof(unsigned int), st));   // running maximum and error word
  // Large row-major tensors take the tile kernel too (row phase only): its TMA ring keeps two tiles in
  // flight per CTA, where the register-fed kernel waits on its loads.  Same arithmetic, same bytes.
  const bool rows_by_tiles = !transpose && rows * cols >= kTileRowsMinElements && (ld * esz) % 16 == 0;
  if (rows_by_tiles) {
    const TileOutputs out = {nullptr, nullptr, nullptr, codes, ws.amax, ws.gmax, ws.gmax + 1, nullptr, 0u, sr16};
    const int32_t rc = x_dtype == METIS_DTYPE_BF16
        ? launch_tile(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr, out, st)
        : launch_tile(static_cast<const float*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr, out, st);
    if (rc) return rc;
  } else if (!transpose) {
    if (x_dtype == METIS_DTYPE_BF16)
      launch_rows(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr,
                  reinterpret_cast<uint32_t*>(codes), ws, st, sr16);
    else
      launch_rows(static_cast<const float*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr,
                  reinterpret_cast<uint32_t*>(codes), ws, st, sr16);
  } else {
    const TileOutputs out = {codes, ws.amax, ws.gmax, nullptr, nullptr, nullptr, ws.gmax + 1, nullptr, rht, sr16};
    const int32_t rc = x_dtype == METIS_DTYPE_BF16
        ? launch_tile(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr, out, st)
        : launch_tile(static_cast<const float*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr, out, st);
    if (rc) return rc;
  }
  METIS_CUDA_OK(cudaGetLastError());
  return launch_finalize(ws, R, C, sf_layout, scales, unit, st, ctr);
}

// Scale pass of the dual quantizer's outputs (either or both) from the block maxima in its workspace.
static int32_t finish_dual(int64_t rows, int64_t cols, int32_t sf_layout, uint8_t* scales, float* unit, const uint8_t* codes_t,
                           uint8_t* scales_t, float* unit_t, float* token_sums_t, void* workspace, bool rowmajor,
                           bool transposed, cudaStream_t st, uint64_t* ctr) {
  const unsigned int* records = static_cast<const unsigned int*>(workspace) + 64;
  float* amax_r = reinterpret_cast<float*>(static_cast<char*>(workspace) + kDualHeaderBytes);
  float* amax_t = amax_r + rows * (cols / 16);
  FinalizeJobs jobs = {};
  int n = 0;
  if (rowmajor) jobs.job[n++] = {amax_r, nullptr, nullptr, rows, cols / 16, sf_layout, scales, unit, 0, nullptr, nullptr, records, 0};
  if (transposed)
    jobs.job[n++] = {amax_t, nullptr, nullptr, cols, rows / 16, sf_layout, scales_t, unit_t, 0,
                     token_sums_t ? reinterpret_cast<const uint2*>(codes_t) : nullptr, token_sums_t, records, 1};
  if (n == 0) return METIS_OK;
  return launch_finalize_jobs(jobs, n, st, ctr);      // job 0 of the launch bumps the Philox offset counter, if there is one
}

extern "C" int64_t metis_nvfp4_quantize_dual_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return kDualHeaderBytes;
  return kDualHeaderBytes + 2 * rows * ceil_div(cols, 16) * (int64_t)sizeof(float);
}

extern "C" int32_t metis_nvfp4_quantize_dual(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                             const float* col_mean, uint32_t flags, uint64_t seed, uint64_t offset,
                                             int32_t sf_layout, uint8_t* codes, uint8_t* scales, float* unit,
                                             uint8_t* codes_t, uint8_t* scales_t, float* unit_t, float* token_sums_t,
                                             void* workspace, int64_t workspace_bytes, void* stream) {
  const bool sr = flags & METIS_Q_STOCHASTIC;
  uint64_t* ctr = (sr && (flags & METIS_Q_OFFSET_ON_DEVICE)) ? reinterpret_cast<uint64_t*>(static_cast<uintptr_t>(offset)) : nullptr;
  if (ctr) offset = 0;
  if ((flags & METIS_Q_OFFSET_ON_DEVICE) && (!sr || !ctr || (reinterpret_cast<uintptr_t>(ctr) & 7u)))
    return fail(METIS_ERR_BAD_ARGUMENT, "METIS_Q_OFFSET_ON_DEVICE needs METIS_Q_STOCHASTIC and an 8-byte aligned device address in offset");
  if (flags & ~(METIS_Q_STOCHASTIC | METIS_Q_OFFSET_ON_DEVICE | METIS_Q_HADAMARD | METIS_Q_SIGN_MASK | METIS_Q_DEFER_ROWMAJOR | METIS_Q_DEFER_TRANSPOSED | METIS_Q_SR16)) return fail(METIS_ERR_BAD_ARGUMENT, "unknown flags 0x%x (the dual quantizer always writes both orientations)", flags);
  if ((flags & METIS_Q_SR16) && !sr) return fail(METIS_ERR_BAD_ARGUMENT, "METIS_Q_SR16 without METIS_Q_STOCHASTIC");
  if ((flags & METIS_Q_DEFER_ROWMAJOR) && (flags & METIS_Q_DEFER_TRANSPOSED)) return fail(METIS_ERR_BAD_ARGUMENT, "only one of the two scale passes can be deferred");
  if ((flags & METIS_Q_SIGN_MASK) && !(flags & METIS_Q_HADAMARD)) return fail(METIS_ERR_BAD_ARGUMENT, "sign bits without METIS_Q_HADAMARD");
  const uint32_t rht = (flags & METIS_Q_HADAMARD) ? ((1u << 16) | (flags >> 16)) : 0u;      // the transposed output only
  if (token_sums_t && rht) return fail(METIS_ERR_BAD_ARGUMENT, "token_sums_t is not available with METIS_Q_HADAMARD (the rotated blocks need weighted sums)");
  if (token_sums_t && rows % 64 != 0) return fail(METIS_ERR_BAD_SHAPE, "token_sums_t needs rows to be a multiple of 64");
  if (!x) return fail(METIS_ERR_BAD_ARGUMENT, "x is null");
  if (x_dtype != METIS_DTYPE_BF16 && x_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown x_dtype %d", x_dtype);
  if (rows <= 0 || cols <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty tensor [%lld, %lld]", (long long)rows, (long long)cols);
  if (rows % 16 != 0 || cols % 16 != 0)
    return fail(METIS_ERR_BAD_SHAPE, "NVFP4 block shape (1, 16) does not divide both dimensions of tensor shape (%lld, %lld)", (long long)rows, (long long)cols);
  if (ld < cols) return fail(METIS_ERR_BAD_ARGUMENT, "ld %lld < cols %lld", (long long)ld, (long long)cols);
  if (sf_layout != METIS_SF_ROWMAJOR && sf_layout != METIS_SF_MMA) return fail(METIS_ERR_BAD_ARGUMENT, "unknown sf_layout %d", sf_layout);
  if (!codes || !scales || !unit || !codes_t || !scales_t || !unit_t || !workspace) return fail(METIS_ERR_BAD_ARGUMENT, "null output pointer");
  const int64_t esz = x_dtype == METIS_DTYPE_BF16 ? 2 : 4;
  if (ld % (16 / esz) != 0 || !aligned16(x) || !aligned16(codes) || !aligned16(scales) || !aligned16(codes_t) || !aligned16(scales_t) || !aligned16(workspace))
    return fail(METIS_ERR_BAD_ALIGNMENT, "x, codes, scales and workspace must be 16-byte aligned, rows of x too");
  if (col_mean && !aligned16(col_mean)) return fail(METIS_ERR_BAD_ALIGNMENT, "col_mean must be 16-byte aligned");
  if (workspace_bytes < metis_nvfp4_quantize_dual_workspace_bytes(rows, cols))
    return fail(METIS_ERR_WORKSPACE, "workspace of %lld bytes, need %lld", (long long)workspace_bytes,
                (long long)metis_nvfp4_quantize_dual_workspace_bytes(rows, cols));
  if (rows >= ((int64_t)1 << 31) || cols >= ((int64_t)1 << 31)) return fail(METIS_ERR_TOO_LARGE, "tensor too large");

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // every CTA of the first pass leaves its maxima and its error word in a record of its own: nothing to zero first
  unsigned int* records = static_cast<unsigned int*>(workspace) + 64;
  float* amax_r = reinterpret_cast<float*>(static_cast<char*>(workspace) + kDualHeaderBytes);
  float* amax_t = amax_r + rows * (cols / 16);
  const TileOutputs out = {codes_t, amax_t, nullptr, codes, amax_r, nullptr, nullptr, records, rht, (flags & METIS_Q_SR16) ? 1u : 0u};
  const int32_t rc = x_dtype == METIS_DTYPE_BF16
      ? launch_tile(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr, out, st)
      : launch_tile(static_cast<const float*>(x), rows, cols, ld, col_mean, sr, seed, offset, ctr, out, st);
  if (rc) return rc;
  METIS_CUDA_OK(cudaGetLastError());
  return finish_dual(rows, cols, sf_layout, scales, unit, codes_t, scales_t, unit_t, token_sums_t, workspace,
                     !(flags & METIS_Q_DEFER_ROWMAJOR), !(flags & METIS_Q_DEFER_TRANSPOSED), st, ctr);
}

extern "C" int32_t metis_nvfp4_quantize_dual_finish(int64_t rows, int64_t cols, uint32_t deferred, int32_t sf_layout,
                                                    uint8_t* scales, float* unit, const uint8_t* codes_t, uint8_t* scales_t,
                                                    float* unit_t, float* token_sums_t, void* workspace,
                                                    int64_t workspace_bytes, void* stream) {
  const bool rowmajor = deferred == METIS_Q_DEFER_ROWMAJOR, transposed = deferred == METIS_Q_DEFER_TRANSPOSED;
  if (!rowmajor && !transposed) return fail(METIS_ERR_BAD_ARGUMENT, "deferred must be METIS_Q_DEFER_ROWMAJOR or METIS_Q_DEFER_TRANSPOSED");
  if (rows <= 0 || cols <= 0 || rows % 16 != 0 || cols % 16 != 0) return fail(METIS_ERR_BAD_SHAPE, "bad shape [%lld, %lld]", (long long)rows, (long long)cols);
  if (sf_layout != METIS_SF_ROWMAJOR && sf_layout != METIS_SF_MMA) return fail(METIS_ERR_BAD_ARGUMENT, "unknown sf_layout %d", sf_layout);
  if (!workspace || !aligned16(workspace) || workspace_bytes < metis_nvfp4_quantize_dual_workspace_bytes(rows, cols))
    return fail(METIS_ERR_WORKSPACE, "the workspace of the quantizing call is needed");
  if (rowmajor && (!scales || !unit || !aligned16(scales))) return fail(METIS_ERR_BAD_ARGUMENT, "scales and unit of the row-major output");
  if (transposed && (!scales_t || !unit_t || !aligned16(scales_t) || (token_sums_t && !codes_t)))
    return fail(METIS_ERR_BAD_ARGUMENT, "scales_t and unit_t of the transposed output (and codes_t for token_sums_t)");
  if (token_sums_t && rows % 64 != 0) return fail(METIS_ERR_BAD_SHAPE, "token_sums_t needs rows to be a multiple of 64");
  return finish_dual(rows, cols, sf_layout, scales, unit, codes_t, scales_t, unit_t, token_sums_t, workspace,
                     rowmajor, transposed, reinterpret_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int64_t metis_col_mean_workspace_bytes(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return col_mean_splits(rows) * cols * (int64_t)sizeof(float);
}

extern "C" int32_t metis_col_mean(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                  float* mean, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x || !mean || !workspace) return fail(METIS_ERR_BAD_ARGUMENT, "null pointer");
  if (x_dtype != METIS_DTYPE_BF16 && x_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown x_dtype %d", x_dtype);
  if (rows <= 0 || cols <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty tensor");
  if (cols % 8 != 0 || ld % 8 != 0 || ld < cols || !aligned16(x))
    return fail(METIS_ERR_BAD_ALIGNMENT, "x must be 16-byte aligned with cols and ld multiples of 8");
  if (workspace_bytes < metis_col_mean_workspace_bytes(rows, cols))
    return fail(METIS_ERR_WORKSPACE, "workspace too small");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t splits = col_mean_splits(rows);
  const int64_t rows_per_split = ceil_div(rows, splits);
  const dim3 g((unsigned)ceil_div(cols, 256), (unsigned)splits);
  // up to 128 rows there is one split: stage 1 writes the mean itself (0 + sum, then the same division)
  const bool single = splits == 1;
  float* partial = single ? mean : static_cast<float*>(workspace);
  const int64_t mean_of_rows = single ? rows : 0;
  if (x_dtype == METIS_DTYPE_BF16)
    METIS_CUDA_OK(launch_overlapped(kLaunchStream, col_partial_sum_kernel<__nv_bfloat16>, g, dim3(kMeanThreads), 0, st,
                                    static_cast<const __nv_bfloat16*>(x), rows, cols, ld, rows_per_split, partial, mean_of_rows));
  else
    METIS_CUDA_OK(launch_overlapped(kLaunchStream, col_partial_sum_kernel<float>, g, dim3(kMeanThreads), 0, st,
                                    static_cast<const float*>(x), rows, cols, ld, rows_per_split, partial, mean_of_rows));
  if (!single)
    METIS_CUDA_OK(launch_overlapped(kLaunchShort, col_mean_finish_kernel, dim3((unsigned)ceil_div(cols, 256)), dim3(256), 0, st,
                                    partial, splits, rows, cols, mean));
  return METIS_OK;
}

// ---- quantizer entry point that brings its own scratch -----------------------------------------------
//
// metis_nvfp4_quantize needs a caller-provided workspace for the per-block maxima.  Some callers
// have no way to provide one: a serving loop whose device memory was carved up once at start-up
// and must not grow, a host binding (cgo, JNI) that holds raw device pointers but no allocator, a
// latency-critical section in which cudaMalloc's implicit device synchronisation is not acceptable.
// For them the scratch lives in this translation unit as a fixed-size device array; the price is
// that every GPU that loads the library keeps these bytes until the process exits, and that the
// tensor size is capped.
namespace metis {

constexpr int64_t kStaticMaxElements = METIS_STATIC_MAX_ELEMENTS;                        // 16 Mi elements
constexpr int64_t kStaticScratchBytes = kWorkspaceHeaderBytes + (kStaticMaxElements / 16) * 4;  // 4 MiB + 256 B

// In device code this name is the array.  In host code it is only a handle for the runtime's symbol
// table, NOT a device address: the address is looked up below with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices] = {};
static std::mutex g_static_scratch_mutex;

// Device address of the array on the CURRENT device, resolved once per device.
static int32_t static_scratch_address(void** out) {
  int dev = -1;
  METIS_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(METIS_ERR_UNSUPPORTED, "device index %d is outside [0, %d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(METIS_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return METIS_OK;
}

}  // namespace metis

extern "C" int32_t metis_nvfp4_quantize_static(const void* x, int32_t x_dtype, int64_t rows, int64_t cols,
                                               int64_t ld, int32_t sf_layout, uint8_t* codes,
                                               uint8_t* scales, float* unit, void* stream) {
  if (!x) return fail(METIS_ERR_BAD_ARGUMENT, "x is null");
  if (x_dtype != METIS_DTYPE_BF16 && x_dtype != METIS_DTYPE_F32) return fail(METIS_ERR_BAD_ARGUMENT, "unknown x_dtype %d", x_dtype);
  if (rows <= 0 || cols <= 0) return fail(METIS_ERR_BAD_SHAPE, "empty tensor [%lld, %lld]", (long long)rows, (long long)cols);
  if (cols % 16 != 0)
    return fail(METIS_ERR_BAD_SHAPE, "NVFP4 block shape (1, 16) does not divide tensor shape (%lld, %lld)", (long long)rows, (long long)cols);
  if (rows > kStaticMaxElements / cols)
    return fail(METIS_ERR_TOO_LARGE, "%lld x %lld elements exceed the built-in scratch (METIS_STATIC_MAX_ELEMENTS = %lld); "
                "use metis_nvfp4_quantize with a caller workspace", (long long)rows, (long long)cols, (long long)kStaticMaxElements);
  if (ld < cols) return fail(METIS_ERR_BAD_ARGUMENT, "ld %lld < cols %lld", (long long)ld, (long long)cols);
  if (sf_layout != METIS_SF_ROWMAJOR && sf_layout != METIS_SF_MMA) return fail(METIS_ERR_BAD_ARGUMENT, "unknown sf_layout %d", sf_layout);
  if (!codes || !scales || !unit) return fail(METIS_ERR_BAD_ARGUMENT, "null output pointer");
  if (ld % 8 != 0 || !aligned16(x) || !aligned16(codes) || !aligned16(scales))
    return fail(METIS_ERR_BAD_ALIGNMENT, "x, codes and scales must be 16-byte aligned and ld a multiple of 8");

  void* scratch = nullptr;
  if (int32_t rc = static_scratch_address(&scratch)) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const WorkspaceView ws = view_workspace(scratch);
  // The array keeps whatever the previous call left.  Only the running maximum and the error word
  // have to start at zero; every block maximum this call reads back is written by this call first.
  METIS_CUDA_OK(cudaMemsetAsync(ws.gmax, 0, 2 * sizeof(unsigned int), st));   // running maximum and error word
  if (x_dtype == METIS_DTYPE_BF16)
    launch_rows(static_cast<const __nv_bfloat16*>(x), rows, cols, ld, nullptr, false, 0, 0, nullptr, reinterpret_cast<uint32_t*>(codes), ws, st);
  else
    launch_rows(static_cast<const float*>(x), rows, cols, ld, nullptr, false, 0, 0, nullptr, reinterpret_cast<uint32_t*>(codes), ws, st);
  METIS_CUDA_OK(cudaGetLastError());
  return launch_finalize(ws, rows, cols, sf_layout, scales, unit, st);
}
