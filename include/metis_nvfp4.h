/*
 * metis_nvfp4.h - C ABI of the B200 (sm_100a) Metis NVFP4 linear-layer library.
 *
 * The reference project (decisivemoments/fp4-post) has no FFI for this path: its
 * Metis layer is eager PyTorch (src/Metis/Metis/quant.py, src/Metis/Metis/bitlinear.py)
 * and its only native surface is a pybind11 module taking torch::Tensor
 * (src/Metis/kernels/src/binding.cpp:12-64).  This header is the boundary a host
 * binding (ctypes, cgo, JNI, a torch extension) loads instead.  Every entry point
 * cites the reference call site whose arithmetic it replaces.
 *
 * Conventions
 *  - extern "C", plain pointers and sizes, no C++ or torch types.
 *  - All data pointers are DEVICE pointers unless stated otherwise.  The caller owns
 *    every buffer, including scratch ("workspace"); the library never allocates device
 *    memory and keeps no pointer after a call returns.  (One exception, stated at its
 *    declaration: metis_nvfp4_quantize_static keeps its scratch inside the library.)
 *  - Every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL is the
 *    legacy default stream) and returns a host-side status: 0 = launched,
 *    negative = argument rejected (nothing was launched).  metis_last_error_string()
 *    describes the last non-zero status of the calling thread.
 *  - Device-side bounded waits (mbarrier, TMEM allocation) never spin forever: on expiry
 *    the kernel writes a positive code to the caller's optional `status` word and exits.
 *  - Kernels are launched with programmatic stream serialization: a kernel's CTAs may become
 *    resident while the previous kernel of the stream drains, and wait on the device
 *    (griddepcontrol.wait) before their first global access, so ordering on the stream is
 *    what it would be with plain launches.  METIS_LAUNCH_OVERLAP=0 in the environment of the
 *    process (read once) gives plain launches.
 *
 * NVFP4 tensor representation (what the quantizers write and the GEMM reads)
 *  - codes : uint8 [R, C/2]; element 2i of a row is the low nibble of byte i, element
 *            2i+1 the high nibble.  A nibble is sign<<3 | e2m1 magnitude code 0..7 with
 *            magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}.
 *  - scales: one E4M3 (float8_e4m3fn) byte per 16 consecutive elements of a row, either
 *            row-major [R, C/16] (METIS_SF_ROWMAJOR) or in the tcgen05 block-scale tile
 *            order (METIS_SF_MMA): tiles of 128 rows x 4 scale columns, 512 bytes each,
 *            byte (r%32)*16 + (r/32%4)*4 + (k%4) inside a tile, tiles ordered
 *            [ceil(R/128)][4*ceil(C/256)].  Padding bytes are written as 0.
 *  - unit  : one fp32 per tensor.  value = e2m1(code) * e4m3(scale) * unit.
 */
#ifndef METIS_NVFP4_H_
#define METIS_NVFP4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define METIS_NVFP4_ABI_VERSION 2

/* element types of dense operands */
#define METIS_DTYPE_BF16 0
#define METIS_DTYPE_F32  1

/* scale-factor layouts */
#define METIS_SF_ROWMAJOR 0
#define METIS_SF_MMA      1

/* quantizer flags */
#define METIS_Q_TRANSPOSE   (1u << 0) /* quantize x^T: blocks run along the rows of x     */
#define METIS_Q_STOCHASTIC  (1u << 1) /* stochastic rounding (Philox4x32-10, seed/offset) */
#define METIS_Q_OFFSET_ON_DEVICE (1u << 2) /* offset = address of a device uint64 counter   */
#define METIS_Q_HADAMARD    (1u << 3) /* rotate every 16-element block of the transposed output by the signed
                                         Hadamard matrix before it is quantized; bits [16, 32) of the flags give
                                         the sign of each of the 16 positions (bit set: minus)                  */
#define METIS_Q_DEFER_ROWMAJOR   (1u << 4) /* dual quantizer: leave the scale pass of the row-major output to ..._dual_finish */
#define METIS_Q_DEFER_TRANSPOSED (1u << 5) /* dual quantizer: leave the scale pass of the transposed output to ..._dual_finish */
#define METIS_Q_SR16        (1u << 6) /* with METIS_Q_STOCHASTIC: 16 random bits per element, in software, instead of
                                         the hardware conversion's 8 (see below) */
#define METIS_Q_SIGN_MASK   0xFFFF0000u

/* status codes (host return values are <= 0, device status words are >= 0) */
#define METIS_OK                 0
#define METIS_ERR_BAD_ARGUMENT  -1
#define METIS_ERR_BAD_SHAPE     -2  /* block of 16 does not divide the quantized dim (quant.py:400-403) */
#define METIS_ERR_BAD_ALIGNMENT -3
#define METIS_ERR_WORKSPACE     -4
#define METIS_ERR_CUDA          -5
#define METIS_ERR_UNSUPPORTED   -6
#define METIS_ERR_TOO_LARGE     -7
#define METIS_DEV_TIMEOUT_TMA    1  /* a bounded mbarrier wait on TMA data expired     */
#define METIS_DEV_TIMEOUT_MMA    2  /* a bounded wait on tensor-core completion expired */
#define METIS_DEV_TIMEOUT_EPI    3  /* a bounded wait on the accumulator hand-off expired */

/* ---- queries ------------------------------------------------------------------------ */

/* ABI version, compiled arch (100 for sm_100a), SM count of the current device (0 if no
 * device).  Any pointer may be NULL.  Replaces nothing in the reference. */
int32_t metis_query(int32_t* abi_version, int32_t* compiled_sm, int32_t* device_sm_count);

/* Thread-local text for the last non-zero status returned to this thread. */
const char* metis_last_error_string(void);

/* Bytes of the scale array for a quantized [R, C] tensor in the given layout. */
int64_t metis_nvfp4_sf_bytes(int64_t R, int64_t C, int32_t sf_layout);

/* Bytes of scratch metis_nvfp4_quantize / metis_rmsnorm_nvfp4_quantize need for a
 * quantized [R, C] tensor (per-block fp32 amax + a 256-byte header). */
int64_t metis_nvfp4_quantize_workspace_bytes(int64_t R, int64_t C);

/* ---- quantizers ----------------------------------------------------------------------- */

/*
 * NVFP4 block quantizer.  Replaces the fake-quant graph
 * _nvfp4_nosr_quantize_dequantize (src/Metis/Metis/quant.py:6-36) reached from
 * Cast2NVFp4e2m1BlockNOSR.quantize_dequantize (quant.py:393-433), and, with
 * METIS_Q_STOCHASTIC, Cast2NVFp4e2m1Block (quant.py:273-388) whose rounding is
 * Cast2Fp4e2m1Random.quant (quant.py:139-147).  Call sites replaced:
 * bitlinear.py:392 (activations), :331 (mean-centred residual), :400-402 (output
 * gradient), :580 (weights).
 *
 *   x         [rows, cols] row-major, leading dimension ld (elements), bf16 or fp32
 *   col_mean  optional fp32 [cols]; x[r][c] - col_mean[c] is quantized instead of x
 *             (the residual of _mean_quant_single, bitlinear.py:311-336)
 *   output    tensor Q of shape [R, C] = [rows, cols], or [cols, rows] with
 *             METIS_Q_TRANSPOSE; C must be a multiple of 16.
 *   codes     uint8 [R, C/2]       scales  E4M3, metis_nvfp4_sf_bytes(R, C, sf_layout)
 *   unit      fp32 [1]             workspace  metis_nvfp4_quantize_workspace_bytes(R, C)
 *
 * Arithmetic (fp32, round-to-nearest mode bit-exact with the reference run on
 * x.float()): s = amax/6 + 1e-9 per block; unit = max(s)/448; scale = e4m3(s/unit);
 * code = round-half-even of |x|/(s/2) folded onto the e2m1 grid; sign bit = (x < 0).
 * Stochastic mode rounds a value up to its upper e2m1 neighbour with the probability of its position between
 * the two neighbours (the reference adds U[-0.5, 0.5) to the folded index before rounding, quant.py:144-145).
 * By default the hardware conversion cvt.rs.satfinite.e2m1x4.f32 does it: 8 random bits per element, up with
 * probability floor(256 p) / 256.  METIS_Q_SR16 selects the software form with 16 random bits per element
 * (floor(index + U), U in steps of 2^-16), about 8 more instructions per element.  The random bits are
 * Philox4x32-10(seed; block index, offset), one call per block of 16.  With METIS_Q_OFFSET_ON_DEVICE the offset is not
 * the argument's value but the content of the device uint64 it points to (8-byte aligned),
 * and the call adds 1 to that counter when its kernels have read it: successive calls on one
 * stream draw fresh bits although their arguments are identical, which is what a captured
 * CUDA graph needs when it is replayed (the reference's torch.rand advances a device-side
 * Philox offset in the same situation).
 *
 * METIS_Q_HADAMARD (with METIS_Q_TRANSPOSE, or on the transposed output of the dual quantizer): the
 * random Hadamard transform of the NVIDIA baseline (_apply_hadamard_blocks, bitlinear.py:125-211, used by
 * _quantize_wgrad_operand, bitlinear.py:395-405) folded into the quantizer.  Every block of 16 values b
 * (16 consecutive tokens of one channel, after the mean has been subtracted) becomes H (s . b), with H the
 * unnormalised 16 x 16 Sylvester matrix and s the signs from the flag bits, in fp32, before amax, scale and
 * codes are taken.  Two operands rotated alike along their contraction dimension give 16 times the plain
 * product (H s is orthogonal up to that factor), so the weight-gradient GEMM runs with alpha = 1/16.
 *
 * Launches: large tensors take a zero-fill of the workspace header, one streaming pass and a scale
 * pass.  Round-to-nearest, untransposed tensors of at most 16384 blocks (rollout-sized
 * activations) take ONE kernel that runs as a single thread-block cluster and does not touch the
 * workspace (it must still be passed and large enough); results are bit-identical.
 */
int32_t metis_nvfp4_quantize(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                             const float* col_mean, uint32_t flags, uint64_t seed, uint64_t offset,
                             int32_t sf_layout, uint8_t* codes, uint8_t* scales, float* unit,
                             void* workspace, int64_t workspace_bytes, void* stream);

/*
 * Both quantizations of one tensor from ONE pass over it: Q = quantize(x) [rows, cols] (blocks along
 * the columns) and Qt = quantize(x^T) [cols, rows] (blocks along the rows).  A training step needs
 * both for every operand: the forward product and dX contract over the last dimension
 * (bitlinear.py:435, :508), dW contracts over the tokens (bitlinear.py:502-505), so the reference's
 * one fake-quantized tensor becomes two packed ones here (call sites bitlinear.py:392, :331,
 * :400-402, :580).  Reads x from HBM once instead of twice; outputs are bit-identical to two calls of
 * metis_nvfp4_quantize (round to nearest; stochastic rounding draws from two disjoint Philox
 * counter spaces).  rows and cols must both be multiples of 16.  flags: METIS_Q_STOCHASTIC, METIS_Q_SR16,
 * METIS_Q_OFFSET_ON_DEVICE, METIS_Q_HADAMARD, METIS_Q_DEFER_*.  Launches: one tile pass (every CTA leaves its largest
 * block maxima in a record of its own in the workspace, so nothing is zeroed first), one scale pass that finishes both
 * outputs.
 *   codes    uint8 [rows, cols/2]   scales    metis_nvfp4_sf_bytes(rows, cols, sf_layout)   unit    fp32 [1]
 *   codes_t  uint8 [cols, rows/2]   scales_t  metis_nvfp4_sf_bytes(cols, rows, sf_layout)   unit_t  fp32 [1]
 *   token_sums_t  optional fp32 [cols]: sum over the rows of x (the tokens) of the quantized values,
 *              token_sums_t[k] = sum_m value(Qt[k, m]), what metis_nvfp4_gemv(Qt, v = NULL) returns up to the order
 *              of the additions (fixed here too).  The weight-gradient product of centred operands needs these
 *              sums (the rank-1 terms of bitlinear.py:502-505 written out); the scale pass forms them from
 *              codes that are still in L2.  NULL = not wanted.  Needs rows % 64 == 0 and no METIS_Q_HADAMARD.
 *   workspace  metis_nvfp4_quantize_dual_workspace_bytes(rows, cols)
 * With METIS_Q_DEFER_ROWMAJOR or METIS_Q_DEFER_TRANSPOSED (one of them) the call writes the codes of both outputs
 * but runs the scale pass of the other output only; scales, unit (and token_sums_t) of the deferred output
 * are written by metis_nvfp4_quantize_dual_finish, given the same shape, layout, pointers and workspace, on
 * any stream that is ordered after this call.  A forward product needs the row-major output of its activation
 * at once and the transposed one only in the backward pass; the weight-gradient product needs the transposed
 * output of the output gradient first: the deferred half leaves the critical path.
 */
int64_t metis_nvfp4_quantize_dual_workspace_bytes(int64_t rows, int64_t cols);
int32_t metis_nvfp4_quantize_dual_finish(int64_t rows, int64_t cols, uint32_t deferred, int32_t sf_layout,
                                         uint8_t* scales, float* unit, const uint8_t* codes_t, uint8_t* scales_t,
                                         float* unit_t, float* token_sums_t, void* workspace,
                                         int64_t workspace_bytes, void* stream);
int32_t metis_nvfp4_quantize_dual(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                  const float* col_mean, uint32_t flags, uint64_t seed, uint64_t offset,
                                  int32_t sf_layout, uint8_t* codes, uint8_t* scales, float* unit,
                                  uint8_t* codes_t, uint8_t* scales_t, float* unit_t, float* token_sums_t,
                                  void* workspace, int64_t workspace_bytes, void* stream);

/*
 * The same round-to-nearest, row-major quantizer for callers that cannot hand over a workspace
 * and must not trigger an allocation: a serving process whose device memory was divided up once
 * at start-up, a host binding that holds raw device pointers but no allocator, code for which
 * cudaMalloc's implicit synchronisation is unacceptable.  This entry point has no counterpart in
 * the reference (which allocates freely through PyTorch).
 *
 * The scratch is a fixed array inside the library: 4 MiB + 256 bytes of device memory on every GPU
 * that loads the library, held until the process exits.  Limit: rows * cols <=
 * METIS_STATIC_MAX_ELEMENTS; larger tensors are rejected with METIS_ERR_TOO_LARGE.  The call
 * allocates nothing (no cudaMalloc/cudaFree, no allocating library routine).
 *  - The first call on each device looks the array's address up (cudaGetSymbolAddress) with that
 *    device current; make that first call before any stream capture begins.  Under the runtime's
 *    lazy module loading the array itself comes into being with the library's first kernel on a
 *    device, whichever entry point launches it: "allocates nothing" is a statement about this call.
 *  - All calls on a device share the one array and it keeps the previous call's contents; the call
 *    clears the part that has to start at zero.  Two calls that overlap on the GPU (different
 *    streams, or threads) race on it: serialise them.
 * Arguments and results are those of metis_nvfp4_quantize without col_mean, flags, seed, offset
 * and workspace; outputs are bit-identical to it.
 */
#define METIS_STATIC_MAX_ELEMENTS (16 * 1024 * 1024)
int32_t metis_nvfp4_quantize_static(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                                    int32_t sf_layout, uint8_t* codes, uint8_t* scales, float* unit,
                                    void* stream);

/*
 * Fused RMSNorm -> NVFP4 quantizer: reads each activation row from HBM once.
 * Replaces RMSNorm.forward (src/Metis/models/llama.py:23-31) followed by the activation
 * quantizer (bitlinear.py:392 -> quant.py:6-36).
 *   y = round_to_x_dtype(x * rsqrt(mean(x^2) + eps)) * gamma     (llama.py:23-31)
 * gamma is bf16 or fp32 [cols]; when x and gamma are both bf16 the product is rounded to
 * bf16 as torch does.  norm_out (optional, dtype of that product, [rows, cols]) receives y.
 * Round-to-nearest only; other outputs as metis_nvfp4_quantize without METIS_Q_TRANSPOSE.
 * Up to 32 rows of 4096 elements (more rows when they are shorter, none past 8192 elements) run as
 * one cluster kernel like the small tensors of metis_nvfp4_quantize.
 */
int32_t metis_rmsnorm_nvfp4_quantize(const void* x, int32_t x_dtype, int64_t rows, int64_t cols,
                                     int64_t ld, const void* gamma, int32_t gamma_dtype, float eps,
                                     int32_t sf_layout, uint8_t* codes, uint8_t* scales, float* unit,
                                     void* norm_out, void* workspace, int64_t workspace_bytes,
                                     void* stream);

/*
 * RMSNorm for the mean-centred quantizer: y = round_to_x_dtype(x * rsqrt(mean(x^2) + eps)) * gamma
 * (src/Metis/models/llama.py:23-31) together with what the next steps need, from one read of x:
 *   norm_out  y, [rows, cols] in the dtype of the product (bf16 when x and gamma are bf16, else fp32)
 *   mean      fp32 [cols], the column mean of y (input_flat.mean(dim=0), bitlinear.py:326): the mean-centred
 *             quantizer cannot start before it exists, so normalisation and quantization are two passes
 *             here; metis_nvfp4_quantize[_dual](y, col_mean = mean) is the second and reads y once
 *   rstd      optional fp32 [rows], rsqrt(mean(x^2) + eps) of every row, for the backward of the norm
 * Deterministic summation order.  workspace: metis_rmsnorm_mean_workspace_bytes(rows, cols).
 */
int64_t metis_rmsnorm_mean_workspace_bytes(int64_t rows, int64_t cols);
int32_t metis_rmsnorm_mean(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                           const void* gamma, int32_t gamma_dtype, float eps, void* norm_out, float* rstd,
                           float* mean, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * codes/scales/unit -> dense [R, C] (ld elements per row), bf16 or fp32:
 * out = e2m1(code) * (e4m3(scale) * unit), the last two steps of quant.py:19-35.
 * If add_row_vec (fp32 [C]) is given it is added to every row (me + QDQ(x - me),
 * bitlinear.py:332).
 */
int32_t metis_nvfp4_dequantize(const uint8_t* codes, const uint8_t* scales, const float* unit,
                               int32_t sf_layout, int64_t R, int64_t C, const float* add_row_vec,
                               void* out, int32_t out_dtype, int64_t ld, void* stream);

/*
 * Column means of x [rows, cols]: mean[c] = (sum_r x[r][c]) / rows in fp32
 * (input_flat.mean(dim=0), bitlinear.py:326).  Deterministic summation order.
 * workspace: at least metis_col_mean_workspace_bytes(rows, cols) bytes (unused, one launch, up to 128 rows).
 */
int64_t metis_col_mean_workspace_bytes(int64_t rows, int64_t cols);
int32_t metis_col_mean(const void* x, int32_t x_dtype, int64_t rows, int64_t cols, int64_t ld,
                       float* mean, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * out[r] = sum_c v[c] * value(Q[r][c])  for a quantized [R, C] tensor (v == NULL: all ones).
 * Gives the rank-1 terms of the mean-centred products: me @ Wq^T (bitlinear.py:332 with
 * :435) and the column sums of the four-term dW expansion.  fp32 output [R].
 */
int32_t metis_nvfp4_gemv(const uint8_t* codes, const uint8_t* scales, const float* unit,
                         int32_t sf_layout, int64_t R, int64_t C, const float* v, float* out,
                         void* stream);

/* ---- GEMM --------------------------------------------------------------------------------- */

/*
 * The rank-r factor of the fused side product: t[m][j] = bf16( float(bf16(yv[m][j] * s[j])) /
 * (unit_a * unit_b) ), i.e. torch.mul(self.s, y) of the low-rank branch (bitlinear.py:752-760)
 * in the activation dtype, expressed in the accumulator units of the residual GEMM that adds
 * T @ U^T.  yv and t are bf16 [M, r] (row pitch ld elements, r a multiple of 8); s is bf16 or
 * fp32 [r] (fp32 is rounded to bf16 first, as s.to(bf16) does); unit_a, unit_b device fp32.
 */
int32_t metis_lowrank_scale(const void* yv, int64_t M, int64_t r, int64_t ld, const void* s,
                            int32_t s_dtype, const float* unit_a, const float* unit_b, void* t,
                            void* stream);

/*
 * D[M,N] = g * ( sum_k A[m,k] B[n,k]  +  sum_j T[m,j] U[n,j] )
 *          + cvec0[m]*rvec0[n] + cvec1[m]*rvec1[n]  ( + C[m,n] )
 * with g = alpha * (*a_unit) * (*b_unit).
 *
 * A [M,K] and B [N,K] are NVFP4 tensors with METIS_SF_MMA scales; the K loop runs on
 * tcgen05 block-scaled MMA (kind::mxf4nvf4, 16-element blocks, UE4M3 scales) with
 * TMA-fed shared-memory stages and the accumulator in tensor memory.  T [M,rank] and
 * U [N,rank] (bf16, rank % 8 == 0, rank <= 256, given in accumulator units, i.e. already
 * divided by (*a_unit)*(*b_unit)) are a rank-r side product issued as kind::f16 MMAs into
 * the same accumulator.  cvec NULL means a vector of ones; a NULL rvec disables its term.
 *
 * Replaces torch.matmul at bitlinear.py:435 (forward), :502-505 (dW), :508 (dX), :748
 * (merged rollout weight) and the vlinear -> s -> ulinear -> add chain (bitlinear.py:752-760),
 * whose native ancestor is lora_fuse (src/Metis/kernels/src/lora/lora_fuse.cu:106-291).
 */
typedef struct metis_gemm_args {
  int64_t M, N, K;
  const uint8_t* a_codes;  const uint8_t* a_scales;  const float* a_unit;
  const uint8_t* b_codes;  const uint8_t* b_scales;  const float* b_unit;
  float alpha;
  int32_t rank;             /* 0: no side product */
  const void* lr_t;  int64_t ldt;   /* bf16 [M, rank] */
  const void* lr_u;  int64_t ldu;   /* bf16 [N, rank] */
  const float* cvec0;  const float* rvec0;
  const float* cvec1;  const float* rvec1;
  const void* c;  int64_t ldc;      /* optional addend, dtype d_dtype */
  void* d;        int64_t ldd;
  int32_t d_dtype;          /* METIS_DTYPE_BF16 or METIS_DTYPE_F32 */
  int32_t reserved;         /* 0.  Two test hooks are accepted: 1 makes the first bounded wait expire (the status
                               word then reads METIS_DEV_TIMEOUT_TMA; results are not meaningful), 8 runs the
                               single-CTA kernel where CTA pairs would be chosen.  Anything else is rejected. */
  int32_t* status;          /* optional device int32: 0, or a METIS_DEV_* code */
  void* stream;
  void* workspace;          /* optional scratch, 16-byte aligned: metis_nvfp4_gemm_workspace_bytes */
  int64_t workspace_bytes;
  int32_t sm_limit;         /* upper bound on the SMs this launch's persistent CTAs occupy; 0: all of them.  A
                               data-parallel step that runs a collective beside this product leaves the
                               collective's kernel its SMs this way.  Per call: launches on other streams and
                               threads are not affected. */
  int32_t reserved2;        /* 0 */
} metis_gemm_args;

int32_t metis_nvfp4_gemm(const metis_gemm_args* args);

/*
 * Scratch that lets a decode-sized product (M <= 128: the rollout path, bitlinear.py:704-751,
 * and the weight gradients of the rank-r factors) split its K loop over otherwise idle SMs:
 * bytes of fp32 partial sums, 0 when the shape is not split.  Without the scratch the same
 * product runs unsplit on fewer SMs; the result is the same up to fp32 summation order.
 */
int64_t metis_nvfp4_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);

/* ---- backward of the unquantized low-rank branch ------------------------------------------------------ */

/*
 * D[Mg, Ng] = A B^T in bf16 with fp32 accumulation on tcgen05 (kind::f16), Ng <= 256: the skinny
 * products of the rank-r branch.  Either operand may be stored with the contraction in its rows:
 *   a_mn_major = 0: a is [Mg, Kg] (row pitch lda);  1: a is [Kg, Mg]
 *   b_mn_major = 0: b is [Ng, Kg] (row pitch ldb);  1: b is [Kg, Ng]
 * so neither grad_output nor a factor is transposed in memory first.  d is fp32 [Mg, ldd].  The K loop
 * is split over the SMs; workspace holds the fp32 partial sums, added in a fixed order.
 * Building block of the two entry points below; replaces torch.matmul in autograd's backward of
 * ulinear (src/Metis/Metis/bitlinear.py:756-757).
 */
int64_t metis_bf16_panel_gemm_workspace_bytes(int64_t Mg, int64_t Ng, int64_t Kg);
int32_t metis_bf16_panel_gemm(const void* a, int32_t a_mn_major, int64_t lda, const void* b, int32_t b_mn_major,
                              int64_t ldb, int64_t Mg, int64_t Ng, int64_t Kg, float* d, int64_t ldd,
                              void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);

/*
 * Gradient through ulinear and the scaling by s (bitlinear.py:752-757: y = torch.mul(self.s, y);
 * y = self.ulinear(y)), as autograd computes it in bf16:
 *   d_ts = bf16(G U)                   G = grad_output [M, N] bf16, U = ulinear.weight [N, r] bf16
 *   d_yv = bf16(d_ts * bf16(s))        the output gradient of vlinear, bf16 [M, r]
 *   ds   = sum_m bf16(d_ts * y_v)      fp32 [r]; y_v = vlinear's output, bf16 [M, r]
 * One pass over G.  s is bf16 or fp32 [r].  r a multiple of 8 up to 256, N a multiple of 8.
 */
int64_t metis_lowrank_dts_workspace_bytes(int64_t M, int64_t N, int64_t r);
int32_t metis_lowrank_dts(const void* g, int64_t ldg, int64_t M, int64_t N, const void* u, int64_t ldu, int64_t r,
                          const void* yv, int64_t ldyv, const void* s, int32_t s_dtype, void* d_yv, int64_t ldd,
                          float* ds, void* workspace, int64_t workspace_bytes, int32_t* status, void* stream);

/*
 * Weight gradient of ulinear: dU = G^T ts [N, r] with ts = bf16(s * y_v) [M, r] (bitlinear.py:756-757
 * through autograd), contraction over the tokens, both operands read as they lie in memory.
 * grad_u is bf16 or fp32 [N, ldgu].  One pass over G.
 */
int64_t metis_lowrank_du_workspace_bytes(int64_t M, int64_t N, int64_t r);
int32_t metis_lowrank_du(const void* g, int64_t ldg, int64_t M, int64_t N, const void* ts, int64_t ldts, int64_t r,
                         void* grad_u, int32_t u_dtype, int64_t ldgu, void* workspace, int64_t workspace_bytes,
                         int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* METIS_NVFP4_H_ */
