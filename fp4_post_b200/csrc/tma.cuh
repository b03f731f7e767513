// TMA / mbarrier plumbing shared by the GEMM and the transposed quantizer: PTX wrappers, the
// bounded wait, and host-side tensor-map creation.
#pragma once

#include "common.cuh"

#include <cuda.h>

namespace metis {

constexpr uint64_t kWaitLimitNs = 400ull * 1000 * 1000;   // every device-side wait gives up after 0.4 s

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
// The *_addr forms take 32-bit shared-memory addresses, so that a caller can keep them in
// (uniform) registers across a loop instead of converting generic pointers every time.
__device__ __forceinline__ void mbar_expect_tx_addr(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_addr(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) { mbar_expect_tx_addr(smem_u32(bar), bytes); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) { mbar_arrive_addr(smem_u32(bar)); }
// One lane of a converged warp (always the same one).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  // may suspend the thread in hardware for up to the hinted time (ns) before it answers
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(2000u) : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false if the phase did not complete within kWaitLimitNs or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = global_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 15u) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > kWaitLimitNs) return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d_addr(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load_addr(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
  tma_load_2d_addr(smem_u32(dst), map, x, y, smem_u32(bar));
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  bulk_load_addr(smem_u32(dst), src, bytes, smem_u32(bar));
}
// TMA tile store shared -> global as one bulk group of the calling thread; elements of the box that lie
// outside the tensor are not written.  x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];\n\tcp.async.bulk.commit_group;"
               ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}
// the calling thread's bulk stores, all but the newest `kPending` groups, have read their shared memory
template <int kPending> __device__ __forceinline__ void bulk_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
// all bulk stores of the calling thread are complete
__device__ __forceinline__ void bulk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// generic-proxy writes to shared memory made before this are visible to the bulk copies issued after it
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

#endif  // __CUDACC__

// ---- host side ----------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D row-major tensor [rows, inner] with a row pitch in bytes; box = [box_rows, box_inner];
// swizzle = 128 or 64 (bytes) or 0 for none; out-of-range elements read as zero and are not written.
static inline int32_t make_map(CUtensorMap* map, CUtensorMapDataType dt, int64_t esz, const void* base, int64_t inner,
                        int64_t rows, int64_t pitch_bytes, int box_inner, int box_rows, const char* what,
                        int swizzle = 128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(METIS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  (void)esz;
  CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
#ifdef METIS_TIMING_KNOBS
  if (const char* e = getenv("METIS_DEV_L2PROMO")) promo = (CUtensorMapL2promotion)atoi(e);
#endif
  const CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(METIS_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with %d", what, (int)r);
  return METIS_OK;
}


}  // namespace metis
