// Shared device/host helpers for the tritonllm_b200 kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/tritonllm_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "tritonllm_b200 kernels are written for sm_100a"
#endif

#define B2_API extern "C" __attribute__((visibility("default")))

// Codes a kernel ORs into the per-device status word when it gives up a bounded wait.
#define B2_DEV_TIMEOUT_FULL 0x1    // consumer gave up waiting for a TMA tile
#define B2_DEV_TIMEOUT_EMPTY 0x2   // producer gave up waiting for a free stage
#define B2_DEV_TIMEOUT_DRAIN 0x4   // producer gave up draining its copies in flight
#define B2_DEV_TIMEOUT_MMA 0x8     // epilogue gave up waiting for tensor-core completion
#define B2_DEV_BAD_INDEX 0x10      // a self-check found an index out of range

namespace b2 {

// ---- host side ------------------------------------------------------------------
// Pointer to the status word of the current device (NULL on failure).
int* device_status_ptr();
int sm_count();
int tunable(int id);
// Optional per-CTA timestamp buffer (8 x int64 per CTA) set with b2_set_trace_buffer; NULL when tracing is off.
long long* trace_buffer(size_t* slots);
enum Tunable { TUNE_ATTN_DECODE_CTAS_PER_SM = 0, TUNE_GEMV_KSPLIT_QKV, TUNE_GEMV_KSPLIT_OUT, TUNE_TMA_L2_PROMOTION, TUNE_ATTN_DECODE_STAGES, TUNE_GEMM_PAIR, TUNE_MOE_FP4_STAGES, TUNE_LAUNCH_OVERLAP, TUNE_MOE_FP4_TOK, TUNE_UNEMBED_STAGES, TUNE_MOE_PREFETCH, TUNE_ATTN_PREFILL_EXP16, TUNE_RMSNORM_WARPS, TUNE_RMSNORM_RING_MIN_ROWS, TUNE_UNEMBED_TILES, TUNE_MOE_FP4_PERSIST, TUNE_MOE_FP4_KSPLIT, TUNE_ATTN_PREFILL_POLY, TUNE_MOE_FP4_FUSE, TUNE_COUNT };

// Encodes a tiled tensor map for a bf16 tensor of up to 5 dims (dim 0 innermost, stride 1).
// strides_bytes[i] is the byte stride of dim i+1.  Returns a B2 status.
int make_tensor_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);
// The same for any element type (uint8 tiles; CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B for FP4 codes, which TMA
// spreads into the 8-bytes-data / 8-bytes-gap layout the FP4 MMA reads: dims in elements, inner extent and box
// multiples of 128 elements, base and strides multiples of 32 bytes).
int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

// Launch with programmatic stream serialization: the grid may be scheduled while the kernel before it on the
// stream is still draining, runs its set-up, and blocks in overlap_wait() until that kernel has completed and
// its writes are visible.  Only for kernels that call overlap_wait() in every thread before they touch global
// memory that an earlier kernel may write or read.  Off unless the tunable "launch_overlap" is 1: replayed from a CUDA
// graph the decode step measured the same with and without it.
template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = tunable(TUNE_LAUNCH_OVERLAP) ? 1 : 0;
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface through launch_status()
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? B2_OK : static_cast<int>(e);
}

// ---- device side ----------------------------------------------------------------
#ifdef __CUDACC__

constexpr uint32_t SPIN_LIMIT = 1u << 22;  // bounded waits: try_wait attempts before giving up
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // ... and the wall-time limit of one wait (2 s)

// Programmatic dependent launch: overlap_start() lets the next kernel on the stream be scheduled as soon as
// every CTA of this grid has started; overlap_wait() blocks until the kernels before this one have completed
// and their memory operations are visible (a no-op for a grid launched the ordinary way).
__device__ __forceinline__ void overlap_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void overlap_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ long long global_timer_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// bf16 pair <-> fp32 (a bf16 is the high half of an fp32)
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// Sum of the two squares of a bf16 pair, each square a bf16 product (one packed HMUL2, rounded to
// nearest even) widened to fp32.
__device__ __forceinline__ float sq_pair_bf16(uint32_t w) {
  __nv_bfloat162 p = *reinterpret_cast<__nv_bfloat162*>(&w);
  p = __hmul2(p, p);
  const uint32_t u = *reinterpret_cast<uint32_t*>(&p);
  return bf16lo(u) + bf16hi(u);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// streaming 128-bit load that does not allocate in L1 (data used once)
__device__ __forceinline__ uint4 ldg128_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ void stg128(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// ---- mbarrier ---------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out (try_wait attempts, or WAIT_LIMIT_NS of wall time, whichever
// comes first) or another thread of the CTA raised *abort_flag.
__device__ __forceinline__ uint64_t wait_clock_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (*abort_flag) return false;
      const uint64_t now = wait_clock_ns();
      if (t0 == 0)
        t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS)
        return false;
    }
  }
  return false;
}

// ---- TMA ------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Asks for a tile to be brought from HBM into L2 without a destination in shared memory: a producer that issues
// these several pipeline steps ahead keeps many more HBM bytes in flight than its ring of shared-memory stages
// holds, and the later copy into shared memory finds the tile in L2.
__device__ __forceinline__ void tma_prefetch_l2_4d(const CUtensorMap* m, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(m), "r"(c0), "r"(c1),
               "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(m), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
// Untiled bulk copies (addresses 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most N of this thread's bulk-store groups still have to READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Orders generic-proxy writes to shared memory before later async-proxy (TMA) accesses.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- warp-level tensor-core pieces for the memory-bound kernels -------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

#endif  // __CUDACC__
}  // namespace b2
