// Library-level entry points: version, status text, the per-device status word,
// tuning knobs and the TMA tensor-map encoder shared by the kernels.
#include <atomic>
#include <cstring>
#include <mutex>

#include "b2_common.cuh"

namespace b2 {

// One status word per device; kernels OR a code into it when a bounded wait runs out.
__device__ int g_device_status = 0;

static constexpr int MAX_DEVICES = 64;
static std::mutex g_mutex;
static int* g_status_ptr[MAX_DEVICES] = {};
static int g_sm_count[MAX_DEVICES] = {};
static std::atomic<int> g_tunables[TUNE_COUNT];
static std::atomic<bool> g_tunables_init{false};

static void init_tunables() {
  bool expected = false;
  if (g_tunables_init.compare_exchange_strong(expected, true)) {
    g_tunables[TUNE_ATTN_DECODE_CTAS_PER_SM] = 1;
    g_tunables[TUNE_GEMV_KSPLIT_QKV] = 0;  // 0 = derive from the SM count
    g_tunables[TUNE_GEMV_KSPLIT_OUT] = 0;
    g_tunables[TUNE_ATTN_DECODE_STAGES] = 3;
    g_tunables[TUNE_GEMM_PAIR] = 1;  // 1: large GEMMs run on CTA pairs (cta_group::2); 2: pairs, one k-block per stage; 0: one CTA per tile
    g_tunables[TUNE_MOE_FP4_STAGES] = 0;  // 0: chosen from the token-tile size
    g_tunables[TUNE_MOE_FP4_TOK] = 0;      // 8 / 16 / 32 / 64: tokens of an expert per CTA (0: by the batch size; 64: the one-shot kernel)
    g_tunables[TUNE_UNEMBED_STAGES] = 0;   // ring depth of the unembedding kernel (0: as deep as shared memory allows)
    g_tunables[TUNE_MOE_PREFETCH] = 0;     // k-blocks of expert weights requested into L2 ahead of the shared-memory ring (0: off; 3-12 measured no faster)
    g_tunables[TUNE_ATTN_PREFILL_EXP16] = 0;   // 1: prefill attention computes its exponentials two at a time on fp16 pairs (measured slower)
    g_tunables[TUNE_RMSNORM_WARPS] = 0;          // warps per CTA of the streaming RMSNorm (0: 16)
    g_tunables[TUNE_RMSNORM_RING_MIN_ROWS] = 0;  // rows from which RMSNorm streams rows through shared memory (0: 512)
    g_tunables[TUNE_UNEMBED_TILES] = 0;          // 1: one weight tile per CTA in the unembedding at every batch size (0: two above 128 sequences)
    g_tunables[TUNE_MOE_FP4_PERSIST] = 4;  // persistent FP4 expert kernel: CTAs per SM (4 / 2 / 1); 0: the one-shot kernel
    g_tunables[TUNE_MOE_FP4_KSPLIT] = 0;   // persistent FP4 expert kernel, last GEMM: 1 = whole k range per unit; else two halves
    g_tunables[TUNE_ATTN_PREFILL_POLY] = 0;   // prefill attention: 2 / 4 = every 2nd / 4th pair of exponentials on the FMA pipe; -1: none; 0: built-in default
    g_tunables[TUNE_MOE_FP4_FUSE] = 0;     // the two expert GEMMs in one persistent launch: 0 = for 32-token parts up to 384 tokens, 1 = never, 2 = always
    g_tunables[TUNE_LAUNCH_OVERLAP] = 0;   // 1: decode kernels are launched with programmatic stream serialization
    g_tunables[TUNE_TMA_L2_PROMOTION] = 0;  // 0 none, 1 = 64 B, 2 = 128 B, 3 = 256 B
  }
}

static std::atomic<long long*> g_trace{nullptr};
static std::atomic<size_t> g_trace_slots{0};
long long* trace_buffer(size_t* slots) {
  *slots = g_trace_slots.load();
  return g_trace.load();
}

int tunable(int id) {
  init_tunables();
  return g_tunables[id].load();
}

int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    g_status_ptr[dev] = static_cast<int*>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 148;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_sm_count[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = 148;
    }
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static std::atomic<EncodeTiledFn> g_encode{nullptr};

static EncodeTiledFn get_encode() {
  EncodeTiledFn fn = g_encode.load();
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || !p) {
    (void)cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(p);
  g_encode.store(fn);
  return fn;
}

int make_tensor_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  return make_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, rank, dims, strides_bytes, box, swizzle);
}

int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return B2_ERR_DRIVER;
  if (!aligned16(base)) return B2_ERR_ALIGN;
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) {
      if (strides_bytes[i] % 16) return B2_ERR_ALIGN;
      s[i] = strides_bytes[i];
    }
  }
  const int pv = tunable(TUNE_TMA_L2_PROMOTION);
  const CUtensorMapL2promotion promo = pv <= 0   ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                       : pv == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                       : pv == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                 : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  CUresult r = fn(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, s,
                  b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B2_OK : B2_ERR_SHAPE;
}

}  // namespace b2

B2_API int b2_version(void) { return 100; }

B2_API const char* b2_status_string(int status) {
  switch (status) {
    case B2_OK: return "ok";
    case B2_ERR_NULL: return "a required pointer is NULL";
    case B2_ERR_SHAPE: return "a size is non-positive or inconsistent";
    case B2_ERR_UNSUPPORTED: return "shape outside what the kernels implement";
    case B2_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case B2_ERR_WORKSPACE: return "workspace missing or too small";
    case B2_ERR_DRIVER: return "a driver entry point could not be resolved";
    case B2_ERR_STATIC_LIMIT: return "problem larger than the fixed scratch of the no-allocation entry point";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown status";
}

B2_API int b2_device_status(int reset, int* status_out) {
  if (!status_out) return B2_ERR_NULL;
  int* p = b2::device_status_ptr();
  if (!p) return B2_ERR_DRIVER;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpy(status_out, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (reset) {
    e = cudaMemset(p, 0, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return B2_OK;
}

namespace b2 {
__global__ void selftest_wait_kernel(int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const bool ok = mbar_wait_bounded(&bar, 0, &abort_flag);  // nothing arrives: runs into the time limit
  if (!ok && threadIdx.x == 0) atomicOr(status, B2_DEV_TIMEOUT_FULL);
}
}  // namespace b2

B2_API int b2_selftest_wait_timeout(void* stream) {
  int* status = b2::device_status_ptr();
  if (!status) return B2_ERR_DRIVER;
  b2::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status);
  return b2::launch_status();
}

B2_API int b2_set_tunable(const char* name, int value) {
  if (!name) return B2_ERR_NULL;
  b2::init_tunables();
  static const char* names[b2::TUNE_COUNT] = {"attn_decode_ctas_per_sm", "gemv_ksplit_qkv", "gemv_ksplit_out",
                                                  "tma_l2_promotion", "attn_decode_stages", "gemm_pair", "moe_fp4_stages", "launch_overlap", "moe_fp4_tok", "unembed_stages", "moe_prefetch", "attn_prefill_exp16", "rmsnorm_warps", "rmsnorm_ring_min_rows", "unembed_tiles", "moe_fp4_persist", "moe_fp4_ksplit", "attn_prefill_poly", "moe_fp4_fuse"};
  for (int i = 0; i < b2::TUNE_COUNT; ++i) {
    if (std::strcmp(name, names[i]) == 0) {
      b2::g_tunables[i] = value;
      return B2_OK;
    }
  }
  return B2_ERR_UNSUPPORTED;
}

B2_API int b2_set_trace_buffer(void* device_buffer, size_t bytes) {
  b2::g_trace_slots = device_buffer ? bytes / (8 * sizeof(long long)) : 0;
  b2::g_trace = static_cast<long long*>(device_buffer);
  return B2_OK;
}
