// RMSNorm (optionally fused with the residual add that precedes it) and in-place RoPE.
//
// Both are HBM-bound.  RMSNorm keeps one row per warp entirely in registers
// (128-bit loads, one read and one write per element, warp-shuffle reduction,
// no shared memory and no block barrier).  RoPE streams q and k once with
// 128-bit loads; the cos/sin row of a token is shared by its 72 heads and
// stays in L1.
#include "b2_common.cuh"

namespace b2 {

// One warp per row; VPL = 16-byte vectors held per lane (row = up to 32*VPL*8 bf16).
template <int VPL, bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ delta,
                                                      const float4* __restrict__ gain, uint4* __restrict__ h_out,
                                                      uint4* __restrict__ y_out, int64_t rows, int nvec, float inv_dim,
                                                      float eps) {
  overlap_start();
  overlap_wait();
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const uint4* xr = x + row * nvec;
  uint4 v[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    v[i] = (c < nvec) ? ldg128_stream(xr + c) : make_uint4(0, 0, 0, 0);
  }
  if (ADD) {
    const uint4* dr = delta + row * nvec;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        const uint4 d = ldg128_stream(dr + c);
        // bf16 tensor add: fp32 sum rounded to bf16, as the next norm reads it
        v[i].x = pack_bf16(bf16lo(v[i].x) + bf16lo(d.x), bf16hi(v[i].x) + bf16hi(d.x));
        v[i].y = pack_bf16(bf16lo(v[i].y) + bf16lo(d.y), bf16hi(v[i].y) + bf16hi(d.y));
        v[i].z = pack_bf16(bf16lo(v[i].z) + bf16lo(d.z), bf16hi(v[i].z) + bf16hi(d.z));
        v[i].w = pack_bf16(bf16lo(v[i].w) + bf16lo(d.w), bf16hi(v[i].w) + bf16hi(d.w));
        stg128(h_out + row * nvec + c, v[i]);
      }
    }
  }
  // Squares are bf16 products (rounded) summed in fp32, as the kernel this replaces does.
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    ss += sq_pair_bf16(v[i].x);
    ss += sq_pair_bf16(v[i].y);
    ss += sq_pair_bf16(v[i].z);
    ss += sq_pair_bf16(v[i].w);
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss * inv_dim + eps);
  uint4* yr = y_out + row * nvec;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      const float4 g0 = __ldg(gain + 2 * c), g1 = __ldg(gain + 2 * c + 1);
      uint4 o;
      o.x = pack_bf16(bf16lo(v[i].x) * r * g0.x, bf16hi(v[i].x) * r * g0.y);
      o.y = pack_bf16(bf16lo(v[i].y) * r * g0.z, bf16hi(v[i].y) * r * g0.w);
      o.z = pack_bf16(bf16lo(v[i].z) * r * g1.x, bf16hi(v[i].z) * r * g1.y);
      o.w = pack_bf16(bf16lo(v[i].w) * r * g1.z, bf16hi(v[i].w) * r * g1.w);
      stg128(yr + c, o);
    }
  }
}


// Many rows: persistent CTAs, one row per warp at a time, rows staged through shared memory by
// bulk async copies.  Each warp owns a ring of row buffers guarded by mbarriers.  A row is pulled
// from its buffer into registers, the buffer is handed straight back to the copy engine for the
// next row of the warp, and the normalised row leaves through coalesced 128-bit stores: every
// buffer of the SM is a load in flight almost all the time, which is what an HBM-bound kernel
// needs, and the warps never run in lock step.  Reading a whole row before writing it keeps
// `out == x` legal.
constexpr int RN_MAX_STAGES = 6;

template <bool ADD, int RN_WARPS, int VPL>
__global__ void __launch_bounds__(RN_WARPS * 32, 1)
rmsnorm_ring_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                    const float4* __restrict__ gain, __nv_bfloat16* __restrict__ h_out,
                    __nv_bfloat16* __restrict__ y_out, int64_t rows, int dim, float inv_dim, float eps, int stages,
                    int* status) {
  extern __shared__ __align__(128) uint8_t rn_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row_bytes = static_cast<uint32_t>(dim) * 2;
  const int nvec = dim >> 3;
  const size_t per_warp = static_cast<size_t>(stages) * row_bytes * (ADD ? 2 : 1);
  uint8_t* xbuf = rn_smem + warp * per_warp;
  uint8_t* dbuf = xbuf + static_cast<size_t>(stages) * row_bytes;
  uint64_t* bar_base = reinterpret_cast<uint64_t*>(rn_smem + RN_WARPS * per_warp);
  uint64_t* bars = bar_base + warp * RN_MAX_STAGES;
  int* abort_flag_s = reinterpret_cast<int*>(bar_base + RN_WARPS * RN_MAX_STAGES);
  if (threadIdx.x == 0) *abort_flag_s = 0;
  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* abort_flag = abort_flag_s;

  const int64_t gw = blockIdx.x + static_cast<int64_t>(gridDim.x) * warp;  // consecutive rows go to different SMs
  const int64_t GW = static_cast<int64_t>(gridDim.x) * RN_WARPS;
  const int64_t n_my = rows > gw ? (rows - gw + GW - 1) / GW : 0;
  const uint32_t tx = row_bytes * (ADD ? 2u : 1u);

  auto issue = [&](int64_t i) {  // lane 0 only; row i of this warp goes to buffer i % stages
    const int s = static_cast<int>(i % stages);
    const int64_t row = gw + i * GW;
    mbar_arrive_expect_tx(&bars[s], tx);
    bulk_load(xbuf + static_cast<size_t>(s) * row_bytes, x + row * dim, row_bytes, &bars[s]);
    if (ADD) bulk_load(dbuf + static_cast<size_t>(s) * row_bytes, delta + row * dim, row_bytes, &bars[s]);
  };
  int64_t issued = 0;
  if (lane == 0)
    for (; issued < n_my && issued < stages; ++issued) issue(issued);
  issued = __shfl_sync(0xffffffffu, issued, 0);

  int64_t i = 0;
  for (; i < n_my; ++i) {
    const int s = static_cast<int>(i % stages);
    const bool ok = mbar_wait_bounded(&bars[s], static_cast<uint32_t>((i / stages) & 1), abort_flag);
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0 && !*abort_flag) atomicOr(status, B2_DEV_TIMEOUT_FULL);
      *abort_flag = 1;
      break;
    }
    const int64_t row = gw + i * GW;
    const uint4* xr = reinterpret_cast<const uint4*>(xbuf + static_cast<size_t>(s) * row_bytes);
    const uint4* dr = reinterpret_cast<const uint4*>(dbuf + static_cast<size_t>(s) * row_bytes);
    uint4 v[VPL];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + 32 * j;
      v[j] = c < nvec ? xr[c] : make_uint4(0, 0, 0, 0);
      if (ADD && c < nvec) {
        const uint4 d = dr[c];
        v[j].x = pack_bf16(bf16lo(v[j].x) + bf16lo(d.x), bf16hi(v[j].x) + bf16hi(d.x));
        v[j].y = pack_bf16(bf16lo(v[j].y) + bf16lo(d.y), bf16hi(v[j].y) + bf16hi(d.y));
        v[j].z = pack_bf16(bf16lo(v[j].z) + bf16lo(d.z), bf16hi(v[j].z) + bf16hi(d.z));
        v[j].w = pack_bf16(bf16lo(v[j].w) + bf16lo(d.w), bf16hi(v[j].w) + bf16hi(d.w));
      }
      ss += sq_pair_bf16(v[j].x);
      ss += sq_pair_bf16(v[j].y);
      ss += sq_pair_bf16(v[j].z);
      ss += sq_pair_bf16(v[j].w);
    }
    // every lane has consumed its part of the buffer (ss depends on all of v): hand it back
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && issued < n_my) issue(issued);
    if (issued < n_my) ++issued;  // same value in every lane
    ss = warp_sum(ss);
    const float r = rsqrtf(ss * inv_dim + eps);
    uint4* yr = reinterpret_cast<uint4*>(y_out + row * dim);
    uint4* hr = reinterpret_cast<uint4*>(h_out + row * dim);
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + 32 * j;
      if (c < nvec) {
        if (ADD) stg128(hr + c, v[j]);
        const float4 g0 = __ldg(gain + 2 * c), g1 = __ldg(gain + 2 * c + 1);
        uint4 o;
        o.x = pack_bf16(bf16lo(v[j].x) * r * g0.x, bf16hi(v[j].x) * r * g0.y);
        o.y = pack_bf16(bf16lo(v[j].y) * r * g0.z, bf16hi(v[j].y) * r * g0.w);
        o.z = pack_bf16(bf16lo(v[j].z) * r * g1.x, bf16hi(v[j].z) * r * g1.y);
        o.w = pack_bf16(bf16lo(v[j].w) * r * g1.z, bf16hi(v[j].w) * r * g1.w);
        stg128(yr + c, o);
      }
    }
  }
  if (lane == 0 && i < n_my) {  // gave up: wait (bounded) for the loads still in flight
    for (int64_t j = i; j < issued; ++j) {
      bool done = false;
      for (uint32_t spin = 0; spin < SPIN_LIMIT && !done; ++spin)
        done = mbar_try_wait(&bars[j % stages], static_cast<uint32_t>((j / stages) & 1));
      if (!done) atomicOr(status, B2_DEV_TIMEOUT_DRAIN);
    }
  }
}

template <bool ADD, int VPL, int W>
static int launch_rmsnorm_ring_w(const void* x, const void* delta, const float* gain, void* h_out, void* y_out,
                                 int64_t rows, int dim, float eps, int* status, cudaStream_t stream) {
  const size_t row_bytes = static_cast<size_t>(dim) * 2 * (ADD ? 2 : 1);
  int stages = static_cast<int>((200 * 1024) / (W * row_bytes));
  if (stages > RN_MAX_STAGES) stages = RN_MAX_STAGES;
  if (stages < 1) return B2_ERR_UNSUPPORTED;
  const size_t smem = W * stages * row_bytes + (W * RN_MAX_STAGES + 2) * sizeof(uint64_t);
  cudaError_t e = cudaFuncSetAttribute(rmsnorm_ring_kernel<ADD, W, VPL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  int64_t grid = (rows + W - 1) / W;
  if (grid > sm_count()) grid = sm_count();
  rmsnorm_ring_kernel<ADD, W, VPL><<<static_cast<unsigned>(grid), W * 32, smem, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
      reinterpret_cast<const float4*>(gain), static_cast<__nv_bfloat16*>(h_out), static_cast<__nv_bfloat16*>(y_out),
      rows, dim, 1.0f / static_cast<float>(dim), eps, stages, status);
  return launch_status();
}

// Warps per CTA: 16 (8 measured slower at 8192 rows although it balances the rows better: 32.8 against 26.4 us);
// the tunable "rmsnorm_warps" (8 / 16 / 32) overrides it for experiments.
template <bool ADD, int VPL>
static int launch_rmsnorm_ring(const void* x, const void* delta, const float* gain, void* h_out, void* y_out,
                               int64_t rows, int dim, float eps, int* status, cudaStream_t stream) {
  const int w = tunable(TUNE_RMSNORM_WARPS);
  if (w == 8) return launch_rmsnorm_ring_w<ADD, VPL, 8>(x, delta, gain, h_out, y_out, rows, dim, eps, status, stream);
  if (w == 32 && static_cast<size_t>(dim) * 2 * (ADD ? 2 : 1) * 32 <= 200 * 1024)
    return launch_rmsnorm_ring_w<ADD, VPL, 32>(x, delta, gain, h_out, y_out, rows, dim, eps, status, stream);
  return launch_rmsnorm_ring_w<ADD, VPL, 16>(x, delta, gain, h_out, y_out, rows, dim, eps, status, stream);
}

template <bool ADD>
static int launch_rmsnorm(const void* x, const void* delta, const float* gain, void* h_out, void* y_out, int64_t rows,
                          int dim, float eps, cudaStream_t stream) {
  if (rows < 0 || dim <= 0) return B2_ERR_SHAPE;
  if (dim % 8 != 0 || dim > 8192) return B2_ERR_UNSUPPORTED;
  if (rows == 0) return B2_OK;  // empty tensors carry NULL data pointers
  if (!x || !gain || !y_out || (ADD && (!delta || !h_out))) return B2_ERR_NULL;
  if (!aligned16(x) || !aligned16(gain) || !aligned16(y_out) || (ADD && (!aligned16(delta) || !aligned16(h_out))))
    return B2_ERR_ALIGN;
  const int nvec = dim / 8;
  const int vpl = (nvec + 31) / 32;
  // The ring of bulk copies pays off where a row needs two input streams (the fused add: 37.9 against 45.1 us at
  // 8192 rows); a plain norm is faster with one warp per row on ordinary 128-bit loads at every size measured
  // (8192 rows: 21.0 against 26.1 us; 65536 rows: 117.8 against 141.3 us = 0.99 of the copy bandwidth).
  const int ring_min = tunable(TUNE_RMSNORM_RING_MIN_ROWS) > 0 ? tunable(TUNE_RMSNORM_RING_MIN_ROWS) : (ADD ? 512 : 0x7fffffff);
  if (rows >= ring_min && static_cast<size_t>(dim) * 2 * (ADD ? 2 : 1) * 16 <= 200 * 1024) {
    // streaming case: per-warp rings of row buffers in shared memory
    int* status = device_status_ptr();
    if (!status) return B2_ERR_DRIVER;
    if (vpl <= 4) return launch_rmsnorm_ring<ADD, 4>(x, delta, gain, h_out, y_out, rows, dim, eps, status, stream);
    if (vpl <= 8) return launch_rmsnorm_ring<ADD, 8>(x, delta, gain, h_out, y_out, rows, dim, eps, status, stream);
    if (vpl <= 12) return launch_rmsnorm_ring<ADD, 12>(x, delta, gain, h_out, y_out, rows, dim, eps, status, stream);
    if (vpl <= 16) return launch_rmsnorm_ring<ADD, 16>(x, delta, gain, h_out, y_out, rows, dim, eps, status, stream);
  }
  // few rows (decode): one warp per CTA so rows spread over the SMs; many rows: 8 warps per CTA
  const int warps = rows >= 4096 ? 8 : 1;
  const dim3 grid(static_cast<unsigned>((rows + warps - 1) / warps)), block(32 * warps);
#define B2_RMS_LAUNCH(V)                                                                                       \
  launch_overlapped(rmsnorm_kernel<V, ADD>, grid, block, 0, stream, static_cast<const uint4*>(x),              \
                    static_cast<const uint4*>(delta), reinterpret_cast<const float4*>(gain),                   \
                    static_cast<uint4*>(h_out), static_cast<uint4*>(y_out), rows, nvec,                        \
                    1.0f / static_cast<float>(dim), eps)
  if (vpl <= 4) B2_RMS_LAUNCH(4);
  else if (vpl <= 8) B2_RMS_LAUNCH(8);
  else if (vpl <= 12) B2_RMS_LAUNCH(12);
  else if (vpl <= 16) B2_RMS_LAUNCH(16);
  else B2_RMS_LAUNCH(32);
#undef B2_RMS_LAUNCH
  return launch_status();
}

// One thread rotates 8 low-half and the 8 paired high-half elements of one head.
__global__ void __launch_bounds__(256) rope_kernel(uint4* __restrict__ q, uint4* __restrict__ k,
                                                   const float4* __restrict__ sin_tab,
                                                   const float4* __restrict__ cos_tab,
                                                   const int64_t* __restrict__ offset_dev, int64_t total, int64_t tokens,
                                                   int n_q, int n_kv, int64_t max_ctx) {
  const int64_t offset = *offset_dev;
  const int heads = n_q + n_kv;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i & 3);           // which 8 of the 32 rotation pairs
    const int64_t th = i >> 2;
    const int head = static_cast<int>(th % heads);
    const int64_t tok = th / heads;                  // b*tokens + t
    const int64_t t = tok % tokens;
    int64_t pos = (t + offset) % max_ctx;
    if (pos < 0) pos += max_ctx;
    uint4* base = head < n_q ? q + (tok * n_q + head) * 8 : k + (tok * n_kv + (head - n_q)) * 8;
    const uint4 lo = base[j], hi = base[4 + j];
    const float4 c0 = __ldg(cos_tab + pos * 8 + 2 * j), c1 = __ldg(cos_tab + pos * 8 + 2 * j + 1);
    const float4 s0 = __ldg(sin_tab + pos * 8 + 2 * j), s1 = __ldg(sin_tab + pos * 8 + 2 * j + 1);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
    uint32_t ol[4], oh[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float a0 = bf16lo(lw[p]), a1 = bf16hi(lw[p]), b0 = bf16lo(hw[p]), b1 = bf16hi(hw[p]);
      ol[p] = pack_bf16(a0 * c[2 * p] - b0 * s[2 * p], a1 * c[2 * p + 1] - b1 * s[2 * p + 1]);
      oh[p] = pack_bf16(b0 * c[2 * p] + a0 * s[2 * p], b1 * c[2 * p + 1] + a1 * s[2 * p + 1]);
    }
    base[j] = make_uint4(ol[0], ol[1], ol[2], ol[3]);
    base[4 + j] = make_uint4(oh[0], oh[1], oh[2], oh[3]);
  }
}

}  // namespace b2

B2_API int b2_rmsnorm(const void* x, const float* gain, void* out, int64_t rows, int dim, float eps, void* stream) {
  return b2::launch_rmsnorm<false>(x, nullptr, gain, nullptr, out, rows, dim, eps, static_cast<cudaStream_t>(stream));
}

B2_API int b2_add_rmsnorm(const void* x, const void* delta, const float* gain, void* h_out, void* y_out, int64_t rows,
                          int dim, float eps, void* stream) {
  if (y_out && (y_out == x || y_out == delta || y_out == h_out)) return B2_ERR_SHAPE;
  return b2::launch_rmsnorm<true>(x, delta, gain, h_out, y_out, rows, dim, eps, static_cast<cudaStream_t>(stream));
}

B2_API int b2_rope_inplace(void* q, void* k, const float* sin_tab, const float* cos_tab, const int64_t* offset_dev,
                           int64_t batch, int64_t tokens, int n_q_heads, int n_kv_heads, int head_dim, int64_t max_ctx,
                           void* stream) {
  if (!q || !k || !sin_tab || !cos_tab || !offset_dev) return B2_ERR_NULL;
  if (batch < 0 || tokens < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_ctx <= 0) return B2_ERR_SHAPE;
  if (head_dim != 64) return B2_ERR_UNSUPPORTED;
  if (!b2::aligned16(q) || !b2::aligned16(k) || !b2::aligned16(sin_tab) || !b2::aligned16(cos_tab)) return B2_ERR_ALIGN;
  const int64_t total = batch * tokens * (n_q_heads + n_kv_heads) * 4;
  if (total == 0) return B2_OK;
  const int block = 256;
  int64_t blocks = (total + block - 1) / block;
  const int64_t cap = static_cast<int64_t>(b2::sm_count()) * 32;
  if (blocks > cap) blocks = cap;
  b2::rope_kernel<<<static_cast<unsigned>(blocks), block, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(q), static_cast<uint4*>(k), reinterpret_cast<const float4*>(sin_tab),
      reinterpret_cast<const float4*>(cos_tab), offset_dev, total, tokens, n_q_heads, n_kv_heads, max_ctx);
  return b2::launch_status();
}
