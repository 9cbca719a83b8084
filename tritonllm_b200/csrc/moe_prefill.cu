// Mixture-of-experts MLP for prompt-sized batches (thousands of tokens): the tokens of an expert are the M rows
// of a grouped GEMM, so every weight tile is used by up to 256 tokens at a time and the work is tensor-bound.
//
//   moe_big_count_kernel    per routed (token, slot): rank of the token inside its expert (atomic counter)
//   moe_big_scan_kernel     per-expert row offsets, and the list of 256-row tiles (each inside one expert's rows)
//   moe_big_gather_kernel   x[token] -> xs[row] in expert-sorted order, routing weight of every row
//   gemm_tc_pair_kernel<192, EPI_MOE_SWIGLU>   act = swiglu(xs W1_e^T + b1_e)      (grouped, CTA pairs, tcgen05)
//   gemm_tc_pair_kernel<192, EPI_MOE_GATE>     y   = (act W2_e^T + b2_e) * gate
//   moe_big_combine_kernel  out[token] = sum of its (up to four) rows of y, fp32, in slot order
//
// The GEMMs run in bf16: block-scaled FP4 x FP8 MMAs would need the activations as two E4M3 terms and so twice the
// MMA work at twice the rate - no faster - while bf16 x bf16 needs none of the per-k-block scale traffic.  The
// expert weights are therefore expanded once per call from MXFP4 to bf16 (exact: an E2M1 value times a power of two
// is a bf16 number) into a scratch the caller provides (moe_upcast_packed_kernel, HBM-bound), and the expansion is
// amortised over all the tokens of the call.
// The order of an expert's rows depends on the order in which the atomics land; every row's result is independent
// of where the row sits, and a token's rows are summed in slot order, so the output does not depend on it.
// Rounding points as in the decode-sized path: act and y are bf16 tensors, the sum over experts is fp32.
#include "gemm_tc.cuh"

namespace b2 {

constexpr int MOEP_TOPK = 4;
constexpr int MOEP_TILE_ROWS = 256;
constexpr int MOEP_MAX_EXPERTS = 1024;

__global__ void __launch_bounds__(256) moe_big_count_kernel(const int16_t* __restrict__ topk_idx, int tokens, int n_experts,
                                                            int* __restrict__ counts, int* __restrict__ rank_of_slot,
                                                            int* __restrict__ status) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(topk_idx) + t);
  const int e[MOEP_TOPK] = {static_cast<int16_t>(raw.x & 0xffffu), static_cast<int16_t>(raw.x >> 16),
                            static_cast<int16_t>(raw.y & 0xffffu), static_cast<int16_t>(raw.y >> 16)};
#pragma unroll
  for (int k = 0; k < MOEP_TOPK; ++k) {
    bool ok = e[k] >= 0 && e[k] < n_experts;
#pragma unroll
    for (int j = 0; j < k; ++j) ok = ok && e[j] != e[k];   // an expert twice for one token would be summed twice
    int rank = -1;
    if (ok)
      rank = atomicAdd(counts + e[k], 1);
    else
      atomicOr(status, B2_DEV_BAD_INDEX);
    rank_of_slot[t * MOEP_TOPK + k] = rank;
  }
}

__global__ void __launch_bounds__(128) moe_big_scan_kernel(const int* __restrict__ counts, int n_experts, int* __restrict__ offsets,
                                                           int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                                                           int* __restrict__ tile_expert, int* __restrict__ n_tiles) {
  __shared__ int s_off[MOEP_MAX_EXPERTS + 1], s_tile[MOEP_MAX_EXPERTS + 1];
  if (threadIdx.x == 0) {
    int run = 0, trun = 0;
    for (int e = 0; e < n_experts; ++e) {
      s_off[e] = run;
      s_tile[e] = trun;
      const int c = counts[e];
      run += c;
      trun += (c + MOEP_TILE_ROWS - 1) / MOEP_TILE_ROWS;
    }
    s_off[n_experts] = run;
    s_tile[n_experts] = trun;
    *n_tiles = trun;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= n_experts; e += blockDim.x) offsets[e] = s_off[e];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
    const int c = s_off[e + 1] - s_off[e];
    for (int i = 0, r = 0; r < c; ++i, r += MOEP_TILE_ROWS) {
      tile_row0[s_tile[e] + i] = s_off[e] + r;
      tile_rows[s_tile[e] + i] = min(MOEP_TILE_ROWS, c - r);
      tile_expert[s_tile[e] + i] = e;
    }
  }
}

// one CTA per routed (token, slot): its row in expert-sorted order, the row's routing weight, the token's activations
__global__ void __launch_bounds__(128) moe_big_gather_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                                             const int16_t* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                                             const int* __restrict__ rank_of_slot, const int* __restrict__ offsets,
                                                             int* __restrict__ row_of_slot, float* __restrict__ gate_of_row,
                                                             __nv_bfloat16* __restrict__ xs, int hidden) {
  const int slot = blockIdx.x;
  const int rank = rank_of_slot[slot];
  const int row = rank < 0 ? -1 : offsets[topk_idx[slot]] + rank;
  if (threadIdx.x == 0) {
    row_of_slot[slot] = row;
    if (row >= 0) gate_of_row[row] = topk_w[slot];
  }
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(slot / MOEP_TOPK) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = __ldg(src + i);
}

__global__ void __launch_bounds__(128) moe_big_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of_slot,
                                                              __nv_bfloat16* __restrict__ out, int64_t ld_out, int hidden) {
  const int t = blockIdx.x;
  int rows[MOEP_TOPK];
#pragma unroll
  for (int k = 0; k < MOEP_TOPK; ++k) rows[k] = row_of_slot[t * MOEP_TOPK + k];
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < MOEP_TOPK; ++k) {
      if (rows[k] < 0) continue;
      const uint4 p = __ldg(reinterpret_cast<const uint4*>(y + static_cast<size_t>(rows[k]) * hidden) + i);
      acc[0] += bf16lo(p.x); acc[1] += bf16hi(p.x); acc[2] += bf16lo(p.y); acc[3] += bf16hi(p.y);
      acc[4] += bf16lo(p.z); acc[5] += bf16hi(p.z); acc[6] += bf16lo(p.w); acc[7] += bf16hi(p.w);
    }
    *(reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ld_out) + i) =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

// Elements 2b (low nibble) and 2b+1 (high nibble) of a code byte times the group scale, as a bf16 pair: the three
// magnitude bits at fp32 bits 22-24 are the E2M1 value times 2^-126, two exact multiplies bring it to value x scale.
__device__ __forceinline__ uint32_t moep_pair(uint32_t byte, float sc) {
  const float lo = __uint_as_float(((byte & 0x07u) << 22) | ((byte & 0x08u) << 28));
  const float hi = __uint_as_float(((byte & 0x70u) << 18) | ((byte & 0x80u) << 24));
  const float two126 = __uint_as_float(0x7e800000u);
  return pack_bf16(__fmul_rn(__fmul_rn(lo, two126), sc), __fmul_rn(__fmul_rn(hi, two126), sc));
}

// MXFP4 in the layout the decode-sized expert kernel reads (codes [E][N][Kp/2], K zero-padded to Kp; scales as
// 512-byte blocks [E][ceil(N/128)][Kp/128][row%32][row/32][group%4]) -> bf16 [E*N][K].  HBM-bound: a CTA takes rows
// in turn, a thread 8 elements (one 32-bit word of codes -> one 16-byte store), so a warp reads 128 contiguous code
// bytes and writes 512 contiguous bytes; three words per thread are in flight.
constexpr int MOEP_UP_THREADS = 128, MOEP_UP_UNROLL = 3;
__global__ void __launch_bounds__(MOEP_UP_THREADS) moe_upcast_packed_kernel(const uint32_t* __restrict__ codes,
                                                                            const uint8_t* __restrict__ sf, uint4* __restrict__ out,
                                                                            int rows_total, int N, int words_per_row,
                                                                            int code_words_per_row, int tiles, int nkb) {
  for (int row = blockIdx.x; row < rows_total; row += gridDim.x) {
    const int e = row / N, r = row - e * N;
    const int tile = r >> 7, rr = r & 127;
    const uint8_t* sf_row = sf + (static_cast<size_t>(e) * tiles + tile) * nkb * 512 + (rr & 31) * 16 + (rr >> 5) * 4;
    const uint32_t* crow = codes + static_cast<size_t>(row) * code_words_per_row;
    uint4* orow = out + static_cast<size_t>(row) * words_per_row;
    for (int w0 = threadIdx.x; w0 < words_per_row; w0 += MOEP_UP_THREADS * MOEP_UP_UNROLL) {
      uint32_t c[MOEP_UP_UNROLL], s[MOEP_UP_UNROLL];
#pragma unroll
      for (int u = 0; u < MOEP_UP_UNROLL; ++u) {
        const int w = w0 + u * MOEP_UP_THREADS;
        const int g = w >> 2;   // 4 words per 32-element group
        c[u] = w < words_per_row ? __ldg(crow + w) : 0u;
        s[u] = w < words_per_row ? static_cast<uint32_t>(__ldg(sf_row + (g >> 2) * 512 + (g & 3))) : 0u;
      }
#pragma unroll
      for (int u = 0; u < MOEP_UP_UNROLL; ++u) {
        const int w = w0 + u * MOEP_UP_THREADS;
        if (w < words_per_row) {
          const float sc = __uint_as_float(s[u] << 23);
          stg128(orow + w, make_uint4(moep_pair(c[u] & 0xffu, sc), moep_pair((c[u] >> 8) & 0xffu, sc),
                                      moep_pair((c[u] >> 16) & 0xffu, sc), moep_pair(c[u] >> 24, sc)));
        }
      }
    }
  }
}

}  // namespace b2

namespace {
size_t al256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
struct MoepLayout {
  size_t counts, offsets, n_tiles, tile_row0, tile_rows, tile_expert, rank_of_slot, row_of_slot, gate_of_row, xs, act, y, total;
  int max_tiles;
};
MoepLayout moep_layout(int64_t tokens, int n_experts, int hidden, int intermediate) {
  MoepLayout L;
  const size_t rows = static_cast<size_t>(tokens) * b2::MOEP_TOPK;
  L.max_tiles = static_cast<int>(rows / b2::MOEP_TILE_ROWS) + n_experts + 1;
  size_t o = 0;
  L.counts = o;       o += al256(sizeof(int) * n_experts);
  L.offsets = o;      o += al256(sizeof(int) * (n_experts + 1));
  L.n_tiles = o;      o += 256;
  L.tile_row0 = o;    o += al256(sizeof(int) * L.max_tiles);
  L.tile_rows = o;    o += al256(sizeof(int) * L.max_tiles);
  L.tile_expert = o;  o += al256(sizeof(int) * L.max_tiles);
  L.rank_of_slot = o; o += al256(sizeof(int) * rows);
  L.row_of_slot = o;  o += al256(sizeof(int) * rows);
  L.gate_of_row = o;  o += al256(sizeof(float) * rows);
  L.xs = o;           o += al256(rows * hidden * 2);
  L.act = o;          o += al256(rows * intermediate * 2);
  L.y = o;            o += al256(rows * hidden * 2);
  L.total = o;
  return L;
}
}  // namespace

B2_API size_t b2_moe_prefill_workspace_bytes(int64_t tokens, int n_experts, int hidden, int intermediate) {
  if (tokens <= 0 || n_experts <= 0 || hidden <= 0 || intermediate <= 0) return 0;
  return moep_layout(tokens, n_experts, hidden, intermediate).total;
}

B2_API int b2_moe_upcast_packed(const void* codes, const void* scale_blocks, void* out, int n_experts, int n, int k, void* stream) {
  if (n_experts <= 0 || n <= 0 || k <= 0) return B2_ERR_SHAPE;
  if (k % 32 != 0) return B2_ERR_UNSUPPORTED;
  if (!codes || !scale_blocks || !out) return B2_ERR_NULL;
  if (!b2::aligned16(codes) || !b2::aligned16(out)) return B2_ERR_ALIGN;
  const int kp = (k + 127) / 128 * 128;
  const int64_t rows = static_cast<int64_t>(n_experts) * n;
  if (rows > 0x7fffffff) return B2_ERR_UNSUPPORTED;
  int64_t blocks = rows;
  const int64_t cap = static_cast<int64_t>(b2::sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  b2::moe_upcast_packed_kernel<<<static_cast<unsigned>(blocks), b2::MOEP_UP_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(codes), static_cast<const uint8_t*>(scale_blocks), static_cast<uint4*>(out),
      static_cast<int>(rows), n, k / 8, kp / 8, (n + 127) / 128, kp / 128);
  return b2::launch_status();
}

B2_API int b2_moe_experts_prefill(const void* x, int64_t ldx, const int16_t* topk_idx, const float* topk_w, const void* w1_bf16,
                                  const float* b1, const void* w2_bf16, const float* b2_, void* out, int64_t ld_out,
                                  void* workspace, size_t workspace_bytes, int64_t tokens, int n_experts, int hidden,
                                  int intermediate, float alpha, float limit, void* stream) {
  using namespace b2;
  if (tokens < 0 || n_experts <= 0 || hidden <= 0 || intermediate <= 0 || ldx < hidden || ld_out < hidden) return B2_ERR_SHAPE;
  if (n_experts > MOEP_MAX_EXPERTS || hidden % 192 || (2 * intermediate) % 192 || hidden % 8 || intermediate % 8 ||
      tokens * MOEP_TOPK > 0x3fffffff)
    return B2_ERR_UNSUPPORTED;
  if (tokens == 0) return B2_OK;
  if (!x || !topk_idx || !topk_w || !w1_bf16 || !b1 || !w2_bf16 || !b2_ || !out || !workspace) return B2_ERR_NULL;
  if (!aligned16(x) || !aligned16(out) || !aligned16(w1_bf16) || !aligned16(w2_bf16) || !aligned16(b1) || !aligned16(b2_) ||
      ldx % 8 || ld_out % 8 || (reinterpret_cast<uintptr_t>(workspace) & 255) || (reinterpret_cast<uintptr_t>(topk_idx) & 7))
    return B2_ERR_ALIGN;
  const MoepLayout L = moep_layout(tokens, n_experts, hidden, intermediate);
  if (workspace_bytes < L.total) return B2_ERR_WORKSPACE;
  int* status = device_status_ptr();
  if (!status) return B2_ERR_DRIVER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* counts = reinterpret_cast<int*>(ws + L.counts);
  int* offsets = reinterpret_cast<int*>(ws + L.offsets);
  int* n_tiles = reinterpret_cast<int*>(ws + L.n_tiles);
  int* tile_row0 = reinterpret_cast<int*>(ws + L.tile_row0);
  int* tile_rows = reinterpret_cast<int*>(ws + L.tile_rows);
  int* tile_expert = reinterpret_cast<int*>(ws + L.tile_expert);
  int* rank_of_slot = reinterpret_cast<int*>(ws + L.rank_of_slot);
  int* row_of_slot = reinterpret_cast<int*>(ws + L.row_of_slot);
  float* gate_of_row = reinterpret_cast<float*>(ws + L.gate_of_row);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ws + L.xs);
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(ws + L.act);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(ws + L.y);
  const int T = static_cast<int>(tokens), rows = T * MOEP_TOPK;

  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * n_experts, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  moe_big_count_kernel<<<(T + 255) / 256, 256, 0, st>>>(topk_idx, T, n_experts, counts, rank_of_slot, status);
  moe_big_scan_kernel<<<1, 128, 0, st>>>(counts, n_experts, offsets, tile_row0, tile_rows, tile_expert, n_tiles);
  moe_big_gather_kernel<<<rows, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, topk_idx, topk_w, rank_of_slot, offsets,
                                             row_of_slot, gate_of_row, xs, hidden);
  int rc = launch_status();
  if (rc != B2_OK) return rc;

  GemmArgs g = {};
  g.M = rows;
  g.tiles_m = n_experts;   // (how the launcher learns the number of experts)
  g.g_tile_row0 = tile_row0;
  g.g_tile_rows = tile_rows;
  g.g_tile_expert = tile_expert;
  g.g_n_tiles = n_tiles;
  g.g_gate = gate_of_row;
  g.alpha = alpha;
  g.limit = limit;
  g.vec_ok = 1;
  // a = swiglu(xs W1 + b1): N = 2 * intermediate interleaved (gate, linear) features, K = hidden
  g.N = 2 * intermediate;
  g.K = hidden;
  g.g_bias = b1;
  g.out = act;
  g.ld_out = intermediate;
  rc = launch_moe_grouped_gemm(EPI_MOE_SWIGLU, xs, hidden, w1_bf16, hidden, g, L.max_tiles, st);
  if (rc != B2_OK) return rc;
  // y = (a W2 + b2) * gate: N = hidden, K = intermediate
  g.N = hidden;
  g.K = intermediate;
  g.g_bias = b2_;
  g.out = y;
  g.ld_out = hidden;
  rc = launch_moe_grouped_gemm(EPI_MOE_GATE, act, intermediate, w2_bf16, intermediate, g, L.max_tiles, st);
  if (rc != B2_OK) return rc;
  moe_big_combine_kernel<<<T, 128, 0, st>>>(y, row_of_slot, static_cast<__nv_bfloat16*>(out), ld_out, hidden);
  return launch_status();
}
