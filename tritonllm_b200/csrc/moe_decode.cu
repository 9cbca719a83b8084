// Mixture-of-experts MLP for decode-sized batches: every routed (token, expert)
// pair runs  a = swiglu(x W1_e + b1_e),  y = (a W2_e + b2_e) * gate,  and a token's output is the sum of
// its experts' y.  Expert weights stay in MXFP4 in HBM (E2M1 codes, two per byte along K, and one E8M0
// scale byte per 32 K elements) and are the only large stream: the op is weight-bandwidth bound.
//
// Two paths share the routing and the combine.  This first part of the file is the conversion path (at most 256
// tokens; plain ExpertWeights; codes turned into bf16 on the CUDA cores, which is its second limit).  The FP4
// tensor-core path (at most 2048 tokens; ExpertWeightsFp4; block-scaled FP4 x FP8 MMAs on the codes as stored) follows
// further down: the routing + quantise launch, the one-shot kernel, its persistent form, and the fused launch of both
// GEMMs, each described where it is defined.
//
//   moe_route_kernel   one CTA: per-expert token lists (stable: tokens ascending), offsets, gate weights
//   moe_gather_kernel  copies each routed token's activation row into expert-sorted order
//   moe_expert_kernel  grid (128-feature tiles, experts); a CTA whose expert got no token returns at once.
//                      Operands are swapped as in the decode projections: the weight tile is the MMA's A
//                      operand (M = 128 features), the expert's tokens are N (rounded to 32, at most 256).
//                        warp 0    TMA: 4 KiB code tiles (128 rows x 32 bytes = 64 K elements) into a raw
//                                  ring, and the tokens' [N x 64] bf16 tiles (128B swizzle) into a B ring
//                        warps 2-9 dequantise: two threads per weight row turn 2 x 16 code bytes into
//                                  128 bytes of bf16 (byte-permute lookup of the eight magnitudes, sign
//                                  bits moved by permute, one packed multiply by the group scale) and
//                                  store them in the 128B-swizzled K-major layout the MMA descriptor
//                                  expects, then fence to the async proxy and arrive
//                        warp 1    tcgen05.mma (M=128, N, K=16) x 4 per tile; commits free both rings
//                        warps 2-5 epilogue: accumulator -> registers -> bias (+ SwiGLU over interleaved
//                                  feature pairs, or * gate) -> bf16 block in shared memory -> full-row
//                                  coalesced stores
//   moe_combine_kernel sums each token's (up to four) per-expert rows in fp32, in slot order
// Rounding points: a and the per-expert y are bf16 tensors, the sum over experts is fp32, the output bf16.
// Every mbarrier wait is bounded.
#include <cuda_bf16.h>

#include "tc_common.cuh"

namespace b2 {

constexpr int MOE_MAX_TOKENS = 2048;        // capacity of the routing metadata (FP4 path: tokens per call)
constexpr int MOE_CONV_MAX_TOKENS = 256;    // conversion path: one CTA takes all tokens of an expert (MMA N <= 256)
constexpr int MOE_MAX_ITEMS = MOE_MAX_TOKENS * 4 / 32 + 128;   // sum over experts of ceil(rows / 32) <= rows / 32 + experts
constexpr int MOE_MAX_EXPERTS = 128;
constexpr int MOE_TOPK = 4;
constexpr int MOE_FT = 128;             // weight rows (output features) per tile
constexpr int MOE_KB = 64;              // K elements per pipeline step
constexpr int MOE_RAW_BYTES = MOE_FT * MOE_KB / 2;   // 4 KiB of codes
constexpr int MOE_A_BYTES = MOE_FT * MOE_KB * 2;     // 16 KiB of bf16
constexpr int MOE_RAW_STAGES = 8;
constexpr int MOE_A_STAGES = 3;
constexpr int MOE_DEQ_WARPS = 8;
constexpr int MOE_THREADS = 64 + 32 * MOE_DEQ_WARPS;
enum { MOE_EPI_SWIGLU = 0, MOE_EPI_GATE = 1 };

struct MoeMeta {          // lives at the start of the workspace
  int counts[MOE_MAX_EXPERTS];
  int offsets[MOE_MAX_EXPERTS + 1];
  int row_of_slot[MOE_MAX_TOKENS * MOE_TOPK];   // (token * 4 + slot) -> row in expert-sorted order
  int slot_of_row[MOE_MAX_TOKENS * MOE_TOPK];   // inverse
  float gate_of_row[MOE_MAX_TOKENS * MOE_TOPK];
  // FP4 path: the non-empty (expert, part of `tok` tokens) pairs, in expert order
  int n_items;
  short item_expert[MOE_MAX_ITEMS];
  short item_part[MOE_MAX_ITEMS];
  int item_done[MOE_MAX_ITEMS];   // fused expert kernel: weight tiles of the first GEMM finished per item (zeroed by the routing kernel)
};

// ------------------------------------------------------------------------------------------- routing
// The routing work of one CTA (any block size that is a multiple of 32).
__device__ __forceinline__ void moe_route_body(const int16_t* __restrict__ topk_idx, const float* __restrict__ topk_w,
                                               int tokens, int n_experts, MoeMeta* meta, int* status, int tok) {
  __shared__ uint32_t mask[MOE_MAX_EXPERTS][MOE_MAX_TOKENS / 32];  // which tokens chose expert e
  __shared__ int offs[MOE_MAX_EXPERTS + 1];
  const int tid = threadIdx.x;
  overlap_start();
  const int words = (tokens + 31) >> 5;   // mask words in use per expert
  for (int i = tid; i < n_experts * words; i += blockDim.x) mask[i / words][i % words] = 0u;
  __syncthreads();
  overlap_wait();
  for (int i = tid; i < MOE_MAX_ITEMS; i += blockDim.x) meta->item_done[i] = 0;
  const int slots = tokens * MOE_TOPK;
  for (int sl = tid; sl < slots; sl += blockDim.x) {
    const int t = sl / MOE_TOPK, e = topk_idx[sl];
    if (e < 0 || e >= n_experts)
      atomicOr(status, B2_DEV_BAD_INDEX);
    else if (atomicOr(&mask[e][t >> 5], 1u << (t & 31)) & (1u << (t & 31)))
      atomicOr(status, B2_DEV_BAD_INDEX);   // the same expert twice for one token: the lists would count it once
  }
  __syncthreads();
  if (tid < 32) {  // counts and exclusive offsets, one warp
    int carry = 0, item_carry = 0;
    for (int base = 0; base < n_experts; base += 32) {
      const int ex = base + tid;
      int c = 0;
      if (ex < n_experts)
        for (int w = 0; w < words; ++w) c += __popc(mask[ex][w]);
      int incl = c;
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (tid >= d) incl += up;
      }
      if (ex < n_experts) {
        meta->counts[ex] = c;
        offs[ex] = carry + incl - c;
        meta->offsets[ex] = carry + incl - c;
      }
      carry += __shfl_sync(0xffffffffu, incl, 31);
      if (tok > 0) {   // the expert's parts of `tok` rows join the item list
        const int parts = (c + tok - 1) / tok;
        int pin = parts;
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, pin, d);
          if (tid >= d) pin += up;
        }
        for (int q = 0; q < parts; ++q) {
          meta->item_expert[item_carry + pin - parts + q] = static_cast<short>(ex);
          meta->item_part[item_carry + pin - parts + q] = static_cast<short>(q);
        }
        item_carry += __shfl_sync(0xffffffffu, pin, 31);
      }
    }
    if (tid == 0) {
      offs[n_experts] = carry;
      meta->offsets[n_experts] = carry;
      meta->n_items = item_carry;
    }
  }
  __syncthreads();
  for (int sl = tid; sl < slots; sl += blockDim.x) {
    const int t = sl / MOE_TOPK, e = topk_idx[sl];
    int row = -1;
    if (e >= 0 && e < n_experts) {
      int rank = 0;  // tokens before t that chose the same expert
      for (int w = 0; w < (t >> 5); ++w) rank += __popc(mask[e][w]);
      rank += __popc(mask[e][t >> 5] & ((1u << (t & 31)) - 1u));
      row = offs[e] + rank;
      meta->slot_of_row[row] = sl;
      meta->gate_of_row[row] = topk_w[sl];
    }
    meta->row_of_slot[sl] = row;
  }
}

__global__ void __launch_bounds__(1024) moe_route_kernel(const int16_t* __restrict__ topk_idx,
                                                         const float* __restrict__ topk_w, int tokens, int n_experts,
                                                         MoeMeta* meta, int* status, int tok) {
  moe_route_body(topk_idx, topk_w, tokens, n_experts, meta, status, tok);
}

// one CTA per routed row: x[token] -> xs[row]
__global__ void __launch_bounds__(128) moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                                         __nv_bfloat16* __restrict__ xs, int hidden, int slots,
                                                         const MoeMeta* __restrict__ meta) {
  const int slot = blockIdx.x;
  if (slot >= slots) return;
  const int row = meta->row_of_slot[slot];
  if (row < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(slot / MOE_TOPK) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = __ldg(src + i);
}

// ------------------------------------------------------------------------------------- expert GEMMs
struct MoeExpertArgs {
  const uint8_t* scales;    // [E][N][K/32] E8M0
  const float* bias;        // [E][N]
  const MoeMeta* meta;
  __nv_bfloat16* out;       // SWIGLU: act [rows][N/2]; GATE: y [rows][N]
  int N, K, nkb, bn_max, b_stages;
  float alpha, limit;
  int* status;
  long long* trace;  // optional [CTA][8] (b2_set_trace_buffer): start ns, end ns, then SM-clock totals of the first
                     // dequantising warp (wait codes, wait A slot, convert) and of the MMA warp (wait A, wait B)
};

struct __align__(16) MoeBarriers {
  uint64_t raw_full[MOE_RAW_STAGES];
  uint64_t raw_empty[MOE_RAW_STAGES];
  uint64_t a_full[MOE_A_STAGES];
  uint64_t a_empty[MOE_A_STAGES];
  uint64_t b_full[4];
  uint64_t b_empty[4];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float moe_swiglu(float g, float l, float alpha, float limit) {
  g = fminf(g, limit);
  l = fmaxf(fminf(l, limit), -limit);
  const float s = __fdividef(g, 1.0f + __expf(-alpha * g));
  return fmaf(s, l, s);
}

// Eight E2M1 codes (nibble i = element i) -> four bf16 pairs, each multiplied by the group scale
// (sc2 = the scale as a bf16 pair).  Magnitudes {0,.5,1,1.5,2,3,4,6} are bf16 0x0000 3F00 3F80 3FC0 4000
// 4040 4080 40C0: two byte-permutes look up the high and low bytes of four codes at once, the sign bits
// (nibble bit 3) are moved to bit 7 of the high bytes with one more permute, a last pair of permutes
// interleaves low and high bytes.
__device__ __forceinline__ void mxfp4_word_to_bf16x8(uint32_t w, uint32_t sc2, uint32_t (&o)[4]) {
  constexpr uint32_t TH0 = 0x3f3f3f00u, TH1 = 0x40404040u, TL0 = 0xc0800000u, TL1 = 0xc0804000u;
  const uint32_t m = w & 0x77777777u, mb = m >> 16;
  const uint32_t sg = w & 0x88888888u;
  const uint32_t sodd = sg & 0x80808080u;          // odd elements: already at bit 7 of byte j (element 2j+1)
  const uint32_t sevn = (sg << 4) & 0x80808080u;   // even elements: bit 7 of byte j (element 2j)
  const uint32_t ha = __byte_perm(TH0, TH1, m) | __byte_perm(sevn, sodd, 0x5140);   // elements 0..3
  const uint32_t hb = __byte_perm(TH0, TH1, mb) | __byte_perm(sevn, sodd, 0x7362);  // elements 4..7
  const uint32_t la = __byte_perm(TL0, TL1, m), lb = __byte_perm(TL0, TL1, mb);
  uint32_t v[4] = {__byte_perm(la, ha, 0x5140), __byte_perm(la, ha, 0x7362), __byte_perm(lb, hb, 0x5140),
                   __byte_perm(lb, hb, 0x7362)};
  const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162*>(&sc2);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 p = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&v[i]), s2);
    o[i] = *reinterpret_cast<const uint32_t*>(&p);
  }
}

template <int EPI>
__global__ void __launch_bounds__(MOE_THREADS, 1)
moe_expert_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const MoeExpertArgs a) {
  const int tile = blockIdx.x, e = blockIdx.y;
  const int n_e = a.meta->counts[e];
  if (n_e <= 0) return;  // no token routed here: this expert's weights are not read at all
  const int row0 = a.meta->offsets[e];
  const int bn = (n_e + 31) & ~31;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw = base;                                                   // MOE_RAW_STAGES x 4 KiB
  uint8_t* atile = raw + MOE_RAW_STAGES * MOE_RAW_BYTES;                 // MOE_A_STAGES x 16 KiB
  uint8_t* btile = atile + MOE_A_STAGES * MOE_A_BYTES;                   // b_stages x bn_max x 128 B
  const int b_stage_bytes = a.bn_max * 128;
  MoeBarriers& bar = *reinterpret_cast<MoeBarriers*>(btile + static_cast<size_t>(a.b_stages) * b_stage_bytes);
  uint8_t* sc_smem = reinterpret_cast<uint8_t*>(&bar + 1);  // the tile's scale bytes: [128 rows][K/32]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int BS = a.b_stages;
  volatile int* abort_flag = &bar.abort_flag;

  if (tid == 0) {
    for (int s = 0; s < MOE_RAW_STAGES; ++s) {
      mbar_init(&bar.raw_full[s], 1);
      mbar_init(&bar.raw_empty[s], MOE_DEQ_WARPS);
    }
    for (int s = 0; s < MOE_A_STAGES; ++s) {
      mbar_init(&bar.a_full[s], MOE_DEQ_WARPS);
      mbar_init(&bar.a_empty[s], 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&bar.b_full[s], 1);
      mbar_init(&bar.b_empty[s], 1);
    }
    mbar_init(&bar.acc_full, 1);
    bar.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  {
    // this tile's scales are one contiguous block of the [E][N][K/32] array (rows past N: zeros)
    const int ng = a.K / 32;
    const int rows_here = min(MOE_FT, a.N - tile * MOE_FT);
    const size_t g0 = (static_cast<size_t>(e) * a.N + static_cast<size_t>(tile) * MOE_FT) * ng;
    const int nbytes = rows_here * ng;
    const uint8_t* src = a.scales + g0;
    if (((reinterpret_cast<uintptr_t>(src) | static_cast<uintptr_t>(nbytes)) & 15) == 0) {
      for (int i = tid; i < nbytes / 16; i += MOE_THREADS)
        reinterpret_cast<uint4*>(sc_smem)[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
    } else {
      for (int i = tid; i < nbytes; i += MOE_THREADS) sc_smem[i] = __ldg(src + i);
    }
    for (int i = nbytes + tid; i < MOE_FT * ng; i += MOE_THREADS) sc_smem[i] = 0;
  }
  int tmem_cols = 32;
  while (tmem_cols < bn) tmem_cols <<= 1;
  if (warp == 1) tmem_alloc(&bar.tmem_base, tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bar.tmem_base;
  const int nkb = a.nkb;
  long long* trace = a.trace ? a.trace + 8ll * (blockIdx.y * gridDim.x + blockIdx.x) : nullptr;
  if (trace && tid == 0) trace[0] = global_timer_ns();

  if (warp == 0) {
    // ===================================== TMA producer =====================================
    const bool leader = elect_one();
    const int xblocks = bn >> 5;  // 32-row pieces of the token tile
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const int rs = kb % MOE_RAW_STAGES, rround = kb / MOE_RAW_STAGES;
      const int bs = kb % BS, bround = kb / BS;
      if (rround > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.raw_empty[rs], (rround - 1) & 1, abort_flag));
      if (ok && bround > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.b_empty[bs], (bround - 1) & 1, abort_flag));
      if (!ok) break;
      if (leader) {
        mbar_arrive_expect_tx(&bar.raw_full[rs], MOE_RAW_BYTES);
        // codes as 16-bit units: 32 bytes of every one of the tile's 128 rows; rows past N read as zero
        tma_load_4d(raw + rs * MOE_RAW_BYTES, &tm_w, &bar.raw_full[rs], kb * (MOE_KB / 4), tile * MOE_FT, e, 0);
        mbar_arrive_expect_tx(&bar.b_full[bs], static_cast<uint32_t>(xblocks) * 32 * 128);
        for (int xb = 0; xb < xblocks; ++xb)
          tma_load_2d(btile + static_cast<size_t>(bs) * b_stage_bytes + xb * 4096, &tm_x, &bar.b_full[bs], kb * MOE_KB,
                      row0 + 32 * xb);
      }
      __syncwarp();
    }
    if (leader && !ok) {
      if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
      *abort_flag = 1;
    }
  } else if (warp == 1) {
    // ===================================== MMA issuer =====================================
    const bool leader = elect_one();
    const uint32_t idesc = umma_idesc_bf16(MOE_FT, bn);
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const int as = kb % MOE_A_STAGES, bs = kb % BS;
      const long long c0 = trace ? clock64() : 0;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.b_full[bs], (kb / BS) & 1, abort_flag));
      const long long c1 = trace ? clock64() : 0;
      ok = ok && __all_sync(0xffffffffu, mbar_wait_bounded(&bar.a_full[as], (kb / MOE_A_STAGES) & 1, abort_flag));
      if (!ok) break;
      if (trace && leader) {
        trace[6] += c1 - c0;
        trace[5] += clock64() - c1;
      }
      tc_fence_after_sync();
      const uint64_t da = umma_desc_k128(smem_u32(atile + as * MOE_A_BYTES));
      const uint64_t db = umma_desc_k128(smem_u32(btile + static_cast<size_t>(bs) * b_stage_bytes));
      if (leader) {
#pragma unroll
        for (int k = 0; k < MOE_KB / 16; ++k) umma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
        umma_commit(&bar.a_empty[as]);
        umma_commit(&bar.b_empty[bs]);
      }
      __syncwarp();
    }
    if (leader) {
      if (ok) {
        umma_commit(&bar.acc_full);
      } else {
        if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    // ===================================== dequantise =====================================
    const int d = (warp - 2) * 32 + lane;   // 0..255
    const int r = d >> 1, h = d & 1;        // weight row of the tile, which half of the 64-element k-block
    const uint8_t* srow = sc_smem + r * (a.K / 32) + h;
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      const int rs = kb % MOE_RAW_STAGES, as = kb % MOE_A_STAGES;
      const uint32_t s_cur = srow[2 * kb];
      const bool tr = trace && d == 0;
      const long long k0 = tr ? clock64() : 0;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.raw_full[rs], (kb / MOE_RAW_STAGES) & 1, abort_flag));
      if (!ok) break;
      const long long k1 = tr ? clock64() : 0;
      const uint4 c = *reinterpret_cast<const uint4*>(raw + rs * MOE_RAW_BYTES + r * 32 + h * 16);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.raw_empty[rs]);  // the codes are in registers
      if (kb >= MOE_A_STAGES) {
        ok = __all_sync(0xffffffffu,
                        mbar_wait_bounded(&bar.a_empty[as], (kb / MOE_A_STAGES - 1) & 1, abort_flag));
        if (!ok) break;
      }
      const long long k2 = tr ? clock64() : 0;
      const uint32_t sb = s_cur << 7;              // E8M0 byte in the bf16 exponent field: 2^(s-127)
      const uint32_t sc2 = sb | (sb << 16);
      uint8_t* arow = atile + as * MOE_A_BYTES + r * 128;
      const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {   // 8 elements = one 16-byte chunk of the bf16 row
        uint32_t o[4];
        mxfp4_word_to_bf16x8(cw[q], sc2, o);
        *reinterpret_cast<uint4*>(arow + (((4 * h + q) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_proxy_async_smem();  // the tensor core reads this tile through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.a_full[as]);
      if (tr) {
        trace[2] += k1 - k0;
        trace[3] += k2 - k1;
        trace[4] += clock64() - k2;
      }
    }
    if (!ok) {
      if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_FULL);
      *abort_flag = 1;
    }
  }

  if (warp >= 2 && warp < 6) {
    // ===================================== epilogue (the first four dequantising warps) =====================================
    const int lane_grp = warp & 3;                   // TMEM lanes 32*(warp%4) .. +31
    const int fr = lane_grp * 32 + lane;             // feature row inside the tile
    const int f = tile * MOE_FT + fr;
    const uint32_t trow = tmem + (static_cast<uint32_t>(lane_grp * 32) << 16);
    bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_full, 0, abort_flag));
    if (!ok) {
      if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
      *abort_flag = 1;
    }
    tc_fence_after_sync();
    // every stage has been consumed: the raw and A rings now hold the bf16 output block [tokens][features]
    __nv_bfloat16* dump = reinterpret_cast<__nv_bfloat16*>(base);
    constexpr int OUT_F = EPI == MOE_EPI_SWIGLU ? MOE_FT / 2 : MOE_FT;   // output features per tile
    const float bias = f < a.N ? __ldg(a.bias + static_cast<size_t>(e) * a.N + f) : 0.f;
    for (int c = 0; c < bn; c += 32) {
      float v[32];
      if (ok) {
        tmem_ld_32x32(trow + c, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int tok = c + i;
        float x = v[i] + bias;
        if (EPI == MOE_EPI_SWIGLU) {
          // features are interleaved: even = gate, odd = linear; the partner sits in the neighbouring lane
          const float other = __shfl_xor_sync(0xffffffffu, x, 1);
          if ((lane & 1) == 0) dump[tok * OUT_F + (fr >> 1)] = __float2bfloat16_rn(moe_swiglu(x, other, a.alpha, a.limit));
        } else {
          const float g = tok < n_e ? a.meta->gate_of_row[row0 + tok] : 0.f;
          dump[tok * OUT_F + fr] = __float2bfloat16_rn(x * g);
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // coalesced write-out: 16-byte pieces, a row's pieces on consecutive threads
    constexpr int PIECES = OUT_F / 8;                // 8 (SwiGLU: 128 B per token) or 16 (256 B)
    const int out_n = EPI == MOE_EPI_SWIGLU ? a.N / 2 : a.N;
    const int t4 = (warp - 2) * 32 + lane;
    for (int it = t4; it < n_e * PIECES; it += 128) {
      const int tok = it / PIECES, pc = it - tok * PIECES;
      const int col = tile * OUT_F + pc * 8;
      if (col + 8 <= out_n)
        *reinterpret_cast<uint4*>(a.out + static_cast<size_t>(row0 + tok) * out_n + col) =
            *reinterpret_cast<const uint4*>(dump + tok * OUT_F + pc * 8);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (trace && tid == 0) {
    trace[1] = global_timer_ns();
    trace[7] = n_e;
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, tmem_cols);
  }
}

// out[t] = sum over the token's slots of y[row_of_slot]   (fp32, slot order)
// y2 (optional): the rows' second partial sums, when the last GEMM ran with its k range split in two
__global__ void __launch_bounds__(128) moe_combine_kernel(const __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ out,
                                                          int64_t ld_out, int hidden, int tokens,
                                                          const MoeMeta* __restrict__ meta,
                                                          const __nv_bfloat16* __restrict__ y2 = nullptr) {
  overlap_start();
  overlap_wait();
  const int t = blockIdx.x;
  if (t >= tokens) return;
  int rows[MOE_TOPK];
#pragma unroll
  for (int k = 0; k < MOE_TOPK; ++k) rows[k] = meta->row_of_slot[t * MOE_TOPK + k];
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < MOE_TOPK; ++k) {
      if (rows[k] < 0) continue;
      const uint4 p = __ldg(reinterpret_cast<const uint4*>(y + static_cast<size_t>(rows[k]) * hidden) + i);
      acc[0] += bf16lo(p.x); acc[1] += bf16hi(p.x); acc[2] += bf16lo(p.y); acc[3] += bf16hi(p.y);
      acc[4] += bf16lo(p.z); acc[5] += bf16hi(p.z); acc[6] += bf16lo(p.w); acc[7] += bf16hi(p.w);
      if (y2) {
        const uint4 q = __ldg(reinterpret_cast<const uint4*>(y2 + static_cast<size_t>(rows[k]) * hidden) + i);
        acc[0] += bf16lo(q.x); acc[1] += bf16hi(q.x); acc[2] += bf16lo(q.y); acc[3] += bf16hi(q.y);
        acc[4] += bf16lo(q.z); acc[5] += bf16hi(q.z); acc[6] += bf16lo(q.w); acc[7] += bf16hi(q.w);
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    *(reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ld_out) + i) = o;
  }
}

// =====================================================================================================
// The same expert GEMMs on the tensor cores' own FP4 path: tcgen05.mma.kind::mxf8f6f4.block_scale takes
// the E2M1 codes and their E8M0 scales as they are, so no instruction is spent on conversion and the
// kernel only has to keep HBM busy.  The other operand must then be an 8-bit float: every activation
// row is split into two block-scaled E4M3 terms (x = hi + lo, each with one E8M0 scale per 32 elements),
// which reproduces bf16 inputs exactly (a bf16 mantissa is two E4M3 mantissas wide), and both terms are
// accumulated into the same fp32 accumulator.
//   weights   codes [E][N][Kp/2], Kp = K rounded up to 128, zero padded (TMA type 16U4_ALIGN16B needs it);
//             scales as ready-made 512-byte blocks [E][N/128][Kp/128][r%32][r/32][group%4]
//   moe_route_quant_kernel   the routing (last CTA) and, one CTA per routed (token, slot) pair, the token's bf16 row ->
//             hi / lo E4M3 rows and their scale bytes at the pair's place in the expert-sorted order (the gather)
//   moe_expert_fp4_kernel   warp 0: TMA (codes 8 KiB -> padded 16 KiB tile, the scale block, the tokens' hi and lo
//             tiles); warps 2-5: per stage, the tokens' scale bytes into the same block layout, later the epilogue;
//             warp 1: tcgen05.cp of the scale blocks into tensor memory, then 4 MMAs (K = 32 each) whose N covers the
//             tokens' hi rows and lo rows side by side; the epilogue adds the two halves of the accumulator.
// =====================================================================================================
__device__ __forceinline__ uint16_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint16_t v) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(v));
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
// E8M0 byte that brings a group with maximum magnitude `amax` into [128, 256): well inside E4M3's range
__device__ __forceinline__ uint32_t moe_block_scale_byte(float amax) {
  const int eb = static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu) - 7;
  return static_cast<uint32_t>(eb < 1 ? 1 : (eb > 253 ? 253 : eb));
}

// Eight consecutive values of a row -> their two block-scaled E4M3 terms.  The four threads of an aligned quad hold the
// 32 elements of one scale group (the whole warp must call this together): qb[term] = the 8 codes, sbyte[term] = the
// group's E8M0 scale byte.
__device__ __forceinline__ void moe_quant8(float (&v)[8], uint32_t (&qb)[2][2], uint32_t (&sbyte)[2]) {
#pragma unroll
  for (int term = 0; term < 2; ++term) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const uint32_t sb = moe_block_scale_byte(amax);
    const float inv = __uint_as_float((254u - sb) << 23), sc = __uint_as_float(sb << 23);
    uint16_t q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q[i] = f32x2_to_e4m3x2(v[2 * i] * inv, v[2 * i + 1] * inv);
      const float2 d = e4m3x2_to_f32x2(q[i]);
      v[2 * i] -= d.x * sc;       // exact: what the first term could not hold
      v[2 * i + 1] -= d.y * sc;
    }
    qb[term][0] = q[0] | (static_cast<uint32_t>(q[1]) << 16);
    qb[term][1] = q[2] | (static_cast<uint32_t>(q[3]) << 16);
    sbyte[term] = sb;
  }
}

// One CTA per row; a thread owns 8 consecutive elements, four threads one 32-element group.  With `meta` the CTA is
// a routed (token, slot) pair: it reads the token's row and writes the row of the expert-sorted order (the gather).
// Row src_row of x -> row `row` of the two E4M3 terms and their scale bytes (the whole CTA works on the row).
__device__ __forceinline__ void moe_quant_row(const __nv_bfloat16* __restrict__ x, int64_t ldx, int K,
                                              uint8_t* __restrict__ q_hi, uint8_t* __restrict__ q_lo,
                                              uint8_t* __restrict__ sf_hi, uint8_t* __restrict__ sf_lo, int sf_stride,
                                              int row, int src_row) {
  const int chunks = K / 8;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(src_row) * ldx);
  for (int base = 0; base < chunks; base += blockDim.x) {   // uniform trip count: the shuffles need whole warps
    const int c = base + threadIdx.x;
    const bool live = c < chunks;
    float v[8];
    if (live) {
      const uint4 p = __ldg(src + c);
      v[0] = bf16lo(p.x); v[1] = bf16hi(p.x); v[2] = bf16lo(p.y); v[3] = bf16hi(p.y);
      v[4] = bf16lo(p.z); v[5] = bf16hi(p.z); v[6] = bf16lo(p.w); v[7] = bf16hi(p.w);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    uint32_t qb[2][2];
    uint32_t sbyte[2];
    moe_quant8(v, qb, sbyte);
    if (live) {
      *reinterpret_cast<uint2*>(q_hi + static_cast<size_t>(row) * K + 8 * c) = make_uint2(qb[0][0], qb[0][1]);
      *reinterpret_cast<uint2*>(q_lo + static_cast<size_t>(row) * K + 8 * c) = make_uint2(qb[1][0], qb[1][1]);
      if ((c & 3) == 0) {
        sf_hi[static_cast<size_t>(row) * sf_stride + (c >> 2)] = static_cast<uint8_t>(sbyte[0]);
        sf_lo[static_cast<size_t>(row) * sf_stride + (c >> 2)] = static_cast<uint8_t>(sbyte[1]);
      }
    }
  }
  // groups past K (the weights are zero there) get a harmless scale of 1
  for (int g = K / 32 + threadIdx.x; g < sf_stride; g += blockDim.x) {
    sf_hi[static_cast<size_t>(row) * sf_stride + g] = 127;
    sf_lo[static_cast<size_t>(row) * sf_stride + g] = 127;
  }
}

// One CTA per routed (token, slot) pair, after the routing kernel: the token's row -> the pair's row of the sorted order.
__global__ void __launch_bounds__(128) moe_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int K,
                                                        uint8_t* __restrict__ q_hi, uint8_t* __restrict__ q_lo,
                                                        uint8_t* __restrict__ sf_hi, uint8_t* __restrict__ sf_lo, int sf_stride,
                                                        const MoeMeta* __restrict__ meta) {
  overlap_start();
  overlap_wait();
  const int row = meta->row_of_slot[blockIdx.x];
  if (row < 0) return;
  moe_quant_row(x, ldx, K, q_hi, q_lo, sf_hi, sf_lo, sf_stride, row, blockIdx.x / MOE_TOPK);
}

// Routing and the first quantise / gather pass in one launch: CTA `slots` (the last) does the routing for the kernels
// that follow; CTA sl < slots quantises the row of routed pair sl and finds its place in the expert-sorted order by
// itself: (tokens' distinct valid experts below e) + (earlier tokens that chose e), which is what the routing CTA
// writes into row_of_slot at the same time.
constexpr int MOE_RQ_THREADS = 256;
__global__ void __launch_bounds__(MOE_RQ_THREADS)
moe_route_quant_kernel(const int16_t* __restrict__ topk_idx, const float* __restrict__ topk_w, int tokens, int n_experts,
                       MoeMeta* meta, int* status, int tok, const __nv_bfloat16* __restrict__ x, int64_t ldx, int K,
                       uint8_t* __restrict__ q_hi, uint8_t* __restrict__ q_lo, uint8_t* __restrict__ sf_hi,
                       uint8_t* __restrict__ sf_lo, int sf_stride) {
  const int slots = tokens * MOE_TOPK;
  if (static_cast<int>(blockIdx.x) == slots) {
    moe_route_body(topk_idx, topk_w, tokens, n_experts, meta, status, tok);
    return;
  }
  overlap_start();
  overlap_wait();
  __shared__ int s_cnt[MOE_RQ_THREADS / 32];
  const int sl = blockIdx.x, t = sl / MOE_TOPK;
  const int e = topk_idx[sl];
  if (e < 0 || e >= n_experts) return;   // flagged by the routing CTA; the pair has no row
  int cnt = 0;
  for (int u = threadIdx.x; u < tokens; u += blockDim.x) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(topk_idx) + u);
    const int id[4] = {static_cast<int16_t>(raw.x & 0xffffu), static_cast<int16_t>(raw.x >> 16),
                       static_cast<int16_t>(raw.y & 0xffffu), static_cast<int16_t>(raw.y >> 16)};
#pragma unroll
    for (int k = 0; k < MOE_TOPK; ++k) {
      const int ek = id[k];
      if (ek < 0 || ek >= n_experts) continue;
      bool first = true;   // a repeated id counts once, as in the routing CTA's bit masks
#pragma unroll
      for (int j = 0; j < k; ++j) first = first && id[j] != ek;
      if (first && (ek < e || (ek == e && u < t))) ++cnt;
    }
  }
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  if ((threadIdx.x & 31) == 0) s_cnt[threadIdx.x >> 5] = cnt;
  __syncthreads();
  int row = 0;
#pragma unroll
  for (int w = 0; w < MOE_RQ_THREADS / 32; ++w) row += s_cnt[w];
  moe_quant_row(x, ldx, K, q_hi, q_lo, sf_hi, sf_lo, sf_stride, row, t);
}

constexpr int FP4_KB = 128;                       // K elements per pipeline stage (4 MMA steps of 32)
constexpr int FP4_A_BYTES = MOE_FT * FP4_KB;      // 16 KiB in shared memory (8 KiB in HBM)
constexpr int FP4_A_TX = MOE_FT * FP4_KB / 2;     // bytes the TMA transaction counts for it
constexpr int FP4_MAX_STAGES = 8;
constexpr int FP4_THREADS = 192;

struct MoeFp4Args {
  const uint8_t* sfa;       // [E][tiles][nkb][512]
  const uint8_t* sf_hi;     // [rows][4*nkb]
  const uint8_t* sf_lo;
  const float* bias;
  const MoeMeta* meta;
  __nv_bfloat16* out;
  int N, nkb, tiles, bn_max, stages, sf_col;
  // SwiGLU epilogue: the activations leave the kernel already split into the two E4M3 terms the second GEMM reads
  uint8_t* q2_hi;           // [rows][K2]
  uint8_t* q2_lo;
  uint8_t* sf2_hi;          // [rows][sf2_stride]
  uint8_t* sf2_lo;
  int K2, sf2_stride;
  int prefetch;             // k-blocks of weights (codes + scale block) requested into L2 ahead of the ring
  int tok;                  // tokens of one expert per CTA (32 or 64); the rest go to the next CTAs along grid.x
  int ksplit;               // persistent kernel, gate epilogue: 1, or 2 = a unit is one half of a tile's k range and the
  int64_t out_half_stride;  //   second half's partial rows go out_half_stride elements further (the combine adds them)
  float alpha, limit;
  int* status;
};

struct __align__(16) MoeFp4Barriers {
  uint64_t full[FP4_MAX_STAGES];
  uint64_t empty[FP4_MAX_STAGES];
  uint64_t sfb_full[FP4_MAX_STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

template <int EPI>
__global__ void __launch_bounds__(FP4_THREADS)
moe_expert_fp4_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_hi,
                      const __grid_constant__ CUtensorMap tm_lo, const MoeFp4Args a) {
  overlap_start();
  overlap_wait();
  // an expert's tokens are handled a.tok (32, or 64 by the tunable) at a time: grid.y walks the list of non-empty (expert, part) pairs the routing
  // kernel wrote (at most rows / tok + experts of them), grid.x the weight tiles, so the CTAs that share a weight
  // tile run in the same wave and all but the first find it in L2.  hi and lo terms sit side by side in the MMA's N
  const int tile = blockIdx.x, item = blockIdx.y;
  if (item >= a.meta->n_items) return;
  const int e = a.meta->item_expert[item], part = a.meta->item_part[item];
  const int n_e = min(a.meta->counts[e] - a.tok * part, a.tok);
  if (n_e <= 0) return;
  const int row0 = a.meta->offsets[e] + a.tok * part;
  const int bn = (n_e + 31) & ~31;
  const int atoms = (2 * bn + 127) >> 7;        // 512-byte scale blocks for the 2 x bn token rows (hi rows, then lo rows)

  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int S = a.stages;
  const int b_stage_bytes = 2 * a.bn_max * 128;                // hi rows, then lo rows, of the token tile
  uint8_t* atile = base;                                        // S x 16 KiB
  uint8_t* btile = atile + static_cast<size_t>(S) * FP4_A_BYTES;   // S x 2 x bn_max x 128
  uint8_t* sfa_s = btile + static_cast<size_t>(S) * b_stage_bytes;      // S x 512
  uint8_t* sfb_s = sfa_s + static_cast<size_t>(S) * 512;        // S x 2 terms x 2 blocks x 512
  MoeFp4Barriers& bar = *reinterpret_cast<MoeFp4Barriers*>(sfb_s + static_cast<size_t>(S) * 2048);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &bar.abort_flag;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&bar.full[s], 1);
      mbar_init(&bar.empty[s], 1);
      mbar_init(&bar.sfb_full[s], 4);
    }
    mbar_init(&bar.acc_full, 1);
    bar.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_hi);
    tma_prefetch_desc(&tm_lo);
  }
  int tmem_cols = 32;
  while (tmem_cols < a.sf_col + 12) tmem_cols <<= 1;   // accumulator, 4 columns of weight scales, 8 of token scales
  if (warp == 1) tmem_alloc(&bar.tmem_base, tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bar.tmem_base;
  const int nkb = a.nkb;

  if (warp == 0) {
    // ===================================== producer =====================================
    const bool leader = elect_one();
    const int xblocks = bn >> 5;
    const uint8_t* sfa_g = a.sfa + (static_cast<size_t>(e) * a.tiles + tile) * nkb * 512;
    bool ok = true;
    const int PF = a.prefetch;
    if (leader)
      for (int kb = 0; kb < PF && kb < nkb; ++kb) {
        tma_prefetch_l2_4d(&tm_w, kb * FP4_KB, tile * MOE_FT, e, 0);
        bulk_prefetch_l2(sfa_g + static_cast<size_t>(kb) * 512, 512);
      }
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const int s = kb % S, round = kb / S;
      if (leader && PF > 0 && kb + PF < nkb) {   // before the wait: the request leaves as early as possible
        tma_prefetch_l2_4d(&tm_w, (kb + PF) * FP4_KB, tile * MOE_FT, e, 0);
        bulk_prefetch_l2(sfa_g + static_cast<size_t>(kb + PF) * 512, 512);
      }
      if (round > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.empty[s], (round - 1) & 1, abort_flag));
      if (!ok) break;
      if (leader) {
        mbar_arrive_expect_tx(&bar.full[s], static_cast<uint32_t>(FP4_A_TX + 512 + 2 * xblocks * 32 * 128));
        tma_load_4d(atile + static_cast<size_t>(s) * FP4_A_BYTES, &tm_w, &bar.full[s], kb * FP4_KB, tile * MOE_FT, e, 0);
        bulk_load(sfa_s + s * 512, sfa_g + static_cast<size_t>(kb) * 512, 512, &bar.full[s]);
        uint8_t* bt = btile + static_cast<size_t>(s) * b_stage_bytes;
        for (int xb = 0; xb < xblocks; ++xb) {
          tma_load_2d(bt + xb * 4096, &tm_hi, &bar.full[s], kb * FP4_KB, row0 + 32 * xb);
          tma_load_2d(bt + (xblocks + xb) * 4096, &tm_lo, &bar.full[s], kb * FP4_KB, row0 + 32 * xb);   // lo rows follow hi rows
        }
      }
      __syncwarp();
    }
    if (leader && !ok) {
      if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
      *abort_flag = 1;
    }
  } else if (warp == 1) {
    // ===================================== MMA issuer =====================================
    const bool leader = elect_one();
    const uint32_t t_sfa = tmem + a.sf_col, t_sfb = t_sfa + 4;
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
      const int s = kb % S;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.full[s], (kb / S) & 1, abort_flag)) &&
           __all_sync(0xffffffffu, mbar_wait_bounded(&bar.sfb_full[s], (kb / S) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after_sync();
      const uint64_t da = umma_desc_k128(smem_u32(atile + static_cast<size_t>(s) * FP4_A_BYTES));
      const uint64_t db = umma_desc_k128(smem_u32(btile + static_cast<size_t>(s) * b_stage_bytes));
      const uint32_t sfb_addr = smem_u32(sfb_s + s * 2048);
      if (leader) {
        tmem_cp_sf_block(t_sfa, umma_desc_sf_block(smem_u32(sfa_s + s * 512)));
        for (int at = 0; at < atoms; ++at) tmem_cp_sf_block(t_sfb + 4 * at, umma_desc_sf_block(sfb_addr + at * 512));
#pragma unroll
        for (int k = 0; k < FP4_KB / 32; ++k)   // 32 elements = 32 bytes of either operand's rows = 2 descriptor units
          umma_fp4_fp8(tmem, da + 2 * k, db + 2 * k, umma_idesc_fp4_fp8(MOE_FT, 2 * bn, k, k), t_sfa, t_sfb, (kb | k) != 0);
        umma_commit(&bar.empty[s]);
      }
      __syncwarp();
    }
    if (leader) {
      if (ok) {
        umma_commit(&bar.acc_full);
      } else {
        if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
        *abort_flag = 1;
      }
    }
  } else {
    // ===================================== token scale blocks, then the epilogue =====================================
    const int t4 = (warp - 2) * 32 + lane;   // 0..127
    const int sf_stride = 4 * nkb;
    // row n2 of the [hi rows; lo rows] token tile: term and token; the four scale bytes of one stage are one word,
    // fetched a stage ahead so that the latency is off the MMA's path
    auto load_tsf = [&](int n2, int kb) -> uint32_t {
      const int term = n2 >= bn, n = n2 - term * bn;
      const uint8_t* sf = term ? a.sf_lo : a.sf_hi;
      return (n2 < 2 * bn && n < n_e) ? __ldg(reinterpret_cast<const uint32_t*>(sf + static_cast<size_t>(row0 + n) * sf_stride) + kb)
                                     : 0x7f7f7f7fu;
    };
    // the words of the next TSF_AHEAD stages are in registers: a load has that many stages to come back from L2
    constexpr int TSF_AHEAD = 4;
    uint32_t nx[TSF_AHEAD][2];
#pragma unroll
    for (int d = 0; d < TSF_AHEAD; ++d) {
      nx[d][0] = d < nkb ? load_tsf(t4, d) : 0x7f7f7f7fu;
      nx[d][1] = (d < nkb && atoms > 1) ? load_tsf(t4 + 128, d) : 0x7f7f7f7fu;
    }
    const int off = (t4 & 31) * 16 + (t4 >> 5) * 4;
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      const int s = kb % S, round = kb / S;
      const uint32_t cur[2] = {nx[0][0], nx[0][1]};
#pragma unroll
      for (int d = 0; d + 1 < TSF_AHEAD; ++d) {
        nx[d][0] = nx[d + 1][0];
        nx[d][1] = nx[d + 1][1];
      }
      if (kb + TSF_AHEAD < nkb) {
        nx[TSF_AHEAD - 1][0] = load_tsf(t4, kb + TSF_AHEAD);
        if (atoms > 1) nx[TSF_AHEAD - 1][1] = load_tsf(t4 + 128, kb + TSF_AHEAD);
      }
      if (round > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.empty[s], (round - 1) & 1, abort_flag));
      if (!ok) break;
      uint8_t* blk = sfb_s + s * 2048;
      *reinterpret_cast<uint32_t*>(blk + off) = cur[0];
      if (atoms > 1) *reinterpret_cast<uint32_t*>(blk + 512 + off) = cur[1];
      fence_proxy_async_smem();   // tcgen05.cp reads the blocks through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.sfb_full[s]);
    }
    if (!ok) {
      if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
      *abort_flag = 1;
    }

    const int lane_grp = warp & 3;
    const int fr = lane_grp * 32 + lane;
    const int f = tile * MOE_FT + fr;
    const uint32_t trow = tmem + (static_cast<uint32_t>(lane_grp * 32) << 16);
    ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_full, 0, abort_flag));
    if (!ok) {
      if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
      *abort_flag = 1;
    }
    tc_fence_after_sync();
    __nv_bfloat16* dump = reinterpret_cast<__nv_bfloat16*>(base);   // the A ring is idle now
    constexpr int OUT_F = EPI == MOE_EPI_SWIGLU ? MOE_FT / 2 : MOE_FT;
    const float bias = f < a.N ? __ldg(a.bias + static_cast<size_t>(e) * a.N + f) : 0.f;
    for (int c = 0; c < bn; c += 32) {
      float v[32];
      if (ok) {   // columns c.. hold the hi term's sums, columns bn + c.. the lo term's
        float w[32];
        tmem_ld_32x32_nowait(trow + c, v);
        tmem_ld_32x32_nowait(trow + bn + c, w);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] += w[i];
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int tok = c + i;
        const float xv = v[i] + bias;
        if (EPI == MOE_EPI_SWIGLU) {
          const float other = __shfl_xor_sync(0xffffffffu, xv, 1);
          if ((lane & 1) == 0) dump[tok * OUT_F + (fr >> 1)] = __float2bfloat16_rn(moe_swiglu(xv, other, a.alpha, a.limit));
        } else {
          const float g = tok < n_e ? a.meta->gate_of_row[row0 + tok] : 0.f;
          dump[tok * OUT_F + fr] = __float2bfloat16_rn(xv * g);
        }
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    constexpr int PIECES = OUT_F / 8;
    const int out_n = EPI == MOE_EPI_SWIGLU ? a.N / 2 : a.N;
    if constexpr (EPI == MOE_EPI_SWIGLU) {
      // the bf16 activations go straight into the form the second GEMM reads: two block-scaled E4M3 terms per row, one
      // scale byte per 32 features (a tile's 64 features are two whole groups); a thread owns 8 features, a quad a group
      const int total = n_e * PIECES;
      for (int base = 0; base < total; base += 128) {   // uniform trip count: the shuffles need whole warps
        const int it = base + t4;
        const bool live = it < total;
        const int tok = live ? it / PIECES : 0, pc = it - (it / PIECES) * PIECES;
        float v[8];
        if (live) {
          const uint4 p = *reinterpret_cast<const uint4*>(dump + tok * OUT_F + pc * 8);
          v[0] = bf16lo(p.x); v[1] = bf16hi(p.x); v[2] = bf16lo(p.y); v[3] = bf16hi(p.y);
          v[4] = bf16lo(p.z); v[5] = bf16hi(p.z); v[6] = bf16lo(p.w); v[7] = bf16hi(p.w);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = 0.f;
        }
        uint32_t qb[2][2];
        uint32_t sbyte[2];
        moe_quant8(v, qb, sbyte);
        const int col = tile * OUT_F + pc * 8;
        if (live && col + 8 <= out_n) {
          const size_t row = static_cast<size_t>(row0 + tok);
          *reinterpret_cast<uint2*>(a.q2_hi + row * a.K2 + col) = make_uint2(qb[0][0], qb[0][1]);
          *reinterpret_cast<uint2*>(a.q2_lo + row * a.K2 + col) = make_uint2(qb[1][0], qb[1][1]);
          if ((pc & 3) == 0) {
            const int g = col >> 5;
            a.sf2_hi[row * a.sf2_stride + g] = static_cast<uint8_t>(sbyte[0]);
            a.sf2_lo[row * a.sf2_stride + g] = static_cast<uint8_t>(sbyte[1]);
            if (g == a.K2 / 32 - 1)   // groups past K2 (the weights are zero there) get a harmless scale of 1
              for (int gg = g + 1; gg < a.sf2_stride; ++gg) {
                a.sf2_hi[row * a.sf2_stride + gg] = 127;
                a.sf2_lo[row * a.sf2_stride + gg] = 127;
              }
          }
        }
      }
    } else {
      for (int it = t4; it < n_e * PIECES; it += 128) {
        const int tok = it / PIECES, pc = it - tok * PIECES;
        const int col = tile * OUT_F + pc * 8;
        if (col + 8 <= out_n)
          *reinterpret_cast<uint4*>(a.out + static_cast<size_t>(row0 + tok) * out_n + col) =
              *reinterpret_cast<const uint4*>(dump + tok * OUT_F + pc * 8);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, tmem_cols);
  }
}


// =====================================================================================================
// The persistent form of moe_expert_fp4_kernel for 32-token parts.  The one-shot kernel spends about a third of a
// CTA's life with nothing in flight (launch, barrier and tensor-memory set-up before its first load; accumulator
// write-out after its last), which is what keeps it near half of the copy bandwidth.  Here a fixed grid of CTAs walks
// the list of (expert part, weight tile) units, unit w = blockIdx.x + i * gridDim.x with the tile index running
// fastest, and the ring of stages simply continues from one unit into the next:
//   warp 0   : TMA producer as before; it also writes the tokens' scale bytes of a stage into the block layout
//              (64 words per stage, fetched FPP_AHEAD k-blocks ahead through a second cursor over the same stream
//              of (unit, k-block) positions), so that no epilogue warp is needed inside the k loop;
//   warp 1   : MMA issuer; one accumulator (64 columns: hi sums | lo sums).  It waits for the epilogue warps to have
//              copied the previous unit's sums into registers (a few hundred clocks) while the producer already
//              fills the ring with the next unit's first stages;
//   warps 2-5: epilogue only: accumulator -> registers, release it, then bias, SwiGLU + requantisation or gate,
//              staged through 4 KiB of shared memory of their own (the ring is never idle here).
// Shared memory per stage: 16 KiB padded codes + 8 KiB token tiles + 512 B + 512 B scale blocks.
// Measured (32 / 256 tokens, whole op): one-shot kernel 133 / 165 us; this kernel with 4 CTAs x 2 stages per SM
// 112 / 134 us, 2 x 4 stages 109 / 141 us, 1 x 8 stages 164 / 232 us.  A variant that gave every CTA an equal
// contiguous share of the (unit, k-block) stream, cutting units between neighbouring CTAs and handing the partial sums
// over through global memory, removed the partly empty last round but came out slower (118 / 149 us): the CTAs that
// are still running in the last round stream faster when the others have finished, and the hand-off is not free.
// =====================================================================================================
constexpr int FPP_BN = 32;            // tokens of an expert per unit
constexpr int FPP_BN_SMALL = 8;       // ... when the batch is so small that an expert gets a handful of tokens: the token
                                      // tiles of a stage shrink from 8 KiB to 2 KiB and an SM holds ten stages instead of eight
__host__ __device__ constexpr int fpp_stage_bytes(int bn) { return FP4_A_BYTES + 2 * bn * 128 + 512 + 512; }
constexpr int FPP_DUMP_BYTES = 4096;
constexpr int FPP_AHEAD = 4;          // k-blocks the token scale words are fetched ahead

struct __align__(16) MoeFppBarriers {
  uint64_t full[FP4_MAX_STAGES];     // 2 arrivals: the TMA transaction's and the scale writer's
  uint64_t empty[FP4_MAX_STAGES];
  uint64_t acc_full;
  uint64_t acc_empty;                // 4 arrivals: one per epilogue warp
  uint32_t tmem_base;
  int abort_flag;
};

struct FppUnit {   // one (expert part, weight tile[, half of the k range]) of the CTA's list
  int e, row0, n_e, tile;
  int kh, kb0, kb1;   // which part of the k range, and its k-blocks [kb0, kb1)
  int side, item;     // fused kernel: which GEMM (0 / 1) and which (expert, part) of the item list
  bool valid;
};
__device__ __forceinline__ FppUnit fpp_unit(const MoeFp4Args& a, int i, int n_units) {
  FppUnit u;
  const int w = static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
  u.valid = w < n_units;
  u.side = u.item = 0;
  if (!u.valid) {
    u.e = u.row0 = u.n_e = u.tile = u.kh = u.kb0 = u.kb1 = 0;
    return u;
  }
  const int per_item = a.tiles * a.ksplit;
  const int item = w / per_item, rem = w - item * per_item;
  u.tile = rem / a.ksplit;
  u.kh = rem - u.tile * a.ksplit;
  u.kb0 = u.kh * a.nkb / a.ksplit;
  u.kb1 = (u.kh + 1) * a.nkb / a.ksplit;
  u.e = a.meta->item_expert[item];
  const int part = a.meta->item_part[item];
  u.n_e = min(a.meta->counts[u.e] - a.tok * part, a.tok);
  u.row0 = a.meta->offsets[u.e] + a.tok * part;
  return u;
}

template <int EPI, int BN>
__global__ void __launch_bounds__(FP4_THREADS)
moe_expert_fp4_persist_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_hi,
                              const __grid_constant__ CUtensorMap tm_lo, const MoeFp4Args a) {
  overlap_start();
  overlap_wait();
  const int n_units = a.meta->n_items * a.tiles * a.ksplit;
  if (static_cast<int>(blockIdx.x) >= n_units) return;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int S = a.stages;
  uint8_t* atile = smem_raw;                                              // S x 16 KiB
  uint8_t* btile = atile + static_cast<size_t>(S) * FP4_A_BYTES;          // S x (32 hi rows, 32 lo rows) x 128
  uint8_t* sfa_s = btile + static_cast<size_t>(S) * (2 * BN * 128);   // S x 512
  uint8_t* sfb_s = sfa_s + static_cast<size_t>(S) * 512;                  // S x 512
  uint8_t* dump_s = sfb_s + static_cast<size_t>(S) * 512;                 // 4 KiB
  MoeFppBarriers& bar = *reinterpret_cast<MoeFppBarriers*>(dump_s + FPP_DUMP_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &bar.abort_flag;
  if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need this alignment
    if (tid == 0) atomicOr(a.status, B2_DEV_BAD_INDEX);
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&bar.full[s], 2);
      mbar_init(&bar.empty[s], 1);
    }
    mbar_init(&bar.acc_full, 1);
    mbar_init(&bar.acc_empty, 4);
    bar.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_hi);
    tma_prefetch_desc(&tm_lo);
  }
  // rows 64..127 of a token scale block are never written again: a harmless scale of 1
  for (int i = tid; i < S * 128; i += FP4_THREADS) reinterpret_cast<uint32_t*>(sfb_s)[i] = 0x7f7f7f7fu;
  fence_proxy_async_smem();
  constexpr int TMEM_COLS = BN == 32 ? 128 : (BN == 16 ? 64 : 32);   // accumulator 2 * BN, weight scales 4, token scales 4
  if (warp == 1) tmem_alloc(&bar.tmem_base, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bar.tmem_base;
  const int nkb = a.nkb;

  if (warp == 0) {
    // ===================================== producer + token scale blocks =====================================
    const bool leader = elect_one();
    const int sf_stride = 4 * nkb;
    struct Cur {
      int i, kb;
      FppUnit u;
    };
    auto next = [&](Cur& c) {
      if (++c.kb >= c.u.kb1) {
        ++c.i;
        c.u = fpp_unit(a, c.i, n_units);
        c.kb = c.u.kb0;
      }
    };
    // row n2 of the [hi rows; lo rows] token tile: the four scale bytes of one k-block are one word
    auto load_tsf = [&](const Cur& c, int n2) -> uint32_t {
      const int term = n2 >= BN, n = n2 - term * BN;
      const uint8_t* sf = term ? a.sf_lo : a.sf_hi;
      return (c.u.valid && n2 < 2 * BN && n < c.u.n_e)
                 ? __ldg(reinterpret_cast<const uint32_t*>(sf + static_cast<size_t>(c.u.row0 + n) * sf_stride) + c.kb)
                 : 0x7f7f7f7fu;
    };
    Cur cur{0, 0, fpp_unit(a, 0, n_units)};
    cur.kb = cur.u.kb0;
    Cur pre = cur;
    uint32_t nx[FPP_AHEAD][2];
#pragma unroll
    for (int d = 0; d < FPP_AHEAD; ++d) {
      nx[d][0] = load_tsf(pre, lane);
      nx[d][1] = load_tsf(pre, lane + 32);
      next(pre);
    }
    const int off = lane * 16;   // row r of the block: (r % 32) * 16 + (r / 32) * 4
    bool ok = true;
    for (int g = 0; cur.u.valid && ok; ++g) {
      const int s = g % S, round = g / S;
      const uint32_t w0 = nx[0][0], w1 = nx[0][1];
#pragma unroll
      for (int d = 0; d + 1 < FPP_AHEAD; ++d) {
        nx[d][0] = nx[d + 1][0];
        nx[d][1] = nx[d + 1][1];
      }
      nx[FPP_AHEAD - 1][0] = load_tsf(pre, lane);
      nx[FPP_AHEAD - 1][1] = load_tsf(pre, lane + 32);
      next(pre);
      if (round > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.empty[s], (round - 1) & 1, abort_flag));
      if (!ok) break;
      if (leader) {
        mbar_arrive_expect_tx(&bar.full[s], static_cast<uint32_t>(FP4_A_TX + 512 + 2 * BN * 128));
        tma_load_4d(atile + static_cast<size_t>(s) * FP4_A_BYTES, &tm_w, &bar.full[s], cur.kb * FP4_KB, cur.u.tile * MOE_FT,
                    cur.u.e, 0);
        bulk_load(sfa_s + s * 512,
                  a.sfa + ((static_cast<size_t>(cur.u.e) * a.tiles + cur.u.tile) * nkb + cur.kb) * 512, 512, &bar.full[s]);
        uint8_t* bt = btile + static_cast<size_t>(s) * (2 * BN * 128);
        tma_load_2d(bt, &tm_hi, &bar.full[s], cur.kb * FP4_KB, cur.u.row0);
        tma_load_2d(bt + BN * 128, &tm_lo, &bar.full[s], cur.kb * FP4_KB, cur.u.row0);   // lo rows follow hi rows
      }
      uint8_t* blk = sfb_s + s * 512;
      if (lane < 2 * BN) *reinterpret_cast<uint32_t*>(blk + off) = w0;
      if (BN == 32) *reinterpret_cast<uint32_t*>(blk + off + 4) = w1;
      fence_proxy_async_smem();   // tcgen05.cp reads the block through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.full[s]);
      next(cur);
    }
    if (leader && !ok) {
      if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
      *abort_flag = 1;
    }
  } else if (warp == 1) {
    // ===================================== MMA issuer =====================================
    const bool leader = elect_one();
    const uint32_t t_sfa = tmem + 2 * BN, t_sfb = t_sfa + 4;
    bool ok = true;
    int g = 0;
    for (int i = 0; ok; ++i) {
      const FppUnit u = fpp_unit(a, i, n_units);
      if (!u.valid) break;
      for (int kb = u.kb0; kb < u.kb1 && ok; ++kb, ++g) {
        const int s = g % S;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.full[s], (g / S) & 1, abort_flag));
        // the previous unit's sums must have left the accumulator
        if (ok && kb == u.kb0 && i > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_empty, (i - 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t da = umma_desc_k128(smem_u32(atile + static_cast<size_t>(s) * FP4_A_BYTES));
        const uint64_t db = umma_desc_k128(smem_u32(btile + static_cast<size_t>(s) * (2 * BN * 128)));
        if (leader) {
          tmem_cp_sf_block(t_sfa, umma_desc_sf_block(smem_u32(sfa_s + s * 512)));
          tmem_cp_sf_block(t_sfb, umma_desc_sf_block(smem_u32(sfb_s + s * 512)));
#pragma unroll
          for (int k = 0; k < FP4_KB / 32; ++k)
            umma_fp4_fp8(tmem, da + 2 * k, db + 2 * k, umma_idesc_fp4_fp8(MOE_FT, 2 * BN, k, k), t_sfa, t_sfb,
                         ((kb - u.kb0) | k) != 0);
          umma_commit(&bar.empty[s]);
          if (kb == u.kb1 - 1) umma_commit(&bar.acc_full);
        }
        __syncwarp();
      }
    }
    if (leader && !ok) {
      if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
      *abort_flag = 1;
    }
  } else {
    // ===================================== epilogue =====================================
    const int t4 = (warp - 2) * 32 + lane;   // 0..127
    const int lane_grp = warp & 3;
    const int fr = lane_grp * 32 + lane;     // feature row of this thread inside the tile
    const uint32_t trow = tmem + (static_cast<uint32_t>(lane_grp * 32) << 16);
    __nv_bfloat16* dump = reinterpret_cast<__nv_bfloat16*>(dump_s);
    constexpr int OUT_F = EPI == MOE_EPI_SWIGLU ? MOE_FT / 2 : MOE_FT;
    constexpr int PIECES = OUT_F / 8;
    const int out_n = EPI == MOE_EPI_SWIGLU ? a.N / 2 : a.N;
    bool ok = true;
    for (int i = 0; ok; ++i) {
      const FppUnit u = fpp_unit(a, i, n_units);
      if (!u.valid) break;
      const int f = u.tile * MOE_FT + fr;
      const float bias = (f < a.N && u.kh == 0) ? __ldg(a.bias + static_cast<size_t>(u.e) * a.N + f) : 0.f;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_full, i & 1, abort_flag));
      if (!ok) {
        if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      float v[32];   // tokens 0 .. BN-1 are meaningful
      if constexpr (BN == 32) {   // columns 0..31 hold the hi term's sums, columns 32..63 the lo term's
        float w[32];
        tmem_ld_32x32_nowait(trow, v);
        tmem_ld_32x32_nowait(trow + BN, w);
        tmem_wait_ld();
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] += w[t];
      } else {                    // one load covers the allocation: hi sums in columns 0..BN-1, lo sums in BN..2BN-1
        float w[32];
        tmem_ld_32x32(trow, w);
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = t < BN ? w[t] + w[(t + BN) & 31] : 0.f;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.acc_empty);   // the MMA warp may start the next unit

      if constexpr (EPI == MOE_EPI_SWIGLU) {
#pragma unroll
        for (int t = 0; t < BN; ++t) {
          const float xv = v[t] + bias;
          const float other = __shfl_xor_sync(0xffffffffu, xv, 1);
          if ((lane & 1) == 0) dump[t * OUT_F + (fr >> 1)] = __float2bfloat16_rn(moe_swiglu(xv, other, a.alpha, a.limit));
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // straight into the form the second GEMM reads: two block-scaled E4M3 terms per row, one scale byte per 32
        // features (a tile's 64 features are two whole groups); a thread owns 8 features, a quad a group
        const int total = u.n_e * PIECES;
        for (int base = 0; base < total; base += 128) {   // uniform trip count: the shuffles need whole warps
          const int it = base + t4;
          const bool live = it < total;
          const int tok = live ? it / PIECES : 0, pc = it - (it / PIECES) * PIECES;
          float q[8];
          if (live) {
            const uint4 p = *reinterpret_cast<const uint4*>(dump + tok * OUT_F + pc * 8);
            q[0] = bf16lo(p.x); q[1] = bf16hi(p.x); q[2] = bf16lo(p.y); q[3] = bf16hi(p.y);
            q[4] = bf16lo(p.z); q[5] = bf16hi(p.z); q[6] = bf16lo(p.w); q[7] = bf16hi(p.w);
          } else {
#pragma unroll
            for (int t = 0; t < 8; ++t) q[t] = 0.f;
          }
          uint32_t qb[2][2];
          uint32_t sbyte[2];
          moe_quant8(q, qb, sbyte);
          const int col = u.tile * OUT_F + pc * 8;
          if (live && col + 8 <= out_n) {
            const size_t row = static_cast<size_t>(u.row0 + tok);
            *reinterpret_cast<uint2*>(a.q2_hi + row * a.K2 + col) = make_uint2(qb[0][0], qb[0][1]);
            *reinterpret_cast<uint2*>(a.q2_lo + row * a.K2 + col) = make_uint2(qb[1][0], qb[1][1]);
            if ((pc & 3) == 0) {
              const int gq = col >> 5;
              a.sf2_hi[row * a.sf2_stride + gq] = static_cast<uint8_t>(sbyte[0]);
              a.sf2_lo[row * a.sf2_stride + gq] = static_cast<uint8_t>(sbyte[1]);
              if (gq == a.K2 / 32 - 1)   // groups past K2 (the weights are zero there) get a harmless scale of 1
                for (int gg = gq + 1; gg < a.sf2_stride; ++gg) {
                  a.sf2_hi[row * a.sf2_stride + gg] = 127;
                  a.sf2_lo[row * a.sf2_stride + gg] = 127;
                }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the dump is free for the next unit
      } else {
        // 128 features x 16 tokens fill the 4 KiB: two passes for 32 tokens
        constexpr int PASS = BN < 16 ? BN : 16;
#pragma unroll
        for (int half = 0; half < BN / PASS; ++half) {
#pragma unroll
          for (int t = 0; t < PASS; ++t) {
            const int tok = PASS * half + t;
            const float gw = tok < u.n_e ? a.meta->gate_of_row[u.row0 + tok] : 0.f;
            dump[t * OUT_F + fr] = __float2bfloat16_rn((v[tok] + bias) * gw);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int n_here = min(u.n_e - PASS * half, PASS);
          for (int it = t4; it < n_here * PIECES; it += 128) {
            const int tok = it / PIECES, pc = it - tok * PIECES;
            const int col = u.tile * OUT_F + pc * 8;
            if (col + 8 <= out_n)
              *reinterpret_cast<uint4*>(a.out + u.kh * a.out_half_stride + static_cast<size_t>(u.row0 + PASS * half + tok) * out_n + col) =
                  *reinterpret_cast<const uint4*>(dump + tok * OUT_F + pc * 8);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}


// =====================================================================================================
// Both expert GEMMs in one persistent launch.  The unit list is the first GEMM's units followed by the second's; the
// CTAs walk it with a stride of the grid as above, so the second GEMM's first units fill the SMs that the first GEMM's
// last, partly empty round would leave idle, and there is no launch boundary between the two.  A unit of the second
// GEMM depends on all weight tiles of the first GEMM for the same (expert, part): each of those counts itself in
// MoeMeta::item_done after storing its rows (release), and the producer warp of the dependent unit waits (bounded,
// acquire) before it requests anything the first GEMM wrote.  Every CTA of the grid is resident (the host sizes the grid
// by registers, shared memory and tensor memory), and a unit only ever waits for units that come earlier in every
// CTA's list, so the waits always end.
// =====================================================================================================
struct MoeFusedArgs {
  const uint8_t* sfa[2];     // per GEMM: weight scale blocks, the input rows' scale bytes (hi, lo), bias
  const uint8_t* sf_hi[2];
  const uint8_t* sf_lo[2];
  const float* bias[2];
  int N[2], nkb[2], tiles[2];
  int ksplit2;               // parts of the second GEMM's k range per weight tile (1 or 2)
  const MoeMeta* meta;
  int* item_done;            // MoeMeta::item_done (zeroed by the routing kernel)
  __nv_bfloat16* out;        // second GEMM: rows [rows][N[1]]; the second half-k partial out_half_stride elements further
  int64_t out_half_stride;
  uint8_t* q2_hi;            // first GEMM's epilogue output = second GEMM's input
  uint8_t* q2_lo;
  uint8_t* sf2_hi;
  uint8_t* sf2_lo;
  int K2, sf2_stride;
  int stages, tok;
  float alpha, limit;
  int* status;
};

__device__ __forceinline__ FppUnit fused_unit(const MoeFusedArgs& a, int i) {
  FppUnit u;
  const int w = static_cast<int>(blockIdx.x) + i * static_cast<int>(gridDim.x);
  const int n_items = a.meta->n_items;
  const int n1 = n_items * a.tiles[0];
  u.valid = w < n1 + n_items * a.tiles[1] * a.ksplit2;
  u.side = 0;
  u.item = 0;
  if (!u.valid) {
    u.e = u.row0 = u.n_e = u.tile = u.kh = u.kb0 = u.kb1 = 0;
    return u;
  }
  if (w < n1) {
    u.item = w / a.tiles[0];
    u.tile = w - u.item * a.tiles[0];
    u.kh = 0;
    u.kb0 = 0;
    u.kb1 = a.nkb[0];
  } else {
    u.side = 1;
    const int w2 = w - n1, per_item = a.tiles[1] * a.ksplit2;
    u.item = w2 / per_item;
    const int rem = w2 - u.item * per_item;
    u.tile = rem / a.ksplit2;
    u.kh = rem - u.tile * a.ksplit2;
    u.kb0 = u.kh * a.nkb[1] / a.ksplit2;
    u.kb1 = (u.kh + 1) * a.nkb[1] / a.ksplit2;
  }
  u.e = a.meta->item_expert[u.item];
  const int part = a.meta->item_part[u.item];
  u.n_e = min(a.meta->counts[u.e] - a.tok * part, a.tok);
  u.row0 = a.meta->offsets[u.e] + a.tok * part;
  return u;
}

template <int BN>
__global__ void __launch_bounds__(FP4_THREADS, 4)
moe_expert_fp4_fused_kernel(const __grid_constant__ CUtensorMap tm_w1, const __grid_constant__ CUtensorMap tm_hi1,
                            const __grid_constant__ CUtensorMap tm_lo1, const __grid_constant__ CUtensorMap tm_w2,
                            const __grid_constant__ CUtensorMap tm_hi2, const __grid_constant__ CUtensorMap tm_lo2,
                            const MoeFusedArgs a) {
  overlap_start();
  overlap_wait();
  const int n_units = a.meta->n_items * (a.tiles[0] + a.tiles[1] * a.ksplit2);
  if (static_cast<int>(blockIdx.x) >= n_units) return;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int S = a.stages;
  uint8_t* atile = smem_raw;                                              // S x 16 KiB
  uint8_t* btile = atile + static_cast<size_t>(S) * FP4_A_BYTES;          // S x (32 hi rows, 32 lo rows) x 128
  uint8_t* sfa_s = btile + static_cast<size_t>(S) * (2 * BN * 128);   // S x 512
  uint8_t* sfb_s = sfa_s + static_cast<size_t>(S) * 512;                  // S x 512
  uint8_t* dump_s = sfb_s + static_cast<size_t>(S) * 512;                 // 4 KiB
  MoeFppBarriers& bar = *reinterpret_cast<MoeFppBarriers*>(dump_s + FPP_DUMP_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &bar.abort_flag;
  if ((smem_u32(smem_raw) & 1023u) != 0) {   // the swizzled tiles need this alignment
    if (tid == 0) atomicOr(a.status, B2_DEV_BAD_INDEX);
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&bar.full[s], 2);
      mbar_init(&bar.empty[s], 1);
    }
    mbar_init(&bar.acc_full, 1);
    mbar_init(&bar.acc_empty, 4);
    bar.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w1);
    tma_prefetch_desc(&tm_hi1);
    tma_prefetch_desc(&tm_lo1);
    tma_prefetch_desc(&tm_w2);
    tma_prefetch_desc(&tm_hi2);
    tma_prefetch_desc(&tm_lo2);
  }
  // rows 64..127 of a token scale block are never written again: a harmless scale of 1
  for (int i = tid; i < S * 128; i += FP4_THREADS) reinterpret_cast<uint32_t*>(sfb_s)[i] = 0x7f7f7f7fu;
  fence_proxy_async_smem();
  constexpr int TMEM_COLS = BN == 32 ? 128 : (BN == 16 ? 64 : 32);   // accumulator 2 * BN, weight scales 4, token scales 4
  if (warp == 1) tmem_alloc(&bar.tmem_base, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bar.tmem_base;

  if (warp == 0) {
    // ===================================== producer + token scale blocks =====================================
    const bool leader = elect_one();
    bool ok = true;
    // A unit of the second GEMM reads what the first GEMM's epilogues wrote for its (expert, part): every weight tile of
    // the first GEMM counts itself in item_done when its rows are stored.  The cursor that runs ahead for the scale
    // words only LOOKS at the count when it enters such a unit (the usual case: complete long ago) and remembers the
    // answer; the blocking wait (bounded), if it is needed at all, is taken when the loading cursor itself reaches the
    // unit - by then every load of this CTA's own earlier units, on whose epilogues the count may depend, has been
    // issued, so the wait cannot keep this CTA's own contribution from happening.
    auto wait_item = [&](const FppUnit& u, bool block) -> bool {
      if (!u.valid || u.side == 0) return true;
      int seen = 0;
      if (lane == 0) {
        const int* cnt = a.item_done + u.item;
        uint64_t t0 = 0;
        for (uint32_t spin = 0; spin < SPIN_LIMIT; ++spin) {
          int v;
          asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(cnt) : "memory");
          if (v >= a.tiles[0]) {
            seen = 1;
            break;
          }
          if (!block) break;
          if ((spin & 63u) == 63u) {
            if (*abort_flag) break;
            const uint64_t now = wait_clock_ns();
            if (t0 == 0)
              t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS)
              break;
          }
        }
      }
      seen = __shfl_sync(0xffffffffu, seen, 0);
      if (!seen && block) ok = false;
      asm volatile("fence.proxy.async;" ::: "memory");   // the TMA loads that follow read other CTAs' generic stores
      return seen != 0;
    };
    struct Cur {
      int i, kb;
      FppUnit u;
    };
    uint32_t ready_mask = 0;   // bit (unit iteration & 31): the look-ahead cursor found the unit's input complete
    auto enter_ahead = [&](const Cur& c) {
      const uint32_t bit = 1u << (c.i & 31);
      ready_mask = wait_item(c.u, false) ? (ready_mask | bit) : (ready_mask & ~bit);
    };
    auto next = [&](Cur& c, bool ahead) {
      if (++c.kb >= c.u.kb1) {
        ++c.i;
        c.u = fused_unit(a, c.i);
        c.kb = c.u.kb0;
        if (ahead) enter_ahead(c);
      }
    };
    // row n2 of the [hi rows; lo rows] token tile: the four scale bytes of one k-block are one word
    auto load_tsf = [&](const Cur& c, int n2) -> uint32_t {
      const int term = n2 >= BN, n = n2 - term * BN;
      const uint8_t* sf = term ? a.sf_lo[c.u.side] : a.sf_hi[c.u.side];
      const int sf_stride = 4 * a.nkb[c.u.side];
      // not through the read-only path: the second GEMM's scale bytes were written during this launch
      return (c.u.valid && ((ready_mask >> (c.i & 31)) & 1u) && n2 < 2 * BN && n < c.u.n_e)
                 ? __ldcg(reinterpret_cast<const uint32_t*>(sf + static_cast<size_t>(c.u.row0 + n) * sf_stride) + c.kb)
                 : 0x7f7f7f7fu;
    };
    Cur cur{0, 0, fused_unit(a, 0)};
    cur.kb = cur.u.kb0;
    Cur pre = cur;
    uint32_t nx[FPP_AHEAD][2];
    auto prime = [&]() {   // the look-ahead cursor restarts at the loading cursor
      pre = cur;
      enter_ahead(pre);
#pragma unroll
      for (int d = 0; d < FPP_AHEAD; ++d) {
        nx[d][0] = load_tsf(pre, lane);
        nx[d][1] = load_tsf(pre, lane + 32);
        next(pre, true);
      }
    };
    if (!wait_item(cur.u, true)) ok = false;   // a CTA whose first unit already belongs to the second GEMM
    prime();
    const int off = lane * 16;   // row r of the block: (r % 32) * 16 + (r / 32) * 4
    for (int g = 0; cur.u.valid && ok; ++g) {
      const int s = g % S, round = g / S;
      const uint32_t w0 = nx[0][0], w1 = nx[0][1];
#pragma unroll
      for (int d = 0; d + 1 < FPP_AHEAD; ++d) {
        nx[d][0] = nx[d + 1][0];
        nx[d][1] = nx[d + 1][1];
      }
      nx[FPP_AHEAD - 1][0] = load_tsf(pre, lane);
      nx[FPP_AHEAD - 1][1] = load_tsf(pre, lane + 32);
      next(pre, true);
      if (round > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.empty[s], (round - 1) & 1, abort_flag));
      if (!ok) break;
      if (leader) {
        mbar_arrive_expect_tx(&bar.full[s], static_cast<uint32_t>(FP4_A_TX + 512 + 2 * BN * 128));
        const int sd = cur.u.side;
        tma_load_4d(atile + static_cast<size_t>(s) * FP4_A_BYTES, sd ? &tm_w2 : &tm_w1, &bar.full[s], cur.kb * FP4_KB,
                    cur.u.tile * MOE_FT, cur.u.e, 0);
        bulk_load(sfa_s + s * 512,
                  a.sfa[sd] + ((static_cast<size_t>(cur.u.e) * a.tiles[sd] + cur.u.tile) * a.nkb[sd] + cur.kb) * 512, 512,
                  &bar.full[s]);
        uint8_t* bt = btile + static_cast<size_t>(s) * (2 * BN * 128);
        tma_load_2d(bt, sd ? &tm_hi2 : &tm_hi1, &bar.full[s], cur.kb * FP4_KB, cur.u.row0);
        tma_load_2d(bt + BN * 128, sd ? &tm_lo2 : &tm_lo1, &bar.full[s], cur.kb * FP4_KB, cur.u.row0);   // lo rows follow hi rows
      }
      uint8_t* blk = sfb_s + s * 512;
      if (lane < 2 * BN) *reinterpret_cast<uint32_t*>(blk + off) = w0;
      if (BN == 32) *reinterpret_cast<uint32_t*>(blk + off + 4) = w1;
      fence_proxy_async_smem();   // tcgen05.cp reads the block through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.full[s]);
      {
        const int before = cur.i;
        next(cur, false);
        // entering a unit whose input the look-ahead cursor did not find complete: wait for it now, then fetch its
        // scale words again (those fetched ahead were placeholders)
        if (cur.i != before && cur.u.valid && cur.u.side == 1 && !((ready_mask >> (cur.i & 31)) & 1u)) {
          if (!wait_item(cur.u, true)) break;
          prime();
        }
      }
    }
    if (leader && !ok) {
      if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
      *abort_flag = 1;
    }
  } else if (warp == 1) {
    // ===================================== MMA issuer =====================================
    const bool leader = elect_one();
    const uint32_t t_sfa = tmem + 2 * BN, t_sfb = t_sfa + 4;
    bool ok = true;
    int g = 0;
    for (int i = 0; ok; ++i) {
      const FppUnit u = fused_unit(a, i);
      if (!u.valid) break;
      for (int kb = u.kb0; kb < u.kb1 && ok; ++kb, ++g) {
        const int s = g % S;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.full[s], (g / S) & 1, abort_flag));
        // the previous unit's sums must have left the accumulator
        if (ok && kb == u.kb0 && i > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_empty, (i - 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after_sync();
        const uint64_t da = umma_desc_k128(smem_u32(atile + static_cast<size_t>(s) * FP4_A_BYTES));
        const uint64_t db = umma_desc_k128(smem_u32(btile + static_cast<size_t>(s) * (2 * BN * 128)));
        if (leader) {
          tmem_cp_sf_block(t_sfa, umma_desc_sf_block(smem_u32(sfa_s + s * 512)));
          tmem_cp_sf_block(t_sfb, umma_desc_sf_block(smem_u32(sfb_s + s * 512)));
#pragma unroll
          for (int k = 0; k < FP4_KB / 32; ++k)
            umma_fp4_fp8(tmem, da + 2 * k, db + 2 * k, umma_idesc_fp4_fp8(MOE_FT, 2 * BN, k, k), t_sfa, t_sfb,
                         ((kb - u.kb0) | k) != 0);
          umma_commit(&bar.empty[s]);
          if (kb == u.kb1 - 1) umma_commit(&bar.acc_full);
        }
        __syncwarp();
      }
    }
    if (leader && !ok) {
      if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
      *abort_flag = 1;
    }
  } else {
    // ===================================== epilogue =====================================
    const int t4 = (warp - 2) * 32 + lane;   // 0..127
    const int lane_grp = warp & 3;
    const int fr = lane_grp * 32 + lane;     // feature row of this thread inside the tile
    const uint32_t trow = tmem + (static_cast<uint32_t>(lane_grp * 32) << 16);
    __nv_bfloat16* dump = reinterpret_cast<__nv_bfloat16*>(dump_s);
    bool ok = true;
    for (int i = 0; ok; ++i) {
      const FppUnit u = fused_unit(a, i);
      if (!u.valid) break;
      const int f = u.tile * MOE_FT + fr;
      const int n_side = a.N[u.side];
      const float bias = (f < n_side && u.kh == 0) ? __ldg(a.bias[u.side] + static_cast<size_t>(u.e) * n_side + f) : 0.f;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_full, i & 1, abort_flag));
      if (!ok) {
        if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      float v[32];   // tokens 0 .. BN-1 are meaningful
      if constexpr (BN == 32) {   // columns 0..31 hold the hi term's sums, columns 32..63 the lo term's
        float w[32];
        tmem_ld_32x32_nowait(trow, v);
        tmem_ld_32x32_nowait(trow + BN, w);
        tmem_wait_ld();
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] += w[t];
      } else {                    // one load covers the allocation: hi sums in columns 0..BN-1, lo sums in BN..2BN-1
        float w[32];
        tmem_ld_32x32(trow, w);
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = t < BN ? w[t] + w[(t + BN) & 31] : 0.f;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.acc_empty);   // the MMA warp may start the next unit

      if (u.side == 0) {
        constexpr int OUT_F = MOE_FT / 2;
        constexpr int PIECES = OUT_F / 8;
        const int out_n = n_side / 2;
#pragma unroll
        for (int t = 0; t < BN; ++t) {
          const float xv = v[t] + bias;
          const float other = __shfl_xor_sync(0xffffffffu, xv, 1);
          if ((lane & 1) == 0) dump[t * OUT_F + (fr >> 1)] = __float2bfloat16_rn(moe_swiglu(xv, other, a.alpha, a.limit));
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // straight into the form the second GEMM reads: two block-scaled E4M3 terms per row, one scale byte per 32
        // features (a tile's 64 features are two whole groups); a thread owns 8 features, a quad a group
        const int total = u.n_e * PIECES;
        for (int base = 0; base < total; base += 128) {   // uniform trip count: the shuffles need whole warps
          const int it = base + t4;
          const bool live = it < total;
          const int tok = live ? it / PIECES : 0, pc = it - (it / PIECES) * PIECES;
          float q[8];
          if (live) {
            const uint4 p = *reinterpret_cast<const uint4*>(dump + tok * OUT_F + pc * 8);
            q[0] = bf16lo(p.x); q[1] = bf16hi(p.x); q[2] = bf16lo(p.y); q[3] = bf16hi(p.y);
            q[4] = bf16lo(p.z); q[5] = bf16hi(p.z); q[6] = bf16lo(p.w); q[7] = bf16hi(p.w);
          } else {
#pragma unroll
            for (int t = 0; t < 8; ++t) q[t] = 0.f;
          }
          uint32_t qb[2][2];
          uint32_t sbyte[2];
          moe_quant8(q, qb, sbyte);
          const int col = u.tile * OUT_F + pc * 8;
          if (live && col + 8 <= out_n) {
            const size_t row = static_cast<size_t>(u.row0 + tok);
            *reinterpret_cast<uint2*>(a.q2_hi + row * a.K2 + col) = make_uint2(qb[0][0], qb[0][1]);
            *reinterpret_cast<uint2*>(a.q2_lo + row * a.K2 + col) = make_uint2(qb[1][0], qb[1][1]);
            if ((pc & 3) == 0) {
              const int gq = col >> 5;
              a.sf2_hi[row * a.sf2_stride + gq] = static_cast<uint8_t>(sbyte[0]);
              a.sf2_lo[row * a.sf2_stride + gq] = static_cast<uint8_t>(sbyte[1]);
              if (gq == a.K2 / 32 - 1)   // groups past K2 (the weights are zero there) get a harmless scale of 1
                for (int gg = gq + 1; gg < a.sf2_stride; ++gg) {
                  a.sf2_hi[row * a.sf2_stride + gg] = 127;
                  a.sf2_lo[row * a.sf2_stride + gg] = 127;
                }
            }
          }
        }
        __threadfence();   // this thread's rows of the second GEMM's input are visible before the item counts this tile
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the dump is free for the next unit
        if (t4 == 0) {
          asm volatile("fence.proxy.async;" ::: "memory");
          asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(a.item_done + u.item) : "memory");
        }
      } else {
        constexpr int OUT_F = MOE_FT;
        constexpr int PIECES = OUT_F / 8;
        const int out_n = n_side;
        // 128 features x 16 tokens fill the 4 KiB: two passes for 32 tokens
        constexpr int PASS = BN < 16 ? BN : 16;
#pragma unroll
        for (int half = 0; half < BN / PASS; ++half) {
#pragma unroll
          for (int t = 0; t < PASS; ++t) {
            const int tok = PASS * half + t;
            const float gw = tok < u.n_e ? a.meta->gate_of_row[u.row0 + tok] : 0.f;
            dump[t * OUT_F + fr] = __float2bfloat16_rn((v[tok] + bias) * gw);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const int n_here = min(u.n_e - PASS * half, PASS);
          for (int it = t4; it < n_here * PIECES; it += 128) {
            const int tok = it / PIECES, pc = it - tok * PIECES;
            const int col = u.tile * OUT_F + pc * 8;
            if (col + 8 <= out_n)
              *reinterpret_cast<uint4*>(a.out + u.kh * a.out_half_stride + static_cast<size_t>(u.row0 + PASS * half + tok) * out_n + col) =
                  *reinterpret_cast<const uint4*>(dump + tok * OUT_F + pc * 8);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace b2

namespace {
size_t moe_align(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
}  // namespace

B2_API size_t b2_moe_decode_workspace_bytes(int64_t tokens, int hidden, int intermediate) {
  if (tokens <= 0 || hidden <= 0 || intermediate <= 0) return 0;
  const size_t rows = static_cast<size_t>(tokens) * b2::MOE_TOPK;
  return moe_align(sizeof(b2::MoeMeta)) + moe_align(rows * hidden * 2) + moe_align(rows * intermediate * 2) +
         moe_align(rows * hidden * 2);
}

B2_API int b2_moe_experts_decode(const void* x, int64_t ldx, const int16_t* topk_idx, const float* topk_w,
                                 const void* w1_codes, const void* w1_scales, const float* b1, const void* w2_codes,
                                 const void* w2_scales, const float* b2_, void* out, int64_t ld_out, void* workspace,
                                 size_t workspace_bytes, int64_t tokens, int n_experts, int hidden, int intermediate,
                                 float alpha, float limit, void* stream) {
  using namespace b2;
  if (tokens < 0 || n_experts <= 0 || hidden <= 0 || intermediate <= 0 || ldx < hidden || ld_out < hidden)
    return B2_ERR_SHAPE;
  if (tokens > MOE_CONV_MAX_TOKENS || n_experts > MOE_MAX_EXPERTS || hidden % 64 || intermediate % 64)
    return B2_ERR_UNSUPPORTED;
  if (tokens == 0) return B2_OK;
  if (!x || !topk_idx || !topk_w || !w1_codes || !w1_scales || !b1 || !w2_codes || !w2_scales || !b2_ || !out ||
      !workspace)
    return B2_ERR_NULL;
  if (!aligned16(x) || !aligned16(out) || !aligned16(w1_codes) || !aligned16(w2_codes) || ldx % 8 || ld_out % 8 ||
      (reinterpret_cast<uintptr_t>(workspace) & 255))
    return B2_ERR_ALIGN;
  if (workspace_bytes < b2_moe_decode_workspace_bytes(tokens, hidden, intermediate)) return B2_ERR_WORKSPACE;
  int* status = device_status_ptr();
  if (!status) return B2_ERR_DRIVER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int T = static_cast<int>(tokens), rows = T * MOE_TOPK;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  MoeMeta* meta = reinterpret_cast<MoeMeta*>(ws);
  ws += moe_align(sizeof(MoeMeta));
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += moe_align(static_cast<size_t>(rows) * hidden * 2);
  __nv_bfloat16* act = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += moe_align(static_cast<size_t>(rows) * intermediate * 2);
  __nv_bfloat16* ybuf = reinterpret_cast<__nv_bfloat16*>(ws);

  moe_route_kernel<<<1, 1024, 0, st>>>(topk_idx, topk_w, T, n_experts, meta, status, 0);
  moe_gather_kernel<<<rows, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), ldx, xs, hidden, rows, meta);

  const int bn_max = ((T < MOE_CONV_MAX_TOKENS ? T : MOE_CONV_MAX_TOKENS) + 31) & ~31;
  const int b_stages = bn_max <= 128 ? 4 : 3;
  const size_t smem = static_cast<size_t>(MOE_RAW_STAGES) * MOE_RAW_BYTES + static_cast<size_t>(MOE_A_STAGES) * MOE_A_BYTES +
                      static_cast<size_t>(b_stages) * bn_max * 128 + sizeof(MoeBarriers) +
                      static_cast<size_t>(MOE_FT) * ((hidden > intermediate ? hidden : intermediate) / 32) + 1024;

  // stage 1: a = swiglu(xs W1 + b1), N = 2 * intermediate interleaved features, K = hidden
  // stage 2: y = (a W2 + b2) * gate,  N = hidden, K = intermediate
  for (int stage = 0; stage < 2; ++stage) {
    const int N = stage == 0 ? 2 * intermediate : hidden;
    const int K = stage == 0 ? hidden : intermediate;
    const void* codes = stage == 0 ? w1_codes : w2_codes;
    CUtensorMap tm_w, tm_x;
    const uint64_t wd[4] = {static_cast<uint64_t>(K / 4), static_cast<uint64_t>(N), static_cast<uint64_t>(n_experts), 1};
    const uint64_t wstr[3] = {static_cast<uint64_t>(K / 2), static_cast<uint64_t>(N) * (K / 2),
                              static_cast<uint64_t>(n_experts) * N * (K / 2)};
    const uint32_t wbox[4] = {MOE_KB / 4, MOE_FT, 1, 1};
    int rc = make_tensor_map_bf16(&tm_w, codes, 4, wd, wstr, wbox, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != B2_OK) return rc;
    const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(rows)};
    const uint64_t xstr[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t xbox[2] = {MOE_KB, 32};
    rc = make_tensor_map_bf16(&tm_x, stage == 0 ? xs : act, 2, xd, xstr, xbox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B2_OK) return rc;
    MoeExpertArgs a;
    a.scales = static_cast<const uint8_t*>(stage == 0 ? w1_scales : w2_scales);
    a.bias = stage == 0 ? b1 : b2_;
    a.meta = meta;
    a.out = stage == 0 ? act : ybuf;
    a.N = N;
    a.K = K;
    a.nkb = K / MOE_KB;
    a.bn_max = bn_max;
    a.b_stages = b_stages;
    a.alpha = alpha;
    a.limit = limit;
    a.status = status;
        {
      size_t slots = 0;
      long long* tb = trace_buffer(&slots);
      // stage 1 uses the first grid-sized block of slots, stage 2 the block after it
      const size_t n1 = static_cast<size_t>((2 * intermediate + MOE_FT - 1) / MOE_FT) * n_experts;
      const size_t need = n1 + static_cast<size_t>((hidden + MOE_FT - 1) / MOE_FT) * n_experts;
      a.trace = slots >= need ? tb + (stage == 0 ? 0 : 8 * n1) : nullptr;
    }
    const dim3 grid(static_cast<unsigned>((N + MOE_FT - 1) / MOE_FT), static_cast<unsigned>(n_experts));
    cudaError_t e;
    if (stage == 0) {
      e = cudaFuncSetAttribute(moe_expert_kernel<MOE_EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      moe_expert_kernel<MOE_EPI_SWIGLU><<<grid, MOE_THREADS, smem, st>>>(tm_w, tm_x, a);
    } else {
      e = cudaFuncSetAttribute(moe_expert_kernel<MOE_EPI_GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      moe_expert_kernel<MOE_EPI_GATE><<<grid, MOE_THREADS, smem, st>>>(tm_w, tm_x, a);
    }
    rc = launch_status();
    if (rc != B2_OK) return rc;
  }
  moe_combine_kernel<<<T, 128, 0, st>>>(ybuf, static_cast<__nv_bfloat16*>(out), ld_out, hidden, T, meta);
  return launch_status();
}

namespace b2 {

// The same sum, followed by what the model does with it next: h = bf16(residual + delta), y = RMSNorm(h) * gain
// (the add that closes the MoE block and the norm that opens the next block or ends the model), one CTA per token.
constexpr int MOE_CN_VPL = 3;   // 16-byte pieces per thread: rows of up to 128 * 3 * 8 = 3072 elements
__global__ void __launch_bounds__(128)
moe_combine_add_norm_kernel(const __nv_bfloat16* __restrict__ y, const MoeMeta* __restrict__ meta,
                            const __nv_bfloat16* __restrict__ residual, int64_t res_stride, const float4* __restrict__ gain,
                            __nv_bfloat16* __restrict__ h_out, int64_t h_stride, __nv_bfloat16* __restrict__ y_out,
                            int64_t y_stride, int hidden, int tokens, float inv_dim, float eps,
                            const __nv_bfloat16* __restrict__ y2) {
  __shared__ float s_ss[4];
  overlap_start();
  overlap_wait();
  const int t = blockIdx.x, nvec = hidden / 8;
  int rows[MOE_TOPK];
#pragma unroll
  for (int k = 0; k < MOE_TOPK; ++k) rows[k] = meta->row_of_slot[t * MOE_TOPK + k];
  uint4 h[MOE_CN_VPL];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < MOE_CN_VPL; ++j) {
    const int i = threadIdx.x + 128 * j;
    h[j] = make_uint4(0, 0, 0, 0);
    if (i < nvec) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < MOE_TOPK; ++k) {
        if (rows[k] < 0) continue;
        const uint4 p = __ldg(reinterpret_cast<const uint4*>(y + static_cast<size_t>(rows[k]) * hidden) + i);
        acc[0] += bf16lo(p.x); acc[1] += bf16hi(p.x); acc[2] += bf16lo(p.y); acc[3] += bf16hi(p.y);
        acc[4] += bf16lo(p.z); acc[5] += bf16hi(p.z); acc[6] += bf16lo(p.w); acc[7] += bf16hi(p.w);
        if (y2) {
          const uint4 q = __ldg(reinterpret_cast<const uint4*>(y2 + static_cast<size_t>(rows[k]) * hidden) + i);
          acc[0] += bf16lo(q.x); acc[1] += bf16hi(q.x); acc[2] += bf16lo(q.y); acc[3] += bf16hi(q.y);
          acc[4] += bf16lo(q.z); acc[5] += bf16hi(q.z); acc[6] += bf16lo(q.w); acc[7] += bf16hi(q.w);
        }
      }
      // the MoE output is a bf16 tensor; the residual add rounds once more
      const uint4 d = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                                 pack_bf16(acc[6], acc[7]));
      const uint4 r = *(reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * res_stride) + i);
      h[j].x = pack_bf16(bf16lo(r.x) + bf16lo(d.x), bf16hi(r.x) + bf16hi(d.x));
      h[j].y = pack_bf16(bf16lo(r.y) + bf16lo(d.y), bf16hi(r.y) + bf16hi(d.y));
      h[j].z = pack_bf16(bf16lo(r.z) + bf16lo(d.z), bf16hi(r.z) + bf16hi(d.z));
      h[j].w = pack_bf16(bf16lo(r.w) + bf16lo(d.w), bf16hi(r.w) + bf16hi(d.w));
      *(reinterpret_cast<uint4*>(h_out + static_cast<size_t>(t) * h_stride) + i) = h[j];
      ss += sq_pair_bf16(h[j].x) + sq_pair_bf16(h[j].y) + sq_pair_bf16(h[j].z) + sq_pair_bf16(h[j].w);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float rstd = rsqrtf((s_ss[0] + s_ss[1] + s_ss[2] + s_ss[3]) * inv_dim + eps);
#pragma unroll
  for (int j = 0; j < MOE_CN_VPL; ++j) {
    const int i = threadIdx.x + 128 * j;
    if (i < nvec) {
      const float4 g0 = __ldg(gain + 2 * i), g1 = __ldg(gain + 2 * i + 1);
      uint4 o;
      o.x = pack_bf16(bf16lo(h[j].x) * rstd * g0.x, bf16hi(h[j].x) * rstd * g0.y);
      o.y = pack_bf16(bf16lo(h[j].y) * rstd * g0.z, bf16hi(h[j].y) * rstd * g0.w);
      o.z = pack_bf16(bf16lo(h[j].z) * rstd * g1.x, bf16hi(h[j].z) * rstd * g1.y);
      o.w = pack_bf16(bf16lo(h[j].w) * rstd * g1.z, bf16hi(h[j].w) * rstd * g1.w);
      *(reinterpret_cast<uint4*>(y_out + static_cast<size_t>(t) * y_stride) + i) = o;
    }
  }
}

}  // namespace b2

// ------------------------------------------------------------------------------- FP4 tensor-core path
namespace {
// Tokens of an expert per unit of the persistent kernel, by the average number of routed rows per expert (4 * tokens /
// experts): up to 4 -> 8, up to 8 -> 16, else 32 (measured, whole op at 32 / 64 / 128 tokens and 32 experts: 8-token
// parts 96 / 123 / 204 us, 16-token parts 100 / 101 / 128 us, 32-token parts 104 / 108 / 112 us).
int moe_part_tokens(int64_t tokens, int n_experts) {
  int part = tokens <= n_experts ? 8 : (tokens <= 2 * n_experts ? 16 : 32);
  // the item list holds at most MOE_MAX_ITEMS (expert, part) pairs: rows / part + experts of them in the worst case
  while (part < 32 && tokens * b2::MOE_TOPK / part + n_experts > b2::MOE_MAX_ITEMS) part *= 2;
  return part;
}
// How b2_moe_experts_decode_fp4 runs under the current tuning knobs; b2_moe_combine_add_rmsnorm must agree with it on
// where the last GEMM's second partial rows are.
struct MoeFp4Plan {
  int tok;      // tokens of an expert per CTA
  int per_sm;   // persistent kernel: CTAs per SM; 0: the one-shot kernel
  int ksplit;   // last GEMM: parts of the k range (2: each weight tile is two units and every row has two partial sums)
};
MoeFp4Plan moe_fp4_plan(int64_t tokens, int intermediate) {
  using namespace b2;
  MoeFp4Plan p{32, 0, 1};
  if (tunable(TUNE_MOE_FP4_TOK) == 32 || tunable(TUNE_MOE_FP4_TOK) == 64) p.tok = tunable(TUNE_MOE_FP4_TOK);
  const int ps = tunable(TUNE_MOE_FP4_PERSIST);
  if (p.tok == FPP_BN && ps != 0) {
    p.per_sm = ps >= 4 ? 4 : (ps >= 2 ? 2 : 1);
    // two halves pay off while the last GEMM's units are fewer than two rounds of CTAs (measured: 32 tokens 114 -> 110 us,
    // 2048 tokens 584 -> 607 us); a half must hold at least two k-blocks
    const int nkb = (intermediate + FP4_KB - 1) / FP4_KB;
    p.ksplit = (tunable(TUNE_MOE_FP4_KSPLIT) == 1 || nkb < 4 || tokens > 512) ? 1 : 2;
  }
  return p;
}
}  // namespace

B2_API size_t b2_moe_fp4_workspace_bytes(int64_t tokens, int hidden, int intermediate) {
  if (tokens <= 0 || hidden <= 0 || intermediate <= 0) return 0;
  const size_t rows = static_cast<size_t>(tokens) * b2::MOE_TOPK;
  const size_t kmax = static_cast<size_t>(hidden > intermediate ? hidden : intermediate);
  const size_t sf_stride = 4 * ((kmax + 127) / 128);
  return b2_moe_decode_workspace_bytes(tokens, hidden, intermediate) + 2 * moe_align(rows * kmax) +
         2 * moe_align(rows * sf_stride);
}

B2_API int b2_moe_experts_decode_fp4(const void* x, int64_t ldx, const int16_t* topk_idx, const float* topk_w,
                                     const void* w1_codes, const void* w1_sf, const float* b1, const void* w2_codes,
                                     const void* w2_sf, const float* b2_, void* out, int64_t ld_out, void* workspace,
                                     size_t workspace_bytes, int64_t tokens, int n_experts, int hidden, int intermediate,
                                     float alpha, float limit, void* stream) {
  using namespace b2;
  if (tokens < 0 || n_experts <= 0 || hidden <= 0 || intermediate <= 0 || ldx < hidden || ld_out < hidden)
    return B2_ERR_SHAPE;
  if (tokens > MOE_MAX_TOKENS || n_experts > MOE_MAX_EXPERTS || hidden % 64 || intermediate % 64)
    return B2_ERR_UNSUPPORTED;
  if (tokens == 0) return B2_OK;
  if (!x || !topk_idx || !topk_w || !w1_codes || !w1_sf || !b1 || !w2_codes || !w2_sf || !b2_ || !workspace)
    return B2_ERR_NULL;   // out may be NULL: the sum over a token's experts is then left to b2_moe_combine_add_rmsnorm
  if (!aligned16(x) || !aligned16(out) || !aligned16(w1_sf) || !aligned16(w2_sf) || ldx % 8 || ld_out % 8 ||
      (reinterpret_cast<uintptr_t>(w1_codes) & 31) || (reinterpret_cast<uintptr_t>(w2_codes) & 31) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255))
    return B2_ERR_ALIGN;
  if (workspace_bytes < b2_moe_fp4_workspace_bytes(tokens, hidden, intermediate)) return B2_ERR_WORKSPACE;
  int* status = device_status_ptr();
  if (!status) return B2_ERR_DRIVER;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int T = static_cast<int>(tokens), rows = T * MOE_TOPK;
  const size_t kmax = static_cast<size_t>(hidden > intermediate ? hidden : intermediate);
  const int sf_stride_max = static_cast<int>(4 * ((kmax + 127) / 128));
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  MoeMeta* meta = reinterpret_cast<MoeMeta*>(ws);
  ws += moe_align(sizeof(MoeMeta));
  // the conversion path's regions for the gathered rows and the bf16 activations hold, here, the second GEMM's input as
  // the SwiGLU epilogue writes it: scale bytes of the two terms, then the two terms' codes
  uint8_t* sf2_hi = ws;
  uint8_t* sf2_lo = ws + moe_align(static_cast<size_t>(rows) * sf_stride_max);
  ws += moe_align(static_cast<size_t>(rows) * hidden * 2);
  uint8_t* q2_hi = ws;
  uint8_t* q2_lo = ws + static_cast<size_t>(rows) * intermediate;
  ws += moe_align(static_cast<size_t>(rows) * intermediate * 2);
  __nv_bfloat16* ybuf = reinterpret_cast<__nv_bfloat16*>(ws);
  ws += moe_align(static_cast<size_t>(rows) * hidden * 2);
  uint8_t* q_hi = ws;
  ws += moe_align(static_cast<size_t>(rows) * kmax);
  uint8_t* q_lo = ws;
  ws += moe_align(static_cast<size_t>(rows) * kmax);
  uint8_t* sf_hi = ws;
  ws += moe_align(static_cast<size_t>(rows) * sf_stride_max);
  uint8_t* sf_lo = ws;

  const int bn_all = ((T < MOE_MAX_TOKENS ? T : MOE_MAX_TOKENS) + 31) & ~31;
  // 32 tokens of an expert per CTA: two stages, four CTAs per SM.  With the item list this beats 64 tokens (three
  // stages, two CTAs per SM) at every size measured (256 tokens: 166 against 183 us; 2048: 769 against 786 us)
  MoeFp4Plan plan = moe_fp4_plan(tokens, intermediate);
  // a handful of tokens per expert: 8- or 16-token parts, 2 CTAs x 5 stages per SM (tunable moe_fp4_tok = 8 / 16 / 32 forces one)
  int part = tunable(TUNE_MOE_FP4_TOK) == 0 ? moe_part_tokens(tokens, n_experts) : tunable(TUNE_MOE_FP4_TOK);
  if (part < 32 && tokens * MOE_TOPK / part + n_experts > MOE_MAX_ITEMS) part = 32;   // a forced size the item list cannot hold
  const bool small_parts = plan.per_sm > 0 && (part == 8 || part == 16);
  if (small_parts) {
    plan.tok = part;
    plan.per_sm = 2;
  }
  const int tok = plan.tok;
  // the first GEMM's input rows are dead when the last GEMM runs: its second partial rows go there
  __nv_bfloat16* ybuf2 = reinterpret_cast<__nv_bfloat16*>(q_hi);
  const int bn_max = bn_all < tok ? bn_all : tok;   // tokens of one expert per CTA; more go to further items of the list
  const int nkb1 = (hidden + FP4_KB - 1) / FP4_KB;
  if (T <= 512) {
    // routing and the first quantise / gather pass in one launch (the last CTA routes, the others place their rows
    // themselves by a scan of the top-k table, which stops paying above a few hundred tokens: 2048 tokens 593 -> 640 us)
    launch_overlapped(moe_route_quant_kernel, dim3(rows + 1), dim3(MOE_RQ_THREADS), 0, st, topk_idx, topk_w, static_cast<int>(T),
                      n_experts, meta, status, tok, static_cast<const __nv_bfloat16*>(x), ldx, hidden, q_hi, q_lo, sf_hi, sf_lo,
                      4 * nkb1);
  } else {
    launch_overlapped(moe_route_kernel, dim3(1), dim3(1024), 0, st, topk_idx, topk_w, static_cast<int>(T), n_experts, meta, status, tok);
    launch_overlapped(moe_quant_kernel, dim3(rows), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(x), ldx, hidden, q_hi, q_lo,
                      sf_hi, sf_lo, 4 * nkb1, static_cast<const MoeMeta*>(meta));
  }
  const int stage_bytes = FP4_A_BYTES + 2 * bn_max * 128 + 512 + 2048;
  // small token tiles: two stages per CTA and four CTAs per SM (start-up and write-out of one CTA hide behind the
  // streaming of the others) beat four stages and two CTAs; larger tiles are limited to two CTAs by tensor memory
  int stages = bn_max <= 32 ? 2 : 3;
  if (tunable(TUNE_MOE_FP4_STAGES) >= 2 && tunable(TUNE_MOE_FP4_STAGES) <= FP4_MAX_STAGES) stages = tunable(TUNE_MOE_FP4_STAGES);
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + sizeof(MoeFp4Barriers) + 1024;

  // Measured, whole op, one fused launch against two launches: 128 tokens 105 / 112 us, 256 tokens 132 / 136 us; with the
  // small parts of small batches the fused kernel loses (4 tokens 65 / 54 us, 32 tokens 124 / 97 us, 64 tokens 118 / 107 us),
  // and so it does with many tokens (512 tokens 214 / 207 us, 1024 tokens 350 / 324 us, 2048 tokens 650 / 603 us): it is
  // the default for 32-token parts up to 384 tokens (tunable moe_fp4_fuse: 1 = never, 2 = always).
  const int fuse = tunable(TUNE_MOE_FP4_FUSE);
  if (plan.per_sm > 0 && fuse != 1 && ((tok == FPP_BN && tokens <= 384) || fuse == 2)) {
    // both GEMMs in one persistent launch (moe_expert_fp4_fused_kernel); its CTAs wait for one another, so the grid is
    // sized to be resident as a whole - if that cannot be established the two-launch path below runs instead
    CUtensorMap tm[2][3];
    MoeFusedArgs fa;
    bool maps_ok = true;
    for (int g = 0; g < 2 && maps_ok; ++g) {
      const int N = g == 0 ? 2 * intermediate : hidden;
      const int K = g == 0 ? hidden : intermediate;
      const int Kp = (K + FP4_KB - 1) / FP4_KB * FP4_KB;
      const uint64_t wd[4] = {static_cast<uint64_t>(Kp), static_cast<uint64_t>(N), static_cast<uint64_t>(n_experts), 1};
      const uint64_t wstr[3] = {static_cast<uint64_t>(Kp / 2), static_cast<uint64_t>(N) * (Kp / 2),
                                static_cast<uint64_t>(n_experts) * N * (Kp / 2)};
      const uint32_t wbox[4] = {FP4_KB, MOE_FT, 1, 1};
      const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(rows)};
      const uint64_t xstr[1] = {static_cast<uint64_t>(K)};
      const uint32_t xbox[2] = {FP4_KB, static_cast<uint32_t>(tok)};
      maps_ok = make_tensor_map(&tm[g][0], CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, g == 0 ? w1_codes : w2_codes, 4, wd, wstr, wbox,
                                CU_TENSOR_MAP_SWIZZLE_128B) == B2_OK &&
                make_tensor_map(&tm[g][1], CU_TENSOR_MAP_DATA_TYPE_UINT8, g == 0 ? q_hi : q2_hi, 2, xd, xstr, xbox,
                                CU_TENSOR_MAP_SWIZZLE_128B) == B2_OK &&
                make_tensor_map(&tm[g][2], CU_TENSOR_MAP_DATA_TYPE_UINT8, g == 0 ? q_lo : q2_lo, 2, xd, xstr, xbox,
                                CU_TENSOR_MAP_SWIZZLE_128B) == B2_OK;
      fa.sfa[g] = static_cast<const uint8_t*>(g == 0 ? w1_sf : w2_sf);
      fa.sf_hi[g] = g == 0 ? sf_hi : sf2_hi;
      fa.sf_lo[g] = g == 0 ? sf_lo : sf2_lo;
      fa.bias[g] = g == 0 ? b1 : b2_;
      fa.N[g] = N;
      fa.nkb[g] = Kp / FP4_KB;
      fa.tiles[g] = (N + MOE_FT - 1) / MOE_FT;
    }
    fa.ksplit2 = plan.ksplit;
    fa.meta = meta;
    fa.item_done = meta->item_done;
    fa.out = ybuf;
    fa.out_half_stride = ybuf2 - ybuf;
    fa.q2_hi = q2_hi;
    fa.q2_lo = q2_lo;
    fa.sf2_hi = sf2_hi;
    fa.sf2_lo = sf2_lo;
    fa.K2 = intermediate;
    fa.sf2_stride = 4 * ((intermediate + FP4_KB - 1) / FP4_KB);
    fa.tok = tok;
    fa.alpha = alpha;
    fa.limit = limit;
    fa.status = status;
    int per_sm = plan.per_sm;
    fa.stages = small_parts ? 5 : FP4_MAX_STAGES / per_sm;
    const size_t psmem = static_cast<size_t>(fa.stages) * fpp_stage_bytes(tok) + FPP_DUMP_BYTES + sizeof(MoeFppBarriers);
    auto kern = tok == 8 ? moe_expert_fp4_fused_kernel<8> : (tok == 16 ? moe_expert_fp4_fused_kernel<16> : moe_expert_fp4_fused_kernel<FPP_BN>);
    int dev = 0, sms = 0, smem_sm = 0, regs_sm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev);
    cudaFuncAttributes attr;
    bool fused_ok = maps_ok &&
                    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(psmem)) == cudaSuccess &&
                    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) == cudaSuccess &&
                    cudaFuncGetAttributes(&attr, kern) == cudaSuccess;
    if (fused_ok) {
      const int regs_cta = ((attr.numRegs * 32 + 255) / 256 * 256) * (FP4_THREADS / 32);   // allocated per warp in units of 256
      const int by_smem = static_cast<int>(smem_sm / (psmem + attr.sharedSizeBytes + 1024));   // 1 KiB per CTA is the system's
      const int by_regs = regs_cta > 0 ? regs_sm / regs_cta : 0;
      const int by_tmem = 512 / (tok == 32 ? 128 : (tok == 16 ? 64 : 32));
      per_sm = std::min(per_sm, std::min(by_smem, std::min(by_regs, by_tmem)));
      fused_ok = per_sm >= 1;
    } else {
      (void)cudaGetLastError();
    }
    if (fused_ok) {
      const long long max_units = static_cast<long long>(fa.tiles[0] + fa.tiles[1] * fa.ksplit2) * (rows / tok + n_experts);
      const unsigned pgrid = static_cast<unsigned>(std::min<long long>(static_cast<long long>(per_sm) * sms, max_units));
      launch_overlapped(kern, dim3(pgrid), dim3(FP4_THREADS), psmem, st, tm[0][0], tm[0][1], tm[0][2], tm[1][0], tm[1][1], tm[1][2], fa);
      const int rc = launch_status();
      if (rc != B2_OK) return rc;
      if (out)
        launch_overlapped(moe_combine_kernel, dim3(T), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(ybuf), static_cast<__nv_bfloat16*>(out),
                          ld_out, hidden, static_cast<int>(T), static_cast<const MoeMeta*>(meta),
                          static_cast<const __nv_bfloat16*>(plan.ksplit == 2 ? ybuf2 : nullptr));
      return launch_status();
    }
  }

  for (int stage = 0; stage < 2; ++stage) {
    const int N = stage == 0 ? 2 * intermediate : hidden;
    const int K = stage == 0 ? hidden : intermediate;
    const int Kp = (K + FP4_KB - 1) / FP4_KB * FP4_KB;
    const int nkb = Kp / FP4_KB;
    // (the first GEMM's rows were quantised and gathered by the routing launch, the second GEMM's by the first GEMM's epilogue)
    const uint8_t* in_hi = stage == 0 ? q_hi : q2_hi;
    const uint8_t* in_lo = stage == 0 ? q_lo : q2_lo;
    CUtensorMap tm_w, tm_hi, tm_lo;
    const uint64_t wd[4] = {static_cast<uint64_t>(Kp), static_cast<uint64_t>(N), static_cast<uint64_t>(n_experts), 1};
    const uint64_t wstr[3] = {static_cast<uint64_t>(Kp / 2), static_cast<uint64_t>(N) * (Kp / 2),
                              static_cast<uint64_t>(n_experts) * N * (Kp / 2)};
    const uint32_t wbox[4] = {FP4_KB, MOE_FT, 1, 1};
    int rc = make_tensor_map(&tm_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, stage == 0 ? w1_codes : w2_codes, 4, wd, wstr, wbox,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B2_OK) return rc;
    const uint64_t xd[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(rows)};
    const uint64_t xstr[1] = {static_cast<uint64_t>(K)};
    const uint32_t xbox[2] = {FP4_KB, small_parts ? static_cast<uint32_t>(tok) : 32u};
    rc = make_tensor_map(&tm_hi, CU_TENSOR_MAP_DATA_TYPE_UINT8, in_hi, 2, xd, xstr, xbox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B2_OK) return rc;
    rc = make_tensor_map(&tm_lo, CU_TENSOR_MAP_DATA_TYPE_UINT8, in_lo, 2, xd, xstr, xbox, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B2_OK) return rc;
    MoeFp4Args a;
    a.sfa = static_cast<const uint8_t*>(stage == 0 ? w1_sf : w2_sf);
    a.sf_hi = stage == 0 ? sf_hi : sf2_hi;
    a.sf_lo = stage == 0 ? sf_lo : sf2_lo;
    a.bias = stage == 0 ? b1 : b2_;
    a.meta = meta;
    a.out = stage == 0 ? nullptr : ybuf;
    a.q2_hi = q2_hi;
    a.q2_lo = q2_lo;
    a.sf2_hi = sf2_hi;
    a.sf2_lo = sf2_lo;
    a.K2 = intermediate;
    a.sf2_stride = 4 * ((intermediate + FP4_KB - 1) / FP4_KB);
    a.N = N;
    a.nkb = nkb;
    a.tiles = (N + MOE_FT - 1) / MOE_FT;
    a.bn_max = bn_max;
    a.stages = stages;
    a.sf_col = 2 * bn_max;
    a.tok = tok;
    a.ksplit = stage == 1 ? plan.ksplit : 1;
    a.out_half_stride = ybuf2 - ybuf;
    a.prefetch = tunable(TUNE_MOE_PREFETCH) < 0 ? 0 : (tunable(TUNE_MOE_PREFETCH) > 32 ? 32 : tunable(TUNE_MOE_PREFETCH));
    a.alpha = alpha;
    a.limit = limit;
    a.status = status;
    const dim3 grid(static_cast<unsigned>(a.tiles), static_cast<unsigned>(rows / tok + n_experts));
    cudaError_t e;
    if (plan.per_sm > 0) {
      // persistent CTAs over the (expert part, weight tile) list: `per_sm` CTAs per SM share the 8 stages an SM has room for
      const int per_sm = plan.per_sm;
      a.stages = small_parts ? 5 : FP4_MAX_STAGES / per_sm;
      if (tunable(TUNE_MOE_FP4_STAGES) >= 2 && tunable(TUNE_MOE_FP4_STAGES) <= a.stages) a.stages = tunable(TUNE_MOE_FP4_STAGES);
      const size_t psmem = static_cast<size_t>(a.stages) * fpp_stage_bytes(tok) + FPP_DUMP_BYTES + sizeof(MoeFppBarriers);
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      const long long max_units = static_cast<long long>(a.tiles) * a.ksplit * (rows / tok + n_experts);
      const unsigned pgrid = static_cast<unsigned>(std::min<long long>(static_cast<long long>(per_sm) * sms, max_units));
      auto kern = stage == 0 ? (tok == 8    ? moe_expert_fp4_persist_kernel<MOE_EPI_SWIGLU, 8>
                                : tok == 16 ? moe_expert_fp4_persist_kernel<MOE_EPI_SWIGLU, 16>
                                            : moe_expert_fp4_persist_kernel<MOE_EPI_SWIGLU, FPP_BN>)
                             : (tok == 8    ? moe_expert_fp4_persist_kernel<MOE_EPI_GATE, 8>
                                : tok == 16 ? moe_expert_fp4_persist_kernel<MOE_EPI_GATE, 16>
                                            : moe_expert_fp4_persist_kernel<MOE_EPI_GATE, FPP_BN>);
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(psmem));
      if (e != cudaSuccess) return static_cast<int>(e);
      launch_overlapped(kern, dim3(pgrid), dim3(FP4_THREADS), psmem, st, tm_w, tm_hi, tm_lo, a);
    } else if (stage == 0) {
      e = cudaFuncSetAttribute(moe_expert_fp4_kernel<MOE_EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      launch_overlapped(moe_expert_fp4_kernel<MOE_EPI_SWIGLU>, grid, dim3(FP4_THREADS), smem, st, tm_w, tm_hi, tm_lo, a);
    } else {
      e = cudaFuncSetAttribute(moe_expert_fp4_kernel<MOE_EPI_GATE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
      launch_overlapped(moe_expert_fp4_kernel<MOE_EPI_GATE>, grid, dim3(FP4_THREADS), smem, st, tm_w, tm_hi, tm_lo, a);
    }
    rc = launch_status();
    if (rc != B2_OK) return rc;
  }
  if (out)
    launch_overlapped(moe_combine_kernel, dim3(T), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(ybuf), static_cast<__nv_bfloat16*>(out),
                      ld_out, hidden, static_cast<int>(T), static_cast<const MoeMeta*>(meta),
                      static_cast<const __nv_bfloat16*>(plan.ksplit == 2 ? ybuf2 : nullptr));
  return launch_status();
}

B2_API int b2_moe_combine_add_rmsnorm(const void* workspace, size_t workspace_bytes, int64_t tokens, int hidden,
                                      int intermediate, const void* residual, int64_t residual_stride, const float* gain,
                                      float eps, void* h_out, int64_t h_stride, void* y_out, int64_t y_stride, void* stream) {
  using namespace b2;
  if (tokens < 0 || hidden <= 0 || intermediate <= 0 || residual_stride < hidden || h_stride < hidden || y_stride < hidden)
    return B2_ERR_SHAPE;
  if (tokens > MOE_MAX_TOKENS || hidden % 64 || intermediate % 64 || hidden > 128 * MOE_CN_VPL * 8) return B2_ERR_UNSUPPORTED;
  if (tokens == 0) return B2_OK;
  if (!workspace || !residual || !gain || !h_out || !y_out) return B2_ERR_NULL;
  if (!aligned16(residual) || !aligned16(gain) || !aligned16(h_out) || !aligned16(y_out) || residual_stride % 8 ||
      h_stride % 8 || y_stride % 8 || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return B2_ERR_ALIGN;
  if (workspace_bytes < b2_moe_fp4_workspace_bytes(tokens, hidden, intermediate)) return B2_ERR_WORKSPACE;
  // the workspace as b2_moe_experts_decode_fp4 laid it out: routing metadata, gathered rows, activations, expert outputs
  const size_t rows = static_cast<size_t>(tokens) * MOE_TOPK;
  const uint8_t* ws = static_cast<const uint8_t*>(workspace);
  const MoeMeta* meta = reinterpret_cast<const MoeMeta*>(ws);
  ws += moe_align(sizeof(MoeMeta)) + moe_align(rows * hidden * 2) + moe_align(rows * intermediate * 2);
  const __nv_bfloat16* y2 =
      moe_fp4_plan(tokens, intermediate).ksplit == 2 ? reinterpret_cast<const __nv_bfloat16*>(ws + moe_align(rows * hidden * 2)) : nullptr;
  launch_overlapped(moe_combine_add_norm_kernel, dim3(static_cast<unsigned>(tokens)), dim3(128), 0,
                    static_cast<cudaStream_t>(stream), reinterpret_cast<const __nv_bfloat16*>(ws), meta,
                    static_cast<const __nv_bfloat16*>(residual), residual_stride, reinterpret_cast<const float4*>(gain),
                    static_cast<__nv_bfloat16*>(h_out), h_stride, static_cast<__nv_bfloat16*>(y_out), y_stride, hidden,
                    static_cast<int>(tokens), 1.0f / static_cast<float>(hidden), eps, y2);
  return launch_status();
}
