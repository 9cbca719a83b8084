// Dense bf16 projections on the 5th-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T  (+ epilogue)
// with A = activations (row-major, K contiguous) and W = weights as the model stores them
// ([out, in], K contiguous), so both operands are K-major and need no transposition.
//
// Tensor-bound.  Large problems (M >= 1024) run on CTA pairs: 256 x BN tiles, tcgen05 cta_group::2 (see
// gemm_tc_pair_kernel below).  Otherwise one persistent CTA per SM walks the list of 128 x BN output tiles:
//   warp 0   : TMA producer - A and W tiles of 64 k-elements (128-byte rows, 128B swizzle) into a
//              ring of shared-memory stages guarded by full/empty mbarriers;
//   warp 1   : one thread issues tcgen05.mma (M = 128, N = BN, K = 16) four times per stage; the
//              fp32 accumulator lives in tensor memory, two buffers of BN columns so the MMAs of
//              tile i+1 run while tile i is being written out; tcgen05.commit releases the stage;
//   warps 2-9: epilogue - tcgen05.ld of the accumulator (one row per thread, two warps per lane quadrant
//              taking alternate 64-column chunks), then the fused tail:
//                EPI_PLAIN    + bias                                    -> bf16 [M, N]
//                EPI_QKV_ROPE + bias, YaRN RoPE on q/k heads, split     -> q, k, v (k/v may be KV-cache rows)
//                EPI_RESIDUAL + bias + residual                         -> bf16 [M, N] (may alias the residual)
//                EPI_ROUTER   round to bf16, + fp32 bias                -> fp32 logits [M, N]
// Every mbarrier wait is bounded; a wait that gives up sets the device status word and the CTA
// drains, frees its tensor memory and returns.
#include "gemm_tc.cuh"

namespace b2 {

constexpr int GT_STAGING_BYTES = GT_EPI_WARPS * 32 * 128;  // one 32 x 64 bf16 block per epilogue warp

struct __align__(16) GemmBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int BN>
__host__ __device__ constexpr int tmem_cols() {
  return 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
}

// ------------------------------------------------------------------------------------------ epilogues
template <int EPI>
__device__ __forceinline__ void epilogue_chunk64(const GemmArgs& a, int m, int n, const float (&lo)[32],
                                                 const float (&hi)[32], long long offset);

// columns n..n+63 of row m: `lo` = columns n..n+31, `hi` = n+32..n+63
template <>
__device__ __forceinline__ void epilogue_chunk64<EPI_PLAIN>(const GemmArgs& a, int m, int n, const float (&lo)[32],
                                                            const float (&hi)[32], long long) {
  __nv_bfloat16* dst = a.out + static_cast<size_t>(m) * a.ld_out + n;
  const bool vec = a.vec_ok && (n + 64 <= a.N);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float(&v)[32] = h ? hi : lo;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int c = n + 32 * h + 8 * g;
      if (vec) {
        const uint4 bb = __ldg(reinterpret_cast<const uint4*>(a.bias + c));
        uint4 o;
        o.x = pack_bf16(v[8 * g + 0] + bf16lo(bb.x), v[8 * g + 1] + bf16hi(bb.x));
        o.y = pack_bf16(v[8 * g + 2] + bf16lo(bb.y), v[8 * g + 3] + bf16hi(bb.y));
        o.z = pack_bf16(v[8 * g + 4] + bf16lo(bb.z), v[8 * g + 5] + bf16hi(bb.z));
        o.w = pack_bf16(v[8 * g + 6] + bf16lo(bb.w), v[8 * g + 7] + bf16hi(bb.w));
        *reinterpret_cast<uint4*>(dst + 32 * h + 8 * g) = o;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (c + e < a.N) dst[32 * h + 8 * g + e] = __float2bfloat16_rn(v[8 * g + e] + __bfloat162float(a.bias[c + e]));
      }
    }
  }
}

template <>
__device__ __forceinline__ void epilogue_chunk64<EPI_RESIDUAL>(const GemmArgs& a, int m, int n, const float (&lo)[32],
                                                               const float (&hi)[32], long long) {
  __nv_bfloat16* dst = a.out + static_cast<size_t>(m) * a.ld_out + n;
  const __nv_bfloat16* res = a.residual + static_cast<size_t>(m) * a.ld_res + n;
  const bool vec = a.vec_ok && (n + 64 <= a.N);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float(&v)[32] = h ? hi : lo;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int c = n + 32 * h + 8 * g;
      if (vec) {
        const uint4 bb = __ldg(reinterpret_cast<const uint4*>(a.bias + c));
        const uint4 rr = *reinterpret_cast<const uint4*>(res + 32 * h + 8 * g);
        uint4 o;
        o.x = pack_bf16(v[8 * g + 0] + bf16lo(bb.x) + bf16lo(rr.x), v[8 * g + 1] + bf16hi(bb.x) + bf16hi(rr.x));
        o.y = pack_bf16(v[8 * g + 2] + bf16lo(bb.y) + bf16lo(rr.y), v[8 * g + 3] + bf16hi(bb.y) + bf16hi(rr.y));
        o.z = pack_bf16(v[8 * g + 4] + bf16lo(bb.z) + bf16lo(rr.z), v[8 * g + 5] + bf16hi(bb.z) + bf16hi(rr.z));
        o.w = pack_bf16(v[8 * g + 6] + bf16lo(bb.w) + bf16lo(rr.w), v[8 * g + 7] + bf16hi(bb.w) + bf16hi(rr.w));
        *reinterpret_cast<uint4*>(dst + 32 * h + 8 * g) = o;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (c + e < a.N)
            dst[32 * h + 8 * g + e] = __float2bfloat16_rn(v[8 * g + e] + __bfloat162float(a.bias[c + e]) +
                                                          __bfloat162float(res[32 * h + 8 * g + e]));
      }
    }
  }
}

template <>
__device__ __forceinline__ void epilogue_chunk64<EPI_ROUTER>(const GemmArgs& a, int m, int n, const float (&lo)[32],
                                                             const float (&hi)[32], long long) {
  float* dst = a.out_f32 + static_cast<size_t>(m) * a.ld_out_f32 + n;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float(&v)[32] = h ? hi : lo;
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const int c = n + 32 * h + e;
      // the bf16 matmul output is rounded to bf16 before the fp32 bias is added
      if (c < a.N) dst[32 * h + e] = round_bf16(v[e]) + (a.bias_f32 ? __ldg(a.bias_f32 + c) : 0.f);
    }
  }
}

// Destination of columns n..n+63 (one head) of row m, or nullptr when the row falls outside the target.
__device__ __forceinline__ __nv_bfloat16* qkv_row_dst(const GemmArgs& a, int m, int n, long long offset) {
  if (n >= a.N || m >= a.M) return nullptr;
  const int head = n >> 6;
  if (head < a.n_q) return a.q_out + (static_cast<size_t>(m) * a.n_q + head) * 64;
  const int b = m / a.tokens, t = m - b * a.tokens;
  const bool is_k = head < a.n_q + a.n_kv;
  const int kvh = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
  const long long row = t + (a.kv_add_offset ? offset : 0);
  if (row < 0 || row >= a.kv_ctx) return nullptr;  // outside the destination: the host is told through the status word
  return (is_k ? a.k_out : a.v_out) + b * a.kv_sb + row * a.kv_sn + kvh * a.kv_sh;
}

// bias, YaRN rotation of q/k heads (pair j / j+32), bf16 pack: o[0..3] = elements 0..31, o[4..7] = 32..63
__device__ __forceinline__ void qkv_row_pack(const GemmArgs& a, int m, int n, const float (&lo)[32],
                                             const float (&hi)[32], long long offset, uint4 (&o)[8]) {
  const int head = n >> 6;
  const int t = m % a.tokens;
  const bool rotate = head < a.n_q + a.n_kv;
  long long pos = (t + offset) % a.max_ctx;
  if (pos < 0) pos += a.max_ctx;
  const float4* cs = reinterpret_cast<const float4*>(a.cos_tab + pos * 32);
  const float4* sn = reinterpret_cast<const float4*>(a.sin_tab + pos * 32);
  uint32_t olo[16], ohi[16];
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const uint2 bl = __ldg(reinterpret_cast<const uint2*>(a.bias + n + 4 * g));
    const uint2 bh = __ldg(reinterpret_cast<const uint2*>(a.bias + n + 32 + 4 * g));
    float x1[4] = {lo[4 * g] + bf16lo(bl.x), lo[4 * g + 1] + bf16hi(bl.x), lo[4 * g + 2] + bf16lo(bl.y),
                   lo[4 * g + 3] + bf16hi(bl.y)};
    float x2[4] = {hi[4 * g] + bf16lo(bh.x), hi[4 * g + 1] + bf16hi(bh.x), hi[4 * g + 2] + bf16lo(bh.y),
                   hi[4 * g + 3] + bf16hi(bh.y)};
    float o1[4], o2[4];
    if (rotate) {
      const float4 c4 = __ldg(cs + g), s4 = __ldg(sn + g);
      const float c[4] = {c4.x, c4.y, c4.z, c4.w}, sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (a.round_before_rope) {  // the projection is a bf16 tensor before it is rotated
          x1[e] = round_bf16(x1[e]);
          x2[e] = round_bf16(x2[e]);
        }
        o1[e] = x1[e] * c[e] - x2[e] * sv[e];
        o2[e] = x2[e] * c[e] + x1[e] * sv[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o1[e] = x1[e];
        o2[e] = x2[e];
      }
    }
    olo[2 * g] = pack_bf16(o1[0], o1[1]);
    olo[2 * g + 1] = pack_bf16(o1[2], o1[3]);
    ohi[2 * g] = pack_bf16(o2[0], o2[1]);
    ohi[2 * g + 1] = pack_bf16(o2[2], o2[3]);
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    o[g] = make_uint4(olo[4 * g], olo[4 * g + 1], olo[4 * g + 2], olo[4 * g + 3]);
    o[4 + g] = make_uint4(ohi[4 * g], ohi[4 * g + 1], ohi[4 * g + 2], ohi[4 * g + 3]);
  }
}

template <>
__device__ __forceinline__ void epilogue_chunk64<EPI_QKV_ROPE>(const GemmArgs& a, int m, int n, const float (&lo)[32],
                                                               const float (&hi)[32], long long offset) {
  __nv_bfloat16* dst = qkv_row_dst(a, m, n, offset);
  if (!dst) return;
  uint4 o[8];
  qkv_row_pack(a, m, n, lo, hi, offset, o);
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int g = 0; g < 8; ++g) d4[g] = o[g];
}

// ------------------------------------------------------------------------------- staged (coalesced) epilogue
// One thread owns one accumulator row, so a direct store would scatter 16-byte pieces over 32 rows per
// instruction and the store path, not the tensor pipe, would set the pace.  Instead the warp parks its
// 32 x 64 bf16 block in shared memory (one 128-byte row per thread, 16-byte chunks XOR-swizzled by the
// row so that neither direction has bank conflicts) and writes it out with every instruction covering
// four full 128-byte rows; the residual of EPI_RESIDUAL comes in the same way.
//   stage: this warp's 32 x 8 uint4; m0: row of lane 0; n: first column of the chunk.
template <int EPI>
__device__ __forceinline__ void epilogue_warp64(const GemmArgs& a, int m0, int lane, int n, const float (&lo)[32],
                                                const float (&hi)[32], long long offset, uint4* stage) {
  const int m = m0 + lane;
  if (EPI == EPI_ROUTER || !a.vec_ok || n + 64 > a.N) {  // fp32 logits, ragged or unaligned tail: direct stores
    if (m < a.M) epilogue_chunk64<EPI>(a, m, n, lo, hi, offset);
    return;
  }
  uint4* my_row = stage + lane * 8;
  const int sw = lane & 7;
  __nv_bfloat16* dst = nullptr;
  uint4 o[8];
  if (EPI == EPI_QKV_ROPE) {
    dst = qkv_row_dst(a, m, n, offset);
    if (dst) qkv_row_pack(a, m, n, lo, hi, offset, o);
  } else {
    if (m < a.M) dst = a.out + static_cast<size_t>(m) * a.ld_out + n;
    uint4 rr[8];
    if (EPI == EPI_RESIDUAL) {
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = 4 * it + (lane >> 3), c = lane & 7;
        if (m0 + r < a.M)
          stage[r * 8 + (c ^ (r & 7))] =
              *reinterpret_cast<const uint4*>(a.residual + static_cast<size_t>(m0 + r) * a.ld_res + n + 8 * c);
      }
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 8; ++c) rr[c] = my_row[c ^ sw];
    }
    if (dst) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float(&v)[32] = c < 4 ? lo : hi;
        const int e = 8 * (c & 3);
        const uint4 bb = __ldg(reinterpret_cast<const uint4*>(a.bias + n + 8 * c));
        float x[8] = {v[e + 0] + bf16lo(bb.x), v[e + 1] + bf16hi(bb.x), v[e + 2] + bf16lo(bb.y), v[e + 3] + bf16hi(bb.y),
                      v[e + 4] + bf16lo(bb.z), v[e + 5] + bf16hi(bb.z), v[e + 6] + bf16lo(bb.w), v[e + 7] + bf16hi(bb.w)};
        if (EPI == EPI_RESIDUAL) {
          x[0] += bf16lo(rr[c].x);
          x[1] += bf16hi(rr[c].x);
          x[2] += bf16lo(rr[c].y);
          x[3] += bf16hi(rr[c].y);
          x[4] += bf16lo(rr[c].z);
          x[5] += bf16hi(rr[c].z);
          x[6] += bf16lo(rr[c].w);
          x[7] += bf16hi(rr[c].w);
        }
        o[c] = make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
      }
    }
  }
  if (dst) {
#pragma unroll
    for (int c = 0; c < 8; ++c) my_row[c ^ sw] = o[c];
  }
  __syncwarp();
  const unsigned long long mine = reinterpret_cast<unsigned long long>(dst);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = 4 * it + (lane >> 3), c = lane & 7;
    const unsigned long long row_dst = __shfl_sync(0xffffffffu, mine, r);
    if (row_dst) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(row_dst) + 8 * c) = stage[r * 8 + (c ^ (r & 7))];
  }
  __syncwarp();  // the block is out before the next chunk overwrites the staging rows
}

// ------------------------------------------------------------------------------- MoE (grouped) epilogues
__device__ __forceinline__ float swiglu_clamped(float g, float l, float alpha, float limit) {
  g = fminf(g, limit);
  l = fmaxf(fminf(l, limit), -limit);
  const float s = __fdividef(g, 1.0f + __expf(-alpha * g));
  return fmaf(s, l, s);
}
// Columns n..n+63 of the 32 rows m0..m0+31 of one expert's output (rows >= m_end belong to the next expert or do not
// exist and are dropped), written through the warp's staging block so that every store covers whole rows.
//   EPI_MOE_SWIGLU: column pairs (2j, 2j+1) = (gate, linear) -> 32 outputs per row at columns n/2..n/2+31
//   EPI_MOE_GATE:   (acc + bias) * gate[row] -> 64 outputs per row
template <int EPI>
__device__ __forceinline__ void epilogue_moe64(const GemmArgs& a, int m0, int lane, int n, const float (&lo)[32],
                                               const float (&hi)[32], int m_end, int expert, uint4* stage) {
  const int m = m0 + lane;
  const bool valid = m < m_end;
  const float4* bias = reinterpret_cast<const float4*>(a.g_bias + static_cast<size_t>(expert) * a.N + n);
  uint4* my_row = stage + lane * 8;
  const int sw = lane & 7;
  __nv_bfloat16* dst = nullptr;
  if (EPI == EPI_MOE_SWIGLU) {
    if (valid) {
      dst = a.out + static_cast<size_t>(m) * a.ld_out + (n >> 1);
#pragma unroll
      for (int g = 0; g < 4; ++g) {   // outputs 8g..8g+7 from columns 16g..16g+15
        const float(&v)[32] = g < 2 ? lo : hi;
        const int e0 = 16 * (g & 1);
        float r[8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 b4 = __ldg(bias + 4 * g + q);
          r[2 * q] = swiglu_clamped(v[e0 + 4 * q] + b4.x, v[e0 + 4 * q + 1] + b4.y, a.alpha, a.limit);
          r[2 * q + 1] = swiglu_clamped(v[e0 + 4 * q + 2] + b4.z, v[e0 + 4 * q + 3] + b4.w, a.alpha, a.limit);
        }
        my_row[g ^ sw] = make_uint4(pack_bf16(r[0], r[1]), pack_bf16(r[2], r[3]), pack_bf16(r[4], r[5]), pack_bf16(r[6], r[7]));
      }
    }
    __syncwarp();
    const unsigned long long mine = reinterpret_cast<unsigned long long>(dst);
#pragma unroll
    for (int it = 0; it < 4; ++it) {   // 8 rows x 64 bytes per instruction
      const int r = 8 * it + (lane >> 2), c = lane & 3;
      const unsigned long long row_dst = __shfl_sync(0xffffffffu, mine, r);
      if (row_dst) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(row_dst) + 8 * c) = stage[r * 8 + (c ^ (r & 7))];
    }
  } else {
    if (valid) {
      dst = a.out + static_cast<size_t>(m) * a.ld_out + n;
      const float gate = __ldg(a.g_gate + m);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float(&v)[32] = c < 4 ? lo : hi;
        const int e = 8 * (c & 3);
        const float4 b0 = __ldg(bias + 2 * c), b1 = __ldg(bias + 2 * c + 1);
        my_row[c ^ sw] = make_uint4(pack_bf16((v[e + 0] + b0.x) * gate, (v[e + 1] + b0.y) * gate),
                                    pack_bf16((v[e + 2] + b0.z) * gate, (v[e + 3] + b0.w) * gate),
                                    pack_bf16((v[e + 4] + b1.x) * gate, (v[e + 5] + b1.y) * gate),
                                    pack_bf16((v[e + 6] + b1.z) * gate, (v[e + 7] + b1.w) * gate));
      }
    }
    __syncwarp();
    const unsigned long long mine = reinterpret_cast<unsigned long long>(dst);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = 4 * it + (lane >> 3), c = lane & 7;
      const unsigned long long row_dst = __shfl_sync(0xffffffffu, mine, r);
      if (row_dst) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(row_dst) + 8 * c) = stage[r * 8 + (c ^ (r & 7))];
    }
  }
  __syncwarp();  // the block is out before the next chunk overwrites the staging rows
}

// ---------------------------------------------------------------------------------------------- kernel
template <int BN, int EPI>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, const GemmArgs a) {
  constexpr int B_BYTES = BN * GT_BK * 2;
  constexpr int STAGE_BYTES = GT_A_BYTES + B_BYTES;
  constexpr uint32_t IDESC = umma_idesc_bf16(GT_BM, BN);
  constexpr int TMEM_COLS = tmem_cols<BN>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmBarriers& bar = *reinterpret_cast<GemmBarriers*>(tiles + static_cast<size_t>(a.stages) * STAGE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = a.stages;
  const int nkb = (a.K + GT_BK - 1) / GT_BK;
  const int n_tiles = a.tiles_m * a.tiles_n;
  volatile int* abort_flag = &bar.abort_flag;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&bar.full[s], 1);
      mbar_init(&bar.empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.acc_full[i], 1);
      mbar_init(&bar.acc_empty[i], GT_EPI_WARPS);
    }
    bar.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  if (warp == 1) tmem_alloc(&bar.tmem_base, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bar.tmem_base;
  if (a.trace && tid == 0) {
    a.trace[8ll * blockIdx.x + 0] = global_timer_ns();
    a.trace[8ll * blockIdx.x + 2] = clock64();
  }

  // Producer and MMA warps walk their loops as whole warps, so tile coordinates, descriptors and barrier
  // addresses stay warp-uniform values; only the TMA / tcgen05 instructions sit under the elected lane.
  if (warp == 0) {
    // ===================================== TMA producer =====================================
    const bool leader = elect_one();
    int it = 0, issued = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const int m0 = (tile / a.tiles_n) * GT_BM, n0 = (tile % a.tiles_n) * BN;  // n fastest: the A tile and all of W stay in L2
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % S, round = it / S;
        if (round > 0 &&
            !__all_sync(0xffffffffu, mbar_wait_bounded(&bar.empty[s], (round - 1) & 1, abort_flag))) {
          if (leader) {
            if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        uint8_t* st = tiles + static_cast<size_t>(s) * STAGE_BYTES;
        if (leader) {
          mbar_arrive_expect_tx(&bar.full[s], STAGE_BYTES);
          tma_load_2d(st, &tm_a, &bar.full[s], kb * GT_BK, m0);
          tma_load_2d(st + GT_A_BYTES, &tm_w, &bar.full[s], kb * GT_BK, n0);
        }
        __syncwarp();
        issued = it + 1;
      }
    }
    __syncwarp();
    if (leader && *abort_flag) {  // wait (bounded) for the copies still in flight before the CTA may exit
      for (int i = issued > S ? issued - S : 0; i < issued; ++i) {
        bool done = false;
        for (uint32_t spin = 0; spin < SPIN_LIMIT && !done; ++spin) done = mbar_try_wait(&bar.full[i % S], (i / S) & 1);
        if (!done) atomicOr(a.status, B2_DEV_TIMEOUT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // ===================================== MMA issuer =====================================
    const bool leader = elect_one();
    int it = 0, tl = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tl) {
      const int buf = tl & 1, use = tl >> 1;
      if (use > 0 && !__all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_empty[buf], (use - 1) & 1, abort_flag))) {
        if (leader) {
          if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + buf * BN;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % S;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bar.full[s], (it / S) & 1, abort_flag))) {
          if (leader) {
            if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_FULL);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(tiles + static_cast<size_t>(s) * STAGE_BYTES);
        const uint64_t da = umma_desc_k128(sa), db = umma_desc_k128(sa + GT_A_BYTES);
        if (leader) {
#pragma unroll
          for (int k = 0; k < GT_BK / 16; ++k)  // 16 elements = 32 bytes = 2 descriptor units along K
            umma_bf16(tmem_d, da + 2 * k, db + 2 * k, IDESC, (kb | k) != 0);
          umma_commit(&bar.empty[s]);  // stage reusable once these MMAs have read it
        }
        __syncwarp();
      }
      if (ok && leader) umma_commit(&bar.acc_full[buf]);
      __syncwarp();
    }
  } else {
    // ===================================== epilogue =====================================
    const int lane_grp = warp & 3;  // a warp may only read TMEM lanes 32*(warp%4) .. +31
    uint4* stage = reinterpret_cast<uint4*>(&bar + 1) + (warp - 2) * 256;  // 4 KiB per epilogue warp
    long long offset = 0;
    if (EPI == EPI_QKV_ROPE) offset = *a.offset;
    int tl = 0;
    bool dead = false;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tl) {
      const int buf = tl & 1;
      if (!dead) {
        const bool ok = mbar_wait_bounded(&bar.acc_full[buf], (tl >> 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
          *abort_flag = 1;
          dead = true;
        }
      }
      if (dead) break;
      tc_fence_after_sync();
      const int m = (tile / a.tiles_n) * GT_BM + lane_grp * 32 + lane;
      const int n0 = (tile % a.tiles_n) * BN;
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 64 * ((warp - 2) >> 2); c < BN; c += 64 * (GT_EPI_WARPS / 4)) {
        float lo[32], hi[32];
        tmem_ld_32x32(trow + c, lo);
        if (BN - c >= 64) {
          tmem_ld_32x32(trow + c + 32, hi);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) hi[i] = 0.f;
        }
        epilogue_warp64<EPI>(a, m - lane, lane, n0 + c, lo, hi, offset, stage);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.acc_empty[buf]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (a.trace && tid == 0) {
    a.trace[8ll * blockIdx.x + 1] = global_timer_ns();
    a.trace[8ll * blockIdx.x + 3] = clock64();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------ CTA-pair kernel
// Same GEMM on 256 x BN tiles computed by two CTAs (a cluster of 2, tcgen05 cta_group::2): per k-block
// each CTA fetches 128 rows of A and BN/2 rows of W, so a tile costs a third less shared-memory fill than
// two 128 x BN tiles; the even CTA of the pair issues the MMAs (M = 256) for both, each CTA's epilogue
// warps write the 128 rows whose accumulator sits in their own tensor memory.
//   full[s]      (leader)  : expect-tx of both CTAs' bytes; the peer's TMA completes on it remotely
//   empty[s]     (both)    : multicast tcgen05.commit from the leader
//   acc_full[b]  (both)    : multicast tcgen05.commit from the leader
//   acc_empty[b] (leader)  : 4 epilogue warps of each CTA arrive (the peer's remotely)
template <int BN, int EPI, int KSUB>
__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                    const GemmArgs a) {
  constexpr int HALF_N = BN / 2;
  constexpr int B_BYTES = HALF_N * GT_BK * 2;
  constexpr int SUB_BYTES = GT_A_BYTES + B_BYTES;      // one 64-element k-block of A and of this CTA's half of W
  constexpr int STAGE_BYTES = KSUB * SUB_BYTES;        // KSUB k-blocks per pipeline stage: one wait and one commit
  constexpr uint32_t IDESC = umma_idesc_bf16(2 * GT_BM, BN);
  constexpr int TMEM_COLS = tmem_cols<BN>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  GemmBarriers& bar = *reinterpret_cast<GemmBarriers*>(tiles + static_cast<size_t>(a.stages) * STAGE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = a.stages;
  const int nkb = (a.K + KSUB * GT_BK - 1) / (KSUB * GT_BK);  // stages per tile; TMA zero-fills k beyond K
  constexpr bool GROUPED = EPI == EPI_MOE_SWIGLU || EPI == EPI_MOE_GATE;   // tiles come from a device-side list
  const int n_tiles = (GROUPED ? __ldg(a.g_n_tiles) : a.tiles_m) * a.tiles_n;   // 256-row tiles
  const uint32_t rank = cluster_cta_rank();            // 0: leader, 1: peer
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  volatile int* abort_flag = &bar.abort_flag;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&bar.full[s], 1);
      mbar_init(&bar.empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar.acc_full[i], 1);
      mbar_init(&bar.acc_empty[i], 2 * GT_EPI_WARPS);
    }
    bar.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_w);
  }
  if (warp == 1) tmem_alloc_pair(&bar.tmem_base, TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anything arrives on them remotely
  tc_fence_after_sync();
  const uint32_t tmem_base = bar.tmem_base;
  if (a.trace && tid == 0) {
    a.trace[8ll * blockIdx.x + 0] = global_timer_ns();
    a.trace[8ll * blockIdx.x + 2] = clock64();
  }

  if (warp == 0) {
    // ===================================== TMA producer (both CTAs) =====================================
    const bool leader_lane = elect_one();
    int it = 0, issued = 0;
    bool ok = true;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
      int m0 = (tile / a.tiles_n) * (2 * GT_BM) + static_cast<int>(rank) * GT_BM;
      int n0 = (tile % a.tiles_n) * BN + static_cast<int>(rank) * HALF_N;
      if (GROUPED) {   // rows of the tile's expert (a tile may run past them: those rows are computed and dropped), its weights
        const int mt = tile / a.tiles_n;
        m0 = __ldg(a.g_tile_row0 + mt) + static_cast<int>(rank) * GT_BM;
        n0 += __ldg(a.g_tile_expert + mt) * a.N;
      }
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % S, round = it / S;
        if (round > 0 &&
            !__all_sync(0xffffffffu, mbar_wait_bounded(&bar.empty[s], (round - 1) & 1, abort_flag))) {
          if (leader_lane) {
            if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        uint8_t* st = tiles + static_cast<size_t>(s) * STAGE_BYTES;
        const uint32_t full_leader = map_to_cta(smem_u32(&bar.full[s]), 0);
        if (leader_lane) {
          if (rank == 0) mbar_arrive_expect_tx(&bar.full[s], 2 * STAGE_BYTES);
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
            tma_load_2d_pair(st + u * SUB_BYTES, &tm_a, full_leader, (kb * KSUB + u) * GT_BK, m0);
            tma_load_2d_pair(st + u * SUB_BYTES + GT_A_BYTES, &tm_w, full_leader, (kb * KSUB + u) * GT_BK, n0);
          }
        }
        __syncwarp();
        issued = it + 1;
      }
    }
    // stay until the leader's MMAs have released every stage this CTA filled: their multicast arrivals
    // must not find this CTA gone
    for (int i = issued > S ? issued - S : 0; i < issued && ok; ++i)
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bar.empty[i % S], (i / S) & 1, abort_flag));
  } else if (warp == 1) {
    // ===================================== MMA issuer (leader CTA only) =====================================
    if (rank == 0) {
      const bool leader_lane = elect_one();
      int it = 0, tl = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++tl) {
        const int buf = tl & 1, use = tl >> 1;
        const long long w0 = a.trace ? clock64() : 0;
        if (use > 0 && !__all_sync(0xffffffffu, mbar_wait_bounded(&bar.acc_empty[buf], (use - 1) & 1, abort_flag))) {
          if (leader_lane) {
            if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
            *abort_flag = 1;
          }
          break;
        }
        if (a.trace && leader_lane) a.trace[8ll * blockIdx.x + 7] += clock64() - w0;
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % S;
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bar.full[s], (it / S) & 1, abort_flag))) {
            if (leader_lane) {
              if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_FULL);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(tiles + static_cast<size_t>(s) * STAGE_BYTES);
          if (leader_lane) {
#pragma unroll
            for (int u = 0; u < KSUB; ++u) {
              const uint64_t da = umma_desc_k128(sa + u * SUB_BYTES), db = umma_desc_k128(sa + u * SUB_BYTES + GT_A_BYTES);
#pragma unroll
              for (int k = 0; k < GT_BK / 16; ++k)
                umma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, IDESC, (kb | u | k) != 0);
            }
            umma_commit_pair(&bar.empty[s], 3);  // the stage is reusable in both CTAs
          }
          __syncwarp();
        }
        if (ok && leader_lane) umma_commit_pair(&bar.acc_full[buf], 3);
        __syncwarp();
      }
    }
  } else {
    // ===================================== epilogue (both CTAs) =====================================
    const int lane_grp = warp & 3;
    uint4* stage = reinterpret_cast<uint4*>(&bar + 1) + (warp - 2) * 256;  // 4 KiB per epilogue warp
    long long offset = 0;
    if (EPI == EPI_QKV_ROPE) offset = *a.offset;
    int tl = 0;
    bool dead = false;
    for (int tile = pair; tile < n_tiles; tile += n_pairs, ++tl) {
      const int buf = tl & 1;
      const long long e0 = a.trace ? clock64() : 0;
      if (!dead) {
        const bool ok = mbar_wait_bounded(&bar.acc_full[buf], (tl >> 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {
          if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
          *abort_flag = 1;
          dead = true;
        }
      }
      if (dead) break;
      const long long e1 = a.trace ? clock64() : 0;
      tc_fence_after_sync();
      int m = (tile / a.tiles_n) * (2 * GT_BM) + static_cast<int>(rank) * GT_BM + lane_grp * 32 + lane;
      const int n0 = (tile % a.tiles_n) * BN;
      int m_end = 0, expert = 0;
      if (GROUPED) {
        const int mt = tile / a.tiles_n, row0 = __ldg(a.g_tile_row0 + mt);
        m = row0 + static_cast<int>(rank) * GT_BM + lane_grp * 32 + lane;
        m_end = row0 + __ldg(a.g_tile_rows + mt);
        expert = __ldg(a.g_tile_expert + mt);
      }
      const uint32_t trow = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 64 * ((warp - 2) >> 2); c < BN; c += 64 * (GT_EPI_WARPS / 4)) {
        float lo[32], hi[32];
        tmem_ld_32x32(trow + c, lo);
        tmem_ld_32x32(trow + c + 32, hi);
        if constexpr (GROUPED)
          epilogue_moe64<EPI>(a, m - lane, lane, n0 + c, lo, hi, m_end, expert, stage);
        else
          epilogue_warp64<EPI>(a, m - lane, lane, n0 + c, lo, hi, offset, stage);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar.acc_empty[buf]), 0));
      if (a.trace && warp == 2 && lane == 0) {
        a.trace[8ll * blockIdx.x + 5] += e1 - e0;
        a.trace[8ll * blockIdx.x + 6] += clock64() - e1;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (a.trace && tid == 0) {
    a.trace[8ll * blockIdx.x + 1] = global_timer_ns();
    a.trace[8ll * blockIdx.x + 3] = clock64();
    a.trace[8ll * blockIdx.x + 4] = n_pairs;
  }
  cluster_sync_all();  // the peer's shared and tensor memory are in use until the leader's last MMA has completed
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------- host
template <int BN, int EPI>
static int launch_gemm_tc(const void* a_ptr, int64_t lda, const void* w_ptr, int64_t ldw, GemmArgs g,
                          cudaStream_t stream) {
  constexpr int STAGE_BYTES = GT_A_BYTES + BN * GT_BK * 2;
  CUtensorMap tm_a, tm_w;
  const uint64_t dims_a[2] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.M)};
  const uint64_t dims_w[2] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.N)};
  const uint64_t str_a[1] = {static_cast<uint64_t>(lda) * 2}, str_w[1] = {static_cast<uint64_t>(ldw) * 2};
  const uint32_t box_a[2] = {GT_BK, GT_BM}, box_w[2] = {GT_BK, BN};
  int rc = make_tensor_map_bf16(&tm_a, a_ptr, 2, dims_a, str_a, box_a, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  rc = make_tensor_map_bf16(&tm_w, w_ptr, 2, dims_w, str_w, box_w, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  g.tiles_m = (g.M + GT_BM - 1) / GT_BM;
  g.tiles_n = (g.N + BN - 1) / BN;
  int stages = (225 * 1024 - GT_STAGING_BYTES) / STAGE_BYTES;
  g.stages = stages > 8 ? 8 : stages;
  g.status = device_status_ptr();
  if (!g.status) return B2_ERR_DRIVER;
  const size_t smem = static_cast<size_t>(g.stages) * STAGE_BYTES + sizeof(GemmBarriers) + GT_STAGING_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long n_tiles = static_cast<long long>(g.tiles_m) * g.tiles_n;
  const int grid = static_cast<int>(n_tiles < sm_count() ? n_tiles : sm_count());
  {
    size_t slots = 0;
    long long* tb = trace_buffer(&slots);
    g.trace = slots >= static_cast<size_t>(grid) ? tb : nullptr;
  }
  gemm_tc_kernel<BN, EPI><<<grid, GT_THREADS, smem, stream>>>(tm_a, tm_w, g);
  return launch_status();
}

// 256 x BN tiles on CTA pairs; falls back to the caller's single-CTA launch when no cluster fits.
template <int BN, int EPI, int KSUB>
static int launch_gemm_tc_pair(const void* a_ptr, int64_t lda, const void* w_ptr, int64_t ldw, GemmArgs g,
                               cudaStream_t stream, bool* launched) {
  constexpr int STAGE_BYTES = KSUB * (GT_A_BYTES + (BN / 2) * GT_BK * 2);
  *launched = false;
  CUtensorMap tm_a, tm_w;
  const uint64_t dims_a[2] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.M)};
  const uint64_t dims_w[2] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.N)};
  const uint64_t str_a[1] = {static_cast<uint64_t>(lda) * 2}, str_w[1] = {static_cast<uint64_t>(ldw) * 2};
  const uint32_t box_a[2] = {GT_BK, GT_BM}, box_w[2] = {GT_BK, BN / 2};
  int rc = make_tensor_map_bf16(&tm_a, a_ptr, 2, dims_a, str_a, box_a, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  rc = make_tensor_map_bf16(&tm_w, w_ptr, 2, dims_w, str_w, box_w, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  g.tiles_m = (g.M + 2 * GT_BM - 1) / (2 * GT_BM);
  g.tiles_n = (g.N + BN - 1) / BN;
  int stages = (225 * 1024 - GT_STAGING_BYTES) / STAGE_BYTES;
  g.stages = stages > 8 ? 8 : stages;
  g.status = device_status_ptr();
  if (!g.status) return B2_ERR_DRIVER;
  const size_t smem = static_cast<size_t>(g.stages) * STAGE_BYTES + sizeof(GemmBarriers) + GT_STAGING_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, EPI, KSUB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * sm_count(), 1, 1);
  cfg.blockDim = dim3(GT_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&n_clusters, gemm_tc_pair_kernel<BN, EPI, KSUB>, &cfg) != cudaSuccess || n_clusters < 1) {
    (void)cudaGetLastError();
    return B2_OK;  // not launched: the caller uses the single-CTA kernel
  }
  const long long n_tiles = static_cast<long long>(g.tiles_m) * g.tiles_n;
  const int pairs = static_cast<int>(n_tiles < n_clusters ? n_tiles : n_clusters);
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  {
    size_t slots = 0;
    long long* tb = trace_buffer(&slots);
    g.trace = slots >= static_cast<size_t>(2 * pairs) ? tb : nullptr;
  }
  e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BN, EPI, KSUB>, tm_a, tm_w, g);
  if (e != cudaSuccess) return static_cast<int>(e);
  *launched = true;
  return launch_status();
}

template <int EPI>
static int launch_moe_grouped_t(const void* a_ptr, int64_t lda, const void* w_ptr, int64_t ldw, GemmArgs g, int max_tiles,
                                cudaStream_t stream) {
  constexpr int BN = 192, KSUB = 2;
  constexpr int STAGE_BYTES = KSUB * (GT_A_BYTES + (BN / 2) * GT_BK * 2);
  CUtensorMap tm_a, tm_w;
  const uint64_t dims_a[2] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.M)};
  const uint64_t dims_w[2] = {static_cast<uint64_t>(g.K), static_cast<uint64_t>(g.tiles_m) * g.N};   // tiles_m carries the expert count in
  const uint64_t str_a[1] = {static_cast<uint64_t>(lda) * 2}, str_w[1] = {static_cast<uint64_t>(ldw) * 2};
  const uint32_t box_a[2] = {GT_BK, GT_BM}, box_w[2] = {GT_BK, BN / 2};
  int rc = make_tensor_map_bf16(&tm_a, a_ptr, 2, dims_a, str_a, box_a, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  rc = make_tensor_map_bf16(&tm_w, w_ptr, 2, dims_w, str_w, box_w, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  g.tiles_m = 0;   // the tile list lives on the device
  g.tiles_n = g.N / BN;
  int stages = (225 * 1024 - GT_STAGING_BYTES) / STAGE_BYTES;
  g.stages = stages > 8 ? 8 : stages;
  g.status = device_status_ptr();
  if (!g.status) return B2_ERR_DRIVER;
  g.trace = nullptr;
  const size_t smem = static_cast<size_t>(g.stages) * STAGE_BYTES + sizeof(GemmBarriers) + GT_STAGING_BYTES + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<BN, EPI, KSUB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * sm_count(), 1, 1);
  cfg.blockDim = dim3(GT_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&n_clusters, gemm_tc_pair_kernel<BN, EPI, KSUB>, &cfg) != cudaSuccess || n_clusters < 1) {
    (void)cudaGetLastError();
    return B2_ERR_UNSUPPORTED;
  }
  const long long upper = static_cast<long long>(max_tiles) * g.tiles_n;   // the list can hold at most this many tiles
  const int pairs = static_cast<int>(upper < n_clusters ? (upper < 1 ? 1 : upper) : n_clusters);
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  e = cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<BN, EPI, KSUB>, tm_a, tm_w, g);
  if (e != cudaSuccess) return static_cast<int>(e);
  return launch_status();
}

// g.tiles_m carries the number of experts in (the rows of w_ptr are experts * g.N)
int launch_moe_grouped_gemm(int epi, const void* a_ptr, int64_t lda, const void* w_ptr, int64_t ldw, GemmArgs g, int max_tiles,
                            cudaStream_t stream) {
  if (g.N % 192 != 0 || g.K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0) return B2_ERR_UNSUPPORTED;
  if (epi == EPI_MOE_SWIGLU) return launch_moe_grouped_t<EPI_MOE_SWIGLU>(a_ptr, lda, w_ptr, ldw, g, max_tiles, stream);
  if (epi == EPI_MOE_GATE) return launch_moe_grouped_t<EPI_MOE_GATE>(a_ptr, lda, w_ptr, ldw, g, max_tiles, stream);
  return B2_ERR_UNSUPPORTED;
}

// Large problems go to the pair kernel (tunable "gemm_pair"), everything else to one CTA per tile.
template <int BN_PAIR, int BN, int EPI>
static int launch_gemm_auto(const void* a_ptr, int64_t lda, const void* w_ptr, int64_t ldw, const GemmArgs& g,
                            cudaStream_t stream) {
  if (tunable(TUNE_GEMM_PAIR) != 0 && g.M >= 1024) {
    bool launched = false;
    // two k-blocks per stage halve the per-stage barrier traffic of the issuing warp; K must be deep enough
    const int rc = (g.K >= 1024 && tunable(TUNE_GEMM_PAIR) != 2)
                       ? launch_gemm_tc_pair<BN_PAIR, EPI, 2>(a_ptr, lda, w_ptr, ldw, g, stream, &launched)
                       : launch_gemm_tc_pair<BN_PAIR, EPI, 1>(a_ptr, lda, w_ptr, ldw, g, stream, &launched);
    if (rc != B2_OK || launched) return rc;
  }
  return launch_gemm_tc<BN, EPI>(a_ptr, lda, w_ptr, ldw, g, stream);
}

static int check_gemm_common(const void* a, int64_t lda, const void* w, int64_t M, int N, int K) {
  if (!a || !w) return B2_ERR_NULL;
  if (M < 0 || N <= 0 || K <= 0 || lda < K) return B2_ERR_SHAPE;
  if (K % 8 != 0 || lda % 8 != 0 || M > 0x7fffffff) return B2_ERR_UNSUPPORTED;  // TMA strides are multiples of 16 B
  if (!aligned16(a) || !aligned16(w)) return B2_ERR_ALIGN;
  return B2_OK;
}

}  // namespace b2

B2_API int b2_linear_bias(const void* x, int64_t ldx, const void* weight, const void* bias, void* out, int64_t ld_out,
                          int64_t M, int N, int K, void* stream) {
  using namespace b2;
  int rc = check_gemm_common(x, ldx, weight, M, N, K);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!bias || !out) return B2_ERR_NULL;
  if (ld_out < N) return B2_ERR_SHAPE;
  GemmArgs g = {};
  g.M = static_cast<int>(M);
  g.N = N;
  g.K = K;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.out = static_cast<__nv_bfloat16*>(out);
  g.ld_out = ld_out;
  g.vec_ok = aligned16(out) && aligned16(bias) && ld_out % 8 == 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (N > 128) return launch_gemm_auto<256, 256, EPI_PLAIN>(x, ldx, weight, K, g, st);
  return launch_gemm_tc<128, EPI_PLAIN>(x, ldx, weight, K, g, st);
}

B2_API int b2_qkv_rope_prefill(const void* x, int64_t ldx, const void* weight, const void* bias, const float* sin_tab,
                               const float* cos_tab, const int64_t* offset_dev, void* q_out, void* k_out, void* v_out,
                               int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, int64_t kv_ctx,
                               int kv_add_offset, int64_t batch, int64_t tokens, int hidden_size, int n_q_heads,
                               int n_kv_heads, int head_dim, int64_t max_ctx, int round_before_rope, void* stream) {
  using namespace b2;
  if (batch < 0 || tokens < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_ctx <= 0 || kv_ctx <= 0) return B2_ERR_SHAPE;
  if (head_dim != 64 || tokens > 0x7fffffff) return B2_ERR_UNSUPPORTED;
  const int N = (n_q_heads + 2 * n_kv_heads) * head_dim;
  const int64_t M = batch * tokens;
  int rc = check_gemm_common(x, ldx, weight, M, N, hidden_size);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!bias || !sin_tab || !cos_tab || !offset_dev || !q_out || !k_out || !v_out) return B2_ERR_NULL;
  if (!aligned16(q_out) || !aligned16(k_out) || !aligned16(v_out) || !aligned16(sin_tab) || !aligned16(cos_tab) ||
      kv_stride_b % 8 || kv_stride_n % 8 || kv_stride_h % 8 || (reinterpret_cast<uintptr_t>(bias) & 7))
    return B2_ERR_ALIGN;
  GemmArgs g = {};
  g.M = static_cast<int>(M);
  g.N = N;
  g.K = hidden_size;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.sin_tab = sin_tab;
  g.cos_tab = cos_tab;
  g.offset = offset_dev;
  g.max_ctx = max_ctx;
  g.tokens = static_cast<int>(tokens);
  g.n_q = n_q_heads;
  g.n_kv = n_kv_heads;
  g.kv_add_offset = kv_add_offset;
  g.round_before_rope = round_before_rope;
  g.q_out = static_cast<__nv_bfloat16*>(q_out);
  g.k_out = static_cast<__nv_bfloat16*>(k_out);
  g.v_out = static_cast<__nv_bfloat16*>(v_out);
  g.kv_sb = kv_stride_b;
  g.kv_sn = kv_stride_n;
  g.kv_sh = kv_stride_h;
  g.kv_ctx = kv_ctx;
  g.vec_ok = 1;  // destinations and strides were checked above: every head row is 16-byte aligned
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (N % 256 == 0) return launch_gemm_auto<256, 256, EPI_QKV_ROPE>(x, ldx, weight, hidden_size, g, st);
  return launch_gemm_tc<128, EPI_QKV_ROPE>(x, ldx, weight, hidden_size, g, st);
}

B2_API int b2_oproj_residual(const void* t, int64_t ldt, const void* weight, const void* bias, const void* residual,
                             int64_t ld_res, void* out, int64_t ld_out, int64_t M, int N, int K, void* stream) {
  using namespace b2;
  int rc = check_gemm_common(t, ldt, weight, M, N, K);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!bias || !residual || !out) return B2_ERR_NULL;
  if (ld_out < N || ld_res < N) return B2_ERR_SHAPE;
  GemmArgs g = {};
  g.M = static_cast<int>(M);
  g.N = N;
  g.K = K;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.residual = static_cast<const __nv_bfloat16*>(residual);
  g.ld_res = ld_res;
  g.out = static_cast<__nv_bfloat16*>(out);
  g.ld_out = ld_out;
  g.vec_ok = aligned16(out) && aligned16(bias) && aligned16(residual) && ld_out % 8 == 0 && ld_res % 8 == 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (N % 192 == 0) return launch_gemm_auto<192, 192, EPI_RESIDUAL>(t, ldt, weight, K, g, st);
  return launch_gemm_tc<128, EPI_RESIDUAL>(t, ldt, weight, K, g, st);
}

B2_API int b2_router_logits(const void* x, int64_t ldx, const void* gate_weight_ek, const float* gate_bias,
                            float* logits, int64_t ld_logits, int64_t M, int n_experts, int K, void* stream) {
  using namespace b2;
  int rc = check_gemm_common(x, ldx, gate_weight_ek, M, n_experts, K);
  if (rc != B2_OK) return rc;
  if (M == 0) return B2_OK;
  if (!logits) return B2_ERR_NULL;
  if (ld_logits < n_experts) return B2_ERR_SHAPE;
  GemmArgs g = {};
  g.M = static_cast<int>(M);
  g.N = n_experts;
  g.K = K;
  g.bias_f32 = gate_bias;
  g.out_f32 = logits;
  g.ld_out_f32 = ld_logits;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_experts <= 32) return launch_gemm_tc<32, EPI_ROUTER>(x, ldx, gate_weight_ek, K, g, st);
  return launch_gemm_tc<128, EPI_ROUTER>(x, ldx, gate_weight_ek, K, g, st);
}
