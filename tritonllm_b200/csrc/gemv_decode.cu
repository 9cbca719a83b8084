// Decode-time projections: a skinny GEMM  y[b, f] = sum_k x[b, k] * W[f, k]  for one token per
// sequence (up to 256 sequences per pass) against a weight matrix streamed from HBM once, with the
// epilogue of the op fused in:
//   EPI_QKV : + bias, YaRN RoPE on q/k heads, q -> q_out, k/v -> KV cache row *offset
//   EPI_OUT : + bias + residual, written into the residual
//
// HBM-bound on W - provided the arithmetic keeps up: warp-level mma.sync runs at a small fraction
// of the tensor-core rate on this chip and caps such a kernel near 20 % of the HBM roofline, so the
// product runs on tcgen05 with the operands swapped: the 128 x 64 weight tile is the M x K operand,
// the activations are the N x K operand (N = sequences, 32..256), the accumulator [128 features x N]
// lives in tensor memory.  Structure:
//   * one CTA per (128-feature tile, K slice); the K slices of a tile form a thread-block cluster
//     sized so that tiles x slices fills the SMs (3 slices for QKV, 6 for o_proj at gpt-oss sizes);
//   * warp 0: TMA producer (weight tile + activation tile per 64-wide k-block, 128-byte rows, 128B
//     swizzle) into a ring of shared-memory stages; warp 1: one thread issues tcgen05.mma;
//   * warps 2-5 (one thread per feature row): the slice's partial sums go from tensor memory to
//     shared memory; after a cluster barrier the CTAs of the cluster add the slices through
//     distributed shared memory in a fixed order (no global scratch, no atomics, deterministic)
//     and run the epilogue, each on its share of the rows, a RoPE pair (j, j+32) per item.
// Bounded waits throughout.
//
// Per-CTA timestamps at 256 sequences (o_proj, 6 slices): accumulators complete at 7.7 us, dumped 9.3, cluster barrier
// 10.1, reduction + epilogue done 20.0, exit 22.2.  The epilogue loop is what grows with the batch: a thread does
// bn / (8 * slices) items one after the other and each item's loads (bias, residual, tables) must return before its
// stores can issue, and it adds the slices one distributed-shared-memory round trip after the other: about 1.6 us per
// item with cold operands as the single-kernel timing has them.  All six warps now share the items (23.8 -> 21.3 us).
// Variants measured and dropped, each removing one of the two chains only: the other slices' sums read four at a time
// (23.5 us); every slice's sums pushed into the shared memory of the CTA that finishes the sequence, local reads
// (24.2 us); three items' operands fetched before the first store (24.2 us); the last two together, with a remote store
// and its address arithmetic per element (30.5 us); the batch split in two halves along grid.z with half the K slices
// (o_proj 26.1 against 21.2 us, QKV 31.1 against 22.3 us: the longer main loop costs more than the smaller reduction saves).
#include <cooperative_groups.h>

#include <map>
#include <mutex>
#include <tuple>

#include "tc_common.cuh"

namespace cg = cooperative_groups;

namespace b2 {

constexpr int SK_THREADS = 192;
constexpr int SK_FT = 128;                       // features per tile (UMMA M)
constexpr int SK_KB = 64;                        // k elements per block
constexpr int SK_W_BYTES = SK_FT * SK_KB * 2;    // 16 KiB
constexpr int SK_MAX_STAGES = 8;
constexpr int SK_MAX_BN = 256;
constexpr int SK_TS = SK_FT + 4;                 // row stride (floats) of the sequence-major accumulator dump
// Bytes of the accumulator dump that reuses the ring: [128][bn + 4] (logits epilogue) or [bn][SK_TS] (the others).
__host__ __device__ constexpr size_t sk_dump_bytes(int bn) {
  return (static_cast<size_t>(SK_FT) * (bn + 4) > static_cast<size_t>(bn) * SK_TS ? static_cast<size_t>(SK_FT) * (bn + 4)
                                                                                  : static_cast<size_t>(bn) * SK_TS) * 4;
}
enum { EPI_QKV = 0, EPI_OUT = 1, EPI_LOGITS = 2 };

struct SkinnyArgs {
  const __nv_bfloat16* bias;
  int batch, bn, k_in, n_out, stages, n_tiles, nkb, epi, kslices;
  int tpc;     // weight tiles per CTA (EPI_LOGITS with many sequences: 2, so that an activation tile fetched from L2 feeds two)
  int vec_ok;  // outputs, bias and residual allow 8-byte accesses at every multiple of four features
  // EPI_QKV
  const float* sin_tab;
  const float* cos_tab;
  const int64_t* offset;
  int64_t offset_stride;            // 0: one position for the whole batch; 1: offset[b] is sequence b's position
  const int32_t* block_table;       // optional [batch][table_stride]: page of a paged KV pool that holds tokens
  int64_t table_stride;             //   page_size * j .. page_size * (j + 1) - 1 of sequence b (the pool is then
  int page_size;                    //   [pages][page_size][heads][64] and cs_b is the page stride)
  int64_t max_ctx, cache_ctx;
  __nv_bfloat16* q_out;
  __nv_bfloat16* cache_k;
  __nv_bfloat16* cache_v;
  int64_t cs_b, cs_n, cs_h;
  int n_q, n_kv;
  // EPI_OUT
  __nv_bfloat16* residual;
  int64_t res_stride;
  // EPI_LOGITS
  __nv_bfloat16* logits;     // [batch][n_out] (optional)
  int64_t logits_stride;
  float* part_max;           // [n_tiles][batch] (optional): per 128-row tile, the largest fp32 sum and its row
  int* part_idx;
  int* status;
  long long* trace;  // optional [grid][8] timestamps (b2_set_trace_buffer)
};

struct __align__(16) SkinnySmem {
  uint64_t full[SK_MAX_STAGES];
  uint64_t empty[SK_MAX_STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

// Four consecutive bf16 values (n of them valid): one 8-byte access when the caller vouches for alignment.
__device__ __forceinline__ void ld_bf16x4(const __nv_bfloat16* p, bool vec, int n, float (&o)[4]) {
  if (vec && n >= 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    o[0] = __uint_as_float(u.x << 16);
    o[1] = __uint_as_float(u.x & 0xffff0000u);
    o[2] = __uint_as_float(u.y << 16);
    o[3] = __uint_as_float(u.y & 0xffff0000u);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = i < n ? __bfloat162float(p[i]) : 0.f;
  }
}
__device__ __forceinline__ void st_bf16x4(__nv_bfloat16* p, bool vec, int n, const float (&v)[4]) {
  if (vec && n >= 4) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (i < n) p[i] = __float2bfloat16_rn(v[i]);
  }
}

// TPC = weight tiles per CTA: 1, or 2 for the unembedding with many sequences (a compile-time constant so that the
// common instantiation keeps straight-line producer / MMA code).
// LG: the unembedding's epilogue (logits / arg-max) instead of the projections' (cluster reduction, bias, RoPE, KV write,
// residual): a compile-time choice so that neither epilogue's registers count against the other (the unembedding runs two
// CTAs per SM and must stay under 170 registers; it needs 84 on its own).
template <int TPC, bool LG>
__global__ void __launch_bounds__(SK_THREADS, 1)
skinny_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const SkinnyArgs a,
                 int b0) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  cg::cluster_group cluster = cg::this_cluster();
  const int S = a.stages, bn = a.bn, KS = a.kslices;
  const int stage_bytes = TPC * SK_W_BYTES + bn * SK_KB * 2;
  // the ring memory is reused for the fp32 dump of the accumulator once the main loop is over
  const size_t ring_bytes = max(static_cast<size_t>(S) * stage_bytes, sk_dump_bytes(bn));
  SkinnySmem& sm = *reinterpret_cast<SkinnySmem*>(tiles + ((ring_bytes + 15) & ~static_cast<size_t>(15)));
  float* dump = reinterpret_cast<float*>(tiles);
  const int dstride = bn + 4;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x * TPC, rank = blockIdx.y;  // first tile of the CTA; cluster = the K slices of one tile (along y)

  overlap_start();
  if (tid == 0 && a.trace) a.trace[(blockIdx.x * KS + rank) * 8 + 0] = global_timer_ns();
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 1);
    }
    mbar_init(&sm.acc_full, 1);
    sm.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_x);
  }
  int tmem_cols = 32;
  while (tmem_cols < TPC * bn) tmem_cols <<= 1;
  if (warp == 1) tmem_alloc(&sm.tmem_base, tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;
  overlap_wait();   // barriers, tensor memory and descriptors were set up while the kernel before this one drained

  const int kb_begin = static_cast<int>((static_cast<long long>(a.nkb) * rank) / KS);
  const int kb_end = static_cast<int>((static_cast<long long>(a.nkb) * (rank + 1)) / KS);
  const int n_my = kb_end - kb_begin;

  if (warp == 0) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      int issued = 0;
      for (int i = 0; i < n_my; ++i) {
        const int s = i % S, round = i / S;
        if (round > 0 && !mbar_wait_bounded(&sm.empty[s], (round - 1) & 1, abort_flag)) {
          if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        uint8_t* st = tiles + static_cast<size_t>(s) * stage_bytes;
        mbar_arrive_expect_tx(&sm.full[s], static_cast<uint32_t>(stage_bytes));
#pragma unroll
        for (int h = 0; h < TPC; ++h)   // rows past n_out (an odd tile count) read as zero
          tma_load_2d(st + h * SK_W_BYTES, &tm_w, &sm.full[s], (kb_begin + i) * SK_KB, (tile + h) * SK_FT);
        tma_load_2d(st + TPC * SK_W_BYTES, &tm_x, &sm.full[s], (kb_begin + i) * SK_KB, b0);
        issued = i + 1;
      }
      if (*abort_flag) {
        for (int i = issued > S ? issued - S : 0; i < issued; ++i) {
          bool done = false;
          for (uint32_t spin = 0; spin < SPIN_LIMIT && !done; ++spin) done = mbar_try_wait(&sm.full[i % S], (i / S) & 1);
          if (!done) atomicOr(a.status, B2_DEV_TIMEOUT_DRAIN);
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(SK_FT, bn);
      bool ok = true;
      for (int i = 0; i < n_my; ++i) {
        const int s = i % S;
        if (!mbar_wait_bounded(&sm.full[s], (i / S) & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(tiles + static_cast<size_t>(s) * stage_bytes);
        const uint64_t dx = umma_desc_k128(sa + TPC * SK_W_BYTES);
#pragma unroll
        for (int h = 0; h < TPC; ++h) {
          const uint64_t dw = umma_desc_k128(sa + h * SK_W_BYTES);
#pragma unroll
          for (int k = 0; k < SK_KB / 16; ++k) umma_bf16(tmem + h * bn, dw + 2 * k, dx + 2 * k, idesc, (i | k) != 0);
        }
        umma_commit(&sm.empty[s]);
      }
      if (ok) {
        umma_commit(&sm.acc_full);  // arrives when every MMA above has completed (and read its stage)
      } else {
        if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
        *abort_flag = 1;
      }
    }
  }
  // ================================ accumulator -> shared memory (warps 2-5) ================================
  bool acc_ok = true;
  auto dump_acc = [&](int h) {   // accumulator of the CTA's h-th tile -> the ring memory, which is idle by now
    const int lane_grp = warp & 3;  // a warp may only read TMEM lanes 32*(warp%4) .. +31
    const int row = lane_grp * 32 + lane;
    const uint32_t trow = tmem + (static_cast<uint32_t>(lane_grp * 32) << 16) + h * bn;
    float* drow = dump + static_cast<size_t>(row) * dstride;
    for (int c = 0; c < bn; c += 32) {
      float v[32];
      if (acc_ok && n_my > 0) {
        tmem_ld_32x32(trow + c, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      if (LG) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(drow + c + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {  // sequence-major: the lanes of a warp (consecutive rows) write consecutive words
#pragma unroll
        for (int i = 0; i < 32; ++i) dump[(c + i) * SK_TS + row] = v[i];
      }
    }
  };
  if (warp >= 2) {
    acc_ok = n_my == 0 || mbar_wait_bounded(&sm.acc_full, 0, abort_flag);
    acc_ok = __all_sync(0xffffffffu, acc_ok);
    if (!acc_ok) {
      if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
      *abort_flag = 1;
    }
    if (a.trace && tid == 64) a.trace[(blockIdx.x * KS + rank) * 8 + 2] = global_timer_ns();
    tc_fence_after_sync();
    // the ring is idle now (every stage was consumed before acc_full fired): overwrite it with the dump
    dump_acc(0);
  }
  tc_fence_before_sync();
  cluster.sync();  // every slice of the tile is in its CTA's shared memory

  if (LG) {
   if (warp >= 2) {
    // ================================ unembedding: logits and per-tile arg-max (one K slice per tile) ================================
    const int e = (warp - 2) * 32 + lane;  // 0..127
    for (int h = 0; h < TPC; ++h) {
      if (h > 0) {   // the next tile of this CTA: its accumulator replaces the dump once every thread is done with it
        named_bar_sync(1, 128);
        tc_fence_after_sync();
        dump_acc(h);
        named_bar_sync(1, 128);
      }
      const int t = tile + h;
      const int f = t * SK_FT + e;
      const int rows = min(SK_FT, a.n_out - t * SK_FT);
      if (rows <= 0 || *abort_flag) continue;
      if (a.logits && f < a.n_out) {   // thread e owns vocabulary row e of the tile: for a sequence, 128 threads write 256 contiguous bytes
        for (int c = 0; c < bn && b0 + c < a.batch; ++c)
          a.logits[static_cast<size_t>(b0 + c) * a.logits_stride + f] = __float2bfloat16_rn(dump[e * dstride + c]);
      }
      if (a.part_max) {                // thread c owns sequence c: the largest fp32 sum of the tile, first row on ties
        for (int c = e; c < bn && b0 + c < a.batch; c += 128) {
          float best = dump[c];
          int arg = 0;
          for (int r = 1; r < rows; ++r) {
            const float v = dump[r * dstride + c];
            if (v > best) {
              best = v;
              arg = r;
            }
          }
          a.part_max[static_cast<size_t>(t) * a.batch + b0 + c] = best;
          a.part_idx[static_cast<size_t>(t) * a.batch + b0 + c] = t * SK_FT + arg;
        }
      }
    }
   }
  } else if (!*abort_flag) {
    // ================================ reduce across the cluster + epilogue ================================
    const int e = tid;  // all six warps: the producer and the MMA warp have nothing left to do
    long long offset = 0, pos = 0;
    bool offset_ok = true;
    const bool per_seq = a.epi == EPI_QKV && (a.offset_stride != 0 || a.block_table != nullptr);
    if (a.epi == EPI_QKV && !per_seq) {
      offset = *a.offset;
      offset_ok = offset >= 0 && offset < a.cache_ctx;
      pos = offset % a.max_ctx;
      if (pos < 0) pos += a.max_ctx;
      if (!offset_ok && e == 0 && tile == 0 && rank == 0) atomicOr(a.status, B2_DEV_BAD_INDEX);
    }
    // items = (sequence, four consecutive row pairs), rows fastest: the 16 lanes of a sequence read 2 x 256
    // contiguous bytes of each slice's dump and write runs of 64-128 contiguous bytes of the output row;
    // this CTA takes every KS-th group of 192 items
    const int items = bn * 16;
    for (int it = rank * SK_THREADS + e; it < items; it += KS * SK_THREADS) {
      const int c = it >> 4, qd = it & 15;
      const int b = b0 + c;
      if (b >= a.batch) continue;
      const int r_lo = a.epi == EPI_QKV ? ((qd >> 3) * 64 + (qd & 7) * 4) : qd * 4;  // RoPE pair (j, j+32) / rows (r, r+64)
      const int r_hi = a.epi == EPI_QKV ? r_lo + 32 : r_lo + 64;
      const int f_lo = tile * SK_FT + r_lo, f_hi = tile * SK_FT + r_hi;
      const int n_lo = min(4, a.n_out - f_lo), n_hi = min(4, a.n_out - f_hi);   // valid features of each quad
      if (n_lo <= 0) continue;
      // epilogue operands first, so their latency overlaps the remote shared-memory reads
      float bias_lo[4], bias_hi[4], cs[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
      float res_lo[4] = {0.f, 0.f, 0.f, 0.f}, res_hi[4] = {0.f, 0.f, 0.f, 0.f};
      ld_bf16x4(a.bias + f_lo, a.vec_ok, n_lo, bias_lo);
      ld_bf16x4(a.bias + f_hi, a.vec_ok, n_hi, bias_hi);
      __nv_bfloat16* dst_lo = nullptr;
      __nv_bfloat16* dst_hi = nullptr;
      bool rotate = false;
      long long kv_row = static_cast<long long>(b) * a.cs_b + offset * a.cs_n;   // element offset of the token's K/V row
      if (per_seq) {   // this sequence's own position, and its page when the KV store is paged
        offset = a.offset[static_cast<size_t>(b) * a.offset_stride];
        offset_ok = offset >= 0 && offset < a.cache_ctx;
        pos = offset % a.max_ctx;
        if (pos < 0) pos += a.max_ctx;
        if (!offset_ok) {
          if (qd == 0 && tile == 0) atomicOr(a.status, B2_DEV_BAD_INDEX);
        } else if (a.block_table) {
          const long long page = a.block_table[static_cast<size_t>(b) * a.table_stride + offset / a.page_size];
          kv_row = page * a.cs_b + (offset % a.page_size) * a.cs_n;
          if (page < 0) {
            offset_ok = false;
            if (qd == 0 && tile == 0) atomicOr(a.status, B2_DEV_BAD_INDEX);
          }
        } else {
          kv_row = static_cast<long long>(b) * a.cs_b + offset * a.cs_n;
        }
      }
      if (a.epi == EPI_QKV) {
        const int head = tile * 2 + (qd >> 3), jj = (qd & 7) * 4;
        rotate = head < a.n_q + a.n_kv;
        if (rotate && a.vec_ok) {
          const float4 c4 = __ldg(reinterpret_cast<const float4*>(a.cos_tab + pos * 32 + jj));
          const float4 s4 = __ldg(reinterpret_cast<const float4*>(a.sin_tab + pos * 32 + jj));
          cs[0] = c4.x; cs[1] = c4.y; cs[2] = c4.z; cs[3] = c4.w;
          sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
        } else if (rotate) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            cs[q] = __ldg(a.cos_tab + pos * 32 + jj + q);
            sn[q] = __ldg(a.sin_tab + pos * 32 + jj + q);
          }
        }
        if (head < a.n_q) {
          dst_lo = a.q_out + (static_cast<size_t>(b) * a.n_q + head) * 64 + jj;
        } else if (offset_ok) {
          const bool is_k = head < a.n_q + a.n_kv;
          const int kvh = is_k ? head - a.n_q : head - a.n_q - a.n_kv;
          dst_lo = (is_k ? a.cache_k : a.cache_v) + kv_row + kvh * a.cs_h + jj;
        }
        dst_hi = dst_lo ? dst_lo + 32 : nullptr;
      } else {
        __nv_bfloat16* res = a.residual + static_cast<size_t>(b) * a.res_stride;
        dst_lo = res + f_lo;
        dst_hi = res + f_hi;
        ld_bf16x4(dst_lo, a.vec_ok, n_lo, res_lo);
        ld_bf16x4(dst_hi, a.vec_ok, n_hi, res_hi);
      }
      float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
      for (int rr = 0; rr < KS; ++rr) {  // fixed order: deterministic sums
        const float* remote = cluster.map_shared_rank(dump, rr) + c * SK_TS;
        const float4 pl = *reinterpret_cast<const float4*>(remote + r_lo);
        const float4 ph = *reinterpret_cast<const float4*>(remote + r_hi);
        lo.x += pl.x; lo.y += pl.y; lo.z += pl.z; lo.w += pl.w;
        hi.x += ph.x; hi.y += ph.y; hi.z += ph.z; hi.w += ph.w;
      }
      if (!dst_lo) continue;  // K/V of a position outside the cache: nothing is written
      float vl[4] = {lo.x + bias_lo[0], lo.y + bias_lo[1], lo.z + bias_lo[2], lo.w + bias_lo[3]};
      float vh[4] = {hi.x + bias_hi[0], hi.y + bias_hi[1], hi.z + bias_hi[2], hi.w + bias_hi[3]};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (rotate) {
          const float rl = vl[q] * cs[q] - vh[q] * sn[q], rh = vh[q] * cs[q] + vl[q] * sn[q];
          vl[q] = rl;
          vh[q] = rh;
        }
        vl[q] += res_lo[q];
        vh[q] += res_hi[q];
      }
      st_bf16x4(dst_lo, a.vec_ok, n_lo, vl);
      st_bf16x4(dst_hi, a.vec_ok, n_hi, vh);
    }
  }
  cluster.sync();  // peers may still be reading this CTA's shared memory
  if (tid == 0 && a.trace) a.trace[(blockIdx.x * KS + rank) * 8 + 3] = global_timer_ns();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, tmem_cols);
  }
}

static int skinny_bn(int64_t batch) {
  const int64_t b = batch > SK_MAX_BN ? SK_MAX_BN : batch;
  return static_cast<int>((b + 31) / 32 * 32);
}

static size_t skinny_smem_bytes(int bn, int nkb, int ks, int* stages_out, int max_stages = SK_MAX_STAGES, int tpc = 1) {
  const int stage_bytes = tpc * SK_W_BYTES + bn * SK_KB * 2;
  int stages = (200 * 1024) / stage_bytes;
  stages = stages > max_stages ? max_stages : stages;
  const int per_slice = (nkb + ks - 1) / ks;
  stages = stages > per_slice ? per_slice : stages;
  size_t ring = static_cast<size_t>(stages) * stage_bytes;
  const size_t dump = sk_dump_bytes(bn);
  if (dump > ring) ring = dump;
  if (stages_out) *stages_out = stages;
  return ((ring + 15) & ~static_cast<size_t>(15)) + sizeof(SkinnySmem) + 1024;
}

static int choose_kslices(int n_tiles, int nkb, int bn) {
  static std::mutex mu;
  static std::map<std::tuple<int, int, int, int>, int> cache;  // (device, n_tiles, nkb, bn) -> ks
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  const auto key = std::make_tuple(dev, n_tiles, nkb, bn);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  int best = 1;
  int start = sm_count() / n_tiles;
  start = start > 8 ? 8 : start < 1 ? 1 : start;
  if (start > nkb) start = nkb;
  for (int ks = start; ks >= 1; --ks) {
    const size_t smem = skinny_smem_bytes(bn, nkb, ks, nullptr);
    if (cudaFuncSetAttribute(skinny_tc_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess) {
      (void)cudaGetLastError();
      continue;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, ks, 1);
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ks;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&n_clusters, skinny_tc_kernel<1, false>, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      continue;
    }
    if (n_clusters >= n_tiles) {
      best = ks;
      break;
    }
  }
  cache[key] = best;
  return best;
}

static int launch_skinny(const void* x, int64_t x_stride, const void* w, SkinnyArgs a, cudaStream_t stream) {
  a.n_tiles = (a.n_out + SK_FT - 1) / SK_FT;
  a.nkb = a.k_in / SK_KB;
  a.status = device_status_ptr();
  if (!a.status) return B2_ERR_DRIVER;
  // K slices per tile = cluster size: the largest (at most 8, the portable limit, and at most one per
  // k-block) for which all n_tiles clusters can be resident at once - a cluster must fit inside one GPC,
  // so this is asked of the occupancy calculator rather than derived from the SM count.
  int ks = a.epi == EPI_LOGITS ? 1 : choose_kslices(a.n_tiles, a.nkb, skinny_bn(a.batch));
  if (a.epi != EPI_LOGITS) {
    const int forced = tunable(a.epi == EPI_QKV ? TUNE_GEMV_KSPLIT_QKV : TUNE_GEMV_KSPLIT_OUT);
    if (forced > 0) ks = forced > 8 ? 8 : forced;
    if (ks > a.nkb) ks = a.nkb;
  }
  a.kslices = ks;
  {
    size_t slots = 0;
    long long* tb = trace_buffer(&slots);
    a.trace = slots >= static_cast<size_t>(a.n_tiles) * ks ? tb : nullptr;
  }
  CUtensorMap tm_w, tm_x;
  const uint64_t wd[2] = {static_cast<uint64_t>(a.k_in), static_cast<uint64_t>(a.n_out)};
  const uint64_t ws[1] = {static_cast<uint64_t>(a.k_in) * 2};
  const uint32_t wb[2] = {SK_KB, SK_FT};
  int rc = make_tensor_map_bf16(&tm_w, w, 2, wd, ws, wb, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  // sequences in passes of up to 256; each pass streams W again (from L2 when it fits)
  for (int b0 = 0; b0 < a.batch; b0 += SK_MAX_BN) {
    a.bn = skinny_bn(a.batch - b0);
    const uint64_t xd[2] = {static_cast<uint64_t>(a.k_in), static_cast<uint64_t>(a.batch)};
    const uint64_t xs[1] = {static_cast<uint64_t>(x_stride) * 2};
    const uint32_t xb[2] = {SK_KB, static_cast<uint32_t>(a.bn)};
    rc = make_tensor_map_bf16(&tm_x, x, 2, xd, xs, xb, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != B2_OK) return rc;
    // the unembedding has many more tiles than SMs: with half the ring two CTAs share an SM and one streams while
    // the other sets up or writes out (32 sequences: 267 -> 213 us); at 256 sequences a stage is too large for that
    int max_stages = SK_MAX_STAGES;
    a.tpc = 1;
    if (a.epi == EPI_LOGITS) {
      const int forced = tunable(TUNE_UNEMBED_STAGES);
      const int stage_bytes = SK_W_BYTES + a.bn * SK_KB * 2;
      if (a.bn <= 128) max_stages = (108 * 1024) / stage_bytes;   // 5 / 4 / 3 stages at 32 / 64 / 128 sequences
      if (forced > 0) max_stages = forced > SK_MAX_STAGES ? SK_MAX_STAGES : forced;
      // many sequences: the activation tile of a k-block (32 KB at 256 sequences) is twice the weight tile and every
      // CTA re-reads it from L2, which then bounds the kernel; a CTA that takes two weight tiles halves that traffic
      // (two accumulators of 256 columns fill tensor memory)
      if (a.bn > 128 && tunable(TUNE_UNEMBED_TILES) != 1) a.tpc = 2;
    }
    const size_t smem = skinny_smem_bytes(a.bn, a.nkb, ks, &a.stages, max_stages, a.tpc);
    auto kern = a.epi != EPI_LOGITS ? skinny_tc_kernel<1, false>
                                    : (a.tpc == 2 ? skinny_tc_kernel<2, true> : skinny_tc_kernel<1, true>);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.n_tiles + a.tpc - 1) / a.tpc, ks, 1);
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ks;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see launch_overlapped
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tunable(TUNE_LAUNCH_OVERLAP) ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, kern, tm_w, tm_x, a, b0);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return static_cast<int>(e);
    }
  }
  return launch_status();
}

// token[b] = row of the largest per-tile maximum, the smallest row on ties; one warp per sequence
__global__ void unembed_argmax_reduce_kernel(const float* __restrict__ part_max, const int* __restrict__ part_idx, int n_tiles,
                                             int batch, long long* __restrict__ token_ids) {
  overlap_start();
  overlap_wait();
  const int b = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (b >= batch) return;
  float best = -3.0e38f;
  int arg = 0x7fffffff;
  for (int t = lane; t < n_tiles; t += 32) {
    const float v = part_max[static_cast<size_t>(t) * batch + b];
    const int i = part_idx[static_cast<size_t>(t) * batch + b];
    if (v > best || (v == best && i < arg)) {
      best = v;
      arg = i;
    }
  }
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, arg, d);
    if (ov > best || (ov == best && oi < arg)) {
      best = ov;
      arg = oi;
    }
  }
  if (lane == 0) token_ids[b] = arg;
}

}  // namespace b2

B2_API size_t b2_unembed_workspace_bytes(int64_t batch, int vocab) {
  if (batch <= 0 || vocab <= 0) return 0;
  return static_cast<size_t>((vocab + b2::SK_FT - 1) / b2::SK_FT) * static_cast<size_t>(batch) * 8;
}

B2_API int b2_unembed_decode(const void* hidden, int64_t hidden_stride_b, const void* weight, void* logits,
                             int64_t logits_stride_b, int64_t* token_ids, void* workspace, size_t workspace_bytes,
                             int64_t batch, int hidden_size, int vocab, void* stream) {
  using namespace b2;
  if (batch < 0 || hidden_size <= 0 || vocab <= 0 || (logits && logits_stride_b < vocab)) return B2_ERR_SHAPE;
  if (hidden_size % SK_KB != 0 || batch > 0x7fffffff) return B2_ERR_UNSUPPORTED;
  if (batch == 0) return B2_OK;
  if (!hidden || !weight || (!logits && !token_ids)) return B2_ERR_NULL;
  if (!aligned16(hidden) || !aligned16(weight) || hidden_stride_b % 8 != 0) return B2_ERR_ALIGN;
  const int n_tiles = (vocab + SK_FT - 1) / SK_FT;
  if (token_ids) {
    if (!workspace) return B2_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) || workspace_bytes < b2_unembed_workspace_bytes(batch, vocab))
      return B2_ERR_WORKSPACE;
  }
  SkinnyArgs a = {};
  a.epi = EPI_LOGITS;
  a.batch = static_cast<int>(batch);
  a.k_in = hidden_size;
  a.n_out = vocab;
  a.logits = static_cast<__nv_bfloat16*>(logits);
  a.logits_stride = logits_stride_b;
  if (token_ids) {
    a.part_max = static_cast<float*>(workspace);
    a.part_idx = reinterpret_cast<int*>(a.part_max + static_cast<size_t>(n_tiles) * batch);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = launch_skinny(hidden, hidden_stride_b, weight, a, st);
  if (rc != B2_OK || !token_ids) return rc;
  const int warps = 8;
  launch_overlapped(unembed_argmax_reduce_kernel, dim3(static_cast<unsigned>((batch + warps - 1) / warps)), dim3(warps * 32),
                    0, st, static_cast<const float*>(a.part_max), static_cast<const int*>(a.part_idx), n_tiles,
                    static_cast<int>(batch), reinterpret_cast<long long*>(token_ids));
  return launch_status();
}

B2_API int b2_qkv_rope_kv_decode(const void* hidden, int64_t hidden_stride_b, const void* weight, const void* bias,
                                 const float* sin_tab, const float* cos_tab, const int64_t* offset_dev, void* q_out,
                                 void* cache_k, void* cache_v, int64_t cache_stride_b, int64_t cache_stride_n,
                                 int64_t cache_stride_h, int64_t cache_ctx, int64_t batch, int hidden_size,
                                 int n_q_heads, int n_kv_heads, int head_dim, int64_t max_ctx, void* stream) {
  using namespace b2;
  if (batch < 0 || hidden_size <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_ctx <= 0 || cache_ctx <= 0)
    return B2_ERR_SHAPE;
  if (head_dim != 64 || hidden_size % SK_KB != 0 || batch > 0x7fffffff) return B2_ERR_UNSUPPORTED;
  if (batch == 0) return B2_OK;
  if (!hidden || !weight || !bias || !sin_tab || !cos_tab || !offset_dev || !q_out || !cache_k || !cache_v)
    return B2_ERR_NULL;
  if (!aligned16(hidden) || !aligned16(weight) || hidden_stride_b % 8 != 0) return B2_ERR_ALIGN;
  SkinnyArgs a = {};
  a.epi = EPI_QKV;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.batch = static_cast<int>(batch);
  a.k_in = hidden_size;
  a.n_out = (n_q_heads + 2 * n_kv_heads) * head_dim;
  a.sin_tab = sin_tab;
  a.cos_tab = cos_tab;
  a.offset = offset_dev;
  a.max_ctx = max_ctx;
  a.cache_ctx = cache_ctx;
  a.q_out = static_cast<__nv_bfloat16*>(q_out);
  a.cache_k = static_cast<__nv_bfloat16*>(cache_k);
  a.cache_v = static_cast<__nv_bfloat16*>(cache_v);
  a.cs_b = cache_stride_b;
  a.cs_n = cache_stride_n;
  a.cs_h = cache_stride_h;
  a.n_q = n_q_heads;
  a.n_kv = n_kv_heads;
  const auto al8 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; };
  a.vec_ok = al8(q_out) && al8(cache_k) && al8(cache_v) && al8(bias) && aligned16(sin_tab) && aligned16(cos_tab) &&
             cache_stride_b % 4 == 0 && cache_stride_n % 4 == 0 && cache_stride_h % 4 == 0;
  return launch_skinny(hidden, hidden_stride_b, weight, a, static_cast<cudaStream_t>(stream));
}

B2_API int b2_qkv_rope_kv_decode_ragged(const void* hidden, int64_t hidden_stride_b, const void* weight, const void* bias,
                                        const float* sin_tab, const float* cos_tab, const int64_t* positions_dev,
                                        void* q_out, void* kv_k, void* kv_v, int64_t kv_stride_b, int64_t kv_stride_n,
                                        int64_t kv_stride_h, int64_t kv_ctx, const int32_t* block_table,
                                        int64_t table_stride, int page_size, int64_t batch, int hidden_size,
                                        int n_q_heads, int n_kv_heads, int head_dim, int64_t max_ctx, void* stream) {
  using namespace b2;
  if (batch < 0 || hidden_size <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_ctx <= 0 || kv_ctx <= 0)
    return B2_ERR_SHAPE;
  if (block_table && (page_size <= 0 || table_stride <= 0 || table_stride * page_size < kv_ctx)) return B2_ERR_SHAPE;
  if (head_dim != 64 || hidden_size % SK_KB != 0 || batch > 0x7fffffff) return B2_ERR_UNSUPPORTED;
  if (batch == 0) return B2_OK;
  if (!hidden || !weight || !bias || !sin_tab || !cos_tab || !positions_dev || !q_out || !kv_k || !kv_v)
    return B2_ERR_NULL;
  if (!aligned16(hidden) || !aligned16(weight) || hidden_stride_b % 8 != 0) return B2_ERR_ALIGN;
  SkinnyArgs a = {};
  a.epi = EPI_QKV;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.batch = static_cast<int>(batch);
  a.k_in = hidden_size;
  a.n_out = (n_q_heads + 2 * n_kv_heads) * head_dim;
  a.sin_tab = sin_tab;
  a.cos_tab = cos_tab;
  a.offset = positions_dev;
  a.offset_stride = 1;
  a.block_table = block_table;
  a.table_stride = table_stride;
  a.page_size = page_size;
  a.max_ctx = max_ctx;
  a.cache_ctx = kv_ctx;
  a.q_out = static_cast<__nv_bfloat16*>(q_out);
  a.cache_k = static_cast<__nv_bfloat16*>(kv_k);
  a.cache_v = static_cast<__nv_bfloat16*>(kv_v);
  a.cs_b = kv_stride_b;
  a.cs_n = kv_stride_n;
  a.cs_h = kv_stride_h;
  a.n_q = n_q_heads;
  a.n_kv = n_kv_heads;
  const auto al8 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; };
  a.vec_ok = al8(q_out) && al8(kv_k) && al8(kv_v) && al8(bias) && aligned16(sin_tab) && aligned16(cos_tab) &&
             kv_stride_b % 4 == 0 && kv_stride_n % 4 == 0 && kv_stride_h % 4 == 0;
  return launch_skinny(hidden, hidden_stride_b, weight, a, static_cast<cudaStream_t>(stream));
}

B2_API int b2_oproj_residual_decode(const void* t, int64_t t_stride_b, const void* weight, const void* bias,
                                    void* residual, int64_t residual_stride_b, int64_t batch, int k_in, int n_out,
                                    void* stream) {
  using namespace b2;
  if (batch < 0 || k_in <= 0 || n_out <= 0 || residual_stride_b < n_out) return B2_ERR_SHAPE;
  if (k_in % SK_KB != 0 || batch > 0x7fffffff) return B2_ERR_UNSUPPORTED;
  if (batch == 0) return B2_OK;
  if (!t || !weight || !bias || !residual) return B2_ERR_NULL;
  if (!aligned16(t) || !aligned16(weight) || t_stride_b % 8 != 0) return B2_ERR_ALIGN;
  SkinnyArgs a = {};
  a.epi = EPI_OUT;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.batch = static_cast<int>(batch);
  a.k_in = k_in;
  a.n_out = n_out;
  a.residual = static_cast<__nv_bfloat16*>(residual);
  a.res_stride = residual_stride_b;
  a.vec_ok = (reinterpret_cast<uintptr_t>(residual) & 7u) == 0 && (reinterpret_cast<uintptr_t>(bias) & 7u) == 0 &&
             residual_stride_b % 4 == 0;
  return launch_skinny(t, t_stride_b, weight, a, static_cast<cudaStream_t>(stream));
}
