// Decode attention (one query token per sequence) over a contiguous KV cache:
// GQA with per-head sinks and an optional sliding window.
//
// HBM-bound: every K and V row of the visible range is read exactly once and shared by the G
// query heads of its group.  The cache is [B, ctx, Hkv, 64]: the 8 KV heads of one token are one
// contiguous 1 KiB row, so the kernel is organised to read whole token rows (a CTA that reads a
// single head touches 128 bytes of every DRAM page and tops out near 75 % of the copy bandwidth):
//   * a CTA streams ALL (up to 8) KV heads of a 32-key tile; consumer warp w owns head w;
//   * persistent grid (one CTA per SM); the list of 32-key tiles of all (sequence, head group)
//     units is cut into equal contiguous chunks, one per CTA, computed on the device from
//     *start_q, so the load is balanced for any position and window and the launch can be
//     captured in a CUDA graph;
//   * a producer warp issues one TMA copy per head (128-byte rows, 128B swizzle, so ldmatrix reads
//     are conflict-free) for K and V of a tile, back to back, into a ring of shared-memory stages
//     guarded by mbarriers; each consumer warp does S = Q K^T and O += P V for its head on
//     mma.sync m16n8k16 (rows = the G heads of the group) with an exp2-domain online softmax in
//     registers - no shared state between warps;
//   * a CTA that covered a whole unit writes the output itself; otherwise every warp leaves a
//     partial (m, l, acc) in the workspace and the last CTA to arrive at that unit (atomic
//     counter) merges the partials; the sink joins the denominator at that point.
// Every mbarrier wait is bounded; on a timeout the CTA raises a shared abort flag, records the
// code in the device status word, drains its copies and returns.
#include <math_constants.h>

#include <mutex>

#include "b2_common.cuh"

namespace b2 {

constexpr int AD_TK = 32;          // keys per tile
constexpr int AD_D = 64;           // head dim
constexpr int AD_HG = 8;           // KV heads per CTA tile = consumer warps
constexpr int AD_THREADS = (AD_HG + 1) * 32;
constexpr int AD_GMAX = 8;         // query heads per kv head (rows of the mma tile in use)
constexpr int AD_HEAD_TILE = AD_TK * AD_D * 2;          // 4 KiB: one head's K (or V) rows of a tile
constexpr int AD_STAGE_BYTES = 2 * AD_HG * AD_HEAD_TILE;  // 64 KiB: K and V, 8 heads
constexpr int AD_MAX_STAGES = 3;
constexpr float AD_M_INIT = -1.0e30f;
constexpr int AD_MAX_CTAS_PER_SM = 1;
constexpr int AD_SLOT_ROWS = AD_HG * AD_GMAX;  // rows of one partial slot

struct AttnDecodeArgs {
  const __nv_bfloat16* q;
  const void* sinks;
  __nv_bfloat16* out;
  const void* start_q;
  float* part_acc;  // [grid*2][AD_SLOT_ROWS][AD_D]
  float* part_ml;   // [grid*2][AD_SLOT_ROWS][2]
  int* counters;    // [units]
  int* status;
  float scale_log2;  // sm_scale * log2(e)
  int batch, n_kv_heads, group, n_kv_ctx, window;
  int sinks_is_f32, start_q_is_i64, stages;
  long long* trace;  // optional [grid][8] timestamps
  int hg;  // KV heads per CTA tile (<= AD_HG): fewer when the whole problem is small, so more SMs take part
  // ragged / paged variant only
  const int32_t* block_table;   // optional [batch][table_stride]: page holding keys page_size*j .. of sequence b
  long long table_stride;
  int page_size;                // multiple of AD_TK
};

constexpr int AD_RAGGED_MAX_BATCH = 2048;   // per-sequence tile counts and positions live in shared memory

// Where a CTA stands in the list of 32-key tiles when sequences have their own lengths: sequence b, head group
// hgi, tile t of the `tiles` tiles of that sequence.  The list is sequence-major, then head group, then tile;
// pfx[b] = tiles (of one head group) of the sequences before b.
struct AdCursor {
  int b, hgi, t, tiles;
  __device__ __forceinline__ void seek(long long g, const int* pfx, int batch, int n_hg) {
    int lo = 0, hi = batch - 1;   // largest b with pfx[b] * n_hg <= g
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (static_cast<long long>(pfx[mid]) * n_hg <= g) lo = mid; else hi = mid - 1;
    }
    b = lo;
    tiles = pfx[b + 1] - pfx[b];
    const int r = static_cast<int>(g - static_cast<long long>(pfx[b]) * n_hg);
    hgi = r / tiles;
    t = r - hgi * tiles;
  }
  __device__ __forceinline__ void next(const int* pfx, int batch, int n_hg) {
    if (++t == tiles) {
      t = 0;
      if (++hgi == n_hg) {
        hgi = 0;
        if (++b < batch) tiles = pfx[b + 1] - pfx[b];
      }
    }
  }
};
// visible key range of a sequence whose new token sits at position sq, and where its first tile starts
__device__ __forceinline__ void ad_range(long long sq, int n_kv_ctx, int window, int& lo, int& hi, int& lo_al) {
  long long h = sq + 1 < n_kv_ctx ? sq + 1 : n_kv_ctx;
  if (h < 0) h = 0;
  long long l = window > 0 ? sq - window + 1 : 0;
  if (l < 0) l = 0;
  if (l > h) l = h;
  lo = static_cast<int>(l);
  hi = static_cast<int>(h);
  lo_al = lo & ~(AD_TK - 1);
}

// Shared memory: `stages` x 64 KiB of tiles (1024-byte aligned), then this struct.
struct __align__(16) AttnDecodeSmem {
  uint64_t full[AD_MAX_STAGES];
  uint64_t empty[AD_MAX_STAGES];
  int abort_flag;
  int is_last;
};

__device__ __forceinline__ float load_sink_log2(const AttnDecodeArgs& a, int head) {
  if (!a.sinks) return 0.f;
  const float s = a.sinks_is_f32 ? static_cast<const float*>(a.sinks)[head]
                                 : __bfloat162float(static_cast<const __nv_bfloat16*>(a.sinks)[head]);
  return s * 1.4426950408889634f;
}

// RAGGED = false: one position for the whole batch (the reference's contract).  RAGGED = true: start_q is an
// array with one position per sequence and the KV store may be paged; tiles then start at multiples of 32 keys
// (so that a tile never straddles a page) and keys before the window are masked like keys after the position.
template <bool RAGGED>
__global__ void __launch_bounds__(AD_THREADS, 1)
attn_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const AttnDecodeArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int S = a.stages;
  AttnDecodeSmem& sm = *reinterpret_cast<AttnDecodeSmem*>(tiles + static_cast<size_t>(S) * AD_STAGE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  overlap_start();
  if (tid == 0 && a.trace) a.trace[blockIdx.x * 8 + 0] = global_timer_ns();
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], AD_HG);
    }
    sm.abort_flag = 0;
    sm.is_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  __syncthreads();
  overlap_wait();   // everything above ran while the kernel before this one was finishing

  // ---- work partition, identical in every CTA ------------------------------------------------
  const int HGR = a.hg;                                        // heads per group in this launch
  const int n_hg = (a.n_kv_heads + HGR - 1) / HGR;            // head groups per sequence
  const int units = a.batch * n_hg;                           // unit = (sequence, head group)
  int lo = 0, hi = 0, tpu = 1;                                 // uniform case: the same for every unit
  long long total;
  // ragged case: positions and the running tile count of every sequence, after the barriers in shared memory
  int* s_pfx = reinterpret_cast<int*>(&sm + 1);                // [batch + 1]
  int* s_pos = s_pfx + (AD_RAGGED_MAX_BATCH + 1);              // [batch], clamped to int
  if constexpr (RAGGED) {
    for (int b = tid; b < a.batch; b += AD_THREADS) {
      long long sq = a.start_q_is_i64 ? static_cast<const long long*>(a.start_q)[b]
                                      : static_cast<long long>(static_cast<const int*>(a.start_q)[b]);
      sq = sq < -1 ? -1 : (sq > 0x3fffffff ? 0x3fffffff : sq);
      int l, h, la;
      ad_range(sq, a.n_kv_ctx, a.window, l, h, la);
      s_pos[b] = static_cast<int>(sq);
      s_pfx[b + 1] = max(1, (h - la + AD_TK - 1) / AD_TK);
    }
    __syncthreads();
    if (warp == 0) {   // inclusive scan, 32 sequences at a time
      int carry = 0;
      for (int base = 0; base < a.batch; base += 32) {
        const int b = base + lane;
        int v = b < a.batch ? s_pfx[b + 1] : 0;
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, v, d);
          if (lane >= d) v += up;
        }
        if (b < a.batch) s_pfx[b + 1] = carry + v;
        carry += __shfl_sync(0xffffffffu, v, 31);
      }
      if (lane == 0) s_pfx[0] = 0;
    }
    __syncthreads();
    total = static_cast<long long>(s_pfx[a.batch]) * n_hg;
  } else {
    const long long sq = a.start_q_is_i64 ? *static_cast<const long long*>(a.start_q)
                                          : static_cast<long long>(*static_cast<const int*>(a.start_q));
    int lo_al;
    ad_range(sq, a.n_kv_ctx, a.window, lo, hi, lo_al);
    tpu = max(1, (hi - lo + AD_TK - 1) / AD_TK);      // tiles per unit
    total = static_cast<long long>(units) * tpu;
  }
  long long chunk = (total + gridDim.x - 1) / gridDim.x;
  // short units (window layers, short contexts): hand out whole units, so nothing has to be merged
  if (!RAGGED && tpu <= 16) chunk = (chunk + tpu - 1) / tpu * tpu;
  const long long g_begin = min(total, chunk * blockIdx.x);
  const long long g_end = min(total, g_begin + chunk);
  const int n_my = static_cast<int>(g_end - g_begin);

  volatile int* abort_flag = &sm.abort_flag;

  if (warp == AD_HG) {
    // ================================ producer ================================
    if (lane == 0) {
      int issued = 0;
      AdCursor pcur = {0, 0, 0, 1};
      for (int i = 0; i < n_my; ++i) {
        const int s = i % S, round = i / S;
        if (round > 0 && !mbar_wait_bounded(&sm.empty[s], (round - 1) & 1, abort_flag)) {
          if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        const long long g = g_begin + i;
        int b, h0, c_key, c_seq;   // sequence, first head, and the copy's coordinates along keys and sequences / pages
        if constexpr (RAGGED) {
          if (i == 0) pcur.seek(g, s_pfx, a.batch, n_hg);
          b = pcur.b;
          h0 = pcur.hgi * HGR;
          int l, h, la;
          ad_range(s_pos[b], a.n_kv_ctx, a.window, l, h, la);
          const int key0 = la + pcur.t * AD_TK;
          if (a.block_table) {
            c_seq = __ldg(a.block_table + static_cast<size_t>(b) * a.table_stride + key0 / a.page_size);
            c_key = key0 % a.page_size;
            if (c_seq < 0) {   // an unmapped page: record it and read page 0 (the keys are masked or garbage either way)
              atomicOr(a.status, B2_DEV_BAD_INDEX);
              c_seq = 0;
            }
          } else {
            c_seq = b;
            c_key = key0;
          }
          pcur.next(s_pfx, a.batch, n_hg);
        } else {
          const int u = static_cast<int>(g / tpu), t = static_cast<int>(g - static_cast<long long>(u) * tpu);
          b = u / n_hg;
          h0 = (u - b * n_hg) * HGR;
          c_seq = b;
          c_key = lo + t * AD_TK;
        }
        const int nh = min(HGR, a.n_kv_heads - h0);
        uint8_t* st = tiles + static_cast<size_t>(s) * AD_STAGE_BYTES;
        mbar_arrive_expect_tx(&sm.full[s], static_cast<uint32_t>(nh) * 2 * AD_HEAD_TILE);
        // one copy per head, K then V, back to back: together they read whole 1 KiB token rows
        for (int h = 0; h < nh; ++h) tma_load_4d(st + h * AD_HEAD_TILE, &tm_k, &sm.full[s], 0, h0 + h, c_key, c_seq);
        for (int h = 0; h < nh; ++h)
          tma_load_4d(st + (AD_HG + h) * AD_HEAD_TILE, &tm_v, &sm.full[s], 0, h0 + h, c_key, c_seq);
        issued = i + 1;
      }
      if (*abort_flag) {
        // Consumers have stopped: wait (bounded) for every copy still in flight before the CTA may exit.
        for (int i = issued > S ? issued - S : 0; i < issued; ++i) {
          bool done = false;
          for (uint32_t spin = 0; spin < SPIN_LIMIT && !done; ++spin) done = mbar_try_wait(&sm.full[i % S], (i / S) & 1);
          if (!done) atomicOr(a.status, B2_DEV_TIMEOUT_DRAIN);
        }
      }
    }
  } else {
    // ================================ consumers: warp w owns KV head slot w ================================
    const int g8 = lane >> 2, t4 = lane & 3;
    const int G = a.group, HQ = a.n_kv_heads * a.group;
    float m_run = AD_M_INIT, l_run = 0.f;
    int lo_tile0 = lo;   // first key of the unit's first tile (ragged: lo rounded down to a multiple of 32)
    float o[AD_D / 8][4];
    uint32_t qa[AD_D / 16][2];
    int cur_u = -1, seg_tiles = 0, cur_b = 0, cur_head = 0;
    bool active = false;  // does this warp's head exist in the current unit?
    AdCursor ccur = {0, 0, 0, 1};
    long long cur_u_begin = 0;   // ragged: index of the unit's first tile in the global list

    auto begin_unit = [&](int u) {
      cur_u = u;
      seg_tiles = 0;
      m_run = AD_M_INIT;
      l_run = 0.f;
#pragma unroll
      for (int n = 0; n < AD_D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
      cur_b = u / n_hg;
      if constexpr (RAGGED) {
        int la;
        ad_range(s_pos[cur_b], a.n_kv_ctx, a.window, lo, hi, la);
        tpu = ccur.tiles;
        cur_u_begin = (static_cast<long long>(s_pfx[cur_b]) * n_hg) + static_cast<long long>(u - cur_b * n_hg) * tpu;
        lo_tile0 = la;
      }
      cur_head = (u - cur_b * n_hg) * HGR + warp;
      active = warp < HGR && cur_head < a.n_kv_heads;
      const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
          a.q + (static_cast<size_t>(cur_b) * HQ + static_cast<size_t>(active ? cur_head : 0) * G + g8) * AD_D);
      const bool ld = active && g8 < G;
#pragma unroll
      for (int ks = 0; ks < AD_D / 16; ++ks) {
        qa[ks][0] = ld ? __ldg(qrow + ks * 8 + t4) : 0u;      // dims 16ks + 2t, +1
        qa[ks][1] = ld ? __ldg(qrow + ks * 8 + 4 + t4) : 0u;  // dims 16ks + 8 + 2t, +1
      }
    };

    // Ends the segment of unit cur_u: write the output, or a partial that the last CTA of the unit merges.
    auto end_unit = [&]() {
      const int u = cur_u;
      float l = l_run;  // every lane of a quad holds the same m and a quarter of l
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      const bool whole = (seg_tiles == tpu);
      const size_t out_row = (static_cast<size_t>(cur_b) * HQ + static_cast<size_t>(cur_head) * G + g8) * AD_D;
      if (whole) {
        if (active && g8 < G) {
          const float inv = 1.0f / (l + exp2f(load_sink_log2(a, cur_head * G + g8) - m_run));
#pragma unroll
          for (int n = 0; n < AD_D / 8; ++n)
            *reinterpret_cast<uint32_t*>(a.out + out_row + 8 * n + 2 * t4) = pack_bf16(o[n][0] * inv, o[n][1] * inv);
        }
        return;
      }
      // partial slot: 0 when this unit is the first of the CTA's chunk, else 1
      const long long u_begin = RAGGED ? cur_u_begin : static_cast<long long>(u) * tpu;
      const size_t slot = static_cast<size_t>(blockIdx.x) * 2 + (u_begin <= g_begin ? 0 : 1);
      const size_t prow = slot * AD_SLOT_ROWS + warp * AD_GMAX + g8;
      if (active) {
#pragma unroll
        for (int n = 0; n < AD_D / 8; ++n)
          *reinterpret_cast<float2*>(a.part_acc + prow * AD_D + 8 * n + 2 * t4) = make_float2(o[n][0], o[n][1]);
        if (t4 == 0) {
          a.part_ml[prow * 2] = m_run;
          a.part_ml[prow * 2 + 1] = l;
        }
      }
      __threadfence();
      named_bar_sync(1, AD_HG * 32);
      const int c_first = static_cast<int>(u_begin / chunk), c_last = static_cast<int>((u_begin + tpu - 1) / chunk);
      if (tid == 0) {
        const int old = atomicAdd(a.counters + u, 1);
        const int last = (old == c_last - c_first);
        if (last) a.counters[u] = 0;  // leave the workspace ready for the next launch
        sm.is_last = last;
      }
      named_bar_sync(1, AD_HG * 32);
      if (sm.is_last && active) {
        __threadfence();
        // lane -> row g8 of this head, 16 dims starting at 16*t4
        const size_t rsub = static_cast<size_t>(warp) * AD_GMAX + g8;
        // One pass, four parts per round trip: all loads of a round are independent, the combine is online.
        float m = AD_M_INIT, lsum = 0.f;
        float acc[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = 0.f;
        for (int c0 = c_first; c0 <= c_last; c0 += 4) {
          float pm[4], pl[4];
          float4 pa[4][4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int c = min(c0 + k, c_last);  // the tail repeats the last part; its weight is zeroed below
            // part c is slot 0 of its CTA when this unit is the first of that CTA's chunk
            const size_t sl = static_cast<size_t>(c) * 2 + (chunk * c >= u_begin ? 0 : 1);
            const size_t pr = sl * AD_SLOT_ROWS + rsub;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + pr * 2));
            pm[k] = ml.x;
            pl[k] = ml.y;
            const float4* src = reinterpret_cast<const float4*>(a.part_acc + pr * AD_D + 16 * t4);
#pragma unroll
            for (int e = 0; e < 4; ++e) pa[k][e] = __ldcg(src + e);
          }
          float m_new = m;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (c0 + k <= c_last) m_new = fmaxf(m_new, pm[k]);
          const float f0 = exp2f(m - m_new);
          lsum *= f0;
#pragma unroll
          for (int e = 0; e < 16; ++e) acc[e] *= f0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float f = c0 + k <= c_last ? exp2f(pm[k] - m_new) : 0.f;
            lsum += pl[k] * f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[4 * e] += pa[k][e].x * f; acc[4 * e + 1] += pa[k][e].y * f;
              acc[4 * e + 2] += pa[k][e].z * f; acc[4 * e + 3] += pa[k][e].w * f;
            }
          }
          m = m_new;
        }
        if (g8 < G) {
          const float inv = 1.0f / (lsum + exp2f(load_sink_log2(a, cur_head * G + g8) - m));
          uint4 w0, w1;
          w0.x = pack_bf16(acc[0] * inv, acc[1] * inv);   w0.y = pack_bf16(acc[2] * inv, acc[3] * inv);
          w0.z = pack_bf16(acc[4] * inv, acc[5] * inv);   w0.w = pack_bf16(acc[6] * inv, acc[7] * inv);
          w1.x = pack_bf16(acc[8] * inv, acc[9] * inv);   w1.y = pack_bf16(acc[10] * inv, acc[11] * inv);
          w1.z = pack_bf16(acc[12] * inv, acc[13] * inv); w1.w = pack_bf16(acc[14] * inv, acc[15] * inv);
          uint4* dst = reinterpret_cast<uint4*>(a.out + out_row + 16 * t4);
          dst[0] = w0;
          dst[1] = w1;
        }
      }
      named_bar_sync(1, AD_HG * 32);  // is_last is reused by the next segment
    };

    bool dead = false;
    for (int i = 0; i < n_my; ++i) {
      const long long g = g_begin + i;
      int u, t;
      if constexpr (RAGGED) {
        if (i == 0) ccur.seek(g, s_pfx, a.batch, n_hg);
        u = ccur.b * n_hg + ccur.hgi;
        t = ccur.t;
      } else {
        u = static_cast<int>(g / tpu);
        t = static_cast<int>(g - static_cast<long long>(u) * tpu);
      }
      if (u != cur_u) {
        if (cur_u >= 0) end_unit();
        begin_unit(u);
      }
      if constexpr (RAGGED) ccur.next(s_pfx, a.batch, n_hg);
      const int s = i % S;
      // A warp that gave up keeps walking the tile list without touching data, so that the
      // named barriers of end_unit() still see all consumer warps.
      if (!dead) {
        const bool ok = mbar_wait_bounded(&sm.full[s], (i / S) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) {  // warp-uniform decision
          if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_FULL);
          *abort_flag = 1;
          dead = true;
        }
      }
      ++seg_tiles;
      if (dead) continue;
      if (a.trace && tid == 0 && i == 0) a.trace[blockIdx.x * 8 + 1] = global_timer_ns();
      if (active) {
        const int key0 = lo_tile0 + t * AD_TK;
        uint8_t* st = tiles + static_cast<size_t>(s) * AD_STAGE_BYTES;
        const uint32_t kbase = smem_u32(st + warp * AD_HEAD_TILE);
        uint8_t* vtile = st + (AD_HG + warp) * AD_HEAD_TILE;
        const uint32_t vbase = smem_u32(vtile);
        const bool ragged = key0 + AD_TK > hi;
        if (ragged) {
          // keys >= hi hold whatever the cache holds: make their V rows zero so 0 * garbage cannot be NaN
          for (int j = lane; j < AD_TK * 8; j += 32) {
            const int row = j >> 3, ch = j & 7;
            if (key0 + row >= hi) *reinterpret_cast<uint4*>(vtile + row * 128 + ((ch ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
          }
          __syncwarp();
        }
        // ---- S = Q K^T for 32 keys: 4 n-tiles x 4 k-steps
        float sacc[4][4];
#pragma unroll
        for (int n = 0; n < 4; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
        {
          const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
          for (int ks = 0; ks < AD_D / 16; ++ks) {
            const int ch = 2 * ks + (mat & 1);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const int krow = half * 16 + (mat >> 1) * 8 + rr;
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4(kbase + krow * 128 + ((ch ^ (krow & 7)) << 4), b0, b1, b2, b3);
              mma_bf16_16816(sacc[2 * half], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
              mma_bf16_16816(sacc[2 * half + 1], qa[ks][0], 0u, qa[ks][1], 0u, b2, b3);
            }
          }
        }
        // ---- online softmax on row g8 (c0,c1 of each n-tile: keys key0 + 8n + 2t, +1)
        float x[8];
#pragma unroll
        for (int n = 0; n < 4; ++n) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int key = key0 + 8 * n + 2 * t4 + e;
            x[2 * n + e] = (key < hi && (!RAGGED || key >= lo)) ? sacc[n][e] * a.scale_log2 : -CUDART_INF_F;
          }
        }
        float mx = fmaxf(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), fmaxf(fmaxf(x[4], x[5]), fmaxf(x[6], x[7])));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float alpha = exp2f(m_run - m_new);
        float p[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) p[e] = exp2f(x[e] - m_new);
        l_run = l_run * alpha + ((p[0] + p[1]) + (p[2] + p[3])) + ((p[4] + p[5]) + (p[6] + p[7]));
        m_run = m_new;
#pragma unroll
        for (int n = 0; n < AD_D / 8; ++n) {
          o[n][0] *= alpha;
          o[n][1] *= alpha;
        }
        // ---- O += P V: 2 k-steps (16 keys each) x 8 n-tiles (8 dims each)
        {
          const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
          for (int kstep = 0; kstep < 2; ++kstep) {
            const uint32_t pa0 = pack_bf16(p[4 * kstep], p[4 * kstep + 1]);      // keys 2t, 2t+1 of this k-step
            const uint32_t pa2 = pack_bf16(p[4 * kstep + 2], p[4 * kstep + 3]);  // keys 8+2t, +1
            const int vrow = kstep * 16 + (mat & 1) * 8 + rr;
#pragma unroll
            for (int np = 0; np < AD_D / 16; ++np) {
              const int ch = 2 * np + (mat >> 1);
              uint32_t b0, b1, b2, b3;
              ldmatrix_x4_trans(vbase + vrow * 128 + ((ch ^ (vrow & 7)) << 4), b0, b1, b2, b3);
              mma_bf16_16816(o[2 * np], pa0, 0u, pa2, 0u, b0, b1);
              mma_bf16_16816(o[2 * np + 1], pa0, 0u, pa2, 0u, b2, b3);
            }
          }
        }
        if (ragged) fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.empty[s]);
    }
    if (a.trace && tid == 0) a.trace[blockIdx.x * 8 + 2] = global_timer_ns();
    if (cur_u >= 0) end_unit();
  }
  __syncthreads();
  if (tid == 0 && a.trace) a.trace[blockIdx.x * 8 + 3] = global_timer_ns();
}

static size_t attn_decode_smem_bytes(int stages) {
  return static_cast<size_t>(stages) * AD_STAGE_BYTES + sizeof(AttnDecodeSmem) + 1024;
}

}  // namespace b2

B2_API size_t b2_attn_decode_workspace_bytes(int64_t batch, int n_kv_heads, int group) {
  (void)group;
  if (batch <= 0 || n_kv_heads <= 0) return 0;
  const size_t units = static_cast<size_t>(batch) * n_kv_heads;  // head groups may be as small as one head
  const size_t max_grid = static_cast<size_t>(b2::sm_count()) * b2::AD_MAX_CTAS_PER_SM;
  const size_t counters = (units * sizeof(int) + 255) & ~static_cast<size_t>(255);
  const size_t ml = max_grid * 2 * b2::AD_SLOT_ROWS * 2 * sizeof(float);
  const size_t acc = max_grid * 2 * b2::AD_SLOT_ROWS * b2::AD_D * sizeof(float);
  return counters + ml + acc;
}

namespace {
// Shared launch path.  Uniform: start_q_dev points at ONE position, k/v are [batch, n_kv_ctx, heads, 64] at the given
// strides.  Ragged: start_q_dev points at `batch` positions; with a block table k/v are a pool of pages
// [n_pages, page_size, heads, 64] (kv_stride_b = page stride) and n_kv_ctx the capacity of a sequence.
int attn_decode_launch(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                       int64_t batch, int n_kv_heads, int group, int head_dim, int64_t n_kv_ctx, int64_t kv_stride_b,
                       int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale, int window, const void* start_q_dev,
                       int start_q_is_i64, void* workspace, size_t workspace_bytes, void* stream, bool ragged,
                       const int32_t* block_table, int64_t table_stride, int page_size, int64_t n_pages) {
  using namespace b2;
  if (!q || !k || !v || !out || !start_q_dev) return B2_ERR_NULL;
  if (batch < 0 || n_kv_heads <= 0 || group <= 0 || n_kv_ctx <= 0 || window < 0) return B2_ERR_SHAPE;
  if (head_dim != AD_D || group > AD_GMAX) return B2_ERR_UNSUPPORTED;
  if (batch * n_kv_heads > 0x3fffffff || n_kv_ctx > 0x3fffffff) return B2_ERR_UNSUPPORTED;
  if (ragged && batch > AD_RAGGED_MAX_BATCH) return B2_ERR_UNSUPPORTED;
  if (block_table) {
    if (page_size <= 0 || n_pages <= 0 || table_stride <= 0 || table_stride * page_size < n_kv_ctx) return B2_ERR_SHAPE;
    if (page_size % AD_TK != 0) return B2_ERR_UNSUPPORTED;   // a 32-key tile must lie inside one page
  }
  if (!aligned16(q) || !aligned16(out)) return B2_ERR_ALIGN;
  if (batch == 0) return B2_OK;
  if (!workspace) return B2_ERR_WORKSPACE;
  if (workspace_bytes < b2_attn_decode_workspace_bytes(batch, n_kv_heads, group)) return B2_ERR_WORKSPACE;
  if (!aligned16(workspace)) return B2_ERR_ALIGN;
  int* status = device_status_ptr();
  if (!status) return B2_ERR_DRIVER;

  CUtensorMap tm_k, tm_v;
  const uint64_t dims[4] = {static_cast<uint64_t>(AD_D), static_cast<uint64_t>(n_kv_heads),
                            static_cast<uint64_t>(block_table ? page_size : n_kv_ctx),
                            static_cast<uint64_t>(block_table ? n_pages : batch)};
  const uint64_t strides[3] = {static_cast<uint64_t>(kv_stride_h) * 2, static_cast<uint64_t>(kv_stride_n) * 2,
                               static_cast<uint64_t>(kv_stride_b) * 2};
  const uint32_t box[4] = {AD_D, 1, AD_TK, 1};
  int rc = make_tensor_map_bf16(&tm_k, k, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  rc = make_tensor_map_bf16(&tm_v, v, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;

  int grid = sm_count() * AD_MAX_CTAS_PER_SM;
  {
    const int g = tunable(TUNE_ATTN_DECODE_CTAS_PER_SM);  // experiments: a smaller grid (values > 8 are CTA counts)
    if (g > 8 && g < grid) grid = g;
  }
  AttnDecodeArgs a;
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.sinks = sinks;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.start_q = start_q_dev;
  const size_t units = static_cast<size_t>(batch) * n_kv_heads;
  const size_t counters = (units * sizeof(int) + 255) & ~static_cast<size_t>(255);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  a.counters = reinterpret_cast<int*>(ws);
  a.part_ml = reinterpret_cast<float*>(ws + counters);
  a.part_acc = reinterpret_cast<float*>(ws + counters + static_cast<size_t>(grid) * 2 * AD_SLOT_ROWS * 2 * sizeof(float));
  a.status = status;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.batch = static_cast<int>(batch);
  a.n_kv_heads = n_kv_heads;
  a.group = group;
  a.n_kv_ctx = static_cast<int>(n_kv_ctx);
  a.window = window;
  a.sinks_is_f32 = sinks_is_f32;
  a.start_q_is_i64 = start_q_is_i64;
  a.block_table = block_table;
  a.table_stride = table_stride;
  a.page_size = page_size;
  {
    size_t slots = 0;
    long long* tb = trace_buffer(&slots);
    a.trace = slots >= static_cast<size_t>(grid) ? tb : nullptr;
  }
  // Heads per CTA tile: all 8 when there is plenty of work (whole 1 KiB token rows per tile); fewer when
  // the visible range is short, so that the tiles spread over more SMs.  Only host-known bounds are
  // used (the position itself lives on the device).
  {
    const int64_t max_keys = window > 0 && window < n_kv_ctx ? window : n_kv_ctx;
    const int64_t tiles_per_seq = (max_keys + AD_TK - 1) / AD_TK + 1;
    int hg = AD_HG;
    // (only for windowed layers: their units are handed out whole, so smaller groups cost no merging)
    while (!ragged && window > 0 && max_keys <= 512 && hg > 1 &&
           batch * ((n_kv_heads + hg - 1) / hg) * tiles_per_seq < 2 * static_cast<int64_t>(grid))
      hg >>= 1;
    a.hg = hg;
  }
  const int stages = tunable(TUNE_ATTN_DECODE_STAGES);
  a.stages = stages < 1 ? 1 : stages > AD_MAX_STAGES ? AD_MAX_STAGES : stages;

  cudaError_t e;
  if (ragged) {
    const size_t smem = attn_decode_smem_bytes(a.stages) + (2 * AD_RAGGED_MAX_BATCH + 1) * sizeof(int);
    e = cudaFuncSetAttribute(attn_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    launch_overlapped(attn_decode_kernel<true>, dim3(grid), dim3(AD_THREADS), smem, static_cast<cudaStream_t>(stream), tm_k, tm_v, a);
  } else {
    const size_t smem = attn_decode_smem_bytes(a.stages);
    e = cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    launch_overlapped(attn_decode_kernel<false>, dim3(grid), dim3(AD_THREADS), smem, static_cast<cudaStream_t>(stream), tm_k, tm_v, a);
  }
  return launch_status();
}
}  // namespace

B2_API int b2_attn_decode(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                          int64_t batch, int n_kv_heads, int group, int head_dim, int64_t n_kv_ctx,
                          int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale, int window,
                          const void* start_q_dev, int start_q_is_i64, void* workspace, size_t workspace_bytes,
                          void* stream) {
  return attn_decode_launch(q, k, v, sinks, sinks_is_f32, out, batch, n_kv_heads, group, head_dim, n_kv_ctx, kv_stride_b,
                            kv_stride_n, kv_stride_h, sm_scale, window, start_q_dev, start_q_is_i64, workspace,
                            workspace_bytes, stream, false, nullptr, 0, 0, 0);
}

B2_API int b2_attn_decode_ragged(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                                 int64_t batch, int n_kv_heads, int group, int head_dim, int64_t n_kv_ctx,
                                 int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale,
                                 int window, const void* positions_dev, int positions_are_i64,
                                 const int32_t* block_table, int64_t table_stride, int page_size, int64_t n_pages,
                                 void* workspace, size_t workspace_bytes, void* stream) {
  return attn_decode_launch(q, k, v, sinks, sinks_is_f32, out, batch, n_kv_heads, group, head_dim, n_kv_ctx, kv_stride_b,
                            kv_stride_n, kv_stride_h, sm_scale, window, positions_dev, positions_are_i64, workspace,
                            workspace_bytes, stream, true, block_table, table_stride, page_size, n_pages);
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library hand the kernels their inputs and outputs but have no way to give
// them scratch: a serving process whose memory pool is fully carved up at start-up, a plugin
// running under a runtime that owns the allocator, or code that runs where cudaMalloc is not
// permitted.  For them the split-KV partials and the per-unit arrival counters live in the
// fixed array below, which is part of the library image: every GPU that loads the library holds
// these bytes until the process exits.
//
// The array is shared by every call on the device.  It keeps whatever the last call left in it,
// so the counters are cleared on the stream before each launch, and two calls whose kernels can
// overlap on the GPU (different streams, or different host threads) race on it: serialise them.
constexpr size_t AD_STATIC_MAX_UNITS = 4096;   // batch * n_kv_heads
constexpr size_t AD_STATIC_MAX_CTAS = 160;     // SM count * AD_MAX_CTAS_PER_SM (148 on B200)
constexpr size_t AD_STATIC_COUNTER_BYTES = AD_STATIC_MAX_UNITS * sizeof(int);
constexpr size_t AD_STATIC_BYTES = AD_STATIC_COUNTER_BYTES +
                                   AD_STATIC_MAX_CTAS * 2 * b2::AD_SLOT_ROWS * 2 * sizeof(float) +
                                   AD_STATIC_MAX_CTAS * 2 * b2::AD_SLOT_ROWS * b2::AD_D * sizeof(float);  // ~5.4 MiB

static __device__ __align__(256) unsigned char g_attn_decode_static_scratch[AD_STATIC_BYTES];

// Device address of the array on the current device.  The array's name is only a host-side
// handle here; the kernel needs the address cudaGetSymbolAddress returns for this device.
static void* attn_decode_static_scratch_ptr(int* rc) {
  static void* ptrs[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *rc = e != cudaSuccess ? static_cast<int>(e) : B2_ERR_UNSUPPORTED;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_decode_static_scratch);
    if (e != cudaSuccess || !p) {
      (void)cudaGetLastError();
      *rc = e != cudaSuccess ? static_cast<int>(e) : B2_ERR_DRIVER;
      return nullptr;
    }
    ptrs[dev] = p;
  }
  *rc = B2_OK;
  return ptrs[dev];
}

B2_API size_t b2_attn_decode_static_max_units(void) { return AD_STATIC_MAX_UNITS; }

B2_API int b2_attn_decode_static(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32,
                                 void* out, int64_t batch, int n_kv_heads, int group, int head_dim, int64_t n_kv_ctx,
                                 int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale,
                                 int window, const void* start_q_dev, int start_q_is_i64, void* stream) {
  if (batch < 0 || n_kv_heads <= 0) return B2_ERR_SHAPE;
  if (batch == 0) return B2_OK;
  // The fixed scratch bounds the problem: refuse anything it cannot hold.
  if (static_cast<size_t>(batch) * static_cast<size_t>(n_kv_heads) > AD_STATIC_MAX_UNITS) return B2_ERR_STATIC_LIMIT;
  if (b2_attn_decode_workspace_bytes(batch, n_kv_heads, group) > AD_STATIC_BYTES) return B2_ERR_STATIC_LIMIT;
  int rc = B2_OK;
  void* scratch = attn_decode_static_scratch_ptr(&rc);  // first call on a device resolves the address
  if (!scratch) return rc;
  // Counters must start at zero whatever an earlier (possibly abandoned) call left behind.
  cudaError_t e = cudaMemsetAsync(scratch, 0, AD_STATIC_COUNTER_BYTES, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  return b2_attn_decode(q, k, v, sinks, sinks_is_f32, out, batch, n_kv_heads, group, head_dim, n_kv_ctx, kv_stride_b,
                        kv_stride_n, kv_stride_h, sm_scale, window, start_q_dev, start_q_is_i64, scratch,
                        AD_STATIC_BYTES, stream);
}
