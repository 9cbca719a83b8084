// Prefill attention: causal GQA softmax attention with per-head sinks and an optional sliding
// window, for T query tokens at absolute positions start_q .. start_q+T-1 against a contiguous
// K/V tensor (fresh k/v of the prompt, or the KV cache itself), head_dim 64.
//
// At head_dim 64 the exponential unit, not the tensor pipe, is the first limit (one exp per score
// against 256 flops), so the kernel is organised around keeping the softmax warps busy.  A work unit is
// 128 consecutive query tokens of one query head; the kernel is persistent: two CTAs per SM (half of
// tensor memory and ~112 KiB of shared memory each) walk the unit list, heaviest units (latest
// positions) first and in serpentine order so that every CTA gets the same mix.  Inside a CTA
//   warp 0   : TMA producer, whole-warp loop with one elected lane issuing: the Q tile of each unit
//              (two buffers, so the next unit's Q arrives early), then K and V blocks (64 keys x 64 dims,
//              128-byte rows, 128B swizzle) through a five-stage ring that runs across unit
//              boundaries, straight from the [B, T, H, 64] layout;
//   warp 1   : walks the block list as a whole warp (descriptors stay warp-uniform), one elected lane
//              issues the tcgen05 MMAs: S_j = Q K_j^T (M=128, N=64, K=64) into one of three S buffers in
//              tensor memory, always three blocks ahead of the softmax - also across a unit boundary -
//              and O += P_j V_j (M=128, N=64, K=64) with P_j read from tensor memory (the A operand),
//              V_j as an MN-major shared-memory operand and O accumulating in tensor memory;
//   warps 2-5: one thread per query row: S row -> registers in one pass, row max, exp2 on the
//              special-function unit, row sum, bf16 pack of P_j over the first half of the buffer S_j
//              came from.  The running maximum is only advanced (and O rescaled in tensor memory) when
//              it grows by more than 2^8, so the rescale is rare.  Blocks that touch the causal
//              diagonal, the window edge or the end of the keys carry a second bf16 term of P (in the
//              second half of the same buffer), so rows with few visible keys keep fp32-like weights.
//              After the last block of a unit they read O, hand the accumulator back to the MMA warp
//              and store the rows.
// The tensor pipe executes one thread's MMAs in issue order, which is what lets S_{j+3} overwrite the
// buffer of S_j / P_j right after P_j V_j has been issued, with no barrier in between.  The round trip
// "P written -> MMA warp wakes -> P V and Q K issued behind the other CTA's MMAs -> completion seen by
// the softmax warps" was measured at about 1300 clocks against 1800 per block: with two S buffers and
// separate P buffers every block waited some 250 clocks for its S and again for its P buffer; the
// third buffer takes both waits off the softmax warps' path.  The sink logit joins the denominator at
// the end.  All waits are bounded.
//
// Where a block's ~1650 clocks go (per-phase SM-clock counters of a -DAP_PHASE_TRACE=1 build, T = 8192): 830 in the
// 64 exponentials per row and their stores (512 would be the special-function unit alone; the other CTA's warp on the
// same sub-core shares it), ~250 each in the first synchronising instruction after the store burst and in
// load-latency + row maximum, ~300 in bookkeeping; a unit boundary costs another ~4500 (2400-3000 of it the wait for
// the last P V to come back through the MMA warp, whose own loop needs ~800 clocks per block to issue eight MMAs and
// three commits).  Variants measured on the same case and dropped, each within +-2 % or slower: eight softmax warps
// splitting the columns of a row (exchange of row maxima through shared memory, 25 % slower), fetching the next
// block's scores before the store drain, packed fp32x2 arithmetic, moving the rescale vote behind the exponentials,
// requesting the next unit's Q tile three blocks into the current unit, and writing a unit's output one block late
// (after the first block of the next unit: 5 % slower, the larger loop body spills).
#include <math_constants.h>

#include <algorithm>

#include "tc_common.cuh"

namespace b2 {

constexpr int AP_BM = 128;       // query rows per unit
constexpr int AP_BN = 64;        // keys per block
constexpr int AP_D = 64;
constexpr int AP_THREADS = 192;
constexpr int AP_DEFAULT_POLY = 0;   // pairs of exponentials per pair computed on the FMA pipe (0: none); tunable "attn_prefill_poly"
constexpr int AP_STAGES = 5;     // K+V blocks in flight per CTA (S = Q K^T runs three blocks ahead of O += P V)
constexpr int AP_NSP = 3;        // S / P buffers in tensor memory
constexpr int AP_Q_BYTES = AP_BM * AP_D * 2;     // 16 KiB
constexpr int AP_KV_BYTES = AP_BN * AP_D * 2;    // 8 KiB
constexpr float AP_M_INIT = -1.0e30f;
constexpr float AP_RESCALE_STEP = 8.0f;          // log2 units the maximum may lag behind
// tensor-memory columns of a CTA: three S buffers (64 fp32 each; P_j, 64 bf16 packed in pairs, overwrites columns
// 0..31 of the buffer of S_j and its second term columns 32..63), O (64 fp32)
constexpr uint32_t AP_COL_S = 0, AP_COL_O = AP_NSP * AP_BN, AP_TMEM_COLS = 256;
static_assert(AP_COL_O + AP_D <= AP_TMEM_COLS, "tensor-memory budget of one of two CTAs per SM");

struct AttnPrefillArgs {
  const void* sinks;
  __nv_bfloat16* out;  // [B, T, Hq*64]
  const void* start_q;
  int* status;
  float scale_log2;
  int T, Tk, n_q_heads, group, window;
  int sinks_is_f32, start_q_is_i64;
  int n_qblk, n_units;  // query blocks per sequence; units = n_qblk * n_q_heads * batch
  long long* trace;     // optional [CTA][8] (b2_set_trace_buffer): start ns, end ns, units, blocks
};

// Diagnostic build (-DAP_PHASE_TRACE=1): every softmax warp adds up the SM clocks it spends per phase of a block; the
// trace buffer then needs four rows of 8 slots per CTA, row = (warp - 2) * gridDim.x + blockIdx.x: slot 2 = the warp's
// whole loop (low 32 bits) and store drain + arrive (high), slot 3 = blocks (low) and rescale vote / P wait (high),
// slots 4..7 = wait for S, tensor-memory load issue, load latency + row maximum, exponentials + pack + stores.
// `cases.py attn_prefill --phase-trace` prints them.
#ifndef AP_PHASE_TRACE
#define AP_PHASE_TRACE 0
#endif
#if AP_PHASE_TRACE
#define AP_CLK(var) const uint32_t var = static_cast<uint32_t>(clock())
#define AP_ACC(acc, t1, t0) acc += (t1) - (t0)
#else
#define AP_CLK(var)
#define AP_ACC(acc, t1, t0)
#endif

struct AttnPrefillSmem {   // placed at the 1024-byte aligned start of dynamic shared memory
  uint8_t q[2][AP_Q_BYTES];
  uint8_t k[AP_STAGES][AP_KV_BYTES];
  uint8_t v[AP_STAGES][AP_KV_BYTES];
  uint64_t q_full[2];
  uint64_t q_empty[2];  // MMA -> producer: every S = Q K^T of the unit has been computed
  uint64_t kv_full[AP_STAGES];
  uint64_t kv_empty[AP_STAGES];
  uint64_t s_full[AP_NSP];   // MMA -> softmax: S_j is in buffer j%3
  uint64_t p_full[AP_NSP];   // softmax -> MMA: P_j is in buffer j%3
  // MMA -> softmax: O += P_j V_j has completed (slot j%3; awaited only to rescale or read O).  Three slots, like the
  // S buffers: a softmax thread that has seen S_j knows that P_{j-3} V_{j-3} (issued before Q K_j^T) has completed,
  // i.e. every earlier phase of slot j%3, so its rare parity waits on this slot can never be one phase off.
  uint64_t pv_done[AP_NSP];
  uint64_t o_free;      // softmax -> MMA: O of the finished unit has been read
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// One work unit: 128 query rows of one head, and the key blocks they can see.
struct ApUnit {
  int q0, head, b, kvh;
  int p_first;  // absolute position of row 0
  int blk_lo;   // first visible 64-key block
  int nblk;     // number of visible blocks (0: nothing to attend to)
};

__device__ __forceinline__ ApUnit ap_unit(const AttnPrefillArgs& a, int u, int sq) {
  ApUnit w;
  const int per_q = a.n_units / a.n_qblk;             // heads * batch
  const int qblk = a.n_qblk - 1 - u / per_q;          // heaviest query blocks first
  const int rem = u % per_q;
  w.b = rem / a.n_q_heads;
  w.head = rem % a.n_q_heads;
  w.kvh = w.head / a.group;
  w.q0 = qblk * AP_BM;
  w.p_first = sq + w.q0;
  const int p_last = sq + min(w.q0 + AP_BM, a.T) - 1;  // position of the last real row
  const int hi = min(p_last + 1, a.Tk);                // keys [lo, hi) can be visible
  const int lo = a.window > 0 ? max(w.p_first - a.window + 1, 0) : 0;
  w.blk_lo = min(lo, hi) / AP_BN;
  w.nblk = hi > lo ? (hi + AP_BN - 1) / AP_BN - w.blk_lo : 0;
  return w;
}
// Does any row of the unit see a masked key in its block j (causal diagonal, window edge, end of keys)?
__device__ __forceinline__ bool ap_block_is_masked(const AttnPrefillArgs& a, const ApUnit& w, int j) {
  const int key0 = (w.blk_lo + j) * AP_BN;
  return (key0 + AP_BN - 1 > w.p_first) || (key0 + AP_BN > a.Tk) ||
         (a.window > 0 && key0 < w.p_first + AP_BM - a.window);
}
// The i-th unit of this CTA: rounds of gridDim.x units, every other round walked backwards.
__device__ __forceinline__ int ap_unit_index(int i) {
  const int g = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  return i * g + ((i & 1) ? g - 1 - c : c);
}

// EXP16 (tunable "attn_prefill_exp16", off): the probabilities are computed two per special-function instruction on
// fp16 pairs (see ex2_f16x2), which halves the work of the exponential unit.  Measured 5 % SLOWER than one fp32
// exponential per score (config 3 full causal: 285.7 against 271.4 us; parity still green): the pack and unpack
// conversions cost more issue slots than the exponential unit gives back, i.e. the softmax warps are bound by
// instruction issue and dependency latency, not by that unit.  Kept as the record of the experiment.
// POLY (tunable "attn_prefill_poly", off): on blocks without masked scores, one pair of exponentials in every POLY pairs
// is computed on the FMA pipe (ex2_poly) instead of the special-function unit, which two CTAs' softmax warps share.
// Measured slower (config 3 full causal: 259 us without, 277 us with every 4th pair, 299 us with every 2nd; parity
// green): like the fp16-pair experiment it says the softmax warps are not waiting for the special-function unit.
template <bool EXP16, int POLY>
__global__ void __launch_bounds__(AP_THREADS, 2)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const AttnPrefillArgs a) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  AttnPrefillSmem& sm = *reinterpret_cast<AttnPrefillSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if ((smem_u32(smem_raw) & 1023u) != 0) {  // the swizzled tiles need this alignment; never seen to fail
    if (tid == 0) atomicOr(a.status, B2_DEV_BAD_INDEX);
    return;
  }

  // A launch that follows a failed wait on this device does nothing: the status word stays set until the
  // host has read and cleared it, so a failure costs one time limit, not one per CTA.
  if (tid == 0) sm.abort_flag = *static_cast<volatile int*>(a.status);
  __syncthreads();
  if (sm.abort_flag != 0) return;
  __syncthreads();
  if (tid == 0) {
    for (int s = 0; s < AP_STAGES; ++s) {
      mbar_init(&sm.kv_full[s], 1);
      mbar_init(&sm.kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sm.q_full[s], 1);
      mbar_init(&sm.q_empty[s], 1);
    }
    for (int s = 0; s < AP_NSP; ++s) {
      mbar_init(&sm.pv_done[s], 1);
      mbar_init(&sm.s_full[s], 1);
      mbar_init(&sm.p_full[s], 4);
    }
    mbar_init(&sm.o_free, 4);
    sm.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) tmem_alloc(&sm.tmem_base, AP_TMEM_COLS);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;
  long long* trace = a.trace ? a.trace + 8ll * blockIdx.x : nullptr;
  if (trace && tid == 0) trace[0] = global_timer_ns();

  const long long sq64 = a.start_q_is_i64 ? *static_cast<const long long*>(a.start_q)
                                          : static_cast<long long>(*static_cast<const int*>(a.start_q));
  const int sq = static_cast<int>(sq64 < 0 ? 0 : (sq64 > 0x3fffffff ? 0x3fffffff : sq64));  // fits in 31 bits

  if (warp == 0) {
    // ===================================== TMA producer =====================================
    const bool leader = elect_one();
    int g = 0, ui = 0;  // blocks and (non-empty) units issued so far
    bool ok = true;
    for (int i = 0; ok; ++i) {
      const int u = ap_unit_index(i);
      if (u >= a.n_units) break;
      const ApUnit w = ap_unit(a, u, sq);
      if (w.nblk == 0) continue;
      const int qb = ui & 1;
      if (ui >= 2) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm.q_empty[qb], ((ui >> 1) - 1) & 1, abort_flag));
      if (!ok) break;
      if (leader) {
        mbar_arrive_expect_tx(&sm.q_full[qb], AP_Q_BYTES);
        tma_load_4d(sm.q[qb], &tm_q, &sm.q_full[qb], 0, w.head, w.q0, w.b);
      }
      __syncwarp();
      for (int j = 0; j < w.nblk; ++j, ++g) {
        const int s = g % AP_STAGES, round = g / AP_STAGES;
        if (round > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm.kv_empty[s], (round - 1) & 1, abort_flag));
        if (!ok) break;
        const int key0 = (w.blk_lo + j) * AP_BN;
        if (leader) {
          mbar_arrive_expect_tx(&sm.kv_full[s], 2 * AP_KV_BYTES);
          tma_load_4d(sm.k[s], &tm_k, &sm.kv_full[s], 0, w.kvh, key0, w.b);
          tma_load_4d(sm.v[s], &tm_v, &sm.kv_full[s], 0, w.kvh, key0, w.b);
        }
        __syncwarp();
      }
      if (ok) ++ui;
    }
    if (leader) {
      if (!ok) {
        if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_EMPTY);
        *abort_flag = 1;
      }
      if (*abort_flag) {  // wait (bounded) for what may still be in flight before the CTA may exit
        for (int qb = 0; qb < 2 && qb <= ui; ++qb) {
          const int uu = ui - qb;  // the two most recent Q loads: units ui (if started) and ui-1
          bool done = false;
          for (uint32_t spin = 0; spin < SPIN_LIMIT && !done; ++spin) done = mbar_try_wait(&sm.q_full[uu & 1], (uu >> 1) & 1);
        }
        for (int gg = g > AP_STAGES ? g - AP_STAGES : 0; gg < g; ++gg) {
          bool done = false;
          for (uint32_t spin = 0; spin < SPIN_LIMIT && !done; ++spin)
            done = mbar_try_wait(&sm.kv_full[gg % AP_STAGES], (gg / AP_STAGES) & 1);
          if (!done) atomicOr(a.status, B2_DEV_TIMEOUT_DRAIN);
        }
      }
    }
  } else if (warp == 1) {
    // ===================================== MMA issuer =====================================
    // Two cursors over the CTA's flat stream of blocks: S = Q K^T runs three blocks ahead of O += P V,
    // across unit boundaries too.
    const bool leader = elect_one();
    constexpr uint32_t IDESC_QK = umma_idesc_bf16(AP_BM, AP_BN);
    constexpr uint32_t IDESC_PV = umma_idesc_bf16_b_mn(AP_BM, AP_D);
    struct Cursor {
      int i, j, ui, g;  // unit iteration of this CTA, block inside the unit, non-empty unit count, flat block index
      ApUnit w;
      bool valid;
    };
    auto seek = [&](Cursor& c) {  // moves c.i forward to the next unit that has blocks
      for (;; ++c.i) {
        const int u = ap_unit_index(c.i);
        if (u >= a.n_units) {
          c.valid = false;
          return;
        }
        c.w = ap_unit(a, u, sq);
        if (c.w.nblk > 0) {
          c.valid = true;
          return;
        }
      }
    };
    auto advance = [&](Cursor& c) {
      ++c.g;
      if (++c.j >= c.w.nblk) {
        c.j = 0;
        ++c.ui;
        ++c.i;
        seek(c);
      }
    };
    Cursor cq{0, 0, 0, 0, {}, false}, cp{0, 0, 0, 0, {}, false};
    seek(cq);
    cp = cq;
    bool ok = true;
    auto wait_kv = [&](const Cursor& c) -> bool {
      return __all_sync(0xffffffffu,
                        mbar_wait_bounded(&sm.kv_full[c.g % AP_STAGES], (c.g / AP_STAGES) & 1, abort_flag));
    };
    auto issue_qk = [&](const Cursor& c) -> bool {  // K of this block has landed
      const int qb = c.ui & 1;
      if (c.j == 0 && !__all_sync(0xffffffffu, mbar_wait_bounded(&sm.q_full[qb], (c.ui >> 1) & 1, abort_flag)))
        return false;
      tc_fence_after_sync();
      const uint64_t dq = umma_desc_k128(smem_u32(sm.q[qb]));
      const uint64_t dk = umma_desc_k128(smem_u32(sm.k[c.g % AP_STAGES]));
      const uint32_t ts = tmem + AP_COL_S + (c.g % AP_NSP) * AP_BN;
      if (leader) {
#pragma unroll
        for (int k = 0; k < AP_D / 16; ++k) umma_bf16(ts, dq + 2 * k, dk + 2 * k, IDESC_QK, k != 0);
        umma_commit(&sm.s_full[c.g % AP_NSP]);
        if (c.j == c.w.nblk - 1) umma_commit(&sm.q_empty[qb]);  // the unit's Q tile is no longer needed
      }
      __syncwarp();
      return true;
    };
    for (int ahead = 0; ahead < AP_NSP && ok && cq.valid; ++ahead) {
      ok = wait_kv(cq) && issue_qk(cq);
      if (ok) advance(cq);
    }
    while (ok && cp.valid) {
      // K of the block three ahead is usually there long before P of this one: take that wait off the critical path
      if (cq.valid) ok = wait_kv(cq);
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm.p_full[cp.g % AP_NSP], (cp.g / AP_NSP) & 1, abort_flag));
      if (!ok) break;
      if (cp.j == 0 && cp.ui > 0) {  // the previous unit's O must have been read out
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&sm.o_free, (cp.ui - 1) & 1, abort_flag));
        if (!ok) break;
      }
      tc_fence_after_sync();
      const int s = cp.g % AP_STAGES;
      const uint64_t dv = umma_desc_k128(smem_u32(sm.v[s]));
      const uint32_t tp = tmem + AP_COL_S + (cp.g % AP_NSP) * AP_BN;   // P_j: first half of the buffer S_j came in
      const uint32_t tl = tp + AP_BN / 2;                              // its second bf16 term: second half
      const bool masked = ap_block_is_masked(a, cp.w, cp.j);
      if (leader) {
#pragma unroll
        for (int k = 0; k < AP_BN / 16; ++k)  // 16 keys: 8 packed P columns, 16 V rows (2048 B)
          umma_bf16_ts(tmem + AP_COL_O, tp + 8 * k, dv + 128 * k, IDESC_PV, (cp.j | k) != 0);
        if (masked) {  // second bf16 term of P
#pragma unroll
          for (int k = 0; k < AP_BN / 16; ++k) umma_bf16_ts(tmem + AP_COL_O, tl + 8 * k, dv + 128 * k, IDESC_PV, 1u);
        }
        umma_commit(&sm.kv_empty[s]);
        umma_commit(&sm.pv_done[cp.g % AP_NSP]);
      }
      __syncwarp();
      // the buffer of this block is free for the block three ahead: the pipe runs it after the MMAs just issued
      if (cq.valid) {
        ok = issue_qk(cq);
        if (ok) advance(cq);
      }
      advance(cp);
    }
    if (!ok && leader) {
      if (!*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
      *abort_flag = 1;
    }
  } else {
    // ===================================== softmax / output =====================================
    const int lane_grp = warp & 3;                 // a warp may only touch TMEM lanes 32*(warp%4) .. +31
    const int r = lane_grp * 32 + lane;            // query row of this thread inside the unit
    const uint32_t trow = tmem + (static_cast<uint32_t>(lane_grp * 32) << 16);
    const float scale_log2 = a.scale_log2;
    int g0 = 0, ui = 0;                            // flat block index of the unit's first block; non-empty units done
    bool dead = false;
    auto give_up = [&]() {
      if (lane == 0 && !*abort_flag) atomicOr(a.status, B2_DEV_TIMEOUT_MMA);
      *abort_flag = 1;
      dead = true;
    };

#if AP_PHASE_TRACE
    uint32_t ph_s = 0, ph_ld = 0, ph_mx = 0, ph_ex = 0, ph_st = 0, ph_pw = 0;
    const uint32_t ph_begin = static_cast<uint32_t>(clock());
#endif
    for (int i = 0; !dead; ++i) {
      const int u = ap_unit_index(i);
      if (u >= a.n_units) break;
      const ApUnit w = ap_unit(a, u, sq);
      const int pos = w.p_first + r;               // absolute position of this thread's row
      const bool row_ok = w.q0 + r < a.T;
      uint4* dst = reinterpret_cast<uint4*>(
          a.out + ((static_cast<size_t>(w.b) * a.T + w.q0 + r) * a.n_q_heads + w.head) * AP_D);
      if (w.nblk == 0) {  // nothing visible: the output rows are zero
        if (row_ok) {
#pragma unroll
          for (int q4 = 0; q4 < AP_D / 8; ++q4) dst[q4] = make_uint4(0u, 0u, 0u, 0u);
        }
        continue;
      }
      float m_run = AP_M_INIT, l_run = 0.f;
      for (int j = 0; j < w.nblk && !dead; ++j) {
        const int g = g0 + j;
        const int buf = g % AP_NSP;
        AP_CLK(c0);
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.s_full[buf], (g / AP_NSP) & 1, abort_flag))) {
          give_up();
          break;
        }
        tc_fence_after_sync();
        AP_CLK(c1);
        AP_ACC(ph_s, c1, c0);
        // ---- the whole S row of this thread, one pass
        float sv[AP_BN];
        const uint32_t ts = trow + AP_COL_S + buf * AP_BN;
        tmem_ld_32x32_nowait(ts, *reinterpret_cast<float(*)[32]>(&sv[0]));
        tmem_ld_32x32_nowait(ts + 32, *reinterpret_cast<float(*)[32]>(&sv[32]));
        tmem_wait_ld();
        AP_CLK(c2);
        AP_ACC(ph_ld, c2, c1);
        const bool masked = ap_block_is_masked(a, w, j);
        if (masked) {
          const int key0 = (w.blk_lo + j) * AP_BN;
          const int vis_hi = min(pos, a.Tk - 1) - key0;                        // last visible column
          const int vis_lo = (a.window > 0 ? pos - a.window + 1 : 0) - key0;   // first visible column
#pragma unroll
          for (int c = 0; c < AP_BN; ++c)
            if (c > vis_hi || c < vis_lo) sv[c] = -CUDART_INF_F;
        }
        float mx0 = max3(sv[0], sv[1], sv[2]), mx1 = max3(sv[3], sv[4], sv[5]);
        float mx2 = max3(sv[6], sv[7], sv[8]), mx3 = max3(sv[9], sv[10], sv[11]);
#pragma unroll
        for (int c = 12; c + 7 < AP_BN; c += 8) {
          mx0 = max3(mx0, sv[c], sv[c + 1]);
          mx1 = max3(mx1, sv[c + 2], sv[c + 3]);
          mx2 = max3(mx2, sv[c + 4], sv[c + 5]);
          mx3 = max3(mx3, sv[c + 6], sv[c + 7]);
        }
        mx0 = max3(mx0, sv[60], sv[61]);  // 12 + 6*8 = 60: columns 60..63 remain
        mx1 = max3(mx1, sv[62], sv[63]);
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // ---- advance the running maximum only when it lags by more than 2^8
        const float m_blk = mx * scale_log2;
        const bool grow = m_blk > m_run + AP_RESCALE_STEP;
        float alpha = 1.f;
        if (grow) {
          alpha = ex2_approx(m_run - m_blk);
          m_run = m_blk;
        }
#if AP_PHASE_TRACE
        const uint32_t c2b = static_cast<uint32_t>(clock()) + (__float_as_uint(m_run) & 0u);   // after the maximum is known
#endif
        if (j > 0 && __any_sync(0xffffffffu, grow)) {  // rare: bring O to the new maximum, in tensor memory
          // every MMA issued so far must have finished with O
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.pv_done[(g - 1) % AP_NSP], ((g - 1) / AP_NSP) & 1, abort_flag))) {
            give_up();
            break;
          }
          tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < AP_D; c += 32) {
            float ov[32];
            tmem_ld_32x32(trow + AP_COL_O + c, ov);
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] *= alpha;
            tmem_st_32x32(trow + AP_COL_O + c, ov);
          }
        }
        // ---- probabilities, row sum, bf16 pack into the P buffer
        AP_CLK(c3);
        AP_ACC(ph_mx, c2b, c2);
        AP_ACC(ph_pw, c3, c2b);
        const float neg_m = -m_run;
        // P overwrites the scores it was computed from (they are in registers by now); the P V that read the
        // previous contents of this buffer ran before the Q K^T that produced these scores
        const uint32_t tp = ts;
        float sum0 = 0.f, sum1 = 0.f;
        if (!masked) {
#pragma unroll
          for (int c = 0; c < AP_BN; c += 32) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              float p0, p1;
              if constexpr (EXP16) {
                const uint32_t ph = ex2_f16x2(f32x2_to_f16x2(fmaf(sv[c + e], scale_log2, neg_m), fmaf(sv[c + e + 1], scale_log2, neg_m)));
                p0 = f16lo_to_f32(ph);
                p1 = f16hi_to_f32(ph);
              } else {
                if (POLY > 0 && ((e >> 1) % (POLY > 0 ? POLY : 1)) == (POLY > 0 ? POLY : 1) - 1) {
                  p0 = ex2_poly(fmaf(sv[c + e], scale_log2, neg_m));
                  p1 = ex2_poly(fmaf(sv[c + e + 1], scale_log2, neg_m));
                } else {
                  p0 = ex2_approx(fmaf(sv[c + e], scale_log2, neg_m));
                  p1 = ex2_approx(fmaf(sv[c + e + 1], scale_log2, neg_m));
                }
              }
              sum0 += p0;
              sum1 += p1;
              pk[e >> 1] = pack_bf16(p0, p1);
            }
            tmem_st_32x16(tp + (c >> 1), pk);
          }
        } else {
#pragma unroll
          for (int c = 0; c < AP_BN; c += 32) {
            uint32_t pk[16], pl[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              // a masked score is -inf: 2^(-inf) = 0
              float p0, p1;
              if constexpr (EXP16) {
                const uint32_t ph = ex2_f16x2(f32x2_to_f16x2(fmaf(sv[c + e], scale_log2, neg_m), fmaf(sv[c + e + 1], scale_log2, neg_m)));
                p0 = f16lo_to_f32(ph);
                p1 = f16hi_to_f32(ph);
              } else {
                p0 = ex2_approx(fmaf(sv[c + e], scale_log2, neg_m));
                p1 = ex2_approx(fmaf(sv[c + e + 1], scale_log2, neg_m));
              }
              sum0 += p0;
              sum1 += p1;
              pk[e >> 1] = pack_bf16(p0, p1);
              pl[e >> 1] = pack_bf16(p0 - bf16lo(pk[e >> 1]), p1 - bf16hi(pk[e >> 1]));
            }
            tmem_st_32x16(tp + (c >> 1), pk);
            tmem_st_32x16(ts + AP_BN / 2 + (c >> 1), pl);
          }
        }
        AP_CLK(c4);
        AP_ACC(ph_ex, c4, c3);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.p_full[buf]);
        AP_CLK(c5);
        AP_ACC(ph_st, c5, c4);
        l_run = l_run * alpha + (sum0 + sum1);
      }
      if (dead) break;

      // ---- the unit's last P V has completed: read O, hand the accumulator back, store the rows
      const int gl = g0 + w.nblk - 1;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&sm.pv_done[gl % AP_NSP], (gl / AP_NSP) & 1, abort_flag))) {
        give_up();
        break;
      }
      tc_fence_after_sync();
      float o[AP_D];
      tmem_ld_32x32_nowait(trow + AP_COL_O, *reinterpret_cast<float(*)[32]>(&o[0]));
      tmem_ld_32x32_nowait(trow + AP_COL_O + 32, *reinterpret_cast<float(*)[32]>(&o[32]));
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.o_free);
      if (row_ok) {
        float sink = 0.f;
        if (a.sinks)
          sink = a.sinks_is_f32 ? static_cast<const float*>(a.sinks)[w.head]
                                : __bfloat162float(static_cast<const __nv_bfloat16*>(a.sinks)[w.head]);
        const float z = l_run + exp2f(sink * 1.4426950408889634f - m_run);
        const float inv = 1.0f / z;
#pragma unroll
        for (int q4 = 0; q4 < AP_D / 8; ++q4) {
          uint4 t;
          t.x = pack_bf16(o[8 * q4 + 0] * inv, o[8 * q4 + 1] * inv);
          t.y = pack_bf16(o[8 * q4 + 2] * inv, o[8 * q4 + 3] * inv);
          t.z = pack_bf16(o[8 * q4 + 4] * inv, o[8 * q4 + 5] * inv);
          t.w = pack_bf16(o[8 * q4 + 6] * inv, o[8 * q4 + 7] * inv);
          dst[q4] = t;
        }
      }
      g0 += w.nblk;
      ++ui;
    }
#if AP_PHASE_TRACE
    if (trace && lane == 0) trace += 8ll * gridDim.x * (warp - 2);   // diagnostic buffer: four rows per CTA
    if (trace && lane == 0) {
#else
    if (trace && warp == 2 && lane == 0) {
#endif
      trace[2] = ui;
      trace[3] = g0;
#if AP_PHASE_TRACE
      trace[3] = static_cast<long long>(g0) | (static_cast<long long>(ph_pw) << 32);
      trace[2] = static_cast<long long>(static_cast<uint32_t>(clock()) - ph_begin) | (static_cast<long long>(ph_st) << 32);
      trace[4] = ph_s;
      trace[5] = ph_ld;
      trace[6] = ph_mx;
      trace[7] = ph_ex;
#endif
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (trace && tid == 0) trace[1] = global_timer_ns();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, AP_TMEM_COLS);
  }
}

}  // namespace b2

B2_API int b2_attn_prefill(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                           int64_t batch, int64_t tokens, int64_t n_kv_ctx, int n_kv_heads, int group, int head_dim,
                           int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale, int window,
                           const void* start_q_dev, int start_q_is_i64, void* stream) {
  using namespace b2;
  if (batch < 0 || tokens < 0 || n_kv_ctx <= 0 || n_kv_heads <= 0 || group <= 0 || window < 0) return B2_ERR_SHAPE;
  if (head_dim != AP_D || tokens > 0x3fffffff || n_kv_ctx > 0x3fffffff || batch > 65535 ||
      static_cast<int64_t>(n_kv_heads) * group > 65535)
    return B2_ERR_UNSUPPORTED;
  if (batch == 0 || tokens == 0) return B2_OK;
  if (!q || !k || !v || !out || !start_q_dev) return B2_ERR_NULL;
  if (!aligned16(q) || !aligned16(out)) return B2_ERR_ALIGN;
  int* status = device_status_ptr();
  if (!status) return B2_ERR_DRIVER;
  const int hq = n_kv_heads * group;

  CUtensorMap tm_q, tm_k, tm_v;
  const uint64_t qd[4] = {AP_D, static_cast<uint64_t>(hq), static_cast<uint64_t>(tokens), static_cast<uint64_t>(batch)};
  const uint64_t qs[3] = {AP_D * 2ull, static_cast<uint64_t>(hq) * AP_D * 2, static_cast<uint64_t>(tokens) * hq * AP_D * 2};
  const uint64_t kd[4] = {AP_D, static_cast<uint64_t>(n_kv_heads), static_cast<uint64_t>(n_kv_ctx),
                          static_cast<uint64_t>(batch)};
  const uint64_t ks[3] = {static_cast<uint64_t>(kv_stride_h) * 2, static_cast<uint64_t>(kv_stride_n) * 2,
                          static_cast<uint64_t>(kv_stride_b) * 2};
  const uint32_t qbox[4] = {AP_D, 1, AP_BM, 1};
  const uint32_t kbox[4] = {AP_D, 1, AP_BN, 1};
  int rc = make_tensor_map_bf16(&tm_q, q, 4, qd, qs, qbox, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  rc = make_tensor_map_bf16(&tm_k, k, 4, kd, ks, kbox, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;
  rc = make_tensor_map_bf16(&tm_v, v, 4, kd, ks, kbox, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != B2_OK) return rc;

  AttnPrefillArgs a;
  a.sinks = sinks;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.start_q = start_q_dev;
  a.status = status;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.T = static_cast<int>(tokens);
  a.Tk = static_cast<int>(n_kv_ctx);
  a.n_q_heads = hq;
  a.group = group;
  a.window = window;
  a.sinks_is_f32 = sinks_is_f32;
  a.start_q_is_i64 = start_q_is_i64;
  a.n_qblk = static_cast<int>((tokens + AP_BM - 1) / AP_BM);
  const int64_t units = static_cast<int64_t>(a.n_qblk) * hq * batch;
  if (units > 0x7fffffff) return B2_ERR_UNSUPPORTED;
  a.n_units = static_cast<int>(units);

  const size_t smem = sizeof(AttnPrefillSmem);
  const bool exp16 = tunable(TUNE_ATTN_PREFILL_EXP16) != 0;
  const int poly = tunable(TUNE_ATTN_PREFILL_POLY) < 0 ? 0 : (tunable(TUNE_ATTN_PREFILL_POLY) == 0 ? AP_DEFAULT_POLY : tunable(TUNE_ATTN_PREFILL_POLY));
  auto kernel = exp16 ? attn_prefill_kernel<true, 0>
                      : (poly == 2 ? attn_prefill_kernel<false, 2> : (poly == 4 ? attn_prefill_kernel<false, 4> : attn_prefill_kernel<false, 0>));
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return B2_ERR_DRIVER;
  const int grid = static_cast<int>(std::min<int64_t>(units, 2ll * sms));  // persistent: two CTAs per SM
  {
    size_t slots = 0;
    long long* tb = trace_buffer(&slots);
    a.trace = slots >= static_cast<size_t>(grid) ? tb : nullptr;
  }
  kernel<<<grid, AP_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, a);
  return launch_status();
}
