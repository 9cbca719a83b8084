// Argument block and epilogue ids of the tcgen05 GEMM kernels (gemm_tc.cu), shared with the MoE prompt path.
#pragma once

#include "tc_common.cuh"

namespace b2 {

constexpr int GT_BM = 128;
constexpr int GT_BK = 64;
constexpr int GT_EPI_WARPS = 8;                     // two per tensor-memory lane quadrant, alternating 64-column chunks
constexpr int GT_THREADS = 64 + 32 * GT_EPI_WARPS;
constexpr int GT_A_BYTES = GT_BM * GT_BK * 2;  // 16 KiB
enum { EPI_PLAIN = 0, EPI_QKV_ROPE = 1, EPI_RESIDUAL = 2, EPI_ROUTER = 3, EPI_MOE_SWIGLU = 4, EPI_MOE_GATE = 5 };

struct GemmArgs {
  int M, N, K, tiles_m, tiles_n, stages;
  int vec_ok;  // outputs/bias/residual are 16-byte aligned with leading dimensions that are multiples of 8
  const __nv_bfloat16* bias;
  const float* bias_f32;
  __nv_bfloat16* out;
  int64_t ld_out;
  const __nv_bfloat16* residual;
  int64_t ld_res;
  float* out_f32;
  int64_t ld_out_f32;
  // EPI_QKV_ROPE
  const float* sin_tab;
  const float* cos_tab;
  const int64_t* offset;
  int64_t max_ctx;
  int tokens, n_q, n_kv, kv_add_offset, round_before_rope;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_out;
  __nv_bfloat16* v_out;
  int64_t kv_sb, kv_sn, kv_sh, kv_ctx;
  // grouped GEMM over expert-sorted rows (EPI_MOE_*): a device-side list of 256-row tiles, each inside one expert's
  // block of rows; W is [experts * N, K], N and ld_out are per expert
  const int* g_tile_row0;    // [tiles] first row of the tile
  const int* g_tile_rows;    // [tiles] valid rows (1..256)
  const int* g_tile_expert;  // [tiles]
  const int* g_n_tiles;      // device scalar: tiles in the list
  const float* g_bias;       // fp32 [experts][N]
  const float* g_gate;       // fp32 [rows]: routing weight of every sorted row (EPI_MOE_GATE)
  float alpha, limit;        // clamped SwiGLU (EPI_MOE_SWIGLU)
  int* status;
  long long* trace;  // optional [CTA][8] (b2_set_trace_buffer): start ns, end ns, start clock, end clock
};


// Grouped GEMM of the MoE prompt path on CTA pairs: for every listed tile, rows [row0, row0 + rows) of a_ptr times the
// tile's expert's block of w_ptr ([experts * N, K] bf16), epilogue `epi` (EPI_MOE_SWIGLU: + bias, clamped SwiGLU over
// interleaved column pairs -> out [rows, N / 2]; EPI_MOE_GATE: (+ bias) * gate[row] -> out [rows, N]).  N % 192 == 0.
int launch_moe_grouped_gemm(int epi, const void* a_ptr, int64_t lda, const void* w_ptr, int64_t ldw, GemmArgs g, int max_tiles,
                            cudaStream_t stream);

}  // namespace b2
