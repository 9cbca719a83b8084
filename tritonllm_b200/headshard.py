"""Optional head-sharded attention block for long-context prefill on several GPUs.

The default multi-GPU mode shards sequences and needs no collective.  One long prompt cannot be split that
way, so this mode splits the attention of ONE sequence by KV head instead: with 8 KV heads and ``world``
ranks, rank r owns KV heads ``r*h .. r*h+h-1`` (h = 8 / world) and the query heads of their GQA groups
(query head q uses KV head q // group, attention_tt_tma.py:43), i.e. a row slice of the QKV weight.  Every
rank runs the norm (replicated), its slice of the QKV projection with RoPE, and the prefill attention of its
heads over the full sequence; ONE all-gather of the per-rank outputs ``[T, h*group*64]`` bf16 (8 MiB per rank
at T = 8192, h = 1) restores ``[T, 4096]`` in every rank's own memory, and the o_proj + residual runs
replicated.  The reference has no multi-GPU code; the block computed is AttentionBlock.forward with
``cache=None`` (tritonllm/gpt_oss/triton/model.py:471-573).

The collective is NCCL's (``torch.distributed``); the kernels only ever read this GPU's memory.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class AttentionShard:
    """The slice of one AttentionBlock's parameters that rank ``rank`` of ``world`` needs for its heads (QKV rows
    and sinks), plus what every rank keeps whole (norm gain, o_proj)."""
    wqkv: torch.Tensor     # [(hq + 2*hkv) * d, hidden]: this rank's q rows, then its k rows, then its v rows
    bqkv: torch.Tensor
    sinks: torch.Tensor    # [hq]
    n_q_heads: int         # hq = hkv * group
    n_kv_heads: int        # hkv
    rank: int
    world: int


def shard_attention_weights(wqkv, bqkv, sinks, rank: int, world: int, n_q_heads=64, n_kv_heads=8, head_dim=64) -> AttentionShard:
    """Row slices of the fused QKV weight [(Hq + 2*Hkv)*d, hidden] (q rows, k rows, v rows, model.py:454-457,
    507) for the KV heads rank ``rank`` owns and the query heads of their groups."""
    if n_kv_heads % world:
        raise ValueError(f"{n_kv_heads} KV heads cannot be split over {world} ranks")
    group = n_q_heads // n_kv_heads
    hkv = n_kv_heads // world
    hq = hkv * group
    d = head_dim
    q0, k0, v0 = 0, n_q_heads * d, (n_q_heads + n_kv_heads) * d
    rows = torch.cat([torch.arange(q0 + rank * hq * d, q0 + (rank + 1) * hq * d),
                      torch.arange(k0 + rank * hkv * d, k0 + (rank + 1) * hkv * d),
                      torch.arange(v0 + rank * hkv * d, v0 + (rank + 1) * hkv * d)]).to(wqkv.device)
    return AttentionShard(wqkv.index_select(0, rows).contiguous(), bqkv.index_select(0, rows).contiguous(),
                          sinks[rank * hq:(rank + 1) * hq].contiguous(), hq, hkv, rank, world)


def gather_heads(o_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather of the per-rank attention outputs [rows, f_local] into [rows, world * f_local], rank r's features
    at columns r*f_local .. (heads are owned in rank order, so this is the layout o_proj expects).  One collective;
    the gathered data lands in this rank's own memory before anything reads it."""
    if not dist.is_initialized():      # a single process: nothing to gather
        return o_local
    world = dist.get_world_size(group)
    if world == 1:
        return o_local
    rows, f = o_local.shape
    stacked = torch.empty((world * rows, f), dtype=o_local.dtype, device=o_local.device)   # rank-major blocks
    dist.all_gather_into_tensor(stacked, o_local.contiguous(), group=group)
    return stacked.view(world, rows, f).permute(1, 0, 2).reshape(rows, world * f)


def attention_heads_local(x, norm_gain, shard: AttentionShard, sin, cos, max_context_length, sm_scale, sliding_window,
                          eps=1e-5, head_dim=64) -> torch.Tensor:
    """This rank's part of the block: norm, its slice of the QKV projection with RoPE, prefill attention of its heads
    over the whole sequence.  x [B, T, hidden] -> [B*T, n_q_heads_local * head_dim]."""
    from . import ops
    B, T, _ = x.shape
    position = torch.zeros(1, dtype=torch.int64, device=x.device)
    n = ops.rmsnorm_forward(x, norm_gain, eps)
    q, k, v = ops.qkv_rope_prefill(n, shard.wqkv, shard.bqkv, sin, cos, max_context_length, position, shard.n_q_heads,
                                   shard.n_kv_heads, head_dim)
    o_local = ops.attention(q.view(B, T, shard.n_kv_heads, shard.n_q_heads // shard.n_kv_heads, head_dim), k, v, shard.sinks,
                            sm_scale, sliding_window, position)
    return o_local.reshape(B * T, -1)


def attention_block_headsharded(x, norm_gain, shard: AttentionShard, wo, bo, sin, cos, max_context_length, sm_scale,
                                sliding_window, eps=1e-5, head_dim=64, group=None, timings: dict | None = None):
    """AttentionBlock.forward(x, cache=None) with the heads split over the ranks of ``group``: x [B, T, hidden]
    (the same on every rank) -> [B, T, hidden] (the same on every rank).  ``timings``, when a dict, receives CUDA
    events around the all-gather (keys ``gather_start`` / ``gather_end``)."""
    from . import ops
    B, T, _ = x.shape
    o_local = attention_heads_local(x, norm_gain, shard, sin, cos, max_context_length, sm_scale, sliding_window, eps, head_dim)
    if timings is not None:
        timings["gather_start"] = torch.cuda.Event(enable_timing=True)
        timings["gather_end"] = torch.cuda.Event(enable_timing=True)
        timings["gather_start"].record()
    o = gather_heads(o_local, group)
    if timings is not None:
        timings["gather_end"].record()
    return ops.out_residual_forward(o.reshape(B, T, -1), wo, bo, x)
