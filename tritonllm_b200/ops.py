"""Host-side mirror of the TritonLLM op call sites for the gpt-oss per-layer path.

Every function keeps the name, argument order and tensor contract of the
function it replaces in ``tritonllm.gpt_oss.triton`` (cited per function) and
forwards to the C ABI of ``libtritonllm_b200.so`` on torch's current stream.
Tensors must be CUDA tensors; there is no CPU path.  Outputs come from a
shape-keyed scratch pool like the reference's, so addresses are stable across
CUDA-graph replays.

One stream at a time: pooled outputs and the workspaces of ``attention_decode``
(arrival counters, split-KV partials), ``moe_experts_decode`` and the
unembedding are process-global, keyed by shape and device like the reference's
pool, not by stream.  Calls of the same shape that overlap on the GPU (two
streams, two threads, two generators stepping concurrently) would share them
and corrupt each other's results; run them on one stream or serialise them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib
from . import scratch_pool

_BF16 = torch.bfloat16


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("tritonllm_b200 ops run on CUDA tensors only (no CPU fallback)")


def _ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


# ----------------------------------------------------------------------------- norms
def rmsnorm_forward(x: torch.Tensor, scale: torch.Tensor, eps: float, out: torch.Tensor | None = None):
    """Drop-in for rmsnorm_forward (tritonllm/gpt_oss/triton/triton_kernels.py:28-35)."""
    _need_cuda(x, scale)
    assert x.dtype == _BF16 and scale.dtype == torch.float32
    assert x.is_contiguous() and scale.is_contiguous() and scale.shape == (x.shape[-1],)
    if out is None:
        out = scratch_pool.get(tuple(x.shape), x.dtype, x.device)
    assert out.shape == x.shape and out.dtype == x.dtype and out.is_contiguous()
    dim = x.shape[-1]
    rows = x.numel() // dim if dim else 0
    _lib.call("b2_rmsnorm", x.data_ptr(), scale.data_ptr(), out.data_ptr(), rows, dim, float(eps), _stream())
    return out


def add_rmsnorm_forward(x: torch.Tensor, delta: torch.Tensor, scale: torch.Tensor, eps: float,
                        h_out: torch.Tensor | None = None, y_out: torch.Tensor | None = None):
    """h = x + delta (bf16), y = rmsnorm(h): the residual add of model.py:572 / 816 fused into the
    RMSNorm that follows it (model.py:476 / 754).  Returns (h, y); h_out may alias x."""
    _need_cuda(x, delta, scale)
    assert x.dtype == _BF16 and delta.dtype == _BF16 and scale.dtype == torch.float32
    assert x.shape == delta.shape and x.is_contiguous() and delta.is_contiguous()
    if h_out is None:
        h_out = torch.empty_like(x)
    if y_out is None:
        y_out = scratch_pool.get(tuple(x.shape), x.dtype, x.device)
    dim = x.shape[-1]
    rows = x.numel() // dim if dim else 0
    _lib.call("b2_add_rmsnorm", x.data_ptr(), delta.data_ptr(), scale.data_ptr(), h_out.data_ptr(), y_out.data_ptr(),
              rows, dim, float(eps), _stream())
    return h_out, y_out


# ------------------------------------------------------------------------------ RoPE
def rope_forward(query, key, sin, cos, max_context_length, offset):
    """Drop-in for rope_forward (triton_kernels.py:90-108): rotates query/key in place."""
    _need_cuda(query, key, sin, cos, offset)
    batch, tokens, n_q, d = query.shape
    batch_k, tokens_k, n_kv, d_k = key.shape
    assert (batch, tokens, d) == (batch_k, tokens_k, d_k)
    assert query.dtype == _BF16 and key.dtype == _BF16 and query.is_contiguous() and key.is_contiguous()
    assert sin.dtype == torch.float32 and cos.dtype == torch.float32 and sin.is_contiguous() and cos.is_contiguous()
    assert sin.shape[-1] == d // 2 and sin.shape[0] >= max_context_length
    assert offset.dtype == torch.int64 and offset.numel() == 1
    _lib.call("b2_rope_inplace", query.data_ptr(), key.data_ptr(), sin.data_ptr(), cos.data_ptr(), offset.data_ptr(),
              batch, tokens, n_q, n_kv, d, int(max_context_length), _stream())


# ---------------------------------------------------------------------------- decode
def qkv_rope_cache_decode_forward(hidden, weight, bias, sin, cos, max_context_length, cache_k, cache_v, offset,
                                  num_q_heads, num_kv_heads, head_dim, weight_scale=None, per_sequence=False):
    """Drop-in for qkv_rope_cache_decode_forward (triton_kernels.py:1109-1255).  Beyond the reference: ``offset``
    may hold one position per sequence (shape [batch]; ``per_sequence=True`` says so for a batch of one)."""
    if weight_scale is not None:
        raise NotImplementedError("fp8 weights (ATTN_FP8) are not part of the B200 path")
    _need_cuda(hidden, weight, bias, sin, cos, cache_k, cache_v, offset)
    batch, num_tokens, hidden_size = hidden.shape
    total_out, hidden_size_weight = weight.shape
    assert num_tokens == 1
    assert hidden_size == hidden_size_weight
    assert total_out == (num_q_heads + 2 * num_kv_heads) * head_dim
    assert bias.shape == (total_out,)
    assert cache_k.shape == cache_v.shape and cache_k.stride() == cache_v.stride()
    assert cache_k.shape[0] == batch and cache_k.shape[2] == num_kv_heads and cache_k.shape[3] == head_dim
    assert offset.dtype == torch.int64 and offset.is_contiguous()
    assert offset.shape == (1,) or offset.shape == (batch,), "one position for the batch, or one per sequence"
    assert hidden.dtype == _BF16 and weight.dtype == _BF16 and bias.dtype == _BF16 and cache_k.dtype == _BF16
    hidden2 = hidden.reshape(batch, hidden_size)
    if hidden2.stride(-1) != 1:
        hidden2 = hidden2.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    bias = bias if bias.is_contiguous() else bias.contiguous()
    assert cache_k.stride(3) == 1 and sin.is_contiguous() and cos.is_contiguous()
    q = scratch_pool.get((batch, num_q_heads, head_dim), hidden.dtype, hidden.device)
    if offset.shape == (1,) and not per_sequence:   # the reference's contract: the whole batch sits at one position
        _lib.call("b2_qkv_rope_kv_decode", hidden2.data_ptr(), hidden2.stride(0), weight.data_ptr(), bias.data_ptr(),
                  sin.data_ptr(), cos.data_ptr(), offset.data_ptr(), q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
                  cache_k.stride(0), cache_k.stride(1), cache_k.stride(2), cache_k.shape[1], batch, hidden_size,
                  num_q_heads, num_kv_heads, head_dim, int(max_context_length), _stream())
    else:
        _lib.call("b2_qkv_rope_kv_decode_ragged", hidden2.data_ptr(), hidden2.stride(0), weight.data_ptr(), bias.data_ptr(),
                  sin.data_ptr(), cos.data_ptr(), offset.data_ptr(), q.data_ptr(), cache_k.data_ptr(), cache_v.data_ptr(),
                  cache_k.stride(0), cache_k.stride(1), cache_k.stride(2), cache_k.shape[1], 0, 0, 0, batch, hidden_size,
                  num_q_heads, num_kv_heads, head_dim, int(max_context_length), _stream())
    return q.reshape(batch, 1, num_q_heads * head_dim)


def out_residual_decode_forward(hidden, weight, bias, residual, weight_scale=None):
    """Drop-in for out_residual_decode_forward (triton_kernels.py:1470-1517): writes into ``residual``."""
    if weight_scale is not None:
        raise NotImplementedError("fp8 weights (ATTN_FP8) are not part of the B200 path")
    _need_cuda(hidden, weight, bias, residual)
    batch, num_tokens, k_in = hidden.shape
    n_out, k_in_w = weight.shape
    assert num_tokens == 1 and k_in == k_in_w
    assert bias.shape == (n_out,)
    assert residual.shape == (batch, 1, n_out)
    assert hidden.dtype == _BF16 and weight.dtype == _BF16 and bias.dtype == _BF16 and residual.dtype == _BF16
    hidden2 = hidden.reshape(batch, k_in)
    if hidden2.stride(-1) != 1:
        hidden2 = hidden2.contiguous()
    out = residual.reshape(batch, n_out)
    assert out.stride(-1) == 1 and out.data_ptr() == residual.data_ptr(), "residual must be updatable in place"
    weight = weight if weight.is_contiguous() else weight.contiguous()
    bias = bias if bias.is_contiguous() else bias.contiguous()
    _lib.call("b2_oproj_residual_decode", hidden2.data_ptr(), hidden2.stride(0), weight.data_ptr(), bias.data_ptr(),
              out.data_ptr(), out.stride(0), batch, k_in, n_out, _stream())
    return out[:, None, :]


_attn_ws: dict[tuple, torch.Tensor] = {}


def _attn_decode_workspace(batch: int, n_kv_heads: int, group: int, device: torch.device) -> torch.Tensor:
    key = (batch, n_kv_heads, group, device)
    ws = _attn_ws.get(key)
    if ws is None:
        nbytes = _lib.load().b2_attn_decode_workspace_bytes(batch, n_kv_heads, group)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)  # zero-filled once; the kernel keeps it reusable
        _attn_ws[key] = ws
    return ws


def attention_decode(q, k, v, sinks, sm_scale, sliding_window, start_q, per_sequence=False):
    """Drop-in for attention_decode (tritonllm/gpt_oss/triton/attention_tt_decode.py:291-410).  Beyond the
    reference: ``start_q`` may hold one position per sequence (length B; ``per_sequence=True`` says so for B = 1)."""
    _need_cuda(q, k, v, start_q)
    bs, n_ctx, n_kv_heads, repeat_kv, head_dim = q.shape
    assert len(start_q) == 1 or len(start_q) == bs, "one position for the batch, or one per sequence"
    ragged = per_sequence or len(start_q) != 1
    bs_k, n_kv_ctx, n_kv_heads_k, head_dim_k = k.shape
    assert v.shape == k.shape and v.stride() == k.stride()
    assert n_ctx == 1 and bs == bs_k and n_kv_heads == n_kv_heads_k and head_dim == head_dim_k
    assert q.dtype == _BF16 and k.dtype == _BF16 and v.dtype == _BF16
    assert k.stride(3) == 1 and start_q.is_contiguous()
    q2 = q.reshape(bs, n_kv_heads * repeat_kv * head_dim)
    if not q2.is_contiguous():
        q2 = q2.contiguous()
    sinks_f32 = 0
    if sinks is not None:
        _need_cuda(sinks)
        assert sinks.numel() == n_kv_heads * repeat_kv and sinks.is_contiguous()
        assert sinks.dtype in (_BF16, torch.float32)
        sinks_f32 = 1 if sinks.dtype == torch.float32 else 0
    assert start_q.dtype in (torch.int32, torch.int64)
    o = scratch_pool.get((bs, n_kv_heads, repeat_kv, head_dim), q.dtype, q.device)
    ws = _attn_decode_workspace(bs, n_kv_heads, repeat_kv, q.device)
    if ragged:
        _lib.call("b2_attn_decode_ragged", q2.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(sinks), sinks_f32, o.data_ptr(),
                  bs, n_kv_heads, repeat_kv, head_dim, n_kv_ctx, k.stride(0), k.stride(1), k.stride(2), float(sm_scale),
                  int(sliding_window or 0), start_q.data_ptr(), 1 if start_q.dtype == torch.int64 else 0, 0, 0, 0, 0,
                  ws.data_ptr(), ws.numel(), _stream())
    else:
        _lib.call("b2_attn_decode", q2.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(sinks), sinks_f32, o.data_ptr(), bs,
                  n_kv_heads, repeat_kv, head_dim, n_kv_ctx, k.stride(0), k.stride(1), k.stride(2), float(sm_scale),
                  int(sliding_window or 0), start_q.data_ptr(), 1 if start_q.dtype == torch.int64 else 0, ws.data_ptr(),
                  ws.numel(), _stream())
    return o.view(bs, 1, n_kv_heads * repeat_kv * head_dim)


# ------------------------------------------------------------------------ paged KV store (decode)
def _check_pool(k_pool, v_pool, block_table, positions, batch, kv_capacity):
    _need_cuda(k_pool, v_pool, block_table, positions)
    assert k_pool.dtype == _BF16 and v_pool.dtype == _BF16 and k_pool.dim() == 4 and k_pool.stride(3) == 1
    assert v_pool.shape == k_pool.shape and v_pool.stride() == k_pool.stride()
    n_pages, page_size = k_pool.shape[0], k_pool.shape[1]
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.shape[0] == batch
    assert block_table.stride(1) == 1
    assert positions.dtype == torch.int64 and positions.shape == (batch,) and positions.is_contiguous()
    if kv_capacity is None:
        kv_capacity = block_table.shape[1] * page_size
    assert kv_capacity <= block_table.shape[1] * page_size
    return n_pages, page_size, int(kv_capacity)


def qkv_rope_paged_decode_forward(hidden, weight, bias, sin, cos, max_context_length, k_pool, v_pool, block_table,
                                  positions, num_q_heads, num_kv_heads, head_dim, kv_capacity=None):
    """``qkv_rope_cache_decode_forward`` for a paged KV store with one position per sequence: k_pool / v_pool
    [pages, page_size, kv_heads, head_dim] bf16, block_table int32 [batch, max_pages] (page of tokens
    page_size*j .. of sequence b), positions int64 [batch].  Token positions[b] of sequence b is written to its
    page; returns q [batch, 1, Hq*D] (pooled).  The reference has no paged store (its Cache is dense,
    model.py:340-433); the arithmetic is that of triton_kernels.py:1109-1255."""
    _need_cuda(hidden, weight, bias, sin, cos)
    batch, num_tokens, hidden_size = hidden.shape
    assert num_tokens == 1 and weight.shape == ((num_q_heads + 2 * num_kv_heads) * head_dim, hidden_size)
    assert hidden.dtype == _BF16 and weight.dtype == _BF16 and bias.dtype == _BF16
    assert k_pool.shape[2] == num_kv_heads and k_pool.shape[3] == head_dim
    _, page_size, cap = _check_pool(k_pool, v_pool, block_table, positions, batch, kv_capacity)
    hidden2 = hidden.reshape(batch, hidden_size)
    if hidden2.stride(-1) != 1:
        hidden2 = hidden2.contiguous()
    assert weight.is_contiguous() and bias.is_contiguous() and sin.is_contiguous() and cos.is_contiguous()
    q = scratch_pool.get((batch, num_q_heads, head_dim), hidden.dtype, hidden.device)
    _lib.call("b2_qkv_rope_kv_decode_ragged", hidden2.data_ptr(), hidden2.stride(0), weight.data_ptr(), bias.data_ptr(),
              sin.data_ptr(), cos.data_ptr(), positions.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(),
              k_pool.stride(0), k_pool.stride(1), k_pool.stride(2), cap, block_table.data_ptr(), block_table.stride(0),
              page_size, batch, hidden_size, num_q_heads, num_kv_heads, head_dim, int(max_context_length), _stream())
    return q.reshape(batch, 1, num_q_heads * head_dim)


def attention_decode_paged(q, k_pool, v_pool, block_table, positions, sinks, sm_scale, sliding_window, kv_capacity=None):
    """``attention_decode`` over a paged KV store with one position per sequence (see
    ``qkv_rope_paged_decode_forward`` for the layout): q [B, 1, Hkv, G, D]; returns [B, 1, Hkv*G*D] (pooled).
    page_size must be a multiple of 32."""
    _need_cuda(q)
    bs, n_ctx, n_kv_heads, repeat_kv, head_dim = q.shape
    assert n_ctx == 1 and q.dtype == _BF16 and k_pool.shape[2] == n_kv_heads and k_pool.shape[3] == head_dim
    n_pages, page_size, cap = _check_pool(k_pool, v_pool, block_table, positions, bs, kv_capacity)
    q2 = q.reshape(bs, n_kv_heads * repeat_kv * head_dim)
    if not q2.is_contiguous():
        q2 = q2.contiguous()
    sinks_f32 = 0
    if sinks is not None:
        _need_cuda(sinks)
        assert sinks.numel() == n_kv_heads * repeat_kv and sinks.is_contiguous() and sinks.dtype in (_BF16, torch.float32)
        sinks_f32 = 1 if sinks.dtype == torch.float32 else 0
    o = scratch_pool.get((bs, n_kv_heads, repeat_kv, head_dim), q.dtype, q.device)
    ws = _attn_decode_workspace(bs, n_kv_heads, repeat_kv, q.device)
    _lib.call("b2_attn_decode_ragged", q2.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), _ptr(sinks), sinks_f32,
              o.data_ptr(), bs, n_kv_heads, repeat_kv, head_dim, cap, k_pool.stride(0), k_pool.stride(1), k_pool.stride(2),
              float(sm_scale), int(sliding_window or 0), positions.data_ptr(), 1, block_table.data_ptr(),
              block_table.stride(0), page_size, n_pages, ws.data_ptr(), ws.numel(), _stream())
    return o.view(bs, 1, n_kv_heads * repeat_kv * head_dim)


# ---------------------------------------------------------------------- MoE front-end
def swiglu(a, alpha, precision_config=None, routing_data=None, limit=None):
    """Drop-in for swiglu (tritonllm/triton_kernels/swiglu.py:85-86).

    ``precision_config`` is the reference's PrecisionConfig (only ``.limit`` is
    read); a bare ``limit=`` works too.  ``routing_data`` must be None.
    """
    if routing_data is not None:
        raise NotImplementedError("swiglu with routing_data (ragged row count) is not part of the B200 path")
    if precision_config is not None:
        limit = getattr(precision_config, "limit", precision_config)
    _need_cuda(a)
    assert a.dtype == _BF16 and a.stride(-1) == 1 and a.shape[-1] % 2 == 0
    n2 = a.shape[-1]
    a2 = a.reshape(-1, n2)
    rows = a2.shape[0]
    out = torch.empty((rows, n2 // 2), dtype=a.dtype, device=a.device)
    _lib.call("b2_swiglu", a2.data_ptr(), a2.stride(0), out.data_ptr(), out.stride(0), rows, n2 // 2, float(alpha),
              float(limit) if limit is not None else 0.0, _stream())
    return out.view(a.shape[:-1] + (n2 // 2,))


@dataclass
class Bitmatrix:
    """Packed expert mask returned by :func:`topk` (uint32 words held as int32).

    ``data`` is the [n_rows, n_words] view of a column-major allocation, as in
    the reference (tritonllm/triton_kernels/topk.py:33-36), ``scratchpad`` the
    zeroed int32 buffer the reference's Bitmatrix carries (tensor.py:173-197).
    """
    data: torch.Tensor
    shape: list
    scratchpad: torch.Tensor


def topk(x, k, apply_softmax=True, dim=1, return_bitmatrix=True, y_indx=None, n_rows=None):
    """Drop-in for topk (tritonllm/triton_kernels/topk.py:86-88), forward only.

    Returns (y_vals fp32 [rows,k], y_indx int16 [rows,k] sorted by expert id, Bitmatrix).
    """
    if y_indx is not None or n_rows is not None:
        raise NotImplementedError("user-provided indices / device row counts are not part of the B200 path")
    assert dim == 1 and return_bitmatrix and x.dim() == 2
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.stride(1) == 1 and x.shape[1] < 32768
    rows, n_expts = x.shape
    dev = x.device
    y_vals = torch.empty((rows, k), dtype=torch.float32, device=dev)
    y_idx = torch.empty((rows, k), dtype=torch.int16, device=dev)
    n_words = (n_expts + 31) // 32
    bm = torch.empty((n_words, (rows + 31) // 32 * 32), dtype=torch.int32, device=dev)
    bm = torch.transpose(bm, 0, 1)[:rows]
    s_cols = (n_expts + 127) // 128 * 128
    scratch = torch.empty((s_cols,), dtype=torch.int32, device=dev)
    _lib.call("b2_topk_softmax", x.data_ptr(), x.stride(0), rows, n_expts, k, 1 if apply_softmax else 0,
              y_vals.data_ptr(), y_idx.data_ptr(), bm.data_ptr(), bm.stride(0), bm.stride(1), scratch.data_ptr(),
              s_cols, _stream())
    return y_vals, y_idx, Bitmatrix(bm, [rows, n_words * 32], scratch)


# --------------------------------------------------------------------------- patching
REPLACED = ("rmsnorm_forward", "rope_forward", "qkv_rope_cache_decode_forward", "out_residual_decode_forward",
            "attention_decode", "attention", "unembedding_decode_forward", "unembedding_decode_argmax_forward",
            "moe", "moe_decode")


def patch(model_module) -> list[str]:
    """Rebinds the op names that ``tritonllm.gpt_oss.triton.model`` imported
    (model.py:11-34) to the functions of this module, so the reference's
    RMSNorm / RotaryEmbedding / AttentionBlock / MLPBlock modules call the B200
    kernels: after it ``TransformerBlock.forward`` (model.py:891-894) launches no
    Triton kernel.  (The dense prefill projections stay the ``F.linear`` calls of
    QKV.forward / OUT.forward; ``qkv_rope_prefill`` / ``out_residual_forward`` are
    the fused forms for a caller that edits those two methods.)
    Returns the names that were rebound."""
    done = []
    for name in REPLACED:
        if hasattr(model_module, name):
            setattr(model_module, name, globals()[name])
            done.append(name)
    return done


def yarn_cos_sin(n_pos: int, head_dim=64, base=150000.0, factor=32.0, orig_ctx=4096, alpha=1.0, beta=32.0,
                 device=None):
    """fp32 cos/sin tables [n_pos, head_dim/2] of the YaRN-scaled rotary embedding, built as
    RotaryEmbedding._compute_cos_sin does (tritonllm/gpt_oss/triton/model.py:259-313)."""
    half = head_dim // 2
    freq = base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim)
    if factor > 1.0:
        conc = 0.1 * math.log(factor) + 1.0
        lo = half * math.log(orig_ctx / (beta * 2 * math.pi)) / math.log(base)
        hi = half * math.log(orig_ctx / (alpha * 2 * math.pi)) / math.log(base)
        ramp = ((torch.arange(half, dtype=torch.float32, device=device) - lo) / (hi - lo)).clamp(0, 1)
        inv_freq = (1.0 / (factor * freq)) * ramp + (1.0 / freq) * (1 - ramp)
    else:
        conc, inv_freq = 1.0, 1.0 / freq
    t = torch.arange(n_pos, dtype=torch.float32, device=device)
    ang = torch.einsum("i,j->ij", t, inv_freq)
    return ang.cos() * conc, ang.sin() * conc


# ------------------------------------------------------------------ prefill projections (tcgen05)
def linear_bias(x, weight, bias):
    """bf16 ``F.linear(x, weight, bias)`` on the tensor cores: QKV.forward / OUT.forward
    (tritonllm/gpt_oss/triton/model.py:136-138, 195-197)."""
    _need_cuda(x, weight, bias)
    assert x.dtype == _BF16 and weight.dtype == _BF16 and bias.dtype == _BF16
    n, k = weight.shape
    assert x.shape[-1] == k and bias.shape == (n,) and weight.is_contiguous() and bias.is_contiguous()
    x2 = x.reshape(-1, k)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], n), dtype=_BF16, device=x.device)
    _lib.call("b2_linear_bias", x2.data_ptr(), x2.stride(0), weight.data_ptr(), bias.data_ptr(), out.data_ptr(),
              out.stride(0), x2.shape[0], n, k, _stream())
    return out.view(x.shape[:-1] + (n,))


def qkv_rope_prefill(x, weight, bias, sin, cos, max_context_length, offset, num_q_heads, num_kv_heads, head_dim,
                     cache_k=None, cache_v=None, round_before_rope=True):
    """The prefill branch of AttentionBlock.forward up to the attention call, fused
    (model.py:506-526): QKV projection + bias, split into heads, RoPE at positions
    offset .. offset+T-1, and - when caches are given - the Cache.extend write
    (model.py:426-433; the caller still advances ``cache.offset``).
    Returns (q [B,T,Hq,D], k, v) where k/v are the caches when given, else new [B,T,Hkv,D]."""
    _need_cuda(x, weight, bias, sin, cos, offset)
    batch, tokens, hidden = x.shape
    n_out, hidden_w = weight.shape
    assert hidden == hidden_w and n_out == (num_q_heads + 2 * num_kv_heads) * head_dim and bias.shape == (n_out,)
    assert x.dtype == _BF16 and weight.dtype == _BF16 and bias.dtype == _BF16
    assert offset.dtype == torch.int64 and offset.numel() == 1
    assert weight.is_contiguous() and bias.is_contiguous() and sin.is_contiguous() and cos.is_contiguous()
    x2 = x.reshape(batch * tokens, hidden)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    q = torch.empty((batch, tokens, num_q_heads, head_dim), dtype=_BF16, device=x.device)
    if cache_k is not None:
        assert cache_v is not None and cache_k.shape == cache_v.shape and cache_k.stride() == cache_v.stride()
        assert cache_k.shape[0] == batch and cache_k.shape[2] == num_kv_heads and cache_k.stride(3) == 1
        k, v, add = cache_k, cache_v, 1
    else:
        k = torch.empty((batch, tokens, num_kv_heads, head_dim), dtype=_BF16, device=x.device)
        v = torch.empty_like(k)
        add = 0
    _lib.call("b2_qkv_rope_prefill", x2.data_ptr(), x2.stride(0), weight.data_ptr(), bias.data_ptr(), sin.data_ptr(),
              cos.data_ptr(), offset.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1),
              k.stride(2), k.shape[1], add, batch, tokens, hidden, num_q_heads, num_kv_heads, head_dim,
              int(max_context_length), 1 if round_before_rope else 0, _stream())
    return q, k, v


def out_residual_forward(t, weight, bias, residual, out=None):
    """``self.out(t) + x`` of the prefill branch (model.py:571-572) in one kernel; ``out`` may be ``residual``."""
    _need_cuda(t, weight, bias, residual)
    n, k = weight.shape
    assert t.shape[-1] == k and residual.shape[-1] == n and bias.shape == (n,)
    assert t.dtype == _BF16 and weight.dtype == _BF16 and bias.dtype == _BF16 and residual.dtype == _BF16
    t2 = t.reshape(-1, k)
    if t2.stride(-1) != 1:
        t2 = t2.contiguous()
    r2 = residual.reshape(-1, n)
    assert r2.stride(-1) == 1 and r2.shape[0] == t2.shape[0]
    if out is None:
        out = torch.empty_like(residual)
    o2 = out.reshape(-1, n)
    assert o2.data_ptr() == out.data_ptr() and o2.stride(-1) == 1
    _lib.call("b2_oproj_residual", t2.data_ptr(), t2.stride(0), weight.data_ptr(), bias.data_ptr(), r2.data_ptr(),
              r2.stride(0), o2.data_ptr(), o2.stride(0), t2.shape[0], n, k, _stream())
    return out


_gate_t: dict[int, tuple] = {}  # id(wg) -> (wg, version, expert-major copy); holding wg keeps the id unique


def _gate_expert_major(wg):
    """The expert-major copy of the reference's [hidden, E] gate weight, made once per tensor object (and
    again if the tensor is modified in place)."""
    hit = _gate_t.get(id(wg))
    if hit is not None and hit[0] is wg and hit[1] == wg._version:
        return hit[2]
    wt = wg.t().contiguous()
    _gate_t[id(wg)] = (wg, wg._version, wt)
    return wt


def norm_router_topk(x, scale, eps, wg, bg, k=4, y_out=None, return_logits=False):
    """``t = self.norm(x)``, ``logits = (t @ wg).float() + bg``, ``topk(logits, k, apply_softmax=True)``
    (tritonllm/gpt_oss/triton/model.py:754, moe.py:46-48, triton_kernels/routing.py:296-297) in one
    launch for decode-sized batches.  x [..., hidden] bf16; returns (t like x, vals fp32 [T, k], idx int16
    [T, k]) and the fp32 logits [T, E] as a fourth value when ``return_logits``."""
    _need_cuda(x, scale, wg)
    assert x.dtype == _BF16 and wg.dtype == _BF16 and scale.dtype == torch.float32 and x.stride(-1) == 1
    hidden, n_experts = wg.shape
    assert x.shape[-1] == hidden and scale.shape == (hidden,)
    x2 = x.reshape(-1, hidden)
    y = torch.empty_like(x) if y_out is None else y_out
    y2 = y.view(-1, hidden)
    assert y2.shape == x2.shape and y2.stride(1) == 1
    rows = x2.shape[0]
    if bg is not None:
        assert bg.dtype == torch.float32 and bg.is_contiguous() and bg.shape == (n_experts,)
    vals = torch.empty((rows, k), dtype=torch.float32, device=x.device)
    idx = torch.empty((rows, k), dtype=torch.int16, device=x.device)
    logits = torch.empty((rows, n_experts), dtype=torch.float32, device=x.device) if return_logits else None
    _lib.call("b2_norm_router_topk", x2.data_ptr(), x2.stride(0), scale.data_ptr(), _gate_expert_major(wg).data_ptr(),
              _ptr(bg), y2.data_ptr(), y2.stride(0), _ptr(logits), n_experts if return_logits else 0, vals.data_ptr(),
              idx.data_ptr(), rows, hidden, n_experts, int(k), float(eps), _stream())
    return (y, vals, idx, logits) if return_logits else (y, vals, idx)


def router_logits(x, wg, bg):
    """``torch.matmul(x, wg).float() + bg`` (tritonllm/gpt_oss/triton/moe.py:46-48): x [T,H] bf16,
    wg [H,E] bf16 as the reference stores it, bg fp32 [E] or None.  The expert-major copy of wg the
    kernel reads is made once per weight tensor object (and again if the tensor is modified in place)."""
    _need_cuda(x, wg)
    assert x.dtype == _BF16 and wg.dtype == _BF16 and x.dim() == 2 and x.shape[1] == wg.shape[0]
    hit = _gate_t.get(id(wg))
    if hit is not None and hit[0] is wg and hit[1] == wg._version:
        wt = hit[2]
    else:
        wt = wg.t().contiguous()
        _gate_t[id(wg)] = (wg, wg._version, wt)
    if bg is not None:
        assert bg.dtype == torch.float32 and bg.is_contiguous() and bg.shape == (wg.shape[1],)
    x2 = x if x.stride(-1) == 1 else x.contiguous()
    logits = torch.empty((x.shape[0], wg.shape[1]), dtype=torch.float32, device=x.device)
    _lib.call("b2_router_logits", x2.data_ptr(), x2.stride(0), wt.data_ptr(), _ptr(bg), logits.data_ptr(),
              logits.stride(0), x.shape[0], wg.shape[1], wg.shape[0], _stream())
    return logits


def attention(q, k, v, sinks, sm_scale, sliding_window, start_q):
    """Drop-in for the prefill ``attention`` (tritonllm/gpt_oss/triton/attention_tt_tma.py:106-166):
    q [B,T,Hkv,G,D], k/v [B,Tk,Hkv,D] (may be strided views of the KV cache), returns [B,T,Hkv*G*D]."""
    _need_cuda(q, k, v, start_q)
    assert len(start_q) == 1
    bs, n_ctx, n_kv_heads, repeat_kv, head_dim = q.shape
    bs_k, n_kv_ctx, n_kv_heads_k, head_dim_k = k.shape
    assert v.shape == k.shape and v.stride() == k.stride() and k.stride(3) == 1
    assert bs == bs_k and n_kv_heads == n_kv_heads_k and head_dim == head_dim_k
    assert q.dtype == _BF16 and k.dtype == _BF16 and v.dtype == _BF16
    q2 = q.reshape(bs, n_ctx, n_kv_heads * repeat_kv, head_dim)
    if not q2.is_contiguous():
        q2 = q2.contiguous()
    sinks_f32 = 0
    if sinks is not None:
        _need_cuda(sinks)
        assert sinks.numel() == n_kv_heads * repeat_kv and sinks.is_contiguous()
        sinks_f32 = 1 if sinks.dtype == torch.float32 else 0
    assert start_q.dtype in (torch.int32, torch.int64)
    o = torch.empty((bs, n_ctx, n_kv_heads * repeat_kv * head_dim), dtype=_BF16, device=q.device)
    _lib.call("b2_attn_prefill", q2.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(sinks), sinks_f32, o.data_ptr(), bs,
              n_ctx, n_kv_ctx, n_kv_heads, repeat_kv, head_dim, k.stride(0), k.stride(1), k.stride(2), float(sm_scale),
              int(sliding_window or 0), start_q.data_ptr(), 1 if start_q.dtype == torch.int64 else 0, _stream())
    return o


def mxfp4_upcast(codes, scales):
    """MXFP4 -> bf16 along the last axis: codes uint8 [..., K/2], scales uint8 [..., K/32]
    (upcast_from_mxfp_torch, tritonllm/triton_kernels/numerics_details/mxfp.py:237-299)."""
    _need_cuda(codes, scales)
    assert codes.dtype == torch.uint8 and scales.dtype == torch.uint8 and codes.is_contiguous() and scales.is_contiguous()
    k = codes.shape[-1] * 2
    assert k % 32 == 0 and scales.shape == codes.shape[:-1] + (k // 32,)
    rows = codes.numel() // codes.shape[-1] if codes.shape[-1] else 0
    out = torch.empty(codes.shape[:-1] + (k,), dtype=_BF16, device=codes.device)
    _lib.call("b2_mxfp4_upcast", codes.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, k, _stream())
    return out


# ------------------------------------------------------------------ MoE experts (decode-sized batches)
class ExpertWeights:
    """MXFP4 expert weights in the layout the kernels read: codes uint8 [E, N, K/2] (K contiguous, low
    nibble = even k), scales uint8 [E, N, K/32], bias fp32 [E, N]."""

    def __init__(self, codes, scales, bias):
        _need_cuda(codes, scales, bias)
        assert codes.dtype == torch.uint8 and scales.dtype == torch.uint8 and bias.dtype == torch.float32
        e, n, k2 = codes.shape
        assert (k2 * 2) % 32 == 0 and scales.shape == (e, n, k2 * 2 // 32) and bias.shape == (e, n)
        assert codes.is_contiguous() and scales.is_contiguous() and bias.is_contiguous()
        self.codes, self.scales, self.bias = codes, scales, bias

    @classmethod
    def from_reference(cls, w_codes_kn, w_scales_gn, bias):
        """From the reference's tensors: packed values of logical shape [E, K, N] stored K-contiguous as
        uint8 [E, K/2, N] with stride(-2) == 1 (quantize_mx4, tritonllm/gpt_oss/triton/moe.py:17-22;
        the layout assert is matmul_ogs.py:412), scales uint8 [E, K/32, N], bias [E, N] (bf16 parameter
        or its fp32 cache)."""
        codes = w_codes_kn.transpose(1, 2).contiguous()    # [E, N, K/2]; a view copy only if not already K-major
        scales = w_scales_gn.transpose(1, 2).contiguous()  # [E, N, K/32]
        return cls(codes, scales, bias.float().contiguous())


class ExpertWeightsFp4:
    """The same weights packed for the tensor cores' block-scaled FP4 path: codes uint8 [E, N, Kp/2] (K padded
    with zeros to a multiple of 128), scales as 512-byte blocks [E, ceil(N/128), Kp/128, 32, 4, 4]."""

    def __init__(self, w: ExpertWeights):
        e, n, k2 = w.codes.shape
        k = 2 * k2
        kp = (k + 127) // 128 * 128
        tiles, nkb = (n + 127) // 128, kp // 128
        self.codes = torch.nn.functional.pad(w.codes, (0, (kp - k) // 2)).contiguous()
        sc = torch.full((e, tiles * 128, nkb * 4), 127, dtype=torch.uint8, device=w.scales.device)
        sc[:, :n, : k // 32] = w.scales
        # [e, tile, j, i, block, kk] -> [e, tile, block, i, j, kk]
        self.sf = sc.view(e, tiles, 4, 32, nkb, 4).permute(0, 1, 4, 3, 2, 5).contiguous()
        self.bias = w.bias
        self.n, self.k = n, k
        assert self.codes.data_ptr() % 32 == 0


_moe_ws: dict = {}
_moe_generation: dict = {}   # workspace address -> number of expert calls that have written it


class PendingMoe:
    """Expert outputs of one ``moe_experts_decode(..., defer_combine=True)`` call, still in the workspace: the
    sum over each token's experts happens in ``moe_combine_add_rmsnorm``, which must be the next user of it."""

    def __init__(self, ws, tokens, hidden, inter):
        self.ws, self.tokens, self.hidden, self.inter = ws, tokens, hidden, inter
        self.generation = _moe_generation.get(ws.data_ptr(), 0)


def moe_combine_add_rmsnorm(pending: PendingMoe, residual, scale, eps, h_out=None, y_out=None):
    """``x.add_(t)`` with t the MoE output (tritonllm/gpt_oss/triton/model.py:816) and the norm that follows
    (model.py:476, 923), fused with the sum over each token's experts that produces t: returns (h, y) like
    ``add_rmsnorm_forward``.  residual [..., hidden] bf16 with pending.tokens rows; h_out may be residual."""
    if _moe_generation.get(pending.ws.data_ptr(), 0) != pending.generation:
        raise RuntimeError("the expert outputs of this PendingMoe were overwritten by a later moe_experts_decode call "
                           "of the same size: combine a deferred call before the next one")
    _need_cuda(residual, scale)
    hidden = pending.hidden
    assert residual.dtype == _BF16 and residual.shape[-1] == hidden and residual.stride(-1) == 1
    r2 = residual.reshape(-1, hidden)
    assert r2.shape[0] == pending.tokens and scale.dtype == torch.float32 and scale.shape == (hidden,)
    h = torch.empty_like(residual) if h_out is None else h_out
    y = torch.empty_like(residual) if y_out is None else y_out
    h2, y2 = h.view(-1, hidden), y.view(-1, hidden)
    _lib.call("b2_moe_combine_add_rmsnorm", pending.ws.data_ptr(), pending.ws.numel(), pending.tokens, hidden, pending.inter,
              r2.data_ptr(), r2.stride(0), scale.data_ptr(), float(eps), h2.data_ptr(), h2.stride(0), y2.data_ptr(),
              y2.stride(0), _stream())
    return h, y


def moe_experts_decode(x, topk_vals, topk_idx, w1, w2, alpha=1.702, limit=7.0, defer_combine=False):
    """moe_decode_experts / moe_experts for at most 2048 tokens (256 with plain ExpertWeights)
    (tritonllm/gpt_oss/triton/moe.py:54-87,118-175): x [T, hidden] bf16; topk_vals fp32 [T, 4] and
    topk_idx int16 [T, 4] as `topk` returns them; returns a new [T, hidden] bf16 tensor - or, with
    ``defer_combine`` (FP4 weights only), a PendingMoe for ``moe_combine_add_rmsnorm``.  w1 / w2 are both
    ExpertWeights (weights converted to bf16 inside the kernel) or both ExpertWeightsFp4 (block-scaled FP4 MMA)."""
    _need_cuda(x, topk_vals, topk_idx)
    assert x.dtype == _BF16 and x.dim() == 2 and x.stride(1) == 1
    t, hidden = x.shape
    assert topk_idx.dtype == torch.int16 and topk_vals.dtype == torch.float32
    assert topk_idx.shape == (t, 4) and topk_vals.shape == (t, 4) and topk_idx.is_contiguous() and topk_vals.is_contiguous()
    fp4 = isinstance(w1, ExpertWeightsFp4)
    assert fp4 == isinstance(w2, ExpertWeightsFp4)
    e = w1.codes.shape[0]
    n1, k1 = (w1.n, w1.k) if fp4 else (w1.codes.shape[1], 2 * w1.codes.shape[2])
    inter = n1 // 2
    assert k1 == hidden and ((w2.n, w2.k) if fp4 else (w2.codes.shape[1], 2 * w2.codes.shape[2])) == (hidden, inter)
    defer_combine = defer_combine and fp4 and t > 0
    out = None if defer_combine else torch.empty((t, hidden), dtype=_BF16, device=x.device)
    if t == 0:
        return out
    lib = _lib.load()
    need = (lib.b2_moe_fp4_workspace_bytes if fp4 else lib.b2_moe_decode_workspace_bytes)(t, hidden, inter)
    key = (x.device, need)
    ws = _moe_ws.get(key)
    if ws is None:
        ws = torch.empty(need, dtype=torch.uint8, device=x.device)
        _moe_ws[key] = ws
    _lib.call("b2_moe_experts_decode_fp4" if fp4 else "b2_moe_experts_decode", x.data_ptr(), x.stride(0),
              topk_idx.data_ptr(), topk_vals.data_ptr(), w1.codes.data_ptr(), (w1.sf if fp4 else w1.scales).data_ptr(),
              w1.bias.data_ptr(), w2.codes.data_ptr(), (w2.sf if fp4 else w2.scales).data_ptr(), w2.bias.data_ptr(),
              _ptr(out), hidden if out is None else out.stride(0), ws.data_ptr(), ws.numel(), t, e, hidden, inter,
              float(alpha), float(limit), _stream())
    _moe_generation[ws.data_ptr()] = _moe_generation.get(ws.data_ptr(), 0) + 1
    return PendingMoe(ws, t, hidden, inter) if defer_combine else out


# ------------------------------------------------------------------ unembedding (decode)
_unembed_ws: dict = {}


def _unembed(hidden, weight, want_logits: bool, want_ids: bool):
    _need_cuda(hidden, weight)
    assert hidden.dtype == _BF16 and weight.dtype == _BF16 and hidden.dim() == 3 and hidden.shape[1] == 1
    batch, _, hs = hidden.shape
    vocab, hs_w = weight.shape
    assert hs == hs_w and weight.is_contiguous()
    x = hidden.reshape(batch, hs)
    if x.stride(-1) != 1:
        x = x.contiguous()
    logits = scratch_pool.get((batch, vocab), _BF16, hidden.device) if want_logits else None
    ids = torch.empty(batch, dtype=torch.int64, device=hidden.device) if want_ids else None
    ws = None
    if want_ids and batch:
        need = _lib.load().b2_unembed_workspace_bytes(batch, vocab)
        key = (hidden.device, need)
        ws = _unembed_ws.get(key)
        if ws is None:
            ws = torch.empty(need, dtype=torch.uint8, device=hidden.device)
            _unembed_ws[key] = ws
    if batch:
        _lib.call("b2_unembed_decode", x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(logits),
                  logits.stride(0) if want_logits else 0, _ptr(ids), _ptr(ws), ws.numel() if ws is not None else 0,
                  batch, hs, vocab, _stream())
    return logits, ids


def unembedding_decode_forward(hidden, weight):
    """bf16 logits [batch, 1, vocab] of one decode token per sequence (pooled), as
    tritonllm/gpt_oss/triton/triton_kernels.py:170-197."""
    return _unembed(hidden, weight, True, False)[0][:, None, :]


def unembedding_decode_argmax_forward(hidden, weight):
    """Greedy token ids [batch] (int64): arg-max of the fp32 logits without materialising them, as
    tritonllm/gpt_oss/triton/triton_kernels.py:363-401."""
    return _unembed(hidden, weight, False, True)[1]


# ------------------------------------------------------------------ embedding lookup and KV-store maintenance
def embedding_forward(tokens, table, out=None):
    """``torch.nn.Embedding`` lookup of Transformer._forward_hidden (tritonllm/gpt_oss/triton/model.py:896-898,
    911): tokens int32/int64 [...] on the device, table [vocab, hidden] bf16; returns [..., hidden] bf16."""
    _need_cuda(tokens, table)
    assert tokens.dtype in (torch.int32, torch.int64) and table.dtype == _BF16 and table.dim() == 2 and table.stride(1) == 1
    tk = tokens.reshape(-1)
    if not tk.is_contiguous():
        tk = tk.contiguous()
    vocab, hidden = table.shape
    if out is None:
        out = torch.empty(tokens.shape + (hidden,), dtype=_BF16, device=table.device)
    o2 = out.view(-1, hidden)
    assert o2.shape[0] == tk.numel() and o2.stride(1) == 1
    _lib.call("b2_embed_gather", table.data_ptr(), table.stride(0), tk.data_ptr(), 1 if tk.dtype == torch.int64 else 0,
              o2.data_ptr(), o2.stride(0), tk.numel(), hidden, vocab, _stream())
    return out


def _kv_rows(k, v):
    _need_cuda(k, v)
    assert k.dtype == _BF16 and v.dtype == _BF16 and k.shape == v.shape and k.dim() == 4
    assert k.is_contiguous() and v.is_contiguous(), "the KV store must be the dense [batch, n_ctx, heads, dim] layout"
    return k.shape[0], k.shape[1], k.shape[2] * k.shape[3] * 2


def kv_slide(k, v, current: int, keep: int) -> None:
    """The data movement of ``Cache.slide_window`` (model.py:391-424), in place: tokens
    current-keep .. current-1 of every sequence move to 0 .. keep-1, the rest of the store becomes zero."""
    batch, n_ctx, row_bytes = _kv_rows(k, v)
    _lib.call("b2_kv_slide", k.data_ptr(), v.data_ptr(), batch, n_ctx, row_bytes, int(current), int(keep), _stream())


def kv_zero_tail(k, v, start: int) -> None:
    """Zeroes tokens start .. n_ctx-1 of every sequence (``Cache.truncate`` / ``Cache.reset``, model.py:354-371)."""
    batch, n_ctx, row_bytes = _kv_rows(k, v)
    _lib.call("b2_kv_zero_tail", k.data_ptr(), v.data_ptr(), batch, n_ctx, row_bytes, int(start), _stream())


# ------------------------------------------------------------------ MoE block behind the reference's call sites
_expert_repack: dict[int, tuple] = {}   # id(reference weight) -> (weight, scales, ExpertWeightsFp4)


def _raw(t):
    """The torch tensor inside one of the reference's wrapped tensors (triton_kernels/tensor.py:99-160)."""
    st = getattr(t, "storage", None)
    if st is not None and not isinstance(t, torch.Tensor):
        return st.data if hasattr(st, "data") else st
    return t


def experts_from_reference(w, w_mx, bias) -> "ExpertWeightsFp4":
    """The kernels' weight layout from what MLPBlock holds (model.py:627-667, 973-989): ``w`` is the wrapped
    MXFP4 value tensor of logical shape [E, K, N] whose uint8 storage is [E, K/2 (+ padding to 128 on
    Blackwell, blackwell_value.py:12-24), N] with K contiguous, ``w_mx`` the wrapped E8M0 scales [E, K/32, N],
    ``bias`` [E, N] (the bf16 parameter or its fp32 cache).  Repacked once per weight object."""
    hit = _expert_repack.get(id(w))
    if hit is not None and hit[0] is w and hit[1] is w_mx:
        return hit[2]
    data, scales = _raw(w), _raw(w_mx)
    k = int(w.shape[-2]) if not isinstance(w, torch.Tensor) else 2 * data.shape[-2]
    assert data.dtype == torch.uint8 and data.dim() == 3 and k % 32 == 0 and data.shape[1] >= k // 2
    packed = ExpertWeightsFp4(ExpertWeights.from_reference(data[:, : k // 2], scales[:, : k // 32], bias))
    _expert_repack[id(w)] = (w, w_mx, packed)
    return packed


def _moe_from_reference(x, wg, w1, w1_mx, w2, w2_mx, bg, b1, b2, experts_per_token, swiglu_limit):
    if x.numel() == 0:
        return x
    assert x.dim() == 2
    logits = router_logits(x, wg, bg)
    vals, idx, _ = topk(logits, experts_per_token)
    e1, e2 = experts_from_reference(w1, w1_mx, b1), experts_from_reference(w2, w2_mx, b2)
    return moe_experts(x, vals, idx, e1, e2, limit=swiglu_limit)


_moe_prefill_ws: dict = {}
_expanded_budget = 0          # bytes per device that resident bf16 copies of expert weights may take (0: none)
_expanded_used: dict = {}     # device -> bytes taken so far


def set_expanded_expert_budget(nbytes: int) -> None:
    """Memory for speed on the prompt path: up to `nbytes` of device memory (per device) may hold the bf16 expansion
    of MXFP4 expert weights from one `moe_experts_prefill` call to the next (3.2 GB per gpt-oss-20b layer, 38 GB for
    the model), which takes the per-call expansion (0.6 ms of 1.7 ms at 8192 tokens) out of every later call.  The
    copy belongs to the `ExpertWeightsFp4` pair it was made from and is not refreshed if their tensors are
    overwritten in place: call `drop_expanded_experts` then.  0 (the default): one shared scratch, expanded per call."""
    global _expanded_budget
    _expanded_budget = int(nbytes)


def drop_expanded_experts(w1=None) -> None:
    """Forgets the resident bf16 copy made for `w1` (or counts every copy as released when w1 is None; the copies
    themselves die with their weight objects)."""
    if w1 is None:
        _expanded_used.clear()
        return
    hit = getattr(w1, "_expanded", None)
    if hit is not None:
        dev = hit[0].device
        _expanded_used[dev] = _expanded_used.get(dev, 0) - hit[0].numel() * 2 - hit[1].numel() * 2
        w1._expanded = None

PREFILL_MOE_MIN_TOKENS = 2049    # from here on the grouped GEMM (tokens as M rows) beats the decode-sized kernel
# ... when the pair's bf16 expansion is resident (no 0.6 ms of expansion per call; measured, grouped GEMMs against the
# decode-sized kernel: 1024 tokens 382 / 328 us, 1536 tokens 392 / 462 us, 2048 tokens 529 / 604 us)
PREFILL_MOE_MIN_TOKENS_RESIDENT = 1280


def moe_experts_prefill(x, topk_vals, topk_idx, w1, w2, alpha=1.702, limit=7.0):
    """moe_experts (tritonllm/gpt_oss/triton/moe.py:54-87) for a prompt-sized batch: x [T, hidden] bf16 with the
    routing `topk` returned; w1 / w2 ExpertWeightsFp4.  The MXFP4 weights are expanded to bf16 into a scratch
    (1.6 GB for the 20b shapes, kept per device and shape) and the tokens of every expert run through one grouped
    tensor-core GEMM per projection.  Returns a new [T, hidden] bf16 tensor."""
    _need_cuda(x, topk_vals, topk_idx)
    assert isinstance(w1, ExpertWeightsFp4) and isinstance(w2, ExpertWeightsFp4)
    assert x.dtype == _BF16 and x.dim() == 2 and x.stride(1) == 1
    t, hidden = x.shape
    assert topk_idx.dtype == torch.int16 and topk_vals.dtype == torch.float32
    assert topk_idx.shape == (t, 4) and topk_vals.shape == (t, 4) and topk_idx.is_contiguous() and topk_vals.is_contiguous()
    e, inter = w1.codes.shape[0], w1.n // 2
    assert w1.k == hidden and (w2.n, w2.k) == (hidden, inter)
    out = torch.empty((t, hidden), dtype=_BF16, device=x.device)
    if t == 0:
        return out
    lib = _lib.load()
    need = lib.b2_moe_prefill_workspace_bytes(t, e, hidden, inter)
    key = (x.device, e, hidden, inter)
    hit = _moe_prefill_ws.get(key)
    if hit is None or hit[0].numel() < need:
        hit = (torch.empty(need, dtype=torch.uint8, device=x.device),
               torch.empty((e * 2 * inter, hidden), dtype=_BF16, device=x.device),
               torch.empty((e * hidden, inter), dtype=_BF16, device=x.device))
        _moe_prefill_ws[key] = hit
    ws, w1b, w2b = hit
    resident = getattr(w1, "_expanded", None)
    if resident is not None and resident[2] is w2:
        w1b, w2b = resident[0], resident[1]            # expanded by an earlier call
    else:
        size = (w1b.numel() + w2b.numel()) * 2
        keep = (_expanded_budget > 0 and _expanded_used.get(x.device, 0) + size <= _expanded_budget
                and not getattr(w1, "_shared_buffer", False))   # views of buffers that change content keep no copy
        if keep:                                       # this pair gets a copy of its own, made once
            w1b, w2b = torch.empty_like(w1b), torch.empty_like(w2b)
        _lib.call("b2_moe_upcast_packed", w1.codes.data_ptr(), w1.sf.data_ptr(), w1b.data_ptr(), e, 2 * inter, hidden, _stream())
        _lib.call("b2_moe_upcast_packed", w2.codes.data_ptr(), w2.sf.data_ptr(), w2b.data_ptr(), e, hidden, inter, _stream())
        if keep:
            w1._expanded = (w1b, w2b, w2)
            _expanded_used[x.device] = _expanded_used.get(x.device, 0) + size
    _lib.call("b2_moe_experts_prefill", x.data_ptr(), x.stride(0), topk_idx.data_ptr(), topk_vals.data_ptr(), w1b.data_ptr(),
              w1.bias.data_ptr(), w2b.data_ptr(), w2.bias.data_ptr(), out.data_ptr(), out.stride(0), ws.data_ptr(), ws.numel(),
              t, e, hidden, inter, float(alpha), float(limit), _stream())
    return out


def _prefill_moe_ok(t, w1, w2) -> bool:
    if not isinstance(w1, ExpertWeightsFp4):
        return False
    # with a resident bf16 copy of this pair the grouped GEMMs have no per-call expansion to amortise
    floor = PREFILL_MOE_MIN_TOKENS_RESIDENT if getattr(w1, "_expanded", None) is not None else PREFILL_MOE_MIN_TOKENS
    return t >= floor and w1.k % 192 == 0 and w1.n % 192 == 0 and w1.k % 8 == 0 and (w1.n // 2) % 8 == 0


def moe_experts(x, topk_vals, topk_idx, w1, w2, alpha=1.702, limit=7.0):
    """moe_experts (tritonllm/gpt_oss/triton/moe.py:54-87) for any number of tokens: the expert GEMMs of
    x [T, hidden] with the routing `topk` returned - the grouped tensor-core GEMM for prompt-sized batches, else the
    decode-sized kernel in calls of at most 2048 tokens."""
    t = x.shape[0]
    if _prefill_moe_ok(t, w1, w2):
        return moe_experts_prefill(x, topk_vals, topk_idx, w1, w2, alpha=alpha, limit=limit)
    block = 2048 if isinstance(w1, ExpertWeightsFp4) else 256
    if t <= block:
        return moe_experts_decode(x, topk_vals, topk_idx, w1, w2, alpha=alpha, limit=limit)
    out = torch.empty_like(x)
    for r0 in range(0, t, block):
        r1 = min(t, r0 + block)
        out[r0:r1] = moe_experts_decode(x[r0:r1], topk_vals[r0:r1], topk_idx[r0:r1], w1, w2, alpha=alpha, limit=limit)
    return out


def moe(x, wg, w1, w1_mx, w2, w2_mx, bg, b1, b2, experts_per_token=4, num_experts=128, swiglu_limit=7.0,
        fused_act=True, interleaved=True):
    """Drop-in for moe (tritonllm/gpt_oss/triton/moe.py:90-95): router matmul + bias, top-k with softmax, expert
    GEMMs with the fused clamped SwiGLU, weighted sum.  Takes the reference's wrapped weight tensors."""
    assert interleaved, "gate / linear features are interleaved in the checkpoint layout"
    return _moe_from_reference(x, wg, w1, w1_mx, w2, w2_mx, bg, b1, b2, experts_per_token, swiglu_limit)


def moe_decode(x, wg, w1, w1_mx, w2, w2_mx, bg, b1, b2, experts_per_token=4, num_experts=128, swiglu_limit=7.0,
               fused_act=True, interleaved=True):
    """Drop-in for moe_decode (tritonllm/gpt_oss/triton/moe.py:178-205); same contract as :func:`moe`."""
    assert interleaved, "gate / linear features are interleaved in the checkpoint layout"
    return _moe_from_reference(x, wg, w1, w1_mx, w2, w2_mx, bg, b1, b2, experts_per_token, swiglu_limit)
