"""KV store, whole-model forward and the batched decode loop on the CUDA path.

Host-side mirror of the reference's inference driver (tritonllm/gpt_oss/triton/model.py):
``ModelConfig`` (:36-53), ``Cache`` (:340-433), ``Transformer._forward_hidden`` / ``forward`` /
``forward_greedy`` / ``prefill`` (:909-936) and ``TokenGenerator`` (:1146-1396).  Every tensor
operation below is a call into this package's ``ops`` (the C ABI); torch only owns the memory, the
stream, the CUDA graph and the random numbers of the sampling branch.

Differences from the reference, all additive:

* the reference's generator holds one sequence; this one holds ``batch_size`` sequences of equal prompt
  length that advance in lock step (the KV store keeps the reference's single position counter for the
  whole batch, model.py:344);
* all layers share ONE position counter tensor, advanced once per step, instead of one per layer;
* a prompt is ingested in slices of sequences so that the activations of a slice stay small;
* the expert GEMMs of a prompt run through the decode-sized kernel in blocks of 2048 tokens;
* optionally every sequence has its own position (``Cache(per_sequence=True)``: prompts of different lengths in
  one batch) and the KV store may be paged (``PagedKVStore``: pages of a shared pool handed out per sequence).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field

import torch

from . import _lib, ops

_OFF = {"0", "false", "no", "off", ""}


@dataclass
class ModelConfig:
    """Field names and defaults of the reference's ModelConfig (model.py:36-53); the 20b checkpoint
    overrides num_hidden_layers=24, num_experts=32."""
    num_hidden_layers: int = 36
    num_experts: int = 128
    experts_per_token: int = 4
    vocab_size: int = 201088
    hidden_size: int = 2880
    intermediate_size: int = 2880
    swiglu_limit: float = 7.0
    head_dim: int = 64
    num_attention_heads: int = 64
    num_key_value_heads: int = 8
    sliding_window: int = 128
    initial_context_length: int = 4096
    rope_theta: float = 150000.0
    rope_scaling_factor: float = 32.0
    rope_ntk_alpha: float = 1.0
    rope_ntk_beta: float = 32.0

    @classmethod
    def gpt_oss_20b(cls, **kw):
        return cls(num_hidden_layers=24, num_experts=32, **kw)


class Cache:
    """Dense KV store of one layer: k, v [batch, n_ctx, kv_heads, d_head] bf16 and the position counter
    ``offset`` int64 (1,) (model.py:340-433).  ``offset`` may be a tensor shared by the stores of all
    layers; then only its owner advances it.  The sliding behaviour and its two environment switches
    (DENSE_CACHE_SLIDING, DENSE_CACHE_SLIDE_CHUNK) follow model.py:345-351."""

    paged = False

    def __init__(self, batch_size, n_ctx, n_kv_heads, d_head=64, device=None, offset: torch.Tensor | None = None,
                 per_sequence: bool = False):
        self.k = torch.zeros((batch_size, n_ctx, n_kv_heads, d_head), dtype=torch.bfloat16, device=device)
        self.v = torch.zeros((batch_size, n_ctx, n_kv_heads, d_head), dtype=torch.bfloat16, device=device)
        self.owns_offset = offset is None
        # one counter for the batch as in the reference, or (per_sequence) one per sequence, shape [batch]
        n_pos = batch_size if per_sequence else 1
        self.offset = torch.zeros((n_pos,), dtype=torch.long, device=device) if offset is None else offset
        self.per_sequence = per_sequence or self.offset.numel() != 1
        self.enable_sliding_window = os.getenv("DENSE_CACHE_SLIDING", "1").strip().lower() not in _OFF
        default_slide_chunk = max(256, min(n_ctx // 8, 4096))
        env = os.getenv("DENSE_CACHE_SLIDE_CHUNK")
        slide_chunk = int(env) if env is not None else default_slide_chunk
        self.slide_chunk = max(1, min(slide_chunk, n_ctx - 1)) if n_ctx > 1 else 0

    def reset(self):
        ops.kv_zero_tail(self.k, self.v, 0)
        if self.owns_offset:
            self.offset.zero_()

    def truncate(self, n_ctx):
        assert n_ctx <= self.k.shape[1]
        ops.kv_zero_tail(self.k, self.v, n_ctx)
        if self.owns_offset:
            self.offset.fill_(n_ctx)
        return self.k, self.v

    def can_slide(self) -> bool:
        return self.enable_sliding_window and self.slide_chunk > 0

    def slide_window(self, keep_last_n: int | None = None, current: int | None = None) -> int:
        """Drops the oldest entries and keeps the newest ``keep_last_n`` (default: capacity - slide_chunk)
        at the front of the store; returns the new position.  Same arithmetic as model.py:391-424."""
        if self.per_sequence:
            raise ValueError("sliding is defined for a store whose sequences share one position")
        if current is None:
            if not self.owns_offset:
                # the owner of a shared counter has already moved it when the loop reaches this layer
                raise ValueError("this Cache shares its position counter: pass `current` (the position before the slide)")
            current = int(self.offset.item())
        capacity = self.k.shape[1]
        if current < capacity or not self.can_slide():
            return current
        if keep_last_n is None:
            keep_last_n = capacity - self.slide_chunk
        keep_last_n = max(1, min(keep_last_n, capacity - 1, current))
        ops.kv_slide(self.k, self.v, current, keep_last_n)
        if self.owns_offset:
            self.offset.fill_(keep_last_n)
        return keep_last_n

    def batch_slice(self, b0: int, b1: int) -> "_CacheView":
        return _CacheView(self.k[b0:b1], self.v[b0:b1], self.offset)


class PagedKVStore:
    """KV store of all layers as pools of pages: per layer k, v [n_pages, page_size, kv_heads, d_head] bf16; ONE
    block table int32 [batch, max_pages] (the page of tokens page_size*j .. of sequence b, -1 = none yet) and ONE
    position vector int64 [batch] shared by the layers.  Pages are handed out on the host from a free list
    (``ensure``) and returned with ``release``; the kernels only read the table.  The reference has no paged store
    (model.py:340-433 is dense): layout and bookkeeping are this library's, the arithmetic on the pages is the
    decode kernels'."""

    def __init__(self, n_layers, batch_size, n_ctx, n_kv_heads, d_head=64, page_size=64, n_pages=None, device=None):
        assert page_size % 32 == 0, "a 32-key attention tile must lie inside one page"
        self.page_size, self.batch_size = page_size, batch_size
        self.max_pages = -(-n_ctx // page_size)
        self.capacity = self.max_pages * page_size
        self.n_pages = n_pages if n_pages is not None else batch_size * self.max_pages
        self.k = [torch.zeros((self.n_pages, page_size, n_kv_heads, d_head), dtype=torch.bfloat16, device=device)
                  for _ in range(n_layers)]
        self.v = [torch.zeros_like(t) for t in self.k]
        self.block_table = torch.full((batch_size, self.max_pages), -1, dtype=torch.int32, device=device)
        self.positions = torch.zeros((batch_size,), dtype=torch.long, device=device)
        self._free = list(range(self.n_pages - 1, -1, -1))
        self._owned = [[] for _ in range(batch_size)]

    def ensure(self, b: int, n_tokens: int) -> None:
        """Makes sure sequence b owns pages for its first ``n_tokens`` tokens."""
        need = -(-n_tokens // self.page_size)
        if need > self.max_pages:
            raise ValueError(f"{n_tokens} tokens exceed the capacity of a sequence ({self.capacity})")
        have = len(self._owned[b])
        if need <= have:
            return
        if need - have > len(self._free):
            raise RuntimeError("the page pool is exhausted")
        new = [self._free.pop() for _ in range(need - have)]
        self._owned[b].extend(new)
        self.block_table[b, have:need] = torch.tensor(new, dtype=torch.int32, device=self.block_table.device)

    def release(self, b: int) -> None:
        self._free.extend(reversed(self._owned[b]))
        self._owned[b] = []
        self.block_table[b].fill_(-1)
        self.positions[b] = 0

    def reset(self) -> None:
        for b in range(self.batch_size):
            self.release(b)

    def layer(self, li: int) -> "_PagedLayer":
        return _PagedLayer(self, li)

    def rows_of(self, b: int, n_tokens: int) -> torch.Tensor:
        """Row index (page * page_size + slot) in the flattened pool of tokens 0 .. n_tokens-1 of sequence b."""
        pages = self.block_table[b, : -(-n_tokens // self.page_size)].long()
        return (pages[:, None] * self.page_size + torch.arange(self.page_size, device=pages.device)[None, :]).reshape(-1)[:n_tokens]


class _PagedLayer:
    """One layer of a PagedKVStore, in the role a Cache plays for a dense store."""
    paged = True
    per_sequence = True
    owns_offset = False

    def __init__(self, store: PagedKVStore, li: int):
        self.store, self.k, self.v = store, store.k[li], store.v[li]
        self.block_table, self.offset = store.block_table, store.positions

    def write_prompt(self, b: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """K/V rows [T, heads, d] of a freshly ingested prompt of sequence b into its pages (Cache.extend's role)."""
        rows = self.store.rows_of(b, k.shape[0])
        self.k.view(-1, *self.k.shape[2:]).index_copy_(0, rows, k)
        self.v.view(-1, *self.v.shape[2:]).index_copy_(0, rows, v)


def check_device_status(where: str) -> None:
    """Raises B2Error when a kernel of this process has recorded a failure in the per-device status word since the
    last check (a bounded wait that gave up, a token id or expert index out of range): such a kernel carries on
    with defined but wrong data, so the results produced since the last check must not be used.  Reads one word
    from the device; call it after a synchronisation point, not inside a captured step."""
    code = _lib.device_status()
    if code:
        raise _lib.B2Error(where, code, f"device status word 0x{code:x} (0x1/0x2/0x4/0x8: a bounded wait gave up; "
                                        "0x10: an index was out of range)")


@dataclass
class _CacheView:
    k: torch.Tensor
    v: torch.Tensor
    offset: torch.Tensor
    paged = False
    per_sequence = False


@dataclass
class LayerWeights:
    """One TransformerBlock (model.py:436-468, 578-667): gains fp32, dense weights bf16 in the reference's
    [out, in] layout, gate weight [hidden, experts] bf16 with fp32 bias, experts as ops.ExpertWeights or
    ops.ExpertWeightsFp4."""
    norm1: torch.Tensor
    wqkv: torch.Tensor
    bqkv: torch.Tensor
    sinks: torch.Tensor
    wo: torch.Tensor
    bo: torch.Tensor
    norm2: torch.Tensor
    wg: torch.Tensor
    bg: torch.Tensor
    w1: object
    w2: object


@dataclass
class ModelWeights:
    embedding: torch.Tensor
    layers: list = field(default_factory=list)
    norm: torch.Tensor | None = None
    unembedding: torch.Tensor | None = None

    @classmethod
    def random(cls, config: ModelConfig, device, seed: int = 0, fp4: bool = True, std: float = 0.02, draw_on=None):
        """Seeded random weights of the architecture (no checkpoint is read): dense weights N(0, std) bf16,
        gains N(1, 0.05), sinks N(0, 1), expert codes uniform over the 16 nibbles with scales 2^-9 .. 2^-4.
        ``draw_on`` names the device whose generator draws the numbers (default: ``device``); "cpu" gives
        the same weights on every machine."""
        target, device = device, (draw_on or device)
        g = torch.Generator(device=device).manual_seed(seed)
        c = config
        H, I, E = c.hidden_size, c.intermediate_size, c.num_experts
        qkv_dim = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim

        def bf(*shape, scale=std):
            return (torch.randn(*shape, device=device, generator=g) * scale).to(torch.bfloat16).to(target)

        def gain():
            return (1.0 + 0.05 * torch.randn(H, device=device, generator=g)).to(target)

        def experts(n, k):
            w = ops.ExpertWeights(
                torch.randint(0, 256, (E, n, k // 2), dtype=torch.uint8, device=device, generator=g).to(target),
                torch.randint(118, 124, (E, n, k // 32), dtype=torch.uint8, device=device, generator=g).to(target),
                (torch.randn(E, n, device=device, generator=g) * 0.05).to(target))
            return ops.ExpertWeightsFp4(w) if fp4 else w

        layers = [LayerWeights(norm1=gain(), wqkv=bf(qkv_dim, H), bqkv=bf(qkv_dim),
                               sinks=torch.randn(c.num_attention_heads, device=device, generator=g).to(torch.bfloat16).to(target),
                               wo=bf(H, c.num_attention_heads * c.head_dim), bo=bf(H), norm2=gain(), wg=bf(H, E),
                               bg=(torch.randn(E, device=device, generator=g) * 0.02).to(target), w1=experts(2 * I, H),
                               w2=experts(H, I))
                  for _ in range(c.num_hidden_layers)]
        return cls(embedding=bf(c.vocab_size, H, scale=1.0), layers=layers, norm=gain(), unembedding=bf(c.vocab_size, H))


class Transformer:
    """Inference forward of the whole model (Transformer, model.py:886-936)."""

    PREFILL_ROWS = 16384     # rows (sequences x tokens) of one prompt slice: the expert weights are expanded once per slice and layer
    MOE_BLOCK = 2048         # tokens per call of the expert kernel (256 when the weights are not FP4-packed)
    FUSED_ROUTER_ROWS = 512  # up to this many rows the norm, the router and the top-k run as one launch

    def __init__(self, config: ModelConfig, weights: ModelWeights, max_context: int | None = None, eps: float = 1e-5):
        self.config, self.w, self.eps = config, weights, eps
        c = config
        self.device = weights.embedding.device
        self.max_context_length = int(max_context or c.initial_context_length * c.rope_scaling_factor)
        self.cos, self.sin = ops.yarn_cos_sin(self.max_context_length, head_dim=c.head_dim, base=c.rope_theta,
                                              factor=c.rope_scaling_factor, orig_ctx=c.initial_context_length,
                                              alpha=c.rope_ntk_alpha, beta=c.rope_ntk_beta, device=self.device)
        self.sm_scale = 1.0 / (c.head_dim ** 0.5)
        self._zero: dict = {}
        self.expert_cache = None   # set by offload_experts()

    def offload_experts(self, resident_layers: int = 0, victim_slots: int = 0):
        """The reference's ``cpu_offload`` mode (Transformer.from_checkpoint(..., cpu_offload=True), model.py:945-962,
        1005-1134): every layer's FP4-packed experts move to pinned host memory and one shared set of GPU buffers
        serves all layers; the first ``resident_layers`` layers keep a copy on the GPU and ``victim_slots`` evicted experts
        are kept in a second-level GPU store.  The step then has a host
        synchronisation per layer (which experts were chosen) and cannot be captured in a CUDA graph."""
        from .expert_cache import ExpertOffloadCache
        assert all(isinstance(p.w1, ops.ExpertWeightsFp4) for p in self.w.layers), "offload works on FP4-packed experts"
        cache = ExpertOffloadCache(self.config.num_experts, self.device)
        for li, p in enumerate(self.w.layers):
            cache.register_layer(li, p.w1, p.w2, keep_on_gpu=li < resident_layers)
            p.w1 = p.w2 = None   # the host copy (or the resident copy) is the only one from here on
            p.offload_layer = li
        cache.init_victim_store(victim_slots)
        self.expert_cache = cache
        return cache

    def window(self, layer_idx: int) -> int:
        return self.config.sliding_window if layer_idx % 2 == 0 else 0   # model.py:448

    def make_caches(self, batch_size: int, n_ctx: int, per_sequence: bool = False) -> list:
        c = self.config
        first = Cache(batch_size, n_ctx, c.num_key_value_heads, c.head_dim, device=self.device, per_sequence=per_sequence)
        return [first] + [Cache(batch_size, n_ctx, c.num_key_value_heads, c.head_dim, device=self.device, offset=first.offset,
                                per_sequence=per_sequence)
                          for _ in range(c.num_hidden_layers - 1)]

    def make_paged_store(self, batch_size: int, n_ctx: int, page_size: int = 64, n_pages: int | None = None) -> PagedKVStore:
        c = self.config
        return PagedKVStore(c.num_hidden_layers, batch_size, n_ctx, c.num_key_value_heads, c.head_dim, page_size, n_pages,
                            device=self.device)

    # ---- one block -------------------------------------------------------------------------------------
    def _moe(self, n2: torch.Tensor, p: LayerWeights) -> torch.Tensor:
        """Router, top-4 with softmax and the expert GEMMs (MLPBlock.forward, model.py:737-816) of
        normalised rows n2 [R, hidden]; returns the MoE output [R, hidden] (not yet added to the residual)."""
        logits = ops.router_logits(n2, p.wg, p.bg)
        vals, idx, _ = ops.topk(logits, self.config.experts_per_token)
        return self._experts(n2, vals, idx, p)

    def _offloaded(self, li: int, idx: torch.Tensor):
        """(w1, w2) of layer li in the shared GPU buffers, holding at least the experts idx names (a host sync)."""
        ids = torch.unique(idx).tolist()
        return self.expert_cache.ensure_experts(li, [e for e in ids if 0 <= e < self.config.num_experts])

    def _experts(self, n2, vals, idx, p: LayerWeights) -> torch.Tensor:
        rows = n2.shape[0]
        w1, w2 = p.w1, p.w2
        if self.expert_cache is not None:   # offload mode: the routed experts are brought into the shared buffers first
            w1, w2 = self._offloaded(p.offload_layer, idx)
        block = self.MOE_BLOCK if isinstance(w1, ops.ExpertWeightsFp4) else min(256, self.MOE_BLOCK)
        if rows <= block:
            # a single call may leave the sum over a token's experts to the add + norm that follows it
            return ops.moe_experts_decode(n2, vals, idx, w1, w2, limit=self.config.swiglu_limit, defer_combine=True)
        if ops._prefill_moe_ok(rows, w1, w2):   # prompt-sized: tokens as the M rows of a grouped GEMM
            return ops.moe_experts_prefill(n2, vals, idx, w1, w2, limit=self.config.swiglu_limit)
        out = torch.empty_like(n2)
        for r0 in range(0, rows, block):
            r1 = min(rows, r0 + block)
            out[r0:r1] = ops.moe_experts_decode(n2[r0:r1], vals[r0:r1], idx[r0:r1], w1, w2,
                                                limit=self.config.swiglu_limit)
        return out

    def _zeros_like(self, x):
        key = (tuple(x.shape), x.device)
        z = self._zero.get(key)
        if z is None:
            z = torch.zeros_like(x)
            self._zero[key] = z
        return z

    def _blocks(self, x: torch.Tensor, caches, position: torch.Tensor, seq_index: int | None = None) -> torch.Tensor:
        """All blocks and the final norm for x [B, T, hidden] at positions position .. position+T-1.  The
        residual add that closes a block (x.add_(t), model.py:816) is fused into the norm that opens the next
        one, and the last one into the final norm."""
        c = self.config
        B, T, H = x.shape
        decode = T == 1 and caches is not None and seq_index is None   # prefill_sequence ingests even a 1-token prompt
        h, delta = x, self._zeros_like(x)
        hbuf, nbuf = torch.empty_like(x), torch.empty_like(x)
        for li, p in enumerate(self.w.layers):
            cache = caches[li] if caches is not None else None
            self._add_norm(h, delta, p.norm1, hbuf, nbuf)
            if decode and cache.paged:
                q = ops.qkv_rope_paged_decode_forward(nbuf, p.wqkv, p.bqkv, self.sin, self.cos, self.max_context_length,
                                                      cache.k, cache.v, cache.block_table, position, c.num_attention_heads,
                                                      c.num_key_value_heads, c.head_dim, kv_capacity=cache.store.capacity)
                att = ops.attention_decode_paged(q.view(B, 1, c.num_key_value_heads, -1, c.head_dim), cache.k, cache.v,
                                                 cache.block_table, position, p.sinks, self.sm_scale, self.window(li),
                                                 kv_capacity=cache.store.capacity)
                h = ops.out_residual_decode_forward(att, p.wo, p.bo, hbuf)
            elif decode:
                per_seq = getattr(cache, "per_sequence", False)
                q = ops.qkv_rope_cache_decode_forward(nbuf, p.wqkv, p.bqkv, self.sin, self.cos, self.max_context_length,
                                                      cache.k, cache.v, position, c.num_attention_heads,
                                                      c.num_key_value_heads, c.head_dim, per_sequence=per_seq)
                att = ops.attention_decode(q.view(B, 1, c.num_key_value_heads, -1, c.head_dim), cache.k, cache.v, p.sinks,
                                           self.sm_scale, self.window(li), position, per_sequence=per_seq)
                h = ops.out_residual_decode_forward(att, p.wo, p.bo, hbuf)
            else:
                dense = cache is not None and not cache.paged
                q, k, v = ops.qkv_rope_prefill(nbuf, p.wqkv, p.bqkv, self.sin, self.cos, self.max_context_length, position,
                                               c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                                               cache_k=cache.k if dense else None, cache_v=cache.v if dense else None)
                att = ops.attention(q.view(B, T, c.num_key_value_heads, -1, c.head_dim), k, v, p.sinks, self.sm_scale,
                                    self.window(li), position)
                if cache is not None and cache.paged:   # a whole prompt of one sequence, ingested from position 0
                    cache.write_prompt(seq_index, k[0], v[0])
                h = ops.out_residual_forward(att, p.wo, p.bo, hbuf, out=hbuf)
            if B * T <= self.FUSED_ROUTER_ROWS and c.num_experts % 32 == 0 and c.experts_per_token <= 4:
                n2, vals, idx = ops.norm_router_topk(h, p.norm2, self.eps, p.wg, p.bg, c.experts_per_token, y_out=nbuf)
                delta = self._experts(n2.view(B * T, H), vals, idx, p)
            else:
                n2 = ops.rmsnorm_forward(h, p.norm2, self.eps, out=nbuf)
                delta = self._moe(n2.view(B * T, H), p)
            if isinstance(delta, torch.Tensor):
                delta = delta.view(B, T, H)
        self._add_norm(h, delta, self.w.norm, hbuf, nbuf)
        return nbuf

    def _add_norm(self, h, delta, gain, hbuf, nbuf):
        """hbuf = h + delta, nbuf = norm(hbuf); delta is a tensor or the pending expert outputs of the last MoE."""
        if isinstance(delta, ops.PendingMoe):
            ops.moe_combine_add_rmsnorm(delta, h, gain, self.eps, h_out=hbuf, y_out=nbuf)
        else:
            ops.add_rmsnorm_forward(h, delta, gain, self.eps, h_out=hbuf, y_out=nbuf)

    # ---- the reference's entry points --------------------------------------------------------------------
    def _forward_hidden(self, tokens: torch.Tensor, caches=None) -> torch.Tensor:
        """tokens [B, T] -> normalised hidden states [B, T, hidden]; with caches the K/V of the T tokens are
        written at the current position and the position advances by T (model.py:909-914)."""
        B, T = tokens.shape
        if caches is None:
            position = torch.zeros(1, dtype=torch.int64, device=self.device)
            return self._blocks(ops.embedding_forward(tokens, self.w.embedding), None, position)
        position = caches[0].offset
        if T == 1:
            out = self._blocks(ops.embedding_forward(tokens, self.w.embedding), caches, position)
            if caches[0].paged:
                position.add_(1)
        elif caches[0].per_sequence:
            raise ValueError("a store with per-sequence positions ingests prompts one sequence at a time: prefill_sequence()")
        else:
            out = torch.empty((B, T, self.config.hidden_size), dtype=torch.bfloat16, device=self.device)
            step = max(1, self.PREFILL_ROWS // T)
            for b0 in range(0, B, step):
                b1 = min(B, b0 + step)
                views = [cch.batch_slice(b0, b1) for cch in caches]
                out[b0:b1] = self._blocks(ops.embedding_forward(tokens[b0:b1], self.w.embedding), views, position)
        for cch in caches:
            if cch.owns_offset:
                cch.offset.add_(T)
        return out

    def prefill_sequence(self, tokens: torch.Tensor, caches, b: int) -> torch.Tensor:
        """Ingests the prompt ``tokens`` [T] of sequence ``b`` alone, from position 0, into a store whose sequences
        have their own positions (dense ``Cache(per_sequence=True)`` layers or the layers of a ``PagedKVStore``) and sets
        that sequence's position to T.  Returns the normalised hidden states [1, T, hidden]."""
        T = tokens.shape[0]
        zero = self._zero.setdefault("pos0", torch.zeros(1, dtype=torch.int64, device=self.device))
        if caches[0].paged:
            caches[0].store.ensure(b, T)
            views = caches
        else:
            assert caches[0].per_sequence
            views = [_CacheView(cch.k[b:b + 1], cch.v[b:b + 1], zero) for cch in caches]
        out = self._blocks(ops.embedding_forward(tokens[None, :], self.w.embedding), views, zero, seq_index=b)
        caches[0].offset[b] = T
        return out

    def forward(self, tokens: torch.Tensor, caches=None) -> torch.Tensor:
        """fp32 logits [B, T, vocab] (model.py:916-919)."""
        x = self._forward_hidden(tokens, caches)
        if x.shape[1] == 1:
            return ops.unembedding_decode_forward(x, self.w.unembedding).float()
        zero_bias = self._zero.setdefault("unembed_bias", torch.zeros(self.w.unembedding.shape[0], dtype=torch.bfloat16,
                                                                      device=self.device))
        return ops.linear_bias(x, self.w.unembedding, zero_bias).float()

    def forward_greedy(self, tokens: torch.Tensor, caches=None) -> torch.Tensor:
        """Token ids [B] of the arg-max logits of a one-token step (model.py:921-925)."""
        x = self._forward_hidden(tokens, caches)
        assert x.shape[1] == 1
        return ops.unembedding_decode_argmax_forward(x, self.w.unembedding)

    def prefill(self, tokens: torch.Tensor, caches) -> torch.Tensor:
        """Fills the KV store for a prompt without the vocabulary projection (model.py:927-929)."""
        return self._forward_hidden(tokens, caches)


class TokenGenerator:
    """Batched counterpart of the reference's TokenGenerator (model.py:1146-1396): ``batch_size`` sequences
    with prompts of one common length, a KV store of ``context`` tokens per sequence, the one-token step
    captured in CUDA graphs (one returning logits, one returning greedy ids; CUDA_GRAPH=0 turns capture off)."""

    def __init__(self, model: Transformer, context: int, batch_size: int = 1, use_cuda_graph: bool | None = None,
                 per_sequence: bool = False, paged: bool = False, page_size: int = 64, n_pages: int | None = None):
        """``per_sequence``: every sequence keeps its own position, so ``generate_ragged`` can take prompts of different
        lengths; ``paged`` (implies per_sequence): the KV store is a PagedKVStore of ``n_pages`` pages of ``page_size``
        tokens (default: enough for every sequence to reach ``context``)."""
        self.model, self.device, self.batch_size = model, model.device, batch_size
        if use_cuda_graph is None:
            use_cuda_graph = os.getenv("CUDA_GRAPH", "1").strip().lower() not in {"0", "false", "no", "off"}
        if model.expert_cache is not None:
            use_cuda_graph = False   # the offload mode asks the host which experts were chosen, once per layer
        self.use_global_cuda_graph = use_cuda_graph
        self.per_sequence = per_sequence or paged
        self.store = model.make_paged_store(batch_size, context, page_size, n_pages) if paged else None
        if paged:
            self.caches = [self.store.layer(li) for li in range(model.config.num_hidden_layers)]
            for b in range(batch_size):          # the capture steps below write one token per sequence
                self.store.ensure(b, 1)
        else:
            self.caches = model.make_caches(batch_size, context, per_sequence=per_sequence)
        self.enable_dense_cache_sliding = not self.per_sequence and all(cache.can_slide() for cache in self.caches)
        self.enable_repeat_pattern_stop = os.getenv("DENSE_REPEAT_PATTERN_STOP", "0").strip().lower() not in _OFF
        self.input_token = torch.zeros((batch_size, 1), dtype=torch.int64, device=self.device)
        self._sampling_graph = self._greedy_graph = None
        self._greedy_token = self.logits = None
        self._noise = None
        self.last_generation_stats = None
        if self.use_global_cuda_graph:
            # one eager step first so that every lazily created buffer exists before capture
            model.forward_greedy(self.input_token, caches=self.caches)
            model.forward(self.input_token, caches=self.caches)
            torch.cuda.synchronize(self.device)
            self._greedy_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._greedy_graph):
                self._greedy_token = model.forward_greedy(self.input_token, caches=self.caches)
            self._sampling_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._sampling_graph):
                self.logits = model.forward(self.input_token, caches=self.caches)[:, 0]
            self._reset_store()

    def _reset_store(self):
        if self.store is not None:
            self.store.reset()
        else:
            for cache in self.caches:
                cache.reset()

    @property
    def max_model_len(self) -> int:
        cap = self.store.capacity if self.store is not None else self.caches[0].k.shape[1]
        return min(self.model.max_context_length, cap)

    def sample_next_token(self, logits: torch.Tensor, temperature: float) -> torch.Tensor:
        """logits fp32 [B, vocab] -> ids [B]; Gumbel-max sampling as model.py:1210-1221."""
        if temperature == 0.0:
            return logits.argmax(dim=-1)
        if self._noise is None or self._noise.shape != logits.shape:
            self._noise = torch.empty_like(logits)
        self._noise.exponential_().log_().neg_().mul_(temperature).add_(logits)
        return self._noise.argmax(dim=-1)

    def _handle_kv_capacity(self, decode_offset: int):
        """model.py:1223-1256: when the store is full either stop or slide every layer's store."""
        if decode_offset < self.max_model_len:
            return True, decode_offset
        if not self.enable_dense_cache_sliding:
            return False, decode_offset
        new_offset = None
        for cache in self.caches:
            kept = cache.slide_window(current=decode_offset)
            assert new_offset is None or new_offset == kept
            new_offset = kept
        return True, new_offset

    @staticmethod
    def _has_repeating_token_pattern(recent_tokens, min_pattern_len=2, max_pattern_len=8, min_repeats=8) -> bool:
        """True when the newest tokens are ``min_repeats`` back-to-back copies of one pattern of 2 to 8 tokens
        (model.py:1258-1276)."""
        n = len(recent_tokens)
        for plen in range(min_pattern_len, max_pattern_len + 1):
            need = plen * min_repeats
            if n < need:
                continue
            tail = recent_tokens[n - need:]
            if all(tail[i] == tail[i % plen] for i in range(need)):
                return True
        return False

    def _step(self, greedy: bool) -> torch.Tensor:
        """One token for every sequence from ``self.input_token``; returns greedy ids [B] or fp32 logits [B, vocab]."""
        if self.use_global_cuda_graph:
            (self._greedy_graph if greedy else self._sampling_graph).replay()
            return self._greedy_token if greedy else self.logits
        if greedy:
            return self.model.forward_greedy(self.input_token, caches=self.caches)
        return self.model.forward(self.input_token, caches=self.caches)[:, 0]

    @torch.inference_mode()
    def generate(self, prompt_tokens, stop_tokens=None, temperature: float = 1.0, max_tokens: int = 0,
                 return_logprobs: bool = False, enable_repeat_pattern_stop: bool | None = None):
        """Yields, per step, the list of the ``batch_size`` new token ids (a plain int when batch_size is 1,
        as the reference does), or (ids, logprobs) with ``return_logprobs``.  ``prompt_tokens``: one list of
        ints (batch 1), a list of equally long lists, or an integer tensor [B, P].  Generation ends after
        ``max_tokens`` steps (0 = until the other conditions), when every sequence has produced a stop token,
        when the KV store is full and sliding is off, or on a repeating pattern (batch 1 only, when enabled).
        A sequence that has stopped keeps stepping with the others; its later tokens are to be ignored."""
        stop = set(stop_tokens or [])
        if enable_repeat_pattern_stop is None:
            enable_repeat_pattern_stop = self.enable_repeat_pattern_stop
        self.last_generation_stats = None
        prompts = torch.as_tensor(prompt_tokens, dtype=torch.int64)
        if prompts.dim() == 1:
            prompts = prompts[None, :]
        if prompts.shape[0] != self.batch_size:
            raise ValueError(f"expected {self.batch_size} prompts, got {prompts.shape[0]}")
        if prompts.shape[1] == 0:
            raise ValueError("empty prompt")
        if prompts.shape[1] > self.max_model_len:
            raise ValueError(f"Prompt is too long: {prompts.shape[1]} tokens exceeds max_model_len={self.max_model_len}. "
                             "Truncate the conversation history before calling generate().")
        prompts = prompts.to(self.device)
        for cache in self.caches:
            cache.reset()
        decode_offset = prompts.shape[1] - 1
        prefill_elapsed = 0.0
        if decode_offset > 0:
            torch.cuda.synchronize(self.device)
            t0 = time.perf_counter()
            self.model.prefill(prompts[:, :-1], self.caches)
            torch.cuda.synchronize(self.device)
            prefill_elapsed = time.perf_counter() - t0
            check_device_status("prefill")
        self.input_token.copy_(prompts[:, -1:])
        greedy = temperature == 0.0 and not return_logprobs
        need_host = bool(stop) or return_logprobs or enable_repeat_pattern_stop
        finished = [False] * self.batch_size
        recent: list[int] = []
        loop_detected = False
        produced = 0
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        while max_tokens == 0 or produced < max_tokens:
            can_continue, decode_offset = self._handle_kv_capacity(decode_offset)
            if not can_continue:
                break
            out = self._step(greedy)
            ids = out if greedy else self.sample_next_token(out, temperature)
            self.input_token.copy_(ids.view(-1, 1))
            decode_offset += 1
            produced += 1
            if return_logprobs:
                lp = torch.log_softmax(out, dim=-1).gather(1, ids.view(-1, 1))[:, 0].tolist()
            ids_host = ids.tolist()
            check_device_status("generate")   # the copy above has synchronised; a failed step must not be yielded
            if self.batch_size == 1:
                yield (ids_host[0], lp[0]) if return_logprobs else ids_host[0]
            else:
                yield (ids_host, lp) if return_logprobs else ids_host
            if enable_repeat_pattern_stop and self.batch_size == 1:
                recent.append(ids_host[0])
                if len(recent) > 64:
                    recent.pop(0)
                if self._has_repeating_token_pattern(recent):
                    loop_detected = True
                    break
            if need_host and stop:
                finished = [f or (t in stop) for f, t in zip(finished, ids_host)]
                if all(finished):
                    break
        torch.cuda.synchronize(self.device)
        check_device_status("generate")
        self.last_generation_stats = {"generated_tokens": produced, "prefill_time_s": prefill_elapsed,
                                      "decode_time_s": time.perf_counter() - t0, "loop_detected": loop_detected}

    @torch.inference_mode()
    def generate_greedy(self, prompts: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Throughput form of ``generate`` at temperature 0 with no stop condition: prompts [B, P] on the
        device, returns the ``new_tokens`` generated ids [B, new_tokens] without touching the host between
        steps (one graph replay and one small copy per step)."""
        assert prompts.shape[0] == self.batch_size and prompts.shape[1] >= 1
        for cache in self.caches:
            cache.reset()
        decode_offset = prompts.shape[1] - 1
        if decode_offset > 0:
            self.model.prefill(prompts[:, :-1], self.caches)
        self.input_token.copy_(prompts[:, -1:])
        out = torch.empty((self.batch_size, new_tokens), dtype=torch.int64, device=self.device)
        for i in range(new_tokens):
            can_continue, decode_offset = self._handle_kv_capacity(decode_offset)
            if not can_continue:
                out = out[:, :i]
                break
            ids = self._step(True)
            self.input_token.copy_(ids.view(-1, 1))
            out[:, i].copy_(ids)
            decode_offset += 1
        torch.cuda.synchronize(self.device)
        check_device_status("generate_greedy")
        return out

    @torch.inference_mode()
    def generate_ragged(self, prompts: list, new_tokens: int, return_first_logits: bool = False):
        """Greedy generation for prompts of DIFFERENT lengths in one batch (needs ``per_sequence`` or ``paged``):
        ``prompts`` is a list of ``batch_size`` token lists.  Every prompt is ingested on its own, then all sequences
        step together, each at its own position.  Returns ids [B, new_tokens]; with ``return_first_logits`` also the
        fp32 logits [B, vocab] of the first step.  Stops early when the longest sequence fills its store."""
        if not self.per_sequence:
            raise ValueError("this generator was built with one position for the whole batch")
        if len(prompts) != self.batch_size or any(len(p) == 0 for p in prompts):
            raise ValueError(f"expected {self.batch_size} non-empty prompts")
        longest = max(len(p) for p in prompts)
        if longest > self.max_model_len:
            raise ValueError(f"Prompt is too long: {longest} tokens exceeds max_model_len={self.max_model_len}.")
        self._reset_store()
        last = []
        for b, p in enumerate(prompts):
            t = torch.as_tensor(p, dtype=torch.int64, device=self.device)
            if self.store is not None:
                self.store.ensure(b, min(self.max_model_len, len(p) + new_tokens))
            if len(p) > 1:
                self.model.prefill_sequence(t[:-1], self.caches, b)
            last.append(int(p[-1]))
        self.input_token.copy_(torch.tensor(last, dtype=torch.int64, device=self.device).view(-1, 1))
        out = torch.empty((self.batch_size, new_tokens), dtype=torch.int64, device=self.device)
        first_logits = None
        n_done = new_tokens
        for i in range(new_tokens):
            if longest - 1 + i >= self.max_model_len:
                n_done = i
                break
            if i == 0 and return_first_logits:
                first_logits = self._step(False).clone()
                ids = first_logits.argmax(dim=-1)
            else:
                ids = self._step(True)
            self.input_token.copy_(ids.view(-1, 1))
            out[:, i].copy_(ids)
        torch.cuda.synchronize(self.device)
        check_device_status("generate_ragged")
        out = out[:, :n_done]
        return (out, first_logits) if return_first_logits else out
