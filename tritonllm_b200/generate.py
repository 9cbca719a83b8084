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
* the expert GEMMs of a prompt run through the decode-sized kernel in blocks of 2048 tokens.
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

    def __init__(self, batch_size, n_ctx, n_kv_heads, d_head=64, device=None, offset: torch.Tensor | None = None):
        self.k = torch.zeros((batch_size, n_ctx, n_kv_heads, d_head), dtype=torch.bfloat16, device=device)
        self.v = torch.zeros((batch_size, n_ctx, n_kv_heads, d_head), dtype=torch.bfloat16, device=device)
        self.owns_offset = offset is None
        self.offset = torch.zeros((1,), dtype=torch.long, device=device) if offset is None else offset
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

    PREFILL_ROWS = 8192      # rows (sequences x tokens) of one prompt slice
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

    def window(self, layer_idx: int) -> int:
        return self.config.sliding_window if layer_idx % 2 == 0 else 0   # model.py:448

    def make_caches(self, batch_size: int, n_ctx: int) -> list:
        c = self.config
        first = Cache(batch_size, n_ctx, c.num_key_value_heads, c.head_dim, device=self.device)
        return [first] + [Cache(batch_size, n_ctx, c.num_key_value_heads, c.head_dim, device=self.device, offset=first.offset)
                          for _ in range(c.num_hidden_layers - 1)]

    # ---- one block -------------------------------------------------------------------------------------
    def _moe(self, n2: torch.Tensor, p: LayerWeights) -> torch.Tensor:
        """Router, top-4 with softmax and the expert GEMMs (MLPBlock.forward, model.py:737-816) of
        normalised rows n2 [R, hidden]; returns the MoE output [R, hidden] (not yet added to the residual)."""
        logits = ops.router_logits(n2, p.wg, p.bg)
        vals, idx, _ = ops.topk(logits, self.config.experts_per_token)
        return self._experts(n2, vals, idx, p)

    def _experts(self, n2, vals, idx, p: LayerWeights) -> torch.Tensor:
        rows = n2.shape[0]
        block = self.MOE_BLOCK if isinstance(p.w1, ops.ExpertWeightsFp4) else min(256, self.MOE_BLOCK)
        if rows <= block:
            # a single call may leave the sum over a token's experts to the add + norm that follows it
            return ops.moe_experts_decode(n2, vals, idx, p.w1, p.w2, limit=self.config.swiglu_limit, defer_combine=True)
        out = torch.empty_like(n2)
        for r0 in range(0, rows, block):
            r1 = min(rows, r0 + block)
            out[r0:r1] = ops.moe_experts_decode(n2[r0:r1], vals[r0:r1], idx[r0:r1], p.w1, p.w2,
                                                limit=self.config.swiglu_limit)
        return out

    def _zeros_like(self, x):
        key = (tuple(x.shape), x.device)
        z = self._zero.get(key)
        if z is None:
            z = torch.zeros_like(x)
            self._zero[key] = z
        return z

    def _blocks(self, x: torch.Tensor, caches, position: torch.Tensor) -> torch.Tensor:
        """All blocks and the final norm for x [B, T, hidden] at positions position .. position+T-1.  The
        residual add that closes a block (x.add_(t), model.py:816) is fused into the norm that opens the next
        one, and the last one into the final norm."""
        c = self.config
        B, T, H = x.shape
        decode = T == 1 and caches is not None
        h, delta = x, self._zeros_like(x)
        hbuf, nbuf = torch.empty_like(x), torch.empty_like(x)
        for li, p in enumerate(self.w.layers):
            cache = caches[li] if caches is not None else None
            self._add_norm(h, delta, p.norm1, hbuf, nbuf)
            if decode:
                q = ops.qkv_rope_cache_decode_forward(nbuf, p.wqkv, p.bqkv, self.sin, self.cos, self.max_context_length,
                                                      cache.k, cache.v, position, c.num_attention_heads,
                                                      c.num_key_value_heads, c.head_dim)
                att = ops.attention_decode(q.view(B, 1, c.num_key_value_heads, -1, c.head_dim), cache.k, cache.v, p.sinks,
                                           self.sm_scale, self.window(li), position)
                h = ops.out_residual_decode_forward(att, p.wo, p.bo, hbuf)
            else:
                q, k, v = ops.qkv_rope_prefill(nbuf, p.wqkv, p.bqkv, self.sin, self.cos, self.max_context_length, position,
                                               c.num_attention_heads, c.num_key_value_heads, c.head_dim,
                                               cache_k=cache.k if cache is not None else None,
                                               cache_v=cache.v if cache is not None else None)
                att = ops.attention(q.view(B, T, c.num_key_value_heads, -1, c.head_dim), k, v, p.sinks, self.sm_scale,
                                    self.window(li), position)
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

    def __init__(self, model: Transformer, context: int, batch_size: int = 1, use_cuda_graph: bool | None = None):
        self.model, self.device, self.batch_size = model, model.device, batch_size
        if use_cuda_graph is None:
            use_cuda_graph = os.getenv("CUDA_GRAPH", "1").strip().lower() not in {"0", "false", "no", "off"}
        self.use_global_cuda_graph = use_cuda_graph
        self.caches = model.make_caches(batch_size, context)
        self.enable_dense_cache_sliding = all(cache.can_slide() for cache in self.caches)
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
            for cache in self.caches:
                cache.reset()

    @property
    def max_model_len(self) -> int:
        return min(self.model.max_context_length, self.caches[0].k.shape[1])

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
