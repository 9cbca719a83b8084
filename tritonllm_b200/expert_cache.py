"""Expert weights in host memory, one shared set of GPU buffers: the optional CPU-offload mode of the MoE block.

Mirrors the role of the reference's ``ExpertCache`` (tritonllm/gpt_oss/triton/expert_cache.py:19-460 and its use in
``MLPBlock.forward``, tritonllm/gpt_oss/triton/model.py:756-800): every layer's expert weights live in (pinned) host
memory, a single set of ``[num_experts, ...]`` GPU buffers is shared by all layers, and before a layer's expert GEMMs
the experts its tokens were routed to are copied into their slots of those buffers - slot e always holds expert e of
*some* layer, and ``gpu_layer[e]`` says which.  A copy is skipped when the slot already holds this layer's expert (the
next token of the same layer usually asks for some of the same experts), layers registered with ``keep_on_gpu=True``
are served by device-to-device copies from a resident copy, and hits and misses are counted as the reference counts
them.  ``init_victim_store(slots)`` adds the reference's second level (``init_victim_cache`` / ``_vc_put`` / ``_vc_get``,
expert_cache.py:227-327): before a slot of the shared buffers is overwritten by another layer's expert, its content is
saved device-to-device into a store of ``slots`` whole experts, least recently used first out, and a later request for
that (layer, expert) is served from there instead of over PCIe (counted as a hit).

The buffers have the layout the FP4 expert kernels read (``ops.ExpertWeightsFp4``: codes ``[E, N, Kp/2]``, scale
blocks ``[E, ceil(N/128), Kp/128, 32, 4, 4]``, bias ``[E, N]``), so ``ensure_experts`` returns a pair of
``ExpertWeightsFp4`` views of the shared buffers that ``ops.moe_experts_decode`` takes as they are.  On a B200 the
mode is only needed for models whose experts do not fit in 180 GB; it trades PCIe copies (13 MB per expert of the 20b
model) and a host synchronisation per layer for memory, and it cannot run inside a CUDA graph.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass

import torch


@dataclass
class _Packed:
    """The three tensors of one projection's packed experts (any device)."""
    codes: torch.Tensor
    sf: torch.Tensor
    bias: torch.Tensor
    n: int
    k: int

    def expert(self, e: int):
        return self.codes[e], self.sf[e], self.bias[e]


def _packed_of(w) -> _Packed:
    return _Packed(w.codes, w.sf, w.bias, int(w.n), int(w.k))


class ExpertOffloadCache:
    def __init__(self, num_experts: int, device, pin_memory: bool | None = None):
        self.num_experts = int(num_experts)
        self.device = torch.device(device)
        self.pin = (self.device.type == "cuda") if pin_memory is None else bool(pin_memory)
        self.host: dict[int, tuple[_Packed, _Packed]] = {}        # layer -> (w1, w2) in host memory
        self.resident: dict[int, tuple[_Packed, _Packed]] = {}    # layers kept on the GPU (served by device copies)
        self.gpu: tuple[_Packed, _Packed] | None = None           # the shared buffers
        self.gpu_layer: list[int] = [-1] * self.num_experts       # which layer's expert each slot holds
        self._hits = 0
        self._misses = 0
        self.victims: tuple[_Packed, _Packed] | None = None              # [slots, ...] copies of evicted experts
        self._victim_of: OrderedDict[tuple[int, int], int] = OrderedDict()   # (layer, expert) -> slot, oldest first
        self._victim_free: list[int] = []

    # ------------------------------------------------------------------ registration
    def _to_host(self, p: _Packed) -> _Packed:
        def host(t):
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.pin)
            h.copy_(t)
            return h
        return _Packed(host(p.codes), host(p.sf), host(p.bias), p.n, p.k)

    def register_layer(self, layer_idx: int, w1, w2, keep_on_gpu: bool = False) -> None:
        """Takes one layer's packed experts (objects with codes / sf / bias / n / k, e.g. ``ops.ExpertWeightsFp4``).
        The first call allocates the shared GPU buffers with this layer's shapes; every layer must have the same."""
        p1, p2 = _packed_of(w1), _packed_of(w2)
        assert p1.codes.shape[0] == self.num_experts and p2.codes.shape[0] == self.num_experts
        if self.gpu is None:
            def like(p):
                return _Packed(torch.empty(p.codes.shape, dtype=p.codes.dtype, device=self.device),
                               torch.empty(p.sf.shape, dtype=p.sf.dtype, device=self.device),
                               torch.empty(p.bias.shape, dtype=p.bias.dtype, device=self.device), p.n, p.k)
            self.gpu = (like(p1), like(p2))
        else:
            for mine, new in zip(self.gpu, (p1, p2)):
                assert mine.codes.shape == new.codes.shape and mine.sf.shape == new.sf.shape and \
                    mine.bias.shape == new.bias.shape, "every layer's experts must have the same packed shapes"
        if keep_on_gpu:
            self.resident[layer_idx] = (_Packed(p1.codes.to(self.device), p1.sf.to(self.device), p1.bias.to(self.device), p1.n, p1.k),
                                        _Packed(p2.codes.to(self.device), p2.sf.to(self.device), p2.bias.to(self.device), p2.n, p2.k))
        else:
            self.host[layer_idx] = (self._to_host(p1), self._to_host(p2))

    def is_cached(self, layer_idx: int) -> bool:
        return layer_idx in self.resident

    def init_victim_store(self, slots: int) -> int:
        """Room on the GPU for ``slots`` evicted experts (call after register_layer).  Returns the slots allocated."""
        assert self.gpu is not None, "register_layer first"
        slots = max(0, int(slots))
        if slots == 0:
            self.victims, self._victim_free = None, []
            self._victim_of.clear()
            return 0
        def room(p):
            return _Packed(torch.empty((slots,) + tuple(p.codes.shape[1:]), dtype=p.codes.dtype, device=self.device),
                           torch.empty((slots,) + tuple(p.sf.shape[1:]), dtype=p.sf.dtype, device=self.device),
                           torch.empty((slots,) + tuple(p.bias.shape[1:]), dtype=p.bias.dtype, device=self.device), p.n, p.k)
        self.victims = (room(self.gpu[0]), room(self.gpu[1]))
        self._victim_free = list(range(slots))
        self._victim_of.clear()
        return slots

    def _save_victim(self, layer_idx: int, e: int) -> None:
        """Slot e of the shared buffers (layer_idx's expert) is about to be overwritten: keep a copy."""
        key = (layer_idx, e)
        slot = self._victim_of.pop(key, None)
        if slot is None:
            slot = self._victim_free.pop() if self._victim_free else self._victim_of.popitem(last=False)[1]
        self._victim_of[key] = slot   # most recently used
        for store, buf in zip(self.victims, self.gpu):
            for d, t in zip(store.expert(slot), buf.expert(e)):
                d.copy_(t, non_blocking=True)

    def _restore_victim(self, layer_idx: int, e: int) -> bool:
        slot = self._victim_of.get((layer_idx, e))
        if slot is None:
            return False
        self._victim_of.move_to_end((layer_idx, e))
        for store, buf in zip(self.victims, self.gpu):
            for d, t in zip(buf.expert(e), store.expert(slot)):
                d.copy_(t, non_blocking=True)
        return True

    # ------------------------------------------------------------------ use
    def _views(self):
        from . import ops
        out = []
        for p in self.gpu:
            w = ops.ExpertWeightsFp4.__new__(ops.ExpertWeightsFp4)
            w.codes, w.sf, w.bias, w.n, w.k = p.codes, p.sf, p.bias, p.n, p.k
            w._shared_buffer = True   # its content changes from call to call: nothing derived from it may be cached
            out.append(w)
        return tuple(out)

    def ensure_experts(self, layer_idx: int, expert_ids):
        """Makes slots ``expert_ids`` of the shared buffers hold layer ``layer_idx``'s experts and returns the buffers
        as a (w1, w2) pair for the expert kernels.  Copies run on the current stream, from pinned memory without
        blocking the host; the caller's kernels on the same stream are ordered after them."""
        assert self.gpu is not None, "register_layer first"
        src = self.resident.get(layer_idx)
        counted = src is None
        if src is None:
            src = self.host[layer_idx]
        for e in expert_ids:
            e = int(e)
            if not 0 <= e < self.num_experts:
                raise IndexError(f"expert id {e} outside 0..{self.num_experts - 1}")
            if self.gpu_layer[e] == layer_idx:
                self._hits += counted
                continue
            prev = self.gpu_layer[e]
            if counted and self.victims is not None:
                # what the slot holds now goes to the victim store first (it may be the very copy asked for next time);
                # then the store is asked for this layer's expert before the host is
                if prev >= 0 and prev not in self.resident:
                    self._save_victim(prev, e)
                if self._restore_victim(layer_idx, e):
                    self._hits += 1
                    self.gpu_layer[e] = layer_idx
                    continue
            self._misses += counted
            for dst, s in zip(self.gpu, src):
                for d, t in zip(dst.expert(e), s.expert(e)):
                    d.copy_(t, non_blocking=True)
            self.gpu_layer[e] = layer_idx
        return self._views()

    def load_all_experts(self, layer_idx: int):
        """Every expert of the layer (prompt-sized batches touch them all)."""
        return self.ensure_experts(layer_idx, range(self.num_experts))

    def hit_rate(self) -> float:
        total = self._hits + self._misses
        return self._hits / total if total else 0.0

    def reset_hit_rate(self) -> None:
        self._hits = self._misses = 0

    def host_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for pair in self.host.values() for p in pair for t in (p.codes, p.sf, p.bias))

    def gpu_bytes(self) -> int:
        pairs = ([self.gpu] if self.gpu else []) + list(self.resident.values()) + ([self.victims] if self.victims else [])
        return sum(t.numel() * t.element_size() for pair in pairs for p in pair for t in (p.codes, p.sf, p.bias))
