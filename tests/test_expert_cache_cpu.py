"""Host logic of the CPU-offload expert cache (tritonllm_b200/expert_cache.py) on CPU tensors: which slot holds which
layer's expert, what is copied when, hit and miss counts, resident layers."""
from types import SimpleNamespace

import pytest
import torch

from tritonllm_b200.expert_cache import ExpertOffloadCache

E, N, K = 4, 6, 8


def _layer(tag: int):
    """Packed experts whose every byte names (layer tag, expert): codes = 16 * tag + e."""
    def pack(n, k):
        codes = torch.stack([torch.full((n, k // 2), 16 * tag + e, dtype=torch.uint8) for e in range(E)])
        sf = torch.stack([torch.full((1, 1, 32, 4, 4), 100 + 16 * tag + e, dtype=torch.uint8) for e in range(E)])
        bias = torch.stack([torch.full((n,), float(16 * tag + e)) for e in range(E)])
        return SimpleNamespace(codes=codes, sf=sf, bias=bias, n=n, k=k)
    return pack(2 * N, K), pack(K, N)


def _slot_tags(cache):
    return [int(cache.gpu[0].codes[e, 0, 0]) for e in range(E)]


def test_slots_follow_the_layers_that_ask_for_them():
    cache = ExpertOffloadCache(E, "cpu", pin_memory=False)
    for li in range(3):
        cache.register_layer(li, *_layer(li))
    assert set(cache.host) == {0, 1, 2} and cache.gpu_layer == [-1] * E
    cache.ensure_experts(0, [1, 3])
    assert cache.gpu_layer == [-1, 0, -1, 0] and _slot_tags(cache)[1] == 1 and _slot_tags(cache)[3] == 3
    cache.ensure_experts(1, [1, 2])                  # layer 1 takes slot 1 over and fills slot 2
    assert cache.gpu_layer == [-1, 1, 1, 0] and _slot_tags(cache)[1:3] == [17, 18]
    for dst, name in ((cache.gpu[0], "w1"), (cache.gpu[1], "w2")):
        assert torch.all(dst.codes[2] == 18) and torch.all(dst.sf[2] == 118) and torch.all(dst.bias[2] == 18.0), name
    cache.ensure_experts(1, [2, 1])                  # both present: nothing to copy
    assert cache.hit_rate() == pytest.approx(2 / 6)  # 4 misses, then 2 hits
    cache.ensure_experts(0, [3])                     # still layer 0's from the first call
    assert cache.hit_rate() == pytest.approx(3 / 7)
    w1, w2 = cache.load_all_experts(2)
    assert cache.gpu_layer == [2] * E and _slot_tags(cache) == [32, 33, 34, 35]
    assert w1.codes is cache.gpu[0].codes and w2.bias is cache.gpu[1].bias and (w1.n, w1.k, w2.n, w2.k) == (2 * N, K, K, N)
    cache.reset_hit_rate()
    assert cache.hit_rate() == 0.0


def test_resident_layers_are_served_from_their_gpu_copy_and_not_counted():
    cache = ExpertOffloadCache(E, "cpu", pin_memory=False)
    cache.register_layer(0, *_layer(0), keep_on_gpu=True)
    cache.register_layer(1, *_layer(1))
    assert cache.is_cached(0) and not cache.is_cached(1) and 0 not in cache.host
    cache.ensure_experts(0, [0, 1])
    assert _slot_tags(cache)[:2] == [0, 1] and cache.hit_rate() == 0.0 and cache._misses == 0
    cache.ensure_experts(1, [0])
    assert _slot_tags(cache)[0] == 16 and cache._misses == 1
    assert cache.host_bytes() > 0 and cache.gpu_bytes() > cache.host_bytes()   # shared buffers + the resident layer


def test_bad_ids_and_shapes_are_refused():
    cache = ExpertOffloadCache(E, "cpu", pin_memory=False)
    cache.register_layer(0, *_layer(0))
    with pytest.raises(IndexError):
        cache.ensure_experts(0, [E])
    w1, w2 = _layer(1)
    w1.codes = w1.codes[:, :-1]
    with pytest.raises(AssertionError):
        cache.register_layer(1, w1, w2)


def test_victim_store_serves_evicted_experts_and_forgets_the_oldest():
    cache = ExpertOffloadCache(E, "cpu", pin_memory=False)
    for li in range(4):
        cache.register_layer(li, *_layer(li))
    assert cache.init_victim_store(2) == 2
    cache.ensure_experts(0, [1])            # miss (host)
    cache.ensure_experts(1, [1])            # miss; layer 0's expert 1 is saved
    assert (0, 1) in cache._victim_of and cache._misses == 2
    cache.ensure_experts(0, [1])            # served by the store: layer 1's copy saved, layer 0's restored
    assert _slot_tags(cache)[1] == 1 and cache._hits == 1 and cache._misses == 2
    assert set(cache._victim_of) == {(0, 1), (1, 1)}
    for buf in cache.gpu:
        assert torch.all(buf.codes[1] == 1) and torch.all(buf.sf[1] == 101) and torch.all(buf.bias[1] == 1.0)
    cache.ensure_experts(2, [1])            # layer 0's copy is saved again (already stored: refreshed, now the newest)
    cache.ensure_experts(3, [1])            # layer 2's copy needs a slot: the oldest entry, layer 1's, goes
    assert set(cache._victim_of) == {(0, 1), (2, 1)} and cache._misses == 4
    cache.ensure_experts(1, [1])            # no longer stored: from the host again
    assert cache._misses == 5 and _slot_tags(cache)[1] == 17
    assert cache.init_victim_store(0) == 0 and cache.victims is None
