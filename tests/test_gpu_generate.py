"""GPU parity of the KV-store maintenance kernels, the embedding lookup, the whole-model forward and the
batched decode loop, all through the C ABI, against the oracle and the reference-generated fixture."""
import numpy as np
import pytest
import torch

from _util import assert_parity, golden, t

import oracle as O

pytestmark = pytest.mark.gpu


def _mods():
    from tritonllm_b200 import _lib, generate, ops
    return ops, generate, _lib


# ----------------------------------------------------------------------------- KV store
@pytest.mark.parametrize("name", ["full_default", "full_keep7", "not_full"])
def test_cache_slide_matches_reference_fixture(name, monkeypatch):
    _, G, _ = _mods()
    monkeypatch.setenv("DENSE_CACHE_SLIDE_CHUNK", "5")
    g = golden("kv_cache")
    k0, v0 = t(g[f"{name}_k0"]).bfloat16(), t(g[f"{name}_v0"]).bfloat16()
    ret, off, current, keep = (int(x) for x in g[f"{name}_ret"])
    c = G.Cache(2, 16, 2, 8, device="cuda")
    assert c.slide_chunk == int(g["slide_chunk"][0])
    c.k.copy_(k0)
    c.v.copy_(v0)
    c.offset.fill_(current)
    got = c.slide_window(keep_last_n=None if keep < 0 else keep)
    assert got == ret and int(c.offset.item()) == off
    assert torch.equal(c.k.float().cpu(), t(g[f"{name}_k1"]))
    assert torch.equal(c.v.float().cpu(), t(g[f"{name}_v1"]))


def test_cache_truncate_matches_reference_fixture():
    _, G, _ = _mods()
    g = golden("kv_cache")
    c = G.Cache(2, 16, 2, 8, device="cuda")
    c.k.copy_(t(g["trunc_k0"]).bfloat16())
    c.v.copy_(t(g["trunc_k0"]).bfloat16())
    c.truncate(9)
    assert int(c.offset.item()) == int(g["trunc_off"][0])
    assert torch.equal(c.k.float().cpu(), t(g["trunc_k1"])) and torch.equal(c.v.float().cpu(), t(g["trunc_k1"]))
    c.reset()
    assert int(c.offset.item()) == 0 and not c.k.any() and not c.v.any()


@pytest.mark.parametrize("B,C,current,keep", [(3, 1024, 1024, 896), (3, 1024, 1024, 100), (2, 512, 512, 512),
                                              (1, 8192, 8192, 7168), (5, 300, 257, 1), (2, 64, 64, 0)])
def test_kv_slide_vs_oracle(B, C, current, keep):
    """Bit-exact move at the model's row size (8 heads x 64): several launches when the shift is smaller than
    what is kept, one when it is larger, nothing moved when everything is kept."""
    ops, _, _ = _mods()
    gen = torch.Generator().manual_seed(7000 + C + keep)
    k = torch.randn(B, C, 8, 64, generator=gen).bfloat16()
    v = torch.randn(B, C, 8, 64, generator=gen).bfloat16()
    kd, vd = k.cuda(), v.cuda()
    ops.kv_slide(kd, vd, current, keep)
    torch.cuda.synchronize()
    for ref, got in ((k, kd), (v, vd)):
        exp = O.kv_slide(ref.view(torch.int16).numpy(), current, keep)
        assert np.array_equal(exp, got.cpu().view(torch.int16).numpy())


def test_kv_slide_rejects_bad_arguments():
    ops, _, L = _mods()
    k = torch.zeros(1, 16, 8, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(L.B2Error):
        ops.kv_slide(k, k.clone(), 17, 4)       # more tokens than the store holds
    with pytest.raises(L.B2Error):
        ops.kv_slide(k, k.clone(), 8, 9)        # keeps more than it has
    with pytest.raises(AssertionError):
        ops.kv_slide(k[:, ::2], k[:, ::2], 4, 2)  # not the dense layout


# ----------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_embedding_lookup_is_exact(dtype):
    ops, _, L = _mods()
    gen = torch.Generator().manual_seed(11)
    table = torch.randn(5000, 2880, generator=gen).bfloat16()
    tokens = torch.randint(0, 5000, (7, 33), generator=gen).to(dtype)
    out = ops.embedding_forward(tokens.cuda(), table.cuda())
    torch.cuda.synchronize()
    assert out.shape == (7, 33, 2880)
    assert torch.equal(out.cpu(), table[tokens.long()])
    assert L.device_status() == 0
    assert ops.embedding_forward(tokens[:0].cuda(), table.cuda()).shape == (0, 33, 2880)


def test_embedding_lookup_records_a_token_outside_the_vocabulary():
    ops, _, L = _mods()
    table = torch.ones(16, 64, dtype=torch.bfloat16, device="cuda")
    out = ops.embedding_forward(torch.tensor([3, 16, -1], device="cuda"), table)
    torch.cuda.synchronize()
    assert L.device_status() & 0x10            # recorded, and cleared by the read
    assert L.device_status() == 0
    assert torch.equal(out.cpu(), torch.ones(3, 64, dtype=torch.bfloat16))


# ----------------------------------------------------------------------------- whole model
def _small_model(fp4: bool, layers=2, vocab=1024, seed=3):
    """A two-layer model at the real hidden sizes (the kernels are built for them) with a small vocabulary;
    returns the GPU model and the same weights as the oracle's dict."""
    ops, G, _ = _mods()
    cfg = G.ModelConfig(num_hidden_layers=layers, num_experts=32, vocab_size=vocab)
    w = G.ModelWeights.random(cfg, "cuda", seed=seed, fp4=False, draw_on="cpu")   # the same weights on every machine
    for p in w.layers:
        p.w2.scales.sub_(5)   # brings the MoE output to the size of the residual stream (random codes are large)
    wo = dict(embedding=w.embedding.cpu(), norm=w.norm.cpu(), unembedding=w.unembedding.cpu(), layers=[])
    for p in w.layers:
        wo["layers"].append(dict(
            norm_gain=p.norm1.cpu(), w_qkv=p.wqkv.cpu(), b_qkv=p.bqkv.cpu(), sinks=p.sinks.cpu(), w_o=p.wo.cpu(),
            b_o=p.bo.cpu(), norm2_gain=p.norm2.cpu(), wg=p.wg.cpu(), bg=p.bg.cpu(),
            w1_codes=p.w1.codes.cpu().numpy(), w1_scales=p.w1.scales.cpu().numpy(), b1=p.w1.bias.cpu(),
            w2_codes=p.w2.codes.cpu().numpy(), w2_scales=p.w2.scales.cpu().numpy(), b2=p.w2.bias.cpu()))
        if fp4:
            p.w1, p.w2 = ops.ExpertWeightsFp4(p.w1), ops.ExpertWeightsFp4(p.w2)
    return G.Transformer(cfg, w, max_context=4096), wo


# Logits after two full layers pass through sixteen bf16-rounded ops (each held to max 2e-2 / rms 4e-3 / cosine
# 0.9999 on its own in the per-op tests) and are themselves rounded to bf16; their independent rounding noise
# adds in quadrature, so the chain is held to four times the per-op bar (cosine 0.9998 = 2 % relative error).
_CHAIN = dict(max_rel=8e-2, rms_rel=1.6e-2, min_cos=0.9998)
# The router logits are bf16 sums (steps of 1/64 at their size): a token whose 4th and 5th logits are closer
# than this may be routed to another expert by a different summation order, in the reference as much as here.
_ROUTER_TIE = 0.02


def _clear_tokens(gaps):
    """[B, S] mask of the tokens whose routing is unambiguous in every layer."""
    clear = torch.stack(gaps).min(dim=0).values >= _ROUTER_TIE
    assert clear.float().mean() > 0.6, "the seed leaves too few unambiguous tokens"
    return clear


@pytest.mark.parametrize("fp4", [True, False])
def test_prompt_then_decode_steps_match_the_oracle(fp4):
    """Prompt of 8 tokens into the KV store, then 5 teacher-forced one-token steps: the logits of step t must
    be the oracle's logits of position t of a store-less forward over the whole sequence."""
    model, wo = _small_model(fp4)
    gen = torch.Generator().manual_seed(21)
    B, P, S = 3, 8, 13
    tokens = torch.randint(0, 1024, (B, S), generator=gen)
    cos, sin = O.yarn_cos_sin(S)
    gaps = []
    ref = O.model_forward(tokens, wo, cos, sin, gaps)                # [B, S, V] fp32
    clear = _clear_tokens(gaps)
    assert clear[:, P:].any(), "no unambiguous decode position: pick another seed"
    td = tokens.cuda()
    # store-less forward of the whole sequence (the prefill kernels)
    full = model.forward(td).cpu()
    assert_parity(ref[clear], full[clear], f"store-less logits fp4={fp4}", **_CHAIN)
    assert torch.nn.functional.cosine_similarity(ref, full, dim=-1).min() > 0.9   # a re-routed token is still close
    caches = model.make_caches(B, 64)
    hidden = model.prefill(td[:, :P], caches)
    assert hidden.shape == (B, P, 2880) and int(caches[0].offset.item()) == P
    for s in range(P, S):
        logits = model.forward(td[:, s:s + 1], caches)
        assert logits.shape == (B, 1, 1024) and logits.dtype == torch.float32
        if clear[:, s].any():
            assert_parity(ref[:, s][clear[:, s]], logits[:, 0].cpu()[clear[:, s]],
                          f"decode logits at position {s} fp4={fp4}", **_CHAIN)
    assert int(caches[0].offset.item()) == S
    # the fused greedy step returns the arg-max of the same logits
    caches2 = model.make_caches(B, 64)
    model.prefill(td[:, :P], caches2)
    ids = model.forward_greedy(td[:, P:P + 1], caches2).cpu()
    top2 = ref[:, P].topk(2, dim=-1)
    sure = ((top2.values[:, 0] - top2.values[:, 1]) > 0.05 * ref[:, P].abs().max()) & clear[:, P]
    assert torch.equal(ids[sure], top2.indices[sure, 0])
    from tritonllm_b200 import _lib
    assert _lib.device_status() == 0


def test_prompt_in_slices_equals_prompt_in_one_pass():
    """Sequences ingested slice by slice write the same K/V as one pass over all of them."""
    model, _ = _small_model(True, layers=1)
    gen = torch.Generator().manual_seed(22)
    tokens = torch.randint(0, 1024, (5, 24), generator=gen).cuda()
    a, b = model.make_caches(5, 32), model.make_caches(5, 32)
    model.prefill(tokens, a)
    model.PREFILL_ROWS = 48                     # two sequences per slice
    try:
        model.prefill(tokens, b)
    finally:
        model.PREFILL_ROWS = type(model).PREFILL_ROWS
    assert torch.equal(a[0].k, b[0].k) and torch.equal(a[0].v, b[0].v)
    assert int(a[0].offset.item()) == int(b[0].offset.item()) == 24


def test_generator_graph_and_eager_agree_and_slide(monkeypatch):
    """The captured step and the eager step produce the same greedy tokens; with a store of 32 tokens and a
    slide chunk of 8 the position drops from 32 to 24 whenever the store is full."""
    _, G, L = _mods()
    monkeypatch.setenv("DENSE_CACHE_SLIDE_CHUNK", "8")
    model, _ = _small_model(True, layers=2)
    gen = torch.Generator().manual_seed(23)
    prompts = torch.randint(0, 1024, (2, 20), generator=gen)
    outs = []
    for graph in (True, False):
        tg = G.TokenGenerator(model, context=32, batch_size=2, use_cuda_graph=graph)
        assert tg.max_model_len == 32 and tg.enable_dense_cache_sliding
        steps = list(tg.generate(prompts.tolist(), temperature=0.0, max_tokens=30))
        assert len(steps) == 30 and all(len(s) == 2 for s in steps)
        assert tg.last_generation_stats["generated_tokens"] == 30
        # 19 prompt tokens stored + 30 steps; the store fills before steps 14, 22 and 30: three slides of 8
        assert int(tg.caches[0].offset.item()) == 19 + 30 - 3 * 8
        outs.append(torch.tensor(steps).T)
        dev = tg.generate_greedy(prompts.cuda(), 30)
        assert torch.equal(dev.cpu(), outs[-1])
    assert torch.equal(outs[0], outs[1])
    assert L.device_status() == 0


def test_offloaded_experts_give_the_same_tokens():
    """The CPU-offload mode (experts in pinned host memory, one shared set of GPU buffers filled per layer with the
    experts the routing chose) computes exactly what the resident model computes, prompt and decode steps alike."""
    _, G, L = _mods()
    gen = torch.Generator().manual_seed(29)
    prompts = torch.randint(0, 1024, (2, 24), generator=gen).cuda()
    model, _ = _small_model(True, layers=3)
    ref = G.TokenGenerator(model, context=64, batch_size=2).generate_greedy(prompts, 12).cpu()
    cache = model.offload_experts(resident_layers=1, victim_slots=6)
    assert model.w.layers[0].w1 is None and cache.is_cached(0) and not cache.is_cached(2)
    tg = G.TokenGenerator(model, context=64, batch_size=2)
    assert not tg.use_global_cuda_graph
    got = tg.generate_greedy(prompts, 12).cpu()
    assert torch.equal(ref, got)
    assert 0.0 <= cache.hit_rate() <= 1.0 and cache._misses > 0 and cache.host_bytes() > 0
    assert len(cache._victim_of) > 0   # two offloaded layers share the slots: evicted experts went to the second level
    assert L.device_status() == 0


def test_generator_stops_and_samples():
    _, G, _ = _mods()
    model, _ = _small_model(True, layers=1)
    tg = G.TokenGenerator(model, context=64, batch_size=1)
    prompt = [5, 17, 900, 4]
    first = next(iter(tg.generate(prompt, temperature=0.0, max_tokens=1)))
    assert isinstance(first, int)
    got = list(tg.generate(prompt, stop_tokens=[first], temperature=0.0))
    assert got == [first]                                         # stops on the stop token
    torch.manual_seed(0)
    pairs = list(tg.generate(prompt, temperature=0.8, max_tokens=4, return_logprobs=True))
    assert len(pairs) == 4 and all(0 <= tok < 1024 and lp <= 0.0 for tok, lp in pairs)
    torch.manual_seed(0)
    assert [p[0] for p in pairs] == list(tg.generate(prompt, temperature=0.8, max_tokens=4))
    with pytest.raises(ValueError):
        list(tg.generate(list(range(65)), temperature=0.0))       # longer than the store
    with pytest.raises(ValueError):
        list(tg.generate([[1, 2], [3, 4]], temperature=0.0))      # two prompts for a batch of one


# ----------------------------------------------------------------------------- checkpoint path
def test_checkpoint_get_decodes_like_the_reference():
    """Checkpoint.get of an expert tensor (decoded on the GPU by the upcast kernel) against what the reference's
    Checkpoint.get returned for the same file."""
    import os
    from tritonllm_b200.checkpoint import Checkpoint
    here = os.path.dirname(os.path.abspath(__file__))
    ck = Checkpoint(os.path.join(here, "golden", "tiny_checkpoint"), "cuda")
    g = golden("checkpoint_ref")
    for name in ("block.0.mlp.mlp1_weight", "block.1.mlp.mlp2_weight"):
        dec = ck.get(name)
        assert dec.dtype == torch.bfloat16 and torch.equal(dec.float().cpu(), t(g[name + "__decoded"]))
    assert torch.equal(ck.get("embedding.weight").float().cpu(), t(g["embedding"]))


@pytest.mark.parametrize("fp4", [True, False])
def test_model_from_checkpoint_equals_model_from_tensors(tmp_path, fp4):
    """A one-layer checkpoint at the real hidden sizes written in the gpt-oss layout, loaded by
    transformer_from_checkpoint: same logits, bit for bit, as the model built from the tensors directly."""
    import json
    from safetensors.torch import save_file
    ops, G, _ = _mods()
    from tritonllm_b200 import checkpoint as C
    cfg = G.ModelConfig(num_hidden_layers=1, num_experts=32, vocab_size=512)
    w = G.ModelWeights.random(cfg, "cuda", seed=9, fp4=False)
    p = w.layers[0]
    H, I, E = 2880, 2880, 32
    tensors = {
        "embedding.weight": w.embedding, "unembedding.weight": w.unembedding, "norm.scale": w.norm.bfloat16(),
        "block.0.attn.norm.scale": p.norm1.bfloat16(), "block.0.attn.qkv.weight": p.wqkv, "block.0.attn.qkv.bias": p.bqkv,
        "block.0.attn.sinks": p.sinks, "block.0.attn.out.weight": p.wo, "block.0.attn.out.bias": p.bo,
        "block.0.mlp.norm.scale": p.norm2.bfloat16(), "block.0.mlp.gate.weight": p.wg.mT.contiguous(),
        "block.0.mlp.gate.bias": p.bg.bfloat16(),
        "block.0.mlp.mlp1_weight.blocks": p.w1.codes.view(E, 2 * I, H // 32, 16), "block.0.mlp.mlp1_weight.scales": p.w1.scales,
        "block.0.mlp.mlp1_bias": p.w1.bias.bfloat16(),
        "block.0.mlp.mlp2_weight.blocks": p.w2.codes.view(E, H, I // 32, 16), "block.0.mlp.mlp2_weight.scales": p.w2.scales,
        "block.0.mlp.mlp2_bias": p.w2.bias.bfloat16()}
    save_file({k: v.contiguous().cpu() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps(dict(num_hidden_layers=1, num_experts=32, vocab_size=512)))
    # the checkpoint stores gains and biases as bf16: give the direct model the same rounded values
    w.norm, p.norm1, p.norm2 = w.norm.bfloat16().float(), p.norm1.bfloat16().float(), p.norm2.bfloat16().float()
    p.bg = p.bg.bfloat16().float()
    p.w1.bias.copy_(p.w1.bias.bfloat16().float())
    p.w2.bias.copy_(p.w2.bias.bfloat16().float())
    if fp4:
        p.w1, p.w2 = ops.ExpertWeightsFp4(p.w1), ops.ExpertWeightsFp4(p.w2)
    direct = G.Transformer(cfg, w, max_context=4096)
    loaded = C.transformer_from_checkpoint(str(tmp_path), fp4=fp4, max_context=4096)
    assert loaded.config == cfg
    tokens = torch.randint(0, 512, (2, 9), generator=torch.Generator().manual_seed(4)).cuda()
    assert torch.equal(direct.forward(tokens), loaded.forward(tokens))
    ca, cb = direct.make_caches(2, 16), loaded.make_caches(2, 16)
    direct.prefill(tokens[:, :8], ca)
    loaded.prefill(tokens[:, :8], cb)
    assert torch.equal(direct.forward_greedy(tokens[:, 8:], ca), loaded.forward_greedy(tokens[:, 8:], cb))


def test_generate_raises_when_a_kernel_recorded_a_failure():
    """A token id outside the vocabulary makes the embedding kernel read row 0 and set the status word; the
    decode loop must raise instead of yielding tokens computed from it."""
    ops, G, _lib = _mods()
    model, _ = _small_model(True)
    tg = G.TokenGenerator(model, context=32, batch_size=2, use_cuda_graph=False)
    bad = torch.tensor([[1, 2, 10 ** 6], [3, 4, 5]])
    with pytest.raises(_lib.B2Error, match="status word"):
        list(tg.generate(bad, temperature=0.0, max_tokens=2))
    assert _lib.device_status() == 0   # the check cleared the word
    good = torch.tensor([[1, 2, 7], [3, 4, 5]])
    assert len(list(tg.generate(good, temperature=0.0, max_tokens=2))) == 2
    with pytest.raises(_lib.B2Error):
        tg.generate_greedy(bad.to("cuda"), 2)
