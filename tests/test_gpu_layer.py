"""Whole attention-block chains through the B200 ops against the oracle and against the output of the
reference's own AttentionBlock.forward (golden fixture), plus a decode step captured in a CUDA graph."""
import numpy as np
import pytest
import torch

import oracle as O
from _util import assert_parity, golden, randn, t

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from tritonllm_b200 import _lib, ops as _ops
    _lib.load()
    assert _lib.device_status() == 0
    yield _ops
    assert _lib.device_status() == 0, "a kernel gave up a bounded wait"


def _params(g, hid=2880):
    bf = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(torch.bfloat16)  # noqa: E731
    return dict(norm_gain=torch.randn(hid, generator=g) * 0.05 + 1, w_qkv=bf(5120, hid, sc=0.02), b_qkv=bf(5120, sc=0.02),
                w_o=bf(hid, 4096, sc=0.02), b_o=bf(hid, sc=0.02), sinks=bf(64))


def _block_prefill(ops, x, p, window, cos_d, sin_d, offset):
    """AttentionBlock.forward(x, cache=None) on the B200 ops: norm -> QKV+RoPE -> attention -> o_proj+residual."""
    d = {k: v.to(DEV) for k, v in p.items()}
    xd = x.to(DEV)
    B, T, _ = x.shape
    n = ops.rmsnorm_forward(xd, d["norm_gain"], 1e-5)
    off = torch.tensor([offset], dtype=torch.int64, device=DEV)
    q, k, v = ops.qkv_rope_prefill(n, d["w_qkv"], d["b_qkv"], sin_d, cos_d, cos_d.shape[0], off, 64, 8, 64)
    a = ops.attention(q.view(B, T, 8, 8, 64), k, v, d["sinks"], 0.125, window, off)
    return ops.out_residual_forward(a, d["w_o"], d["b_o"], xd)


@pytest.mark.parametrize("layer", [0, 1])
def test_config1_block_vs_reference_module(ops, layer):
    """BASELINE config 1 (T=16, 20b dims): the reference's AttentionBlock.forward output (fp32 mode, CPU)."""
    gd = golden("attention_block")
    gen = torch.Generator().manual_seed(1235 + layer)
    r = lambda *s: torch.randn(*s, generator=gen)  # noqa: E731
    x = O.bf16_round(r(1, 16, 2880))
    p = dict(norm_gain=r(2880) * 0.05 + 1, w_qkv=O.bf16_round(r(5120, 2880) * 0.02), b_qkv=O.bf16_round(r(5120) * 0.02),
             w_o=O.bf16_round(r(2880, 4096) * 0.02), b_o=O.bf16_round(r(2880) * 0.02), sinks=O.bf16_round(r(64)))
    chk = np.array([float(a.double().sum()) for a in (x, p["norm_gain"], p["w_qkv"], p["b_qkv"], p["w_o"], p["b_o"],
                                                      p["sinks"])])
    if not np.allclose(chk, gd[f"l{layer}__checksums"], rtol=0, atol=1e-9):
        pytest.skip("torch RNG stream differs from the one that produced the fixture")
    cos, sin = O.yarn_cos_sin(64)
    pb = {k: (v.to(torch.bfloat16) if k != "norm_gain" else v) for k, v in p.items()}
    out = _block_prefill(ops, x.to(torch.bfloat16), pb, 128 if layer % 2 == 0 else 0, cos.to(DEV), sin.to(DEV), 0)
    assert_parity(t(gd[f"l{layer}__t"]), out, f"attention block, layer {layer}, vs the reference module")


@pytest.mark.parametrize("B,T,window,offset", [(2, 300, 128, 0), (1, 700, 0, 0), (2, 130, 0, 40)])
def test_prefill_block_vs_oracle(ops, B, T, window, offset):
    g = torch.Generator().manual_seed(300 + T)
    p = _params(g)
    x = randn(g, B, T, 2880)
    cos, sin = O.yarn_cos_sin(2048)
    ref, *_ = O.attention_block(x, p, window, cos, sin, offset)
    out = _block_prefill(ops, x, p, window, cos.to(DEV), sin.to(DEV), offset)
    assert_parity(ref, out, f"prefill attention block T={T} W={window}")


def test_decode_steps_in_a_cuda_graph(ops):
    """A decode step (norm -> QKV+RoPE+cache -> attention -> o_proj+residual -> norm -> router -> top-k) captured
    once and replayed three times; the position is a device tensor, so each replay handles the next token."""
    g = torch.Generator().manual_seed(400)
    B, ctx, start, E = 8, 256, 100, 32
    p = _params(g)
    gain2 = torch.randn(2880, generator=g) * 0.05 + 1
    wg, bg = randn(g, 2880, E, scale=0.02), torch.randn(E, generator=g) * 0.02
    ck, cv = torch.zeros(B, ctx, 8, 64, dtype=torch.bfloat16), torch.zeros(B, ctx, 8, 64, dtype=torch.bfloat16)
    ck[:, :start], cv[:, :start] = randn(g, B, start, 8, 64), randn(g, B, start, 8, 64)
    xs = [randn(g, B, 1, 2880) for _ in range(3)]
    cos, sin = O.yarn_cos_sin(ctx)
    d = {k: v.to(DEV) for k, v in p.items()}
    gain2_d, wg_d, bg_d, cos_d, sin_d = gain2.to(DEV), wg.to(DEV), bg.to(DEV), cos.to(DEV), sin.to(DEV)
    ckd, cvd = ck.to(DEV), cv.to(DEV)
    x_in = torch.empty(B, 1, 2880, dtype=torch.bfloat16, device=DEV)
    offset = torch.tensor([start], dtype=torch.int64, device=DEV)

    def step(window):
        n = ops.rmsnorm_forward(x_in, d["norm_gain"], 1e-5)
        q = ops.qkv_rope_cache_decode_forward(n, d["w_qkv"], d["b_qkv"], sin_d, cos_d, ctx, ckd, cvd, offset, 64, 8, 64)
        a = ops.attention_decode(q.view(B, 1, 8, 8, 64), ckd, cvd, d["sinks"], 0.125, window, offset)
        h = ops.out_residual_decode_forward(a, d["w_o"], d["b_o"], x_in)           # in place on x_in
        n2 = ops.rmsnorm_forward(h, gain2_d, 1e-5, out=torch.empty_like(h))
        logits = ops.router_logits(n2.view(B, 2880), wg_d, bg_d)
        vals, idx, _ = ops.topk(logits, 4)
        offset.add_(1)
        return h, logits, vals, idx

    x_in.copy_(xs[0])
    step(128)                      # warm-up outside the capture (module load, pools, workspaces)
    ckd.copy_(ck), cvd.copy_(cv), offset.fill_(start)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = step(128)
    ckd.copy_(ck), cvd.copy_(cv), offset.fill_(start)
    ck_ref, cv_ref = ck.clone(), cv.clone()
    for i, x in enumerate(xs):
        x_in.copy_(x)
        graph.replay()
        torch.cuda.synchronize()
        pos = start + i
        n_ref = O.rmsnorm(x, p["norm_gain"], 1e-5)
        q_ref = O.qkv_rope_cache_decode(n_ref, p["w_qkv"], p["b_qkv"], cos, sin, pos, ck_ref, cv_ref, max_ctx=ctx)
        a_ref = O.attention(q_ref.reshape(B, 1, 8, 8, 64), ck_ref, cv_ref, p["sinks"], 0.125, 128, pos)
        h_ref = O.out_residual(a_ref.reshape(B, 4096), p["w_o"], p["b_o"], x.reshape(B, 2880))
        assert_parity(h_ref, outs[0].reshape(B, 2880), f"decode step {i}: residual stream")
        assert_parity(ck_ref[:, pos], ckd[:, pos], f"decode step {i}: cache k row")
        # routing is bit-exact on the logits the GPU produced
        _, idx_ref, _ = O.topk_softmax(outs[1].cpu(), 4)
        assert torch.equal(outs[3].cpu(), idx_ref)
        assert_parity(O.router_logits(O.rmsnorm(h_ref.reshape(B, 1, 2880), gain2, 1e-5).reshape(B, 2880), wg, bg),
                      outs[1], f"decode step {i}: router logits", max_rel=3e-2, rms_rel=8e-3)
    assert int(offset.item()) == start + 3


@pytest.mark.parametrize("world,window", [(8, 0), (2, 128)])
def test_head_sharded_block_equals_unsharded(ops, world, window):
    """The optional long-context mode on one GPU: every rank's share (its slice of the QKV weight, its heads'
    attention) computed in turn, the shares placed side by side as the all-gather would, then the replicated
    o_proj: equal to the unsharded block bit for bit, and within the bar of the oracle."""
    from tritonllm_b200 import headshard
    g = torch.Generator().manual_seed(900 + world)
    p = _params(g)
    B, T = 1, 300
    x = randn(g, B, T, 2880)
    cos, sin = O.yarn_cos_sin(512)
    cos_d, sin_d = cos.to(DEV), sin.to(DEV)
    d = {k: v.to(DEV) for k, v in p.items()}
    xd = x.to(DEV)
    parts = []
    for r in range(world):
        sh = headshard.shard_attention_weights(d["w_qkv"], d["b_qkv"], d["sinks"], r, world)
        parts.append(headshard.attention_heads_local(xd, d["norm_gain"], sh, sin_d, cos_d, cos_d.shape[0], 0.125, window).clone())
    o = torch.cat(parts, dim=1)
    got = ops.out_residual_forward(o.reshape(B, T, -1), d["w_o"], d["b_o"], xd)
    want = _block_prefill(ops, x, p, window, cos_d, sin_d, 0)
    assert torch.equal(got, want)
    ref, *_ = O.attention_block(x, p, window, cos, sin, 0)
    assert_parity(ref, got, f"head-sharded block, {world} ranks")
