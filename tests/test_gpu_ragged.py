"""Per-sequence positions and the paged KV store in the decode kernels (b2_qkv_rope_kv_decode_ragged,
b2_attn_decode_ragged) and in the decode loop.  The reference keeps one position for the whole batch and a dense
store, so the bar is: a sequence in a ragged batch gets what it gets when run alone through the reference-shaped
entry points (bit for bit where no split-KV merge order is involved, within the parity bar otherwise), the CPU
oracle per sequence, and paged == dense bit for bit."""
import pytest
import torch

import oracle as O
from _util import assert_parity, randn

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from tritonllm_b200 import _lib, ops as _ops
    _lib.load()
    assert _lib.device_status() == 0
    yield _ops
    assert _lib.device_status() == 0, "a kernel recorded a failure"


def _paged_copy(g, k, v, page_size, spare=3):
    """Scatters dense stores [B, ctx, H, D] into a pool of shuffled pages; returns (k_pool, v_pool, block_table)."""
    B, ctx, H, D = k.shape
    per = ctx // page_size
    n_pages = B * per + spare
    perm = torch.randperm(n_pages, generator=g)[: B * per].reshape(B, per)
    kp = randn(g, n_pages, page_size, H, D)       # unowned pages hold other data, never zeros
    vp = randn(g, n_pages, page_size, H, D)
    for b in range(B):
        for j in range(per):
            kp[perm[b, j]] = k[b, j * page_size:(j + 1) * page_size]
            vp[perm[b, j]] = v[b, j * page_size:(j + 1) * page_size]
    return kp, vp, perm.to(torch.int32)


@pytest.mark.parametrize("B,ctx,window,positions", [
    (5, 256, 0, [0, 37, 128, 255, 64]),
    (5, 256, 128, [0, 127, 128, 255, 200]),
    (3, 4096, 0, [4095, 1, 2047]),
    (3, 4096, 128, [4095, 1, 2047]),
    (40, 512, 0, None),
    (40, 512, 128, None),
])
def test_attention_decode_with_per_sequence_positions(ops, B, ctx, window, positions):
    g = torch.Generator().manual_seed(1000 + B + window + ctx)
    pos = torch.tensor(positions) if positions is not None else torch.randint(0, ctx, (B,), generator=g)
    q = randn(g, B, 1, 8, 8, 64)
    k, v = randn(g, B, ctx, 8, 64), randn(g, B, ctx, 8, 64)
    sinks = torch.randn(64, generator=g)
    # rows past a sequence's position hold NaN: a kernel that touched them would show it
    for b in range(B):
        k[b, int(pos[b]) + 1:] = float("nan")
        v[b, int(pos[b]) + 1:] = float("nan")
    qd, kd, vd, sd, pd = q.to(DEV), k.to(DEV), v.to(DEV), sinks.to(DEV), pos.to(DEV)
    got = ops.attention_decode(qd, kd, vd, sd, 0.125, window, pd).clone()
    torch.cuda.synchronize()
    for b in range(B):
        ref = O.attention(q[b:b + 1], torch.nan_to_num(k[b:b + 1]), torch.nan_to_num(v[b:b + 1]), sinks, 0.125, window, int(pos[b]))
        assert_parity(ref, got[b:b + 1], f"ragged decode attention, sequence {b} at {int(pos[b])}")
    # the same sequence alone through the reference-shaped entry point (one position for the batch)
    for b in range(min(B, 5)):
        alone = ops.attention_decode(qd[b:b + 1], kd[b:b + 1], vd[b:b + 1], sd, 0.125, window, pd[b:b + 1].clone()).clone()
        # (not bit for bit: the split points of the key range, and with them the merge order, depend on the batch)
        assert_parity(alone, got[b:b + 1], "ragged batch vs sequence alone", max_rel=1e-2, rms_rel=2e-3)
    # paged store: the same tiles and the same split points, other addresses -> bit for bit
    for page_size in (32, 64):
        kp, vp, table = _paged_copy(g, torch.nan_to_num(k, nan=7.0), torch.nan_to_num(v, nan=7.0), page_size)
        kd2, vd2 = torch.nan_to_num(kd, nan=7.0), torch.nan_to_num(vd, nan=7.0)
        dense = ops.attention_decode(qd, kd2, vd2, sd, 0.125, window, pd).clone()
        paged = ops.attention_decode_paged(qd, kp.to(DEV), vp.to(DEV), table.to(DEV), pd, sd, 0.125, window).clone()
        assert torch.equal(dense, paged), f"paged (page {page_size}) vs dense"


def test_ragged_attention_is_graph_capturable_and_positions_live_on_the_device(ops):
    g = torch.Generator().manual_seed(31)
    B, ctx = 6, 192
    q, k, v = randn(g, B, 1, 8, 8, 64), randn(g, B, ctx, 8, 64), randn(g, B, ctx, 8, 64)
    sinks = torch.randn(64, generator=g)
    pos = torch.tensor([3, 50, 100, 0, 150, 99])
    qd, kd, vd, sd, pd = q.to(DEV), k.to(DEV), v.to(DEV), sinks.to(DEV), pos.to(DEV)
    ops.attention_decode(qd, kd, vd, sd, 0.125, 128, pd)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = ops.attention_decode(qd, kd, vd, sd, 0.125, 128, pd)
    for step in range(3):
        graph.replay()
        torch.cuda.synchronize()
        for b in range(B):
            ref = O.attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], sinks, 0.125, 128, int(pos[b]) + step)
            assert_parity(ref, out[b:b + 1], f"replay {step}, sequence {b}")
        pd.add_(1)


@pytest.mark.parametrize("B", [1, 7, 40])
def test_qkv_decode_with_per_sequence_positions(ops, B):
    g = torch.Generator().manual_seed(2000 + B)
    ctx, hid = 128, 2880
    x = randn(g, B, 1, hid)
    w, bias = randn(g, 5120, hid, scale=0.02), randn(g, 5120, scale=0.02)
    pos = torch.randint(0, ctx, (B,), generator=g)
    cos, sin = O.yarn_cos_sin(ctx)
    ck0, cv0 = randn(g, B, ctx, 8, 64), randn(g, B, ctx, 8, 64)
    xd, wd, bd, cd, sd = x.to(DEV), w.to(DEV), bias.to(DEV), cos.to(DEV), sin.to(DEV)
    ck, cv = ck0.to(DEV), cv0.to(DEV)
    qr = ops.qkv_rope_cache_decode_forward(xd, wd, bd, sd, cd, ctx, ck, cv, pos.to(DEV), 64, 8, 64, per_sequence=True).clone()
    torch.cuda.synchronize()
    for b in range(B):
        # alone, through the reference-shaped call: bit for bit (no reduction order depends on the batch)
        ck1, cv1 = ck0[b:b + 1].to(DEV), cv0[b:b + 1].to(DEV)
        q1 = ops.qkv_rope_cache_decode_forward(xd[b:b + 1], wd, bd, sd, cd, ctx, ck1, cv1, pos[b:b + 1].to(DEV), 64, 8, 64).clone()
        assert torch.equal(q1, qr[b:b + 1])
        assert torch.equal(ck1[0], ck[b]) and torch.equal(cv1[0], cv[b])
    b = B - 1
    ckr, cvr = ck0[b:b + 1].clone(), cv0[b:b + 1].clone()
    q_ref = O.qkv_rope_cache_decode(x[b:b + 1], w, bias, cos, sin, int(pos[b]), ckr, cvr, max_ctx=ctx)
    assert_parity(q_ref, qr[b:b + 1], "ragged decode QKV vs oracle")
    assert_parity(ckr[0, int(pos[b])], ck[b, int(pos[b])], "K row vs oracle")

    # paged store: rows land in the sequence's page, nothing else changes
    page = 32
    kp0, vp0, table = _paged_copy(g, ck0, cv0, page)
    kp, vp = kp0.to(DEV), vp0.to(DEV)
    qp = ops.qkv_rope_paged_decode_forward(xd, wd, bd, sd, cd, ctx, kp, vp, table.to(DEV), pos.to(DEV), 64, 8, 64).clone()
    torch.cuda.synchronize()
    assert torch.equal(qp, qr)
    want_k, want_v = kp0.clone(), vp0.clone()
    for b in range(B):
        p = int(pos[b])
        want_k[table[b, p // page], p % page] = ck[b, p].cpu()
        want_v[table[b, p // page], p % page] = cv[b, p].cpu()
    assert torch.equal(kp.cpu(), want_k) and torch.equal(vp.cpu(), want_v)


def test_bad_positions_and_pages_are_recorded_not_followed(ops):
    from tritonllm_b200 import _lib
    g = torch.Generator().manual_seed(5)
    B, ctx, page = 3, 64, 32
    x = randn(g, B, 1, 2880)
    w, bias = randn(g, 5120, 2880, scale=0.02), randn(g, 5120, scale=0.02)
    cos, sin = O.yarn_cos_sin(ctx)
    k, v = randn(g, B, ctx, 8, 64), randn(g, B, ctx, 8, 64)
    kp, vp, table = _paged_copy(g, k, v, page)
    table[1, 1] = -1                                   # sequence 1 has no second page
    pos = torch.tensor([5, 40, 70])                    # 70 is beyond the capacity of 64
    kpd, vpd = kp.to(DEV), vp.to(DEV)
    before_k = kpd.clone()
    ops.qkv_rope_paged_decode_forward(x.to(DEV), w.to(DEV), bias.to(DEV), sin.to(DEV), cos.to(DEV), ctx, kpd, vpd,
                                      table.to(DEV), pos.to(DEV), 64, 8, 64)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0x10
    changed = (kpd != before_k).flatten(1).any(dim=1).nonzero().flatten().tolist()
    assert changed == [int(table[0, 0])]               # only sequence 0 wrote a row
    q = randn(g, B, 1, 8, 8, 64)
    ops.attention_decode_paged(q.to(DEV), kpd, vpd, table.to(DEV), torch.tensor([5, 40, 20]).to(DEV), None, 0.125, 0)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0x10                # sequence 1's visible range reaches the unmapped page
    assert _lib.device_status() == 0
    with pytest.raises(_lib.B2Error):                  # a page size that a 32-key tile could straddle
        ops.attention_decode_paged(q.to(DEV), kpd.view(-1, 16, 8, 64), vpd.view(-1, 16, 8, 64),
                                   torch.zeros(B, 8, dtype=torch.int32, device=DEV), torch.tensor([5, 40, 20]).to(DEV), None,
                                   0.125, 0)


def _tiny_model():
    from tritonllm_b200 import generate as G
    cfg = G.ModelConfig(num_hidden_layers=2, num_experts=32, vocab_size=1024)
    w = G.ModelWeights.random(cfg, "cuda", seed=11, fp4=True, draw_on="cpu")
    return G, G.Transformer(cfg, w, max_context=4096)


def test_ragged_generation_matches_each_sequence_alone_and_paged_matches_dense():
    """Three prompts of different lengths in one batch: the logits of the first step equal (within the bar of a chain
    of rounded ops) what each prompt gives alone in a batch of one with the reference's single position counter; the
    paged store reproduces the dense per-sequence store token for token."""
    G, model = _tiny_model()
    gen = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=gen).tolist() for n in (5, 70, 23)]
    new = 6
    tg = G.TokenGenerator(model, context=128, batch_size=3, per_sequence=True)
    ids, logits = tg.generate_ragged(prompts, new, return_first_logits=True)
    assert ids.shape == (3, new)
    assert tg.caches[0].offset.tolist() == [len(p) - 1 + new for p in prompts]
    tg_eager = G.TokenGenerator(model, context=128, batch_size=3, per_sequence=True, use_cuda_graph=False)
    ids_eager = tg_eager.generate_ragged(prompts, new)
    assert torch.equal(ids, ids_eager)                 # graph replay == eager launches
    for b, p in enumerate(prompts):
        one = G.TokenGenerator(model, context=128, batch_size=1, use_cuda_graph=False)
        for c in one.caches:
            c.reset()
        t = torch.tensor(p, device="cuda")[None, :]
        model.prefill(t[:, :-1], one.caches)
        alone = model.forward(t[:, -1:], caches=one.caches)[:, 0]
        assert_parity(alone[0], logits[b], f"sequence {b} in the ragged batch vs alone", max_rel=8e-2, rms_rel=1.6e-2,
                      min_cos=0.9998)
    for page_size in (32, 64):
        tp = G.TokenGenerator(model, context=128, batch_size=3, paged=True, page_size=page_size, n_pages=3 * (128 // page_size) + 2)
        ids_p, logits_p = tp.generate_ragged(prompts, new, return_first_logits=True)
        assert torch.equal(ids_p, ids) and torch.equal(logits_p, logits)
    # pages go back to the pool
    tp.store.reset()
    assert len(tp.store._free) == tp.store.n_pages and int(tp.store.block_table.max()) == -1
    with pytest.raises(ValueError):
        G.TokenGenerator(model, context=64, batch_size=3, use_cuda_graph=False).generate_ragged(prompts, 2)
