"""GPU parity of the decode-sized MoE expert MLP (b2_moe_experts_decode) through the C ABI."""
import numpy as np
import pytest
import torch

from _util import assert_parity, bf16_from_bits, bf16_ulp_diff, golden

import oracle as O

pytestmark = pytest.mark.gpu


def _ops():
    from tritonllm_b200 import ops
    return ops


def _random_experts(gen, E, N, K, scale_lo=118, scale_hi=123):
    codes = torch.randint(0, 256, (E, N, K // 2), generator=gen, dtype=torch.uint8)
    scales = torch.randint(scale_lo, scale_hi + 1, (E, N, K // 32), generator=gen, dtype=torch.uint8)
    bias = torch.randn(E, N, generator=gen) * 0.1
    return codes, scales, bias


FP4 = [False, True]   # weights converted in the kernel / the tensor cores' block-scaled FP4 path


def _run(x, vals, idx, w1, w2, fp4=False):
    ops = _ops()
    dev = "cuda"
    W1 = ops.ExpertWeights(w1[0].to(dev), w1[1].to(dev), w1[2].to(dev))
    W2 = ops.ExpertWeights(w2[0].to(dev), w2[1].to(dev), w2[2].to(dev))
    if fp4:
        W1, W2 = ops.ExpertWeightsFp4(W1), ops.ExpertWeightsFp4(W2)
    out = ops.moe_experts_decode(x.to(dev), vals.to(dev), idx.to(dev), W1, W2)
    torch.cuda.synchronize()
    from tritonllm_b200 import _lib
    assert _lib.device_status() == 0
    return out.cpu()


def _oracle(x, vals, idx, w1, w2):
    return O.moe_experts(x, vals, idx, w1[0].numpy(), w1[1].numpy(), w1[2], w2[0].numpy(), w2[1].numpy(), w2[2])


@pytest.mark.parametrize("fp4", FP4)
def test_moe_golden(fp4):
    g = golden("moe_experts")
    x = bf16_from_bits(g["x_bf16"])
    vals, idx = torch.from_numpy(g["vals"]), torch.from_numpy(g["idx"])
    w1 = (torch.from_numpy(g["q1"].transpose(0, 2, 1).copy()), torch.from_numpy(g["s1"].transpose(0, 2, 1).copy()),
          torch.from_numpy(g["b1"]))
    w2 = (torch.from_numpy(g["q2"].transpose(0, 2, 1).copy()), torch.from_numpy(g["s2"].transpose(0, 2, 1).copy()),
          torch.from_numpy(g["b2"]))
    out = _run(x, vals, idx, w1, w2, fp4)
    ref = bf16_from_bits(g["out_bf16"])
    assert_parity(ref, out, "moe golden")


@pytest.mark.parametrize("T,E,H,I", [(1, 32, 2880, 2880), (5, 32, 2880, 2880), (32, 32, 2880, 2880),
                                     (256, 32, 2880, 2880), (70, 128, 2880, 2880), (33, 8, 192, 320),
                                     (40, 8, 256, 512)])   # the last: four k-blocks, so the last GEMM runs as two halves of two
@pytest.mark.parametrize("fp4", FP4)
def test_moe_vs_oracle(T, E, H, I, fp4):
    gen = torch.Generator().manual_seed(4000 + T + E)
    x = torch.randn(T, H, generator=gen).bfloat16()
    logits = torch.randn(T, E, generator=gen)
    vals, idx, _ = O.topk_softmax(logits, 4)
    w1 = _random_experts(gen, E, 2 * I, H)
    w2 = _random_experts(gen, E, H, I)
    out = _run(x, vals, idx, w1, w2, fp4)
    ref = _oracle(x, vals, idx, w1, w2)
    assert_parity(ref, out, f"moe T={T} E={E} fp4={fp4}")


@pytest.mark.parametrize("knobs", [{"moe_fp4_fuse": 2, "moe_fp4_tok": 8}, {"moe_fp4_fuse": 2, "moe_fp4_tok": 16},
                                   {"moe_fp4_fuse": 1, "moe_fp4_tok": 32}, {"moe_fp4_fuse": 1, "moe_fp4_ksplit": 1},
                                   {"moe_fp4_persist": 0}, {"moe_fp4_persist": 2}])
def test_moe_fp4_kernel_variants_agree_with_the_oracle(knobs):
    """The FP4 path picks its kernel by batch size (part size, one fused launch or two, half-k units, persistent or
    one-shot); every variant is forced here on the same 72-token batch."""
    from tritonllm_b200 import _lib
    lib = _lib.load()
    T, E, H, I = 72, 32, 2880, 2880
    gen = torch.Generator().manual_seed(4100)
    x = torch.randn(T, H, generator=gen).bfloat16()
    vals, idx, _ = O.topk_softmax(torch.randn(T, E, generator=gen), 4)
    w1, w2 = _random_experts(gen, E, 2 * I, H), _random_experts(gen, E, H, I)
    try:
        for k, v in knobs.items():
            _lib.check("b2_set_tunable", lib.b2_set_tunable(k.encode(), v))
        out = _run(x, vals, idx, w1, w2, True)
    finally:
        for k in knobs:
            _lib.check("b2_set_tunable", lib.b2_set_tunable(k.encode(), 0 if k != "moe_fp4_persist" else 4))
    assert_parity(_oracle(x, vals, idx, w1, w2), out, f"moe fp4 variant {knobs}")


def test_moe_fused_launch_replays_from_a_cuda_graph():
    """96 tokens on 32 experts take the one-launch path (32-token parts); its per-item completion counts are zeroed by
    the routing launch of the same call, so a captured call must give the same rows on every replay."""
    ops = _ops()
    T, E, H, I = 96, 32, 2880, 2880
    gen = torch.Generator().manual_seed(4300)
    x = torch.randn(T, H, generator=gen).bfloat16().cuda()
    vals, idx, _ = O.topk_softmax(torch.randn(T, E, generator=gen), 4)
    vals, idx = vals.cuda(), idx.to(torch.int16).cuda()
    W1, W2 = _packed(_random_experts(gen, E, 2 * I, H)), _packed(_random_experts(gen, E, H, I))
    eager = ops.moe_experts_decode(x, vals, idx, W1, W2).clone()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = ops.moe_experts_decode(x, vals, idx, W1, W2)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.int16), eager.view(torch.int16))
    from tritonllm_b200 import _lib
    assert _lib.device_status() == 0


@pytest.mark.parametrize("fp4", FP4)
def test_moe_all_tokens_one_expert_set(fp4):
    """Every token picks the same four experts: 256 rows per expert, the largest token tile."""
    T, E, H, I = 256, 8, 256, 128
    gen = torch.Generator().manual_seed(4100)
    x = torch.randn(T, H, generator=gen).bfloat16()
    idx = torch.tensor([[1, 3, 4, 6]], dtype=torch.int16).repeat(T, 1)
    vals = torch.softmax(torch.randn(T, 4, generator=gen), dim=1)
    w1 = _random_experts(gen, E, 2 * I, H)
    w2 = _random_experts(gen, E, H, I)
    out = _run(x, vals, idx, w1, w2, fp4)
    assert_parity(_oracle(x, vals, idx, w1, w2), out, "moe one expert set")


@pytest.mark.parametrize("fp4", FP4)
def test_moe_is_deterministic_and_row_independent(fp4):
    """Same token, different batch neighbours: the token's output row must not change bit for bit."""
    E, H, I = 32, 2880, 2880
    gen = torch.Generator().manual_seed(4200)
    x = torch.randn(48, H, generator=gen).bfloat16()
    vals, idx, _ = O.topk_softmax(torch.randn(48, E, generator=gen), 4)
    w1 = _random_experts(gen, E, 2 * I, H)
    w2 = _random_experts(gen, E, H, I)
    full = _run(x, vals, idx, w1, w2, fp4)
    again = _run(x, vals, idx, w1, w2, fp4)
    assert torch.equal(full.view(torch.int16), again.view(torch.int16))
    part = _run(x[7:20].contiguous(), vals[7:20].contiguous(), idx[7:20].contiguous(), w1, w2, fp4)
    assert torch.equal(full[7:20].view(torch.int16), part.view(torch.int16))


def test_moe_rejects_unsupported():
    ops = _ops()
    from tritonllm_b200._lib import B2Error
    gen = torch.Generator().manual_seed(1)
    w1 = _random_experts(gen, 4, 128, 64)
    w2 = _random_experts(gen, 4, 64, 64)
    W1 = ops.ExpertWeights(*[t.cuda() for t in w1])
    W2 = ops.ExpertWeights(*[t.cuda() for t in w2])
    x = torch.zeros(257, 64, dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros(257, 4, dtype=torch.int16, device="cuda")
    vals = torch.zeros(257, 4, device="cuda")
    with pytest.raises(B2Error):
        ops.moe_experts_decode(x, vals, idx, W1, W2)   # more than 256 tokens: not the decode regime
    out = ops.moe_experts_decode(x[:0], vals[:0], idx[:0], W1, W2)
    assert out.shape == (0, 64)


# ----------------------------------------------------------------------------- fused norm + router + top-k
@pytest.mark.parametrize("rows,hidden,E,bias", [(1, 2880, 32, True), (32, 2880, 32, True), (256, 2880, 32, False),
                                                (300, 2880, 128, True), (5, 192, 64, True), (7, 3072, 32, False)])
def test_norm_router_topk_fused(rows, hidden, E, bias):
    """One launch against the three ops it replaces: the normalised row is rmsnorm_forward's up to one bf16 step
    (the sum of squares is added in another order), the logits are the oracle's on the kernel's own row up to one
    bf16 step, and the selection is the oracle's top-k of the kernel's own logits, bit for bit."""
    from tritonllm_b200 import ops
    gen = torch.Generator().manual_seed(900 + rows + E)
    x = (torch.randn(rows, 1, hidden, generator=gen) * 3).bfloat16().cuda()
    gain = (1 + 0.05 * torch.randn(hidden, generator=gen)).cuda()
    wg = (torch.randn(hidden, E, generator=gen) * 0.02).bfloat16().cuda()
    bg = (torch.randn(E, generator=gen) * 0.02).cuda() if bias else None
    y, vals, idx, logits = ops.norm_router_topk(x, gain, 1e-5, wg, bg, 4, return_logits=True)
    y_ref = ops.rmsnorm_forward(x, gain, 1e-5, out=torch.empty_like(x))
    torch.cuda.synchronize()
    assert y.shape == x.shape and int(bf16_ulp_diff(y, y_ref).max()) <= 1
    assert_parity(O.rmsnorm(x.cpu(), gain.cpu(), 1e-5), y, "fused norm vs oracle")
    lg_oracle = O.router_logits(y.cpu().reshape(rows, hidden), wg.cpu(), None if bg is None else bg.cpu())
    assert (logits.cpu() - lg_oracle).abs().max() <= 2 ** -6 * max(1.0, lg_oracle.abs().max().item())   # one bf16 step
    v_ref, i_ref = O.topk_softmax(logits.cpu(), 4)[:2]
    assert torch.equal(idx.cpu(), i_ref) and idx.dtype == torch.int16
    assert torch.allclose(vals.cpu(), v_ref, rtol=1e-5, atol=1e-7)
    # without the logits output, and in place on x
    y2, vals2, idx2 = ops.norm_router_topk(x, gain, 1e-5, wg, bg, 4, y_out=x)
    torch.cuda.synchronize()
    assert y2.data_ptr() == x.data_ptr() and torch.equal(x, y) and torch.equal(idx2, idx) and torch.equal(vals2, vals)


def test_norm_router_topk_rejects_unsupported_shapes():
    from tritonllm_b200 import _lib, ops
    x = torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda")
    g = torch.ones(64, device="cuda")
    with pytest.raises(_lib.B2Error):
        ops.norm_router_topk(x, g, 1e-5, torch.zeros(64, 48, dtype=torch.bfloat16, device="cuda"), None, 4)   # E % 32
    with pytest.raises(_lib.B2Error):
        ops.norm_router_topk(x, g, 1e-5, torch.zeros(64, 32, dtype=torch.bfloat16, device="cuda"), None, 5)   # k > 4
    y, vals, idx = ops.norm_router_topk(x[:0], g, 1e-5, torch.zeros(64, 32, dtype=torch.bfloat16, device="cuda"), None, 4)
    assert y.shape == (0, 64) and vals.shape == (0, 4) and idx.shape == (0, 4)


# ----------------------------------------------------------------------------- FP4 path beyond 256 tokens
@pytest.mark.parametrize("T,E,H,I", [(700, 32, 256, 128), (2048, 8, 256, 128), (1000, 32, 2880, 2880)])
def test_moe_fp4_prompt_sized_blocks(T, E, H, I):
    """Up to 2048 tokens per call: an expert's tokens are spread over CTAs of 64."""
    gen = torch.Generator().manual_seed(4300 + T)
    x = torch.randn(T, H, generator=gen).bfloat16()
    vals, idx, _ = O.topk_softmax(torch.randn(T, E, generator=gen), 4)
    w1 = _random_experts(gen, E, 2 * I, H)
    w2 = _random_experts(gen, E, H, I)
    out = _run(x, vals, idx, w1, w2, True)
    assert_parity(_oracle(x, vals, idx, w1, w2), out, f"moe fp4 T={T} E={E}")


def test_moe_fp4_2048_tokens_on_four_experts():
    """Every token picks the same four experts: 2048 rows per expert, 32 parts each."""
    T, E, H, I = 2048, 8, 256, 128
    gen = torch.Generator().manual_seed(4400)
    x = torch.randn(T, H, generator=gen).bfloat16()
    idx = torch.tensor([[0, 2, 5, 7]], dtype=torch.int16).repeat(T, 1)
    vals = torch.softmax(torch.randn(T, 4, generator=gen), dim=1)
    w1 = _random_experts(gen, E, 2 * I, H)
    w2 = _random_experts(gen, E, H, I)
    out = _run(x, vals, idx, w1, w2, True)
    assert_parity(_oracle(x, vals, idx, w1, w2), out, "moe fp4 2048 rows per expert")
    ops = _ops()
    from tritonllm_b200._lib import B2Error
    W1, W2 = (ops.ExpertWeightsFp4(ops.ExpertWeights(*[t.cuda() for t in w])) for w in (w1, w2))
    with pytest.raises(B2Error):
        ops.moe_experts_decode(torch.zeros(2049, H, dtype=torch.bfloat16, device="cuda"), torch.zeros(2049, 4, device="cuda"),
                               torch.zeros(2049, 4, dtype=torch.int16, device="cuda"), W1, W2)


@pytest.mark.parametrize("T", [1, 32, 256, 700])
def test_moe_deferred_combine_with_add_and_norm(T):
    """The expert sum left to the add + norm that follows: the residual stream is bit-identical to combine-then-add,
    the normalised row equals add_rmsnorm_forward's up to one bf16 step (sum of squares added in another order)."""
    ops = _ops()
    E, H, I = 32, 2880, 2880
    gen = torch.Generator().manual_seed(4500 + T)
    x = torch.randn(T, H, generator=gen).bfloat16().cuda()
    res = torch.randn(T, 1, H, generator=gen).bfloat16().cuda()
    gain = (1 + 0.05 * torch.randn(H, generator=gen)).cuda()
    vals, idx, _ = O.topk_softmax(torch.randn(T, E, generator=gen), 4)
    vals, idx = vals.cuda(), idx.cuda()
    w1 = _random_experts(gen, E, 2 * I, H)
    w2 = _random_experts(gen, E, H, I)
    W1, W2 = (ops.ExpertWeightsFp4(ops.ExpertWeights(*[t.cuda() for t in w])) for w in (w1, w2))
    out = ops.moe_experts_decode(x, vals, idx, W1, W2)
    h_ref, y_ref = ops.add_rmsnorm_forward(res, out.view(T, 1, H), gain, 1e-5)
    pending = ops.moe_experts_decode(x, vals, idx, W1, W2, defer_combine=True)
    assert isinstance(pending, ops.PendingMoe)
    h, y = ops.moe_combine_add_rmsnorm(pending, res, gain, 1e-5)
    torch.cuda.synchronize()
    assert torch.equal(h, h_ref) and int(bf16_ulp_diff(y, y_ref).max()) <= 1
    # in place on the residual
    pending = ops.moe_experts_decode(x, vals, idx, W1, W2, defer_combine=True)
    h2, y2 = ops.moe_combine_add_rmsnorm(pending, res, gain, 1e-5, h_out=res)
    torch.cuda.synchronize()
    assert h2.data_ptr() == res.data_ptr() and torch.equal(res, h_ref) and torch.equal(y2, y)
    from tritonllm_b200 import _lib
    assert _lib.device_status() == 0


def test_moe_flags_an_expert_chosen_twice_by_one_token():
    """The routing lists count an expert once per token; a duplicate id (never produced by `topk`) is recorded in
    the device status word instead of silently summing one expert row twice."""
    ops = _ops()
    from tritonllm_b200 import _lib
    gen = torch.Generator().manual_seed(77)
    T, E, H, I = 4, 8, 256, 128
    dev = "cuda"
    x = (torch.randn(T, H, generator=gen)).to(torch.bfloat16).to(dev)
    w1, w2 = _random_experts(gen, E, 2 * I, H), _random_experts(gen, E, H, I)
    W1 = ops.ExpertWeightsFp4(ops.ExpertWeights(*(t.to(dev) for t in w1)))
    W2 = ops.ExpertWeightsFp4(ops.ExpertWeights(*(t.to(dev) for t in w2)))
    idx = torch.tensor([[0, 1, 2, 3], [1, 1, 4, 5], [0, 2, 4, 6], [1, 3, 5, 7]], dtype=torch.int16, device=dev)
    vals = torch.full((T, 4), 0.25, device=dev)
    assert _lib.device_status() == 0
    ops.moe_experts_decode(x, vals, idx, W1, W2)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0x10
    assert _lib.device_status() == 0


# ----------------------------------------------------------------------------- prompt-sized batches (grouped GEMM)
def _packed(w):
    ops = _ops()
    dev = "cuda"
    return ops.ExpertWeightsFp4(ops.ExpertWeights(w[0].to(dev), w[1].to(dev), w[2].to(dev)))


@pytest.mark.parametrize("E,N,K", [(3, 320, 384), (2, 5760, 2880), (5, 192, 96)])
def test_upcast_of_the_packed_layout_is_exact(E, N, K):
    """b2_moe_upcast_packed reads the padded codes and the 512-byte scale blocks of ExpertWeightsFp4 and must give
    exactly the values the reference's upcast gives for the original tensors."""
    from tritonllm_b200 import _lib
    gen = torch.Generator().manual_seed(E * 1000 + N)
    w = _random_experts(gen, E, N, K, scale_lo=100, scale_hi=140)
    pk = _packed(w)
    out = torch.empty((E * N, K), dtype=torch.bfloat16, device="cuda")
    _lib.call("b2_moe_upcast_packed", pk.codes.data_ptr(), pk.sf.data_ptr(), out.data_ptr(), E, N, K,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    want = torch.from_numpy(O.mxfp4_upcast(w[0].reshape(E * N, K // 2).numpy(), w[1].reshape(E * N, K // 32).numpy()))
    assert torch.equal(out.cpu().float(), want.float())


def _routing(gen, T, E):
    logits = torch.randn(T, E, generator=gen)
    vals, idx = O.topk_softmax(logits, 4)[:2]
    return vals, idx.to(torch.int16)


@pytest.mark.parametrize("T,E,H,I", [(700, 8, 384, 192), (2049, 32, 384, 192), (300, 4, 768, 384)])
def test_moe_prefill_vs_oracle_small_dims(T, E, H, I):
    ops = _ops()
    gen = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    vals, idx = _routing(gen, T, E)
    w1, w2 = _random_experts(gen, E, 2 * I, H), _random_experts(gen, E, H, I)
    out = ops.moe_experts_prefill(x.cuda(), vals.cuda(), idx.cuda(), _packed(w1), _packed(w2))
    torch.cuda.synchronize()
    from tritonllm_b200 import _lib
    assert _lib.device_status() == 0
    assert_parity(_oracle(x, vals, idx, w1, w2), out, f"prompt-sized MoE T={T} E={E}")


def test_moe_prefill_real_dims_against_the_oracle_and_the_decode_sized_kernel():
    ops = _ops()
    gen = torch.Generator().manual_seed(4242)
    T, E, H, I = 3000, 32, 2880, 2880
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16)
    vals, idx = _routing(gen, T, E)
    idx[100:140] = torch.tensor([0, 1, 2, 3], dtype=torch.int16)      # a run of tokens on the same experts
    w1, w2 = _random_experts(gen, E, 2 * I, H), _random_experts(gen, E, H, I, scale_lo=113, scale_hi=118)
    W1, W2 = _packed(w1), _packed(w2)
    xd, vd, idd = x.cuda(), vals.cuda(), idx.cuda()
    out = ops.moe_experts_prefill(xd, vd, idd, W1, W2)
    small = torch.cat([ops.moe_experts_decode(xd[r:r + 1500], vd[r:r + 1500], idd[r:r + 1500], W1, W2) for r in (0, 1500)])
    torch.cuda.synchronize()
    from tritonllm_b200 import _lib
    assert _lib.device_status() == 0
    # both paths multiply exactly and accumulate in fp32: only the order of the sums differs
    assert_parity(small, out, "grouped GEMM vs decode-sized kernel", rms_rel=1e-3)
    sel = torch.cat([torch.arange(0, 24), torch.arange(100, 108), torch.arange(T - 8, T)])
    assert_parity(_oracle(x[sel], vals[sel], idx[sel], w1, w2), out[sel], "prompt-sized MoE, sampled tokens vs oracle")


def test_moe_prefill_resident_expansion_is_the_same_computation():
    """With a budget, the bf16 expansion of an expert pair is made once and kept; results do not change."""
    ops = _ops()
    E, H, I, T = 8, 768, 768, 640
    gen = torch.Generator().manual_seed(4702)
    x = torch.randn(T, H, generator=gen).bfloat16()
    vals, idx = _routing(gen, T, E)
    p1, p2 = _packed(_random_experts(gen, E, 2 * I, H)), _packed(_random_experts(gen, E, H, I))
    args = (x.cuda(), vals.cuda(), idx.cuda(), p1, p2)
    plain = ops.moe_experts_prefill(*args).cpu()
    ops.set_expanded_expert_budget(1 << 30)
    try:
        first = ops.moe_experts_prefill(*args).cpu()
        assert getattr(p1, "_expanded", None) is not None
        second = ops.moe_experts_prefill(*args).cpu()          # no expansion this time
        ops.drop_expanded_experts(p1)
        assert p1._expanded is None
    finally:
        ops.set_expanded_expert_budget(0)
        ops.drop_expanded_experts()
    torch.cuda.synchronize()
    assert torch.equal(plain.view(torch.int16), first.view(torch.int16))
    assert torch.equal(plain.view(torch.int16), second.view(torch.int16))


def test_moe_prefill_config4_shape_and_edges():
    """BASELINE config 4's token count and expert count (16384 tokens, 128 experts, hidden 2880): every token of the
    grouped-GEMM path against the decode-sized kernel run in blocks, plus experts without tokens."""
    ops = _ops()
    gen = torch.Generator().manual_seed(77)
    T, E, H, I = 16384, 128, 2880, 2880
    x = torch.randn(T, H, generator=gen).to(torch.bfloat16).cuda()
    logits = torch.randn(T, E, generator=gen)
    logits[:, 5] = -1e9           # expert 5 never chosen
    logits[:, 100:104] -= 50.0    # nor these
    vals, idx = O.topk_softmax(logits, 4)[:2]
    vd, idd = vals.cuda(), idx.to(torch.int16).cuda()
    gd = torch.Generator(device="cuda").manual_seed(78)

    def experts(n, k, lo, hi):
        w = ops.ExpertWeights(torch.randint(0, 256, (E, n, k // 2), dtype=torch.uint8, device="cuda", generator=gd),
                              torch.randint(lo, hi, (E, n, k // 32), dtype=torch.uint8, device="cuda", generator=gd),
                              torch.randn(E, n, device="cuda", generator=gd) * 0.1)
        return ops.ExpertWeightsFp4(w)
    W1, W2 = experts(2 * I, H, 118, 124), experts(H, I, 113, 118)
    out = ops.moe_experts_prefill(x, vd, idd, W1, W2)
    ref = torch.cat([ops.moe_experts_decode(x[r:r + 2048], vd[r:r + 2048], idd[r:r + 2048], W1, W2) for r in range(0, T, 2048)])
    torch.cuda.synchronize()
    from tritonllm_b200 import _lib
    assert _lib.device_status() == 0
    assert_parity(ref, out, "config 4 shape: grouped GEMM vs decode-sized kernel", rms_rel=1e-3)
    assert torch.equal(ops.moe_experts_prefill(x, vd, idd, W1, W2), out)     # deterministic despite the atomic row order
    bad = idd.clone()
    bad[7, 2] = 500
    bad[9, 1] = bad[9, 0]
    ops.moe_experts_prefill(x, vd, bad, W1, W2)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0x10
