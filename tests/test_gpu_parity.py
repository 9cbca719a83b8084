"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle and the golden
fixtures, on seeded inputs.  Tolerance for bf16 tensors is BASELINE's: max relative error
<= 2e-2 (reference normalisation), rms <= 4e-3, cosine >= 0.9999 per tensor; router indices
and bit masks are compared bit for bit."""
import numpy as np
import pytest
import torch

import oracle as O
from _util import assert_parity, bf16_from_bits, bf16_ulp_diff, golden, randn, t

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from tritonllm_b200 import _lib, ops as _ops
    _lib.load()
    assert _lib.device_status() == 0
    yield _ops
    assert _lib.device_status() == 0, "a kernel gave up a bounded wait"


@pytest.fixture(scope="module")
def tables():
    cos, sin = O.yarn_cos_sin(131072)
    return cos, sin, cos.to(DEV), sin.to(DEV)


# ------------------------------------------------------------------------------ RMSNorm
@pytest.mark.parametrize("rows,dim", [(1, 2880), (5, 2880), (33, 2880), (4099, 2880), (7, 64), (3, 8), (9, 1024),
                                      (4, 4096), (2, 5120), (0, 2880)])
def test_rmsnorm(ops, rows, dim):
    g = torch.Generator().manual_seed(11 + rows + dim)
    x = randn(g, rows, dim)
    gain = randn(g, dim, scale=0.05, shift=1.0, dtype=torch.float32)
    y = ops.rmsnorm_forward(x.to(DEV), gain.to(DEV), 1e-5, out=torch.empty(rows, dim, dtype=torch.bfloat16, device=DEV))
    if rows == 0:
        return
    ref = O.rmsnorm(x, gain, 1e-5)
    assert_parity(ref, y, "rmsnorm")
    ulp = bf16_ulp_diff(ref, y)
    assert ulp.max() <= 1 and (ulp > 0).float().mean() < 0.02  # same arithmetic: at most rounding-boundary flips


def test_rmsnorm_golden_and_in_place(ops):
    gd = golden("rmsnorm")
    x = bf16_from_bits(gd["x_bf16"])
    xd = x.to(DEV)
    y = ops.rmsnorm_forward(xd, t(gd["gain"]).to(DEV), 1e-5)
    assert_parity(t(gd["y"]), y, "rmsnorm vs reference kernel (fp32 mode)", max_rel=1e-2)
    y2 = ops.rmsnorm_forward(xd, t(gd["gain"]).to(DEV), 1e-5, out=xd)  # final-norm call site aliases out = x
    assert y2.data_ptr() == xd.data_ptr() and torch.equal(y2.cpu(), y.cpu())


@pytest.mark.parametrize("rows", [1, 6, 2500])
def test_add_rmsnorm(ops, rows):
    g = torch.Generator().manual_seed(21 + rows)
    x, d = randn(g, rows, 2880), randn(g, rows, 2880, scale=0.5)
    gain = randn(g, 2880, scale=0.05, shift=1.0, dtype=torch.float32)
    h_ref, y_ref = O.add_rmsnorm(x, d, gain, 1e-5)
    xd = x.to(DEV)
    h, y = ops.add_rmsnorm_forward(xd, d.to(DEV), gain.to(DEV), 1e-5, h_out=xd)  # residual updated in place
    assert h.data_ptr() == xd.data_ptr()
    assert torch.equal(h.cpu().view(torch.int16), h_ref.view(torch.int16))  # a bf16 add is exact to the bit
    assert_parity(y_ref, y, "add_rmsnorm")
    assert bf16_ulp_diff(y_ref, y).max() <= 1


# --------------------------------------------------------------------------------- RoPE
@pytest.mark.parametrize("B,T,offset", [(1, 1, 0), (2, 5, 131069), (1, 61, 7), (3, 130, 4000)])
def test_rope(ops, tables, B, T, offset):
    cos, sin, cos_d, sin_d = tables
    g = torch.Generator().manual_seed(31 + T)
    q, k = randn(g, B, T, 64, 64), randn(g, B, T, 8, 64)
    qr, kr = O.rope(q, k, cos, sin, offset, 131072)
    qd, kd = q.to(DEV), k.to(DEV)
    ops.rope_forward(qd, kd, sin_d, cos_d, 131072, torch.tensor([offset], dtype=torch.int64, device=DEV))
    assert_parity(qr, qd, "rope q")
    assert_parity(kr, kd, "rope k")
    # fused multiply-add on the GPU vs separate roundings in torch: one bf16 step, except where
    # x1*cos - x2*sin cancels to a value far smaller than its terms
    for src, ref, got in ((q, qr, qd), (k, kr, kd)):
        ulp = bf16_ulp_diff(ref, got)
        assert (ulp > 1).float().mean() < 1e-4 and (ulp > 0).float().mean() < 0.02
        torch.testing.assert_close(got.cpu().float(), ref.float(), atol=2e-3, rtol=2 ** -7)
        # which elements exceed one step: only those where the two products cancel, i.e. the result is at least
        # eight times smaller than the larger input of its (j, j + 32) pair
        big = torch.maximum(src[..., :32].abs(), src[..., 32:].abs()).float().repeat(1, 1, 1, 2)
        off = ulp > 1
        assert bool((ref.float().abs()[off] * 8 <= big[off]).all()), \
            f"{int(off.sum())} elements differ by more than one bf16 step; not all of them are cancellations"


def test_rope_golden(ops, tables):
    _, _, cos_d, sin_d = tables
    gd = golden("rope")
    qd, kd = bf16_from_bits(gd["q_in"]).to(DEV), bf16_from_bits(gd["k_in"]).to(DEV)
    ops.rope_forward(qd, kd, sin_d, cos_d, 131072, torch.tensor([int(gd["offset"])], dtype=torch.int64, device=DEV))
    # the interpreter truncates its bf16 stores: allow one bf16 step
    assert bf16_ulp_diff(bf16_from_bits(gd["q_out"]), qd).max() <= 1
    assert bf16_ulp_diff(bf16_from_bits(gd["k_out"]), kd).max() <= 1


# ------------------------------------------------------------------------- decode QKV
def _qkv_case(g, B, hid, nq, nkv, ctx):
    d = 64
    x = randn(g, B, 1, hid)
    w = randn(g, (nq + 2 * nkv) * d, hid, scale=0.02)
    b = randn(g, (nq + 2 * nkv) * d, scale=0.02)
    ck = randn(g, B, ctx, nkv, d)
    cv = randn(g, B, ctx, nkv, d)
    return x, w, b, ck, cv


@pytest.mark.parametrize("B,hid,nq,nkv,ctx,offset", [(1, 2880, 64, 8, 16, 0), (3, 2880, 64, 8, 16, 15),
                                                     (32, 2880, 64, 8, 8, 5), (70, 2880, 64, 8, 4, 3),
                                                     (5, 576, 2, 1, 6, 4), (2, 64, 1, 1, 3, 2)])
def test_qkv_rope_cache_decode(ops, tables, B, hid, nq, nkv, ctx, offset):
    cos, sin, cos_d, sin_d = tables
    g = torch.Generator().manual_seed(41 + B + hid)
    x, w, b, ck, cv = _qkv_case(g, B, hid, nq, nkv, ctx)
    ck_ref, cv_ref = ck.clone(), cv.clone()
    q_ref = O.qkv_rope_cache_decode(x, w, b, cos, sin, offset, ck_ref, cv_ref, nq, nkv, 64, max_ctx=131072)
    ckd, cvd = ck.to(DEV), cv.to(DEV)
    q = ops.qkv_rope_cache_decode_forward(x.to(DEV), w.to(DEV), b.to(DEV), sin_d, cos_d, 131072, ckd, cvd,
                                          torch.tensor([offset], dtype=torch.int64, device=DEV), nq, nkv, 64)
    assert_parity(q_ref, q, "decode q")
    assert_parity(ck_ref[:, offset], ckd[:, offset], "decode k row")
    assert_parity(cv_ref[:, offset], cvd[:, offset], "decode v row")
    # every other cache row is untouched
    keep = [i for i in range(ctx) if i != offset]
    assert torch.equal(ckd.cpu()[:, keep], ck[:, keep]) and torch.equal(cvd.cpu()[:, keep], cv[:, keep])


def test_qkv_decode_golden(ops):
    gd = golden("qkv_decode")
    hid, nq, nkv, d, B, ctx = [int(v) for v in gd["dims"]]
    off = int(gd["offset"])
    cos = torch.zeros(off + 1, d // 2)
    sin = torch.zeros(off + 1, d // 2)
    cos[off], sin[off] = t(gd["cos_row"]), t(gd["sin_row"])
    ckd = torch.zeros(B, ctx, nkv, d, dtype=torch.bfloat16, device=DEV)
    cvd = torch.zeros_like(ckd)
    q = ops.qkv_rope_cache_decode_forward(bf16_from_bits(gd["x_bf16"]).to(DEV), bf16_from_bits(gd["w_bf16"]).to(DEV),
                                          bf16_from_bits(gd["b_bf16"]).to(DEV), sin.to(DEV), cos.to(DEV), off + 1, ckd,
                                          cvd, torch.tensor([off], dtype=torch.int64, device=DEV), nq, nkv, d)
    assert_parity(t(gd["q"]), q, "decode q vs reference kernels", max_rel=1e-2)
    assert_parity(t(gd["cache_k"]), ckd, "decode cache_k vs reference kernels", max_rel=1e-2)
    assert_parity(t(gd["cache_v"]), cvd, "decode cache_v vs reference kernels", max_rel=1e-2)


# ----------------------------------------------------------------------- decode o_proj
@pytest.mark.parametrize("B,kin,nout", [(1, 4096, 2880), (4, 4096, 2880), (32, 4096, 2880), (65, 4096, 2880),
                                        (3, 192, 160), (2, 64, 8)])
def test_out_residual_decode(ops, B, kin, nout):
    g = torch.Generator().manual_seed(51 + B + kin)
    x = randn(g, B, 1, kin)
    w = randn(g, nout, kin, scale=0.02)
    b = randn(g, nout, scale=0.02)
    res = randn(g, B, 1, nout)
    ref = O.out_residual(x.reshape(B, kin), w, b, res.reshape(B, nout))
    resd = res.to(DEV)
    out = ops.out_residual_decode_forward(x.to(DEV), w.to(DEV), b.to(DEV), resd)
    assert out.data_ptr() == resd.data_ptr() and out.shape == (B, 1, nout)  # written into the residual
    assert_parity(ref, out.reshape(B, nout), "o_proj + residual")


def test_out_residual_golden(ops):
    gd = golden("out_residual")
    res = bf16_from_bits(gd["res_bf16"])
    B, nout = res.shape
    out = ops.out_residual_decode_forward(bf16_from_bits(gd["t_bf16"])[:, None, :].to(DEV),
                                          bf16_from_bits(gd["w_bf16"]).to(DEV), bf16_from_bits(gd["b_bf16"]).to(DEV),
                                          res[:, None, :].contiguous().to(DEV))
    assert_parity(t(gd["out"]), out.reshape(B, nout), "o_proj vs reference kernel", max_rel=1e-2)


# --------------------------------------------------------------------- decode attention
def _attn_inputs(g, B, ctx, Hkv=8, G=8, sinks_dtype=torch.bfloat16):
    q = randn(g, B, 1, Hkv, G, 64)
    k = randn(g, B, ctx, Hkv, 64)
    v = randn(g, B, ctx, Hkv, 64)
    s = randn(g, Hkv * G, dtype=sinks_dtype)
    return q, k, v, s


@pytest.mark.parametrize("tag", ["dec_a", "dec_b", "dec_c", "dec_d", "dec_e", "dec_f"])
def test_attention_decode_golden(ops, tag):
    gd = golden("attention")
    q, k, v, s = (bf16_from_bits(gd[f"{tag}__{n}"]) for n in ("q", "k", "v", "sinks"))
    window, start = int(gd[f"{tag}__window"]), int(gd[f"{tag}__start"])
    o = ops.attention_decode(q.to(DEV), k.to(DEV), v.to(DEV), s.to(DEV), 0.125, window,
                             torch.tensor([start], dtype=torch.int32, device=DEV))
    o_ref = bf16_from_bits(gd[f"{tag}__o_ref"])        # the reference's attention_ref
    o_ker = bf16_from_bits(gd[f"{tag}__o_kernel"])     # the reference's Triton decode kernel
    assert_parity(o_ref, o, "decode attention vs attention_ref")
    torch.testing.assert_close(o.cpu().float(), o_ref.float(), atol=1e-2, rtol=1e-1)  # the reference's own test bar
    assert_parity(o_ker.reshape(o_ref.shape), o, "decode attention vs reference kernel")


@pytest.mark.parametrize("B,ctx,window,start", [
    (1, 128, 0, 0), (2, 128, 0, 5), (2, 128, 128, 63), (1, 1024, 0, 1023), (2, 2048, 2048, 2047), (2, 4096, 0, 1023),
    (1, 4096, 128, 127), (1, 4096, 128, 128), (3, 4096, 128, 4095), (2, 4096, 0, 4095), (1, 70, 0, 69),
    (2, 200, 0, 500), (33, 512, 0, 300), (1, 8192, 0, 8191)])
def test_attention_decode_vs_oracle(ops, B, ctx, window, start):
    g = torch.Generator().manual_seed(61 + B + ctx + start)
    q, k, v, s = _attn_inputs(g, B, ctx)
    ref = O.attention(q, k, v, s, 0.125, window, start)
    sq = torch.tensor([start], dtype=torch.int64, device=DEV)
    o = ops.attention_decode(q.to(DEV), k.to(DEV), v.to(DEV), s.to(DEV), 0.125, window, sq)
    assert_parity(ref, o, f"decode attention B={B} ctx={ctx} W={window} start={start}")
    o2 = ops.attention_decode(q.to(DEV), k.to(DEV), v.to(DEV), s.to(DEV), 0.125, window, sq).clone()
    assert torch.equal(o.cpu(), o2.cpu()), "second call on the same workspace differs"


def test_attention_decode_ignores_keys_beyond_position(ops):
    """Cache rows at and beyond start_q+1 may hold anything (here NaN): they must not be read into the result."""
    g = torch.Generator().manual_seed(71)
    B, ctx, start = 2, 1024, 700
    q, k, v, s = _attn_inputs(g, B, ctx, sinks_dtype=torch.float32)
    ref = O.attention(q, k[:, :start + 1], v[:, :start + 1], s, 0.125, 0, start)
    k[:, start + 1:] = float("nan")
    v[:, start + 1:] = float("nan")
    o = ops.attention_decode(q.to(DEV), k.to(DEV), v.to(DEV), s.to(DEV), 0.125, 0,
                             torch.tensor([start], dtype=torch.int32, device=DEV))
    assert_parity(ref, o, "decode attention with NaN beyond the position")


def test_attention_decode_strided_cache_and_small_groups(ops):
    """k/v as a slice of a larger cache (non-contiguous batch stride) and a GQA group of 4."""
    g = torch.Generator().manual_seed(72)
    B, ctx, Hkv, G, start = 3, 320, 2, 4, 299
    q = randn(g, B, 1, Hkv, G, 64)
    big_k, big_v = randn(g, B, ctx + 64, Hkv, 64), randn(g, B, ctx + 64, Hkv, 64)
    s = randn(g, Hkv * G)
    ref = O.attention(q, big_k[:, 32:32 + ctx], big_v[:, 32:32 + ctx], s, 0.125, 128, start)
    kd, vd = big_k.to(DEV)[:, 32:32 + ctx], big_v.to(DEV)[:, 32:32 + ctx]
    assert not kd.is_contiguous()
    o = ops.attention_decode(q.to(DEV), kd, vd, s.to(DEV), 0.125, 128, torch.tensor([start], dtype=torch.int64, device=DEV))
    assert_parity(ref, o, "decode attention on a cache slice, G=4")


def test_attention_decode_config2_full_size(ops):
    """BASELINE config 2: B=32, 64 q heads / 8 kv heads, ctx 4096, fp32 sinks, both mask variants."""
    g = torch.Generator().manual_seed(1236)
    B, ctx = 32, 4096
    q, k, v, s = _attn_inputs(g, B, ctx, sinks_dtype=torch.float32)
    qd, kd, vd, sd = q.to(DEV), k.to(DEV), v.to(DEV), s.to(DEV)
    sq = torch.tensor([ctx - 1], dtype=torch.int64, device=DEV)
    for window in (128, 0):
        o = ops.attention_decode(qd, kd, vd, sd, 0.125, window, sq).clone()
        ref = O.attention(q, k, v, s, 0.125, window, ctx - 1)
        assert_parity(ref, o, f"config 2, window={window}")
    # size-independent property: the result does not depend on the order of the visible keys
    perm = torch.randperm(ctx, generator=g)
    o_full = ops.attention_decode(qd, kd, vd, sd, 0.125, 0, sq).clone()
    o_perm = ops.attention_decode(qd, kd[:, perm.to(DEV)].contiguous(), vd[:, perm.to(DEV)].contiguous(), sd, 0.125, 0, sq)
    assert_parity(o_full, o_perm, "permutation invariance")


# ------------------------------------------------------------------------------ SwiGLU
@pytest.mark.parametrize("rows,n", [(1, 8), (9, 48), (7, 2880), (64, 2880), (5, 3), (3, 20)])
def test_swiglu(ops, rows, n):
    g = torch.Generator().manual_seed(81 + rows + n)
    a = randn(g, rows, 2 * n, scale=2.0)
    ref = O.swiglu(a, 1.702, 7.0)
    o = ops.swiglu(a.to(DEV), 1.702, limit=7.0)
    assert_parity(ref, o, "swiglu")
    assert bf16_ulp_diff(ref, o).max() <= 1


def test_swiglu_golden_and_clamp_edges(ops):
    gd = golden("swiglu")
    a = bf16_from_bits(gd["a_bf16"])
    o = ops.swiglu(a.to(DEV), 1.702, limit=7.0)
    assert_parity(t(gd["out_f32"]), o, "swiglu vs swiglu_torch", max_rel=1e-2)
    assert_parity(t(gd["out_moe_f32"]), o, "swiglu vs moe.swiglu", max_rel=1e-2)
    o_nolimit = ops.swiglu(a.to(DEV), 1.702, limit=None)
    assert_parity(O.swiglu(a, 1.702, None), o_nolimit, "swiglu without clamp")


def test_swiglu_config4_rows(ops):
    """BASELINE config 4 row shape ([*, 5760] bf16 ~ N(0,2)); 4096 of the 65536 rows checked against the oracle."""
    g = torch.Generator().manual_seed(1238)
    a = randn(g, 4096, 5760, scale=2.0)
    o = ops.swiglu(a.to(DEV), 1.702, limit=7.0)
    assert_parity(O.swiglu(a, 1.702, 7.0), o, "swiglu config 4")


# ------------------------------------------------------------------------------- top-k
@pytest.mark.parametrize("tag", ["e128", "e32"])
def test_topk_golden_bit_exact(ops, tag):
    gd = golden("topk_router")
    logits = t(gd[f"{tag}__logits"])
    for softmax in (True, False):
        vals, idx, bm = ops.topk(logits.to(DEV), 4, apply_softmax=softmax)
        assert torch.equal(idx.cpu(), t(gd[f"{tag}__idx"]))
        ref_vals = t(gd[f"{tag}__vals" if softmax else f"{tag}__raw"])
        if softmax:
            torch.testing.assert_close(vals.cpu(), ref_vals, atol=1e-6, rtol=1e-5)
        else:
            assert torch.equal(vals.cpu().view(torch.int32), ref_vals.view(torch.int32))
        words = bm.data.cpu().numpy().view(np.uint32)
        assert np.array_equal(words, gd[f"{tag}__bitmatrix"][:, : words.shape[1]])
        assert int(bm.scratchpad.abs().sum()) == 0


@pytest.mark.parametrize("T,E,k", [(16384, 128, 4), (300, 32, 4), (17, 96, 2), (5, 1000, 8), (33, 4, 4)])
def test_topk_vs_oracle(ops, T, E, k):
    g = torch.Generator().manual_seed(91 + T + E)
    logits = torch.randn(T, E, generator=g)
    logits = O.bf16_round(logits)  # router logits are bf16 matmul outputs: plenty of exact ties
    vals_ref, idx_ref, words_ref = O.topk_softmax(logits, k)
    vals, idx, bm = ops.topk(logits.to(DEV), k)
    assert torch.equal(idx.cpu(), idx_ref)
    torch.testing.assert_close(vals.cpu(), vals_ref, atol=1e-6, rtol=1e-5)
    assert np.array_equal(bm.data.cpu().numpy().view(np.uint32).astype(np.int64), words_ref.numpy())


# ------------------------------------------------------------------------------- MXFP4
@pytest.mark.parametrize("rows,k", [(5, 96), (1, 32), (64, 2880), (3, 5760)])
def test_mxfp4_upcast_bit_exact(ops, rows, k):
    """E2M1 codes uniform over the 256 byte values, E8M0 scales in [2^-8, 2^0] (BASELINE config 4) and beyond."""
    g = torch.Generator().manual_seed(95 + rows + k)
    codes = torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8)
    scales = torch.randint(119, 128, (rows, k // 32), generator=g, dtype=torch.uint8)
    scales[0, 0] = 1      # 2^-126
    scales[-1, -1] = 200  # 2^73
    ref = torch.from_numpy(O.mxfp4_upcast(codes.numpy(), scales.numpy())).to(torch.bfloat16)
    got = ops.mxfp4_upcast(codes.to(DEV), scales.to(DEV))
    assert torch.equal(got.cpu().view(torch.int16), ref.view(torch.int16))


def test_mxfp4_golden(ops):
    gd = golden("mxfp4")
    got = ops.mxfp4_upcast(t(gd["codes"]).to(DEV), t(gd["scales"]).to(DEV))
    assert torch.equal(got.cpu().float(), t(gd["up2"]))  # E2M1 x 2^e is exact in bf16
    got = ops.mxfp4_upcast(t(gd["q"]).to(DEV), t(gd["s"]).to(DEV))
    assert torch.equal(got.cpu().float(), t(gd["up"]).to(torch.bfloat16).float())


def test_bounded_wait_times_out_and_context_survives():
    """A wait that nothing will ever satisfy gives up after its time limit, the kernel reports it through
    the device status word, and the same context keeps working (no trap, no hang)."""
    import time
    from tritonllm_b200 import _lib, ops
    assert _lib.device_status() == 0
    t0 = time.time()
    _lib.call("b2_selftest_wait_timeout", torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    waited = time.time() - t0
    status = _lib.device_status()            # reads and clears
    assert status & 0x1, status
    assert 1.0 < waited < 20.0, waited
    x = torch.randn(4, 2880, device="cuda").bfloat16()
    y = ops.rmsnorm_forward(x, torch.ones(2880, device="cuda"), 1e-5)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and _lib.device_status() == 0
