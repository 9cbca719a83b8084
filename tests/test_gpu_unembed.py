"""GPU parity of the decode unembedding (logits and fused greedy arg-max) through the C ABI."""
import pytest
import torch

from _util import assert_parity, golden, t

import oracle as O

pytestmark = pytest.mark.gpu


def _ops():
    from tritonllm_b200 import ops
    return ops


def _check_ids(ids_gpu, acc_ref):
    """The chosen row must carry the maximum of the fp32 sums up to summation-order noise; equal rows -> smaller index."""
    ids_ref = acc_ref.argmax(dim=-1)
    mx = acc_ref.max(dim=-1).values
    got = acc_ref.gather(1, ids_gpu.cpu()[:, None])[:, 0]
    assert torch.all(got >= mx - 1e-4 * mx.abs().clamp_min(1.0)), (ids_gpu.cpu(), ids_ref)
    return ids_ref


def test_unembed_golden():
    ops = _ops()
    g = golden("unembedding")
    x, w = t(g["x"]).bfloat16(), t(g["w"]).bfloat16()      # bf16-representable fp32 values
    logits = ops.unembedding_decode_forward(x.cuda(), w.cuda())
    ids = ops.unembedding_decode_argmax_forward(x.cuda(), w.cuda())
    torch.cuda.synchronize()
    assert logits.shape == (3, 1, 300)
    assert_parity(t(g["logits"]), logits[:, 0].float().cpu(), "unembedding logits vs reference kernel")
    assert torch.equal(ids.cpu(), t(g["ids"]).long())       # includes the exact tie (rows 17 and 201): 17 wins


@pytest.mark.parametrize("B,V,H", [(1, 201088, 2880), (32, 201088, 2880), (256, 50000, 2880), (5, 1000, 192), (300, 4096, 128), (200, 1100, 192)])
def test_unembed_vs_oracle(B, V, H):
    ops = _ops()
    gen = torch.Generator().manual_seed(5000 + B)
    x = torch.randn(B, 1, H, generator=gen).bfloat16()
    w = (torch.randn(V, H, generator=gen) * 0.02).bfloat16()
    xd, wd = x.cuda(), w.cuda()
    logits = ops.unembedding_decode_forward(xd, wd)[:, 0].cpu()
    ids = ops.unembedding_decode_argmax_forward(xd, wd)
    torch.cuda.synchronize()
    acc = x[:, 0].float() @ w.float().T
    assert_parity(acc.bfloat16(), logits, f"unembedding logits B={B} V={V}")
    _check_ids(ids, acc)
    assert ids.dtype == torch.int64 and ids.shape == (B,)


def test_unembed_empty_batch():
    ops = _ops()
    w = torch.zeros(256, 128, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros(0, 1, 128, dtype=torch.bfloat16, device="cuda")
    assert ops.unembedding_decode_forward(x, w).shape == (0, 1, 256)
    assert ops.unembedding_decode_argmax_forward(x, w).shape == (0,)
