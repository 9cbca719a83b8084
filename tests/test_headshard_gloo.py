"""Host-side logic of the optional head-sharded prefill mode, run as two gloo ranks on the CPU: the weight slices
each rank takes, the all-gather and the reassembly of the per-rank attention outputs.  Each rank does its heads'
work with the oracle; the gathered block must equal the oracle's unsharded attention block."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from tritonllm_b200 import headshard


def _params(g, hid=256):
    bf = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc).to(torch.bfloat16)  # noqa: E731
    return dict(norm_gain=torch.randn(hid, generator=g) * 0.05 + 1, w_qkv=bf(5120, hid, sc=0.05), b_qkv=bf(5120, sc=0.02),
                w_o=bf(hid, 4096, sc=0.02), b_o=bf(hid, sc=0.02), sinks=bf(64))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_weight_slices_cover_every_head_once(world):
    g = torch.Generator().manual_seed(1)
    p = _params(g, hid=64)
    seen_q, seen_k, seen_v = [], [], []
    for r in range(world):
        s = headshard.shard_attention_weights(p["w_qkv"], p["b_qkv"], p["sinks"], r, world)
        assert s.n_kv_heads == 8 // world and s.n_q_heads == 64 // world
        nq, nk = s.n_q_heads * 64, s.n_kv_heads * 64
        assert s.wqkv.shape == (nq + 2 * nk, 64) and s.bqkv.shape == (nq + 2 * nk,) and s.sinks.shape == (s.n_q_heads,)
        seen_q.append(s.wqkv[:nq]), seen_k.append(s.wqkv[nq:nq + nk]), seen_v.append(s.wqkv[nq + nk:])
    assert torch.equal(torch.cat(seen_q + seen_k + seen_v), p["w_qkv"])
    with pytest.raises(ValueError):
        headshard.shard_attention_weights(p["w_qkv"], p["b_qkv"], p["sinks"], 0, 3)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(9)   # every rank draws the same block
        B, T, hid, window = 1, 40, 256, 16
        p = _params(g, hid)
        x = torch.randn(B, T, hid, generator=g).bfloat16()
        cos, sin = O.yarn_cos_sin(64)
        s = headshard.shard_attention_weights(p["w_qkv"], p["b_qkv"], p["sinks"], rank, world)
        n = O.rmsnorm(x, p["norm_gain"], 1e-5)
        q, k, v = O.qkv_rope_prefill(n, s.wqkv, s.bqkv, cos, sin, 0, n_q=s.n_q_heads, n_kv=s.n_kv_heads)
        o_local = O.attention(q.reshape(B, T, s.n_kv_heads, 8, 64), k, v, s.sinks, 0.125, window, 0)
        o = headshard.gather_heads(o_local.reshape(B * T, -1))      # the one collective of the mode
        t = O.out_residual_two_step(o, p["w_o"], p["b_o"], x.reshape(B * T, hid)).reshape(B, T, hid)
        ref, _, _, _, a_ref = O.attention_block(x, p, window, cos, sin, 0)
        ret[rank] = (bool(torch.equal(o.reshape(B, T, -1), a_ref)), bool(torch.equal(t, ref)))
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharding_matches_unsharded():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = 30500 + os.getpid() % 1000
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
        assert ret[0] == (True, True) and ret[1] == (True, True)
