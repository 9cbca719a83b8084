"""Single-kernel cases on synthetic inputs, for timing and for profiler captures.

    python cases.py <case> [--iters N] [--batch B] [--ctx L] [--rows R] [--window W]

Each case builds several independent copies of its inputs on the device (together larger than
the 126 MB L2), warms up, captures one call per copy into a CUDA graph, then times `--iters`
replays of that window, bracketed by CUDA events on the launching stream, after a write of a 256 MB buffer and a
read of another (so no call finds its inputs in L2 and L2 holds no dirty lines whose write-back
would land in the window).  Prints one JSON line: algorithmic bytes per call, median
microseconds per call, GB/s and the fraction of the measured HBM copy bandwidth.

Cases: attn_decode, rmsnorm, add_rmsnorm, rope, swiglu, topk, qkv_decode, oproj_decode,
mxfp4, moe_decode, moe_prefill, router_fused, unembed, decode_stack, generate, qkv_prefill, oproj_prefill, router, attn_prefill (the last four are tensor-bound: TFLOP/s is reported too).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch

_ROOT = os.path.dirname(os.path.abspath(__file__))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from tritonllm_b200 import _lib, ops  # noqa: E402


def _peak_gbs():
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _tensor_fields(flops, us):
    """TFLOP/s and the fraction of the measured cuBLAS bf16 burst rate, for the tensor-bound cases."""
    if not flops:
        return {}
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    peak = 1590.0
    if os.path.exists(path):
        with open(path) as f:
            peak = float(json.load(f)["bf16_tflops"])
    tf = flops / us / 1e6
    return {"tflops": round(tf, 1), "frac_of_bf16_peak": round(tf / peak, 3), "peak_tflops": peak}


_REF = {}


def _ref():
    """The reference's own kernel entry points (a TritonLLM checkout under baseline/_ref or $TRITONLLM_REFERENCE),
    for the `--reference` legs: the same inputs through the reference's Triton kernels on the same GPU."""
    if not _REF:
        from tritonllm_b200 import integration
        M = integration.load_reference()
        import gpt_oss.triton.triton_kernels as TK
        from gpt_oss.triton import moe as RM
        from triton_kernels.routing import routing
        _REF.update(M=M, TK=TK, RM=RM, routing=routing)
    return _REF


def _bf(*shape, scale=1.0, dev="cuda"):
    return (torch.randn(*shape, device=dev, dtype=torch.float32) * scale).to(torch.bfloat16)


def build_case(name: str, a):
    """Returns (callable, algorithmic_bytes, description)."""
    dev = "cuda"
    if name == "attn_decode":
        B, L, W = a.batch, a.ctx, a.window
        q = _bf(B, 1, 8, 8, 64)
        k, v = _bf(B, L, 8, 64), _bf(B, L, 8, 64)
        sinks = torch.randn(64, device=dev)
        sq = torch.tensor([L - 1], dtype=torch.int64, device=dev)
        vis = min(W, L) if W else L
        nbytes = B * vis * 8 * 64 * 2 * 2 + 2 * B * 64 * 64 * 2
        if a.reference:
            fn_ref = _ref()["M"].attention_decode
            sinks_bf = sinks.bfloat16()
            return (lambda: fn_ref(q, k, v, sinks_bf, 0.125, W, sq)), nbytes, f"B={B} ctx={L} window={W} (reference kernel)"
        return (lambda: ops.attention_decode(q, k, v, sinks, 0.125, W, sq)), nbytes, f"B={B} ctx={L} window={W}"
    if name in ("rmsnorm", "add_rmsnorm"):
        R = a.rows
        x, d = _bf(R, 2880), _bf(R, 2880)
        gain = torch.ones(2880, device=dev)
        y, h = torch.empty_like(x), torch.empty_like(x)
        if name == "rmsnorm":
            fn = _ref()["TK"].rmsnorm_forward if a.reference else ops.rmsnorm_forward
            return (lambda: fn(x, gain, 1e-5, out=y)), R * 2880 * 4 + 2880 * 4, f"rows={R} dim=2880"
        return (lambda: ops.add_rmsnorm_forward(x, d, gain, 1e-5, h_out=h, y_out=y)), R * 2880 * 8 + 2880 * 4, \
            f"rows={R} dim=2880"
    if name == "rope":
        R = a.rows
        q, k = _bf(1, R, 64, 64), _bf(1, R, 8, 64)
        cos, sin = ops.yarn_cos_sin(max(R, 16), device=dev)
        off = torch.zeros(1, dtype=torch.int64, device=dev)
        fn = _ref()["TK"].rope_forward if a.reference else ops.rope_forward
        return (lambda: fn(q, k, sin, cos, cos.shape[0], off)), R * 72 * 64 * 4 + R * 256, f"tokens={R}"
    if name == "swiglu":
        R = a.rows
        x = _bf(R, 5760, scale=2.0)
        return (lambda: ops.swiglu(x, 1.702, limit=7.0)), R * 5760 * 2 + R * 2880 * 2, f"rows={R} cols=5760"
    if name == "topk":
        R, E = a.rows, a.experts
        x = torch.randn(R, E, device=dev)
        return (lambda: ops.topk(x, 4)), R * E * 4 + R * (16 + 8) + R * ((E + 31) // 32) * 4, f"rows={R} experts={E}"
    if name == "qkv_decode":
        B, ctx = a.batch, 64
        x = _bf(B, 1, 2880)
        w, b = _bf(5120, 2880, scale=0.02), _bf(5120, scale=0.02)
        ck, cv = _bf(B, ctx, 8, 64), _bf(B, ctx, 8, 64)
        cos, sin = ops.yarn_cos_sin(ctx, device=dev)
        off = torch.tensor([5], dtype=torch.int64, device=dev)
        nbytes = 5120 * 2880 * 2 + B * 2880 * 2 + B * 5120 * 2 + 5120 * 2
        fn = _ref()["TK"].qkv_rope_cache_decode_forward if a.reference else ops.qkv_rope_cache_decode_forward
        return (lambda: fn(x, w, b, sin, cos, ctx, ck, cv, off, 64, 8, 64)), nbytes, f"B={B} hidden=2880 out=5120"
    if name == "oproj_decode":
        B = a.batch
        x = _bf(B, 1, 4096)
        w, b = _bf(2880, 4096, scale=0.02), _bf(2880, scale=0.02)
        res = _bf(B, 1, 2880)
        nbytes = 2880 * 4096 * 2 + B * 4096 * 2 + 2 * B * 2880 * 2 + 2880 * 2
        fn = _ref()["TK"].out_residual_decode_forward if a.reference else ops.out_residual_decode_forward
        return (lambda: fn(x, w, b, res)), nbytes, f"B={B} in=4096 out=2880"
    if name == "qkv_prefill":
        R = a.rows
        x = _bf(1, R, 2880)
        w, b = _bf(5120, 2880, scale=0.02), _bf(5120, scale=0.02)
        cos, sin = ops.yarn_cos_sin(max(R, 16), device=dev)
        off = torch.zeros(1, dtype=torch.int64, device=dev)
        fn = lambda: ops.qkv_rope_prefill(x, w, b, sin, cos, cos.shape[0], off, 64, 8, 64)  # noqa: E731
        if a.library:  # cuBLAS on the same shape (GEMM + bias only: no RoPE, split or cache write)
            fn = lambda: torch.nn.functional.linear(x, w, b)  # noqa: E731
        return fn, R * 2880 * 2 + 5120 * 2880 * 2 + R * 5120 * 2, f"M={R} K=2880 N=5120", 2.0 * R * 2880 * 5120
    if name == "oproj_prefill":
        R = a.rows
        t_, res = _bf(R, 4096), _bf(R, 2880)
        w, b = _bf(2880, 4096, scale=0.02), _bf(2880, scale=0.02)
        out = torch.empty_like(res)
        fn = lambda: ops.out_residual_forward(t_, w, b, res, out=out)  # noqa: E731
        if a.library:  # cuBLAS GEMM + bias, then the separate residual add the reference does
            fn = lambda: torch.add(torch.nn.functional.linear(t_, w, b), res, out=out)  # noqa: E731
        return fn, R * 4096 * 2 + 2880 * 4096 * 2 + 2 * R * 2880 * 2, f"M={R} K=4096 N=2880", 2.0 * R * 4096 * 2880
    if name == "mxfp4":
        R = a.rows
        codes = torch.randint(0, 256, (R, 1440), device=dev, dtype=torch.uint8)
        scales = torch.randint(119, 128, (R, 90), device=dev, dtype=torch.uint8)
        return (lambda: ops.mxfp4_upcast(codes, scales)), R * (1440 + 90 + 5760), f"rows={R} K=2880"
    if name == "router_fused":
        R, E = a.rows, a.experts
        x = _bf(R, 1, 2880)
        gain = torch.ones(2880, device=dev)
        wg, bg = _bf(2880, E, scale=0.02), torch.zeros(E, device=dev)
        y = torch.empty_like(x)
        nbytes = R * 2880 * 4 + 2880 * E * 2 + R * 4 * 6
        return (lambda: ops.norm_router_topk(x, gain, 1e-5, wg, bg, 4, y_out=y)), nbytes, f"rows={R} hidden=2880 experts={E}"
    if name == "unembed":
        B, V, H = a.batch, 201088, 2880
        x, w = _bf(B, 1, H), _bf(V, H, scale=0.02)
        nbytes = V * H * 2 + B * H * 2 + B * 8
        return (lambda: ops.unembedding_decode_argmax_forward(x, w)), nbytes, f"B={B} vocab={V} hidden={H} (greedy arg-max)"
    if name == "moe_decode":
        T, E = a.batch, (a.moe_experts or 32)
        H = I = 2880
        x = _bf(T, H)
        logits = torch.randn(T, E, device=dev)
        vals, idx, _ = ops.topk(logits, 4)
        def w(n, k):
            return ops.ExpertWeights(torch.randint(0, 256, (E, n, k // 2), dtype=torch.uint8, device=dev),
                                     torch.randint(118, 124, (E, n, k // 32), dtype=torch.uint8, device=dev),
                                     torch.randn(E, n, device=dev) * 0.1)
        w1, w2 = w(2 * I, H), w(H, I)
        if not a.no_fp4:
            w1, w2 = ops.ExpertWeightsFp4(w1), ops.ExpertWeightsFp4(w2)
        touched = int(torch.unique(idx.long()).numel())
        per_expert = (2 * I) * (H // 2 + H // 32 + 4) + H * (I // 2 + I // 32 + 4)
        nbytes = touched * per_expert + T * H * 2 * 2
        if a.reference:  # moe_decode_experts: routing metadata + two matmul_ogs calls on weights its own quantiser laid out
            R = _ref()
            rw1, rw1s = R["RM"].quantize_mx4(_bf(E, H, 2 * I, scale=0.05))
            rw2, rw2s = R["RM"].quantize_mx4(_bf(E, I, H, scale=0.05))
            b1, b2 = torch.randn(E, 2 * I, device=dev) * 0.1, torch.randn(E, H, device=dev) * 0.1
            expert_fn = R["RM"].moe_decode_experts if T <= 256 else R["RM"].moe_experts

            def ref_moe():
                rdata, gi, si = R["routing"](logits, 4, simulated_ep=1)
                return expert_fn(x, rw1, rw1s, rw2, rw2s, b1, b2, rdata, gi, si)
            return ref_moe, nbytes, f"T={T} E={E} touched={touched} hidden=2880 (reference routing + matmul_ogs)"
        return (lambda: ops.moe_experts_decode(x, vals, idx, w1, w2)), nbytes, f"T={T} E={E} touched={touched} hidden=2880 fp4={not a.no_fp4}"
    if name == "moe_prefill":   # prompt-sized MoE: MXFP4 -> bf16 expansion of all experts + grouped tensor-core GEMMs
        T, E = a.batch, (a.moe_experts or 32)
        H = I = 2880
        x = _bf(T, H)
        vals, idx, _ = ops.topk(torch.randn(T, E, device=dev), 4)
        def w(n, k):
            return ops.ExpertWeightsFp4(ops.ExpertWeights(torch.randint(0, 256, (E, n, k // 2), dtype=torch.uint8, device=dev),
                                                          torch.randint(118, 124, (E, n, k // 32), dtype=torch.uint8, device=dev),
                                                          torch.randn(E, n, device=dev) * 0.1))
        w1, w2 = w(2 * I, H), w(H, I)
        per_expert = (2 * I) * (H // 2 + H // 32 + 4) + H * (I // 2 + I // 32 + 4)
        nbytes = E * per_expert + T * H * 2 * 2
        return (lambda: ops.moe_experts_prefill(x, vals, idx, w1, w2)), nbytes, f"T={T} E={E} hidden=2880 (grouped bf16 GEMM)", \
            2.0 * T * 4 * (2 * I * H + H * I)
    if name == "attn_prefill":
        B, T, W = a.batch, a.ctx, a.window
        q = _bf(B, T, 8, 8, 64)
        k, v = _bf(B, T, 8, 64), _bf(B, T, 8, 64)
        sinks = torch.randn(64, device=dev)
        sq = torch.zeros(1, dtype=torch.int64, device=dev)
        pairs = sum(min(i + 1, W) if W else i + 1 for i in range(T))  # visible (query, key) pairs per head
        fn = lambda: ops.attention(q, k, v, sinks, 0.125, W, sq)  # noqa: E731
        if a.reference:  # attention_tt_tma.attention on cc >= 9: includes its host-side transposes, as the model pays them
            fn_ref, sinks_bf = _ref()["M"].attention, sinks.bfloat16()
            fn = lambda: fn_ref(q, k, v, sinks_bf, 0.125, W, sq)  # noqa: E731
        nbytes = B * T * 64 * 64 * 2 * 2 + 2 * B * T * 8 * 64 * 2
        return fn, nbytes, f"B={B} T={T} window={W}", 4.0 * B * 64 * 64 * pairs
    if name == "router":
        R, E = a.rows, a.experts
        x, wg = _bf(R, 2880), _bf(2880, E, scale=0.02)
        bg = torch.zeros(E, device=dev)
        fn = lambda: ops.router_logits(x, wg, bg)  # noqa: E731
        return fn, R * 2880 * 2 + 2880 * E * 2 + R * E * 4, f"M={R} K=2880 E={E}", 2.0 * R * 2880 * E
    raise SystemExit(f"unknown case {name}")



def decode_stack(a):
    """One decode token through `--layers` gpt-oss-20b layers (attention block + MoE block each, every layer
    with its own random weights and KV cache), the final norm and the unembedding with its greedy arg-max,
    captured in one CUDA graph (the embedding lookup is the only part of a decode step that is left out).
    Prints step time, tokens/s and the bytes the step must read."""
    dev = "cuda"
    B, ctx, L, E = a.batch, a.ctx, a.layers, (a.moe_experts or 32)
    H, I = 2880, 2880
    cos, sin = ops.yarn_cos_sin(ctx, device=dev)
    offset = torch.tensor([ctx - 1], dtype=torch.int64, device=dev)

    def expert_w(n, k):
        w = ops.ExpertWeights(torch.randint(0, 256, (E, n, k // 2), dtype=torch.uint8, device=dev),
                              torch.randint(118, 124, (E, n, k // 32), dtype=torch.uint8, device=dev),
                              torch.randn(E, n, device=dev) * 0.05)
        return w if a.no_fp4 else ops.ExpertWeightsFp4(w)
    layers = []
    for _ in range(L):
        layers.append(dict(
            g1=torch.ones(H, device=dev), g2=torch.ones(H, device=dev),
            wqkv=_bf(5120, H, scale=0.02), bqkv=_bf(5120, scale=0.02), wo=_bf(H, 4096, scale=0.02), bo=_bf(H, scale=0.02),
            sinks=torch.randn(64, device=dev), ck=_bf(B, ctx, 8, 64), cv=_bf(B, ctx, 8, 64),
            wg=_bf(H, E, scale=0.02), bg=torch.randn(E, device=dev) * 0.02, w1=expert_w(2 * I, H), w2=expert_w(H, I)))
    g_final = torch.ones(H, device=dev)
    w_unembed = _bf(201088, H, scale=0.02)
    x0 = _bf(B, 1, H)
    x = torch.empty_like(x0)
    zero = torch.zeros_like(x0)
    hbuf, nbuf = torch.empty_like(x0), torch.empty_like(x0)

    def step():
        h, delta = x, zero
        for li, p in enumerate(layers):
            # residual add of the previous MoE output fused into this layer's first norm
            ops.add_rmsnorm_forward(h, delta, p["g1"], 1e-5, h_out=hbuf, y_out=nbuf)
            q = ops.qkv_rope_cache_decode_forward(nbuf, p["wqkv"], p["bqkv"], sin, cos, ctx, p["ck"], p["cv"], offset, 64, 8, 64)
            att = ops.attention_decode(q.view(B, 1, 8, 8, 64), p["ck"], p["cv"], p["sinks"], 0.125, 128 if li % 2 == 0 else 0, offset)
            h = ops.out_residual_decode_forward(att, p["wo"], p["bo"], hbuf)     # in place on hbuf
            n2 = ops.rmsnorm_forward(h, p["g2"], 1e-5, out=nbuf)
            logits = ops.router_logits(n2.view(B, H), p["wg"], p["bg"])
            vals, idx, _ = ops.topk(logits, 4)
            delta = ops.moe_experts_decode(n2.view(B, H), vals, idx, p["w1"], p["w2"]).view(B, 1, H)
        # last residual add fused into the final norm, then the unembedding with the greedy arg-max
        ops.add_rmsnorm_forward(h, delta, g_final, 1e-5, h_out=hbuf, y_out=nbuf)
        return ops.unembedding_decode_argmax_forward(nbuf, w_unembed)

    x.copy_(x0)
    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    x.copy_(x0)
    with torch.cuda.graph(graph):
        step()
    times = []
    for _ in range(a.iters):
        x.copy_(x0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    assert _lib.device_status() == 0
    ms = statistics.median(times)
    dense = 5120 * H * 2 + H * 4096 * 2 + H * E * 2
    # experts a layer touches: expected number of distinct experts among 4B uniform picks
    touched = E * (1.0 - (1.0 - 4.0 / E) ** B)
    experts = int(touched * ((2 * I) * (H // 2 + H // 32) + H * (I // 2 + I // 32)))
    kv = sum(B * (min(128, ctx) if li % 2 == 0 else ctx) * 8 * 64 * 2 * 2 for li in range(L))
    nbytes = L * (dense + experts) + kv + 201088 * H * 2
    peak, kind = _peak_gbs()
    print(json.dumps({"case": "decode_stack", "shape": f"B={B} ctx={ctx} layers={L} experts={E} fp4={not a.no_fp4}", "ms_per_step": round(ms, 3),
                      "tokens_per_s": round(B / ms * 1e3, 1), "weight_and_kv_bytes": nbytes,
                      "gbs": round(nbytes / ms / 1e6, 1), "frac_of_hbm_peak": round(nbytes / ms / 1e6 / peak, 3),
                      "peak_gbs": peak, "peak_kind": kind, "kernels_per_layer": 12, "iters": a.iters}))


def generate_case(a):
    """Whole-model greedy generation (BASELINE config 5 shape): `--batch` sequences with `--prompt` seeded random
    prompt tokens each are ingested into the KV store, then `--new-tokens` tokens per sequence are generated with
    the step replayed from one CUDA graph.  Random weights of the 20b architecture (`--layers`, `--moe-experts`)."""
    from tritonllm_b200 import generate as G
    dev = "cuda"
    B, P, N = a.batch, a.prompt, a.new_tokens
    cfg = G.ModelConfig(num_hidden_layers=a.layers, num_experts=a.moe_experts or 32)
    model = G.Transformer(cfg, G.ModelWeights.random(cfg, dev, seed=1239, fp4=not a.no_fp4), max_context=max(P + N, 4096))
    tg = G.TokenGenerator(model, context=P + N, batch_size=B, use_cuda_graph=not a.no_graph)
    gen = torch.Generator().manual_seed(1239)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=gen).to(dev)
    for cache in tg.caches:
        cache.reset()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    if a.skip_prefill:
        for cache in tg.caches:     # random K/V stand in for the ingested prompt
            cache.k.normal_()
            cache.v.normal_()
        tg.caches[0].offset.fill_(P - 1)
    elif P > 1:
        model.prefill(prompts[:, :-1], tg.caches)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    tg.input_token.copy_(prompts[:, -1:])
    out = torch.empty((B, N), dtype=torch.int64, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(N):
        ids = tg._step(True)
        tg.input_token.copy_(ids.view(-1, 1))
        out[:, i].copy_(ids)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    assert _lib.device_status() == 0
    assert int(tg.caches[0].offset.item()) == P - 1 + N and int(out.min()) >= 0 and int(out.max()) < cfg.vocab_size
    print(json.dumps({"case": "generate", "shape": f"B={B} prompt={P} new={N} layers={a.layers} experts={cfg.num_experts} fp4={not a.no_fp4}",
                      "prefill_s": round(prefill_s, 3), "prefill_tokens_per_s": round(B * (P - 1) / max(prefill_s, 1e-9), 1),
                      "decode_ms_per_step": round(ms / N, 3), "decode_tokens_per_s": round(B * N / ms * 1e3, 1),
                      "distinct_tokens": int(out.unique().numel())}))


def _parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--copies", type=int, default=0, help="input copies = calls per timed window (0 = auto)")
    ap.add_argument("--no-graph", action="store_true", help="launch from Python instead of replaying a CUDA graph")
    ap.add_argument("--no-fp4", action="store_true",
                    help="moe_decode / decode_stack: convert the expert weights to bf16 in the kernel instead of the FP4 MMA path")
    ap.add_argument("--layers", type=int, default=24, help="decode_stack: number of layers")
    ap.add_argument("--moe-experts", type=int, default=0, help="moe_decode: number of experts (default 32)")
    ap.add_argument("--prompt", type=int, default=2048, help="generate: prompt tokens per sequence")
    ap.add_argument("--new-tokens", type=int, default=256, help="generate: tokens generated per sequence")
    ap.add_argument("--skip-prefill", action="store_true",
                    help="generate: fill the KV store with random values instead of ingesting the prompt")
    ap.add_argument("--library", action="store_true",
                    help="GEMM cases: time torch's cuBLAS path on the same shape instead (the library comparator)")
    ap.add_argument("--reference", action="store_true",
                    help="time the reference's own Triton kernel for the case instead (attn_decode, attn_prefill, moe_decode, "
                         "rmsnorm, rope, qkv_decode, oproj_decode); needs a TritonLLM checkout and triton")
    ap.add_argument("--tune", action="append", default=[], help="name=value tuning knob (b2_set_tunable)")
    ap.add_argument("--expanded-gb", type=float, default=0.0,
                    help="generate / moe_prefill: device memory (GB) that may hold resident bf16 copies of the expert weights for the prompt path")
    ap.add_argument("--phase-trace", action="store_true",
                    help="attn_prefill: also print the softmax warps' per-phase clock counters (diagnostic build of the library)")
    return ap


def make_args(case: str, **kw):
    """The argument namespace of one case with the command line's defaults, for callers that time cases in-process."""
    a = _parser().parse_args([case])
    for k, v in kw.items():
        assert hasattr(a, k), k
        setattr(a, k, v)
    return a


def run_case(a) -> dict:
    """Times one single-kernel case as the module docstring describes and returns the result record."""
    built = build_case(a.case, a)
    fn, nbytes, desc = built[:3]
    flops = built[3] if len(built) > 3 else None
    # several independent copies of the inputs, so a window of back-to-back calls never re-reads
    # what an earlier call of the window left in L2
    n_copies = a.copies if a.copies > 0 else max(2, min(16, -(-(300 << 20) // max(nbytes, 1))))
    fns = [fn] + [build_case(a.case, a)[0] for _ in range(n_copies - 1)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    flush_rd = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream()
    for f in fns:
        f()
    torch.cuda.synchronize()
    graph = None
    if not a.no_graph:
        # replaying a captured window takes the host (Python, ctypes, launch set-up) out of the measurement
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph):
                for f in fns:
                    f()
        except Exception as exc:   # only the reference legs can get here (a host synchronisation inside the op)
            if not a.reference:
                raise
            print(f"# capture failed ({exc!r:.200}); timing eager launches", file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
        stream = torch.cuda.current_stream()
    times = []
    for _ in range(a.iters):
        # evict the inputs from L2, then leave L2 full of clean lines (no write-back lands in the window);
        # the two flush kernels also keep the GPU busy while the host queues the whole window, so the
        # window measures kernels back to back, not launch latency
        flush.fill_(1)
        flush_rd.max()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if graph is not None:
            graph.replay()
        else:
            for f in fns:
                f()
        e1.record(stream)
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / n_copies)
    assert _lib.device_status() == 0
    us = statistics.median(times)
    peak, kind = _peak_gbs()
    gbs = nbytes / us / 1e3
    return {"case": a.case, "shape": desc, "algorithmic_bytes": nbytes, "us_median": round(us, 2),
            "us_min": round(min(times), 2), "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peak, 3),
            "peak_gbs": peak, "peak_kind": kind, "iters": a.iters, "calls_per_window": n_copies, "graph": graph is not None,
            "tune": a.tune, "library": bool(a.library), "reference_kernel": bool(a.reference),
            "algorithmic_flops": flops, **_tensor_fields(flops, us)}


def attn_prefill_phases(a) -> dict:
    """Per-phase SM-clock counters of the prefill attention kernel's softmax warps, per 64-key block, averaged over the
    CTAs.  They exist only in a diagnostic build of the library
    (`TRITONLLM_B200_NVCC_FLAGS=-DAP_PHASE_TRACE=1 python -m tritonllm_b200.build`); a plain build leaves them at zero."""
    import ctypes as C
    fn = build_case("attn_prefill", a)[0]
    fn()
    torch.cuda.synchronize()
    rows = 4 * 1024   # four softmax warps per CTA, 8 slots per row
    buf = torch.zeros(rows * 8, dtype=torch.int64, device="cuda")
    _lib.call("b2_set_trace_buffer", C.c_void_p(buf.data_ptr()), C.c_size_t(buf.numel() * 8))
    try:
        fn()
        torch.cuda.synchronize()
    finally:
        _lib.call("b2_set_trace_buffer", C.c_void_p(0), C.c_size_t(0))
    t = buf.view(rows, 8).cpu()
    t = t[(t[:, 3] & 0xffffffff) > 0]
    if len(t) == 0 or int(t[:, 4:8].sum()) == 0:
        return {"phases": None, "note": "the library was not built with -DAP_PHASE_TRACE=1"}
    blocks = (t[:, 3] & 0xffffffff).double()
    per = lambda col: round(float((col.double() / blocks).mean()), 1)  # noqa: E731
    total, drain = t[:, 2] & 0xffffffff, t[:, 2] >> 32
    named = {"wait_for_S": t[:, 4], "tensor_memory_load_issue": t[:, 5], "load_latency_and_row_max": t[:, 6],
             "rescale_vote_and_P_buffer_wait": t[:, 3] >> 32, "exponentials_pack_stores": t[:, 7], "store_drain_and_arrive": drain}
    out = {k: per(v) for k, v in named.items()}
    out["total_per_block"] = per(total)
    out["bookkeeping_and_unit_ends"] = round(out["total_per_block"] - sum(v for k, v in out.items() if k != "total_per_block"), 1)
    return {"phases": out, "warps": len(t), "blocks_per_cta": round(float(blocks.mean()), 1), "unit": "SM clocks per 64-key block"}


def main():
    a = _parser().parse_args()
    assert torch.cuda.is_available(), "cases need a CUDA device"
    lib = _lib.load()
    for kv in a.tune:
        name, val = kv.split("=")
        _lib.check("b2_set_tunable", lib.b2_set_tunable(name.encode(), int(val)))
    ops.set_expanded_expert_budget(int(a.expanded_gb * (1 << 30)))
    if a.case == "generate":
        return generate_case(a)
    if a.case == "decode_stack":
        decode_stack(a)
        return
    rec = run_case(a)
    if a.case == "attn_prefill" and a.phase_trace:
        rec.update(attn_prefill_phases(a))
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
