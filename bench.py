"""Benchmark of the gpt-oss decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

Headline workload (N = 1 and per rank for N > 1): BASELINE config 2, decode attention for a batch of
32 sequences, 64 query / 8 KV heads, head_dim 64, bf16, KV cache 4096 per sequence, fp32
sinks, scale 1/8, one new token per sequence at position 4095.  One step = one decode token
through the attention of the 24 layers of gpt-oss-20b: the two mask variants alternate
(128-token window on even layers, full causal on odd layers), every layer on its own KV
cache (24 x 268 MB resident, so no launch finds its keys in the 126 MB L2).  The step is
captured once in a CUDA graph; a timed step is one replay.

Prints ONE JSON line.  `value` is algorithmic GB/s of the step with all inputs resident in
HBM; `roofline` is the full-causal launch timed in the same process (a graph holding only the
twelve full-causal launches); `roofline.kernels` times every kernel of the path alone at its
BASELINE size; `e2e` is the headline figure through tritonllm_b200.ops with q, K, V in pinned host
memory (copied to the device inside the timed region) and the result read back; `decode` is the
whole-model tokens/s half of the metric (config 5: real prompt ingestion, 256 generated tokens,
weak and strong sharding).  `--impl reference` times the reference's CPU attention on the host cores
instead (a bounded sample of the same workload).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

B, HQ, HKV, G, D, CTX, WINDOW = 32, 64, 8, 8, 64, 4096, 128
SCALE = 0.125
START_Q = CTX - 1
LAYERS = 24


def algorithmic_bytes(batch: int, visible: int) -> int:
    """K and V rows of the visible range once per KV head, plus q in and o out."""
    return batch * visible * HKV * D * 2 * 2 + 2 * batch * HQ * D * 2


BYTES_FULL = algorithmic_bytes(B, CTX)
BYTES_WINDOW = algorithmic_bytes(B, WINDOW)
BYTES_STEP = (LAYERS // 2) * (BYTES_FULL + BYTES_WINDOW)
# DRAM bytes one full-causal launch moved in an ncu capture of this kernel on this workload (269,243,648 read +
# 4,486,400 written; the second captured launch: 269,256,960 + 389,888).  A recorded constant, not measured in the
# run: the bench never runs under a profiler.  Re-recorded after the kernel gained its per-sequence / paged template.
NCU_TRAFFIC_FULL = 269243648 + 4486400
NCU_TRAFFIC_RECORDED = "2026-11-25, attn_decode_kernel<false> with 3 stages of 64 KiB, one CTA per SM"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Polls SM clock and clock-event reasons through NVML (read-only) from a thread while the
    timed region runs.  The timed loop is a handful of graph launches, so a 2 ms period is enough and keeps the
    thread off the launching thread's interpreter lock."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, cuda_index: int):
        self.samples, self.bits, self.max_mhz, self.err = [], 0, None, None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
                uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # NVML missing: report it, never fail the benchmark
            self.nv, self.err = None, repr(e)

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            except Exception as e:
                self.err = repr(e)
                return
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        sm = sorted(self.samples)
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
               "reasons": sorted(n for b, n in self.REASONS.items() if self.bits & b), "samples": len(sm)}
        if self.err:
            out["error"] = self.err
        return out


def make_inputs(seed: int):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, 1, HKV, G, D, generator=g).to(torch.bfloat16)
    sinks = torch.randn(HQ, generator=g)
    return g, q, sinks


def workload_config():
    return {"workload": "config 2: decode attention, 32 seq x 64q/8kv heads x 64, KV 4096/seq, bf16, "
                        "24 layers per step alternating window-128 / full-causal", "batch_per_gpu": B, "kv_ctx": CTX, "start_q": START_Q,
            "layers_per_step": LAYERS, "launch": "one CUDA graph replay per step",
            "l2": f"inputs larger than L2: {LAYERS} per-layer KV caches of 268 MB each, all read every step"}


# ------------------------------------------------------------------------------------------- CPU arms
def _host_threads() -> int:
    # torchrun exports OMP_NUM_THREADS=1 to its workers; a CPU arm is the only work on the host, so it takes
    # every core the process may run on
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    return torch.get_num_threads()


def _import_reference():
    """Makes the reference importable from the installed copy that travels with the repository (baseline/_ref, or
    $TRITONLLM_REFERENCE); nothing of this repository's package is involved."""
    import importlib
    import types
    root = os.environ.get("TRITONLLM_REFERENCE") or os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(root, "tritonllm")):
        raise ImportError("no installed copy of the reference")
    if root not in sys.path:
        sys.path.insert(0, root)
    try:
        importlib.import_module("termcolor")
    except ImportError:
        sys.modules["termcolor"] = types.ModuleType("termcolor")   # coloured prints only
    importlib.import_module("tritonllm")   # aliases its gpt_oss / triton_kernels sub-packages as top-level modules


def _reference_attention():
    """The reference's own CPU attention (`attention_ref`, pure torch) from an installed copy of the reference when
    one travels with the repository, else the restatement in oracle/.  Returns (callable, kind)."""
    try:
        _import_reference()
        from gpt_oss.triton.attention_ref import attention_ref

        def fn(q, k, v, sinks, scale, window, start_q):
            return attention_ref(q, k, v, sinks, scale, window, torch.tensor([start_q]))
        return fn, "reference"
    except Exception:
        import oracle as O
        return O.attention, "port"


def _cpu_attention_sample(sample_b: int):
    g, q, sinks = make_inputs(1236)
    k = torch.randn(sample_b, CTX, HKV, D, generator=g).to(torch.bfloat16)
    v = torch.randn(sample_b, CTX, HKV, D, generator=g).to(torch.bfloat16)
    return q[:sample_b], k, v, sinks


def run_reference(args, rank: int, world: int):
    """The reference's CPU attention on all host threads, a bounded sample of the workload per step."""
    if rank != 0:
        return
    cores = _host_threads()
    attn, kind = _reference_attention()
    sample_b = 4
    q, k, v, sinks = _cpu_attention_sample(sample_b)

    def step():
        attn(q, k, v, sinks, SCALE, WINDOW, START_Q)
        attn(q, k, v, sinks, SCALE, 0, START_Q)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    nbytes = algorithmic_bytes(sample_b, CTX) + algorithmic_bytes(sample_b, WINDOW)
    val = nbytes / dt / 1e9
    sample = (f"{sample_b} of {B} sequences per step, both mask variants, "
              + ("the reference's attention_ref (torch, fp32) on the CPU" if kind == "reference" else "oracle port of attention_ref, torch CPU fp32"))
    print(json.dumps({
        "impl": "reference", "metric": "fused-layer HBM GB/s", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline_leg():
    cores = _host_threads()
    attn, kind = _reference_attention()
    sample_b = 2
    q, k, v, sinks = _cpu_attention_sample(sample_b)
    attn(q, k, v, sinks, SCALE, 0, START_Q)  # warm-up
    reps, t0 = 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 200):
        attn(q, k, v, sinks, SCALE, WINDOW, START_Q)
        attn(q, k, v, sinks, SCALE, 0, START_Q)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    nbytes = algorithmic_bytes(sample_b, CTX) + algorithmic_bytes(sample_b, WINDOW)
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{sample_b} of {B} sequences, both mask variants, {reps} repetitions, torch CPU fp32"}


def interpreter_leg_child():
    """Child process (TRITON_INTERPRET=1, no GPU visible): the reference's `attention_decode` Triton kernels run by
    the Triton interpreter on the CPU, one sequence of the workload, both mask variants.  Prints one JSON object."""
    _import_reference()
    import gpt_oss.triton.model as M
    g = torch.Generator().manual_seed(1236)
    r = lambda *s: torch.randn(*s, generator=g).bfloat16()  # noqa: E731  (the decode kernels widen to fp32 at load)
    q, k, v, sinks = r(1, 1, HKV, G, D), r(1, CTX, HKV, D), r(1, CTX, HKV, D), r(HQ)
    sq = torch.tensor([START_Q])
    t0 = time.perf_counter()
    o_w = M.attention_decode(q, k, v, sinks, SCALE, WINDOW, sq).clone()   # the result is a pooled buffer
    o_f = M.attention_decode(q, k, v, sinks, SCALE, 0, sq)
    dt = time.perf_counter() - t0
    import oracle as O
    err = max(float((o_w.float() - O.attention(q, k, v, sinks, SCALE, WINDOW, START_Q).float()).abs().max()),
              float((o_f.float() - O.attention(q, k, v, sinks, SCALE, 0, START_Q).float()).abs().max()))
    nbytes = algorithmic_bytes(1, CTX) + algorithmic_bytes(1, WINDOW)
    print(json.dumps({"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "reference",
                      "seconds": dt, "max_abs_diff_vs_oracle": err,
                      "sample": f"1 of {B} sequences, both mask variants, once; the reference's attention_decode kernels under "
                                "TRITON_INTERPRET=1, one interpreter thread"}))


def interpreter_leg():
    """Runs interpreter_leg_child in a child process and returns its record (or why it is unavailable)."""
    env = dict(os.environ, TRITON_INTERPRET="1", CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "interpreter-child"], env=env,
                           capture_output=True, text=True, timeout=240)
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if r.returncode != 0 or not line:
            return {"unavailable": (r.stderr.strip().splitlines() or ["no output"])[-1][:300]}
        return json.loads(line[-1])
    except Exception as exc:
        return {"unavailable": repr(exc)[:300]}


# ------------------------------------------------------------------------------------------- kernel table
# (kernel label, case, overrides, bound): every kernel of the path alone at the size its BASELINE config gives it
KERNEL_CASES = [
    ("A1 rmsnorm (config 3: 8192 rows)", "rmsnorm", dict(rows=8192), "hbm"),
    ("A2 add + rmsnorm (8192 rows)", "add_rmsnorm", dict(rows=8192), "hbm"),
    ("A4 rope in place (8192 tokens)", "rope", dict(rows=8192), "hbm"),
    ("A3 QKV GEMM + bias + RoPE + split (M 8192)", "qkv_prefill", dict(rows=8192), "tensor"),
    ("A9 o_proj GEMM + bias + residual (M 8192)", "oproj_prefill", dict(rows=8192), "tensor"),
    ("A7 prefill attention, full causal (4 x 2048)", "attn_prefill", dict(batch=4, ctx=2048, window=0), "tensor"),
    ("A7 prefill attention, window 128 (4 x 2048)", "attn_prefill", dict(batch=4, ctx=2048, window=128), "tensor"),
    ("A5 decode QKV + RoPE + KV write (32 seq)", "qkv_decode", dict(batch=32), "hbm"),
    ("A5 decode QKV + RoPE + KV write (256 seq)", "qkv_decode", dict(batch=256), "hbm"),
    ("A9 decode o_proj + residual (32 seq)", "oproj_decode", dict(batch=32), "hbm"),
    ("A9 decode o_proj + residual (256 seq)", "oproj_decode", dict(batch=256), "hbm"),
    ("A8 decode attention, full causal (config 2)", "attn_decode", dict(batch=32, ctx=4096, window=0), "hbm"),
    ("A8 decode attention, window 128 (config 2)", "attn_decode", dict(batch=32, ctx=4096, window=128), "hbm"),
    ("A8 decode attention, full causal (256 seq x 2304)", "attn_decode", dict(batch=256, ctx=2304, window=0), "hbm"),
    ("A10 router GEMM (config 4: 16384 x 128)", "router", dict(rows=16384, experts=128), "hbm"),
    ("A11 top-4 + softmax + bitmatrix (16384 x 128)", "topk", dict(rows=16384, experts=128), "hbm"),
    ("A12 clamped SwiGLU (config 4: 65536 x 5760)", "swiglu", dict(rows=65536), "hbm"),
    ("A13 MXFP4 upcast (184320 x 2880)", "mxfp4", dict(rows=184320), "hbm"),
    ("A1+A10+A11 norm + router + top-4, one launch (256 rows, 32 experts)", "router_fused", dict(rows=256, experts=32), "hbm"),
    ("f1 MoE expert MLP, 32 tokens (routing + quantise + 2 GEMMs + combine)", "moe_decode", dict(batch=32), "hbm"),
    ("f1 MoE expert MLP, 256 tokens", "moe_decode", dict(batch=256), "hbm"),
    ("f1 MoE expert MLP, 2048 tokens (prompt-sized)", "moe_decode", dict(batch=2048), "tensor"),
    ("f1 MoE expert MLP, 8192 tokens (MXFP4 -> bf16 expansion + grouped GEMMs)", "moe_prefill", dict(batch=8192, copies=1), "tensor"),
    ("f2 unembedding + arg-max (32 seq)", "unembed", dict(batch=32), "hbm"),
    ("f2 unembedding + arg-max (256 seq)", "unembed", dict(batch=256), "hbm"),
]


def kernel_table(hbm_peak: float, tf_peak: float, peak_kind: str):
    """Times each kernel alone (CUDA-graph windows over input copies larger than L2, CUDA events) and returns the
    per-kernel roofline records."""
    import cases
    rows = []
    for label, case, kw, bound in KERNEL_CASES:
        try:
            a = cases.make_args(case, iters=8, **kw)
            r = cases.run_case(a)
            us = r["us_median"]
            rec = {"kernel": label, "case": case, "bound": bound, "us": us, "algorithmic_bytes": r["algorithmic_bytes"]}
            flops = r.get("algorithmic_flops")
            if case == "moe_decode":   # both GEMMs of every routed row: 2 flops x (2I x H + H x I) x 4 experts per token
                flops = 2.0 * kw["batch"] * 4 * (5760 * 2880 + 2880 * 2880)
            if flops:
                rec["algorithmic_flops"] = flops
            if bound == "tensor":
                ach = flops / us / 1e6
                rec.update(achieved=round(ach, 1), peak=tf_peak, unit="TFLOP/s", frac=round(ach / tf_peak, 3))
            else:
                ach = r["algorithmic_bytes"] / us / 1e3
                rec.update(achieved=round(ach, 1), peak=hbm_peak, unit="GB/s", frac=round(ach / hbm_peak, 3))
            rec["peak_kind"] = f"of {peak_kind}"
            rows.append(rec)
        except Exception as exc:  # reported in the line, never hidden
            rows.append({"kernel": label, "case": case, "error": repr(exc)[:200]})
        torch.cuda.empty_cache()
    return rows


# ------------------------------------------------------------------------------------------- whole-model decode
DECODE_TOTAL, DECODE_PROMPT, DECODE_NEW = 256, 2048, 256


def decode_bytes_per_step(batch: int, position: int) -> int:
    """Bytes one decode step must read at the gpt-oss-20b shape: dense weights and the unembedding once, the
    experts that receive a token (expected number of distinct experts among 4 x batch uniform picks), and the
    visible K/V rows (12 full-causal layers, 12 layers of 128 keys)."""
    H, I, E, L, V = 2880, 2880, 32, 24, 201088
    dense = 5120 * H * 2 + H * 4096 * 2 + H * E * 2
    touched = E * (1.0 - (1.0 - 4.0 / E) ** batch)
    experts = touched * ((2 * I) * (H // 2 + H // 32) + H * (I // 2 + I // 32))
    kv = (L // 2) * batch * ((position + 1) + min(128, position + 1)) * HKV * D * 2 * 2
    return int(L * (dense + experts) + V * H * 2 + kv)


def decode_run(model, dev, rank: int, batch: int, hbm_peak: float):
    """Config 5 on this rank's share: `batch` sequences with 2048-token seeded random prompts are really ingested
    into the KV store, then 256 tokens per sequence are generated greedily, one CUDA-graph replay per step."""
    from tritonllm_b200 import generate as GEN
    from tritonllm_b200 import ops as OPS
    # memory for speed on the prompt side: the bf16 expansion of every layer's experts (38 GB for this model) stays
    # resident instead of being redone by every prompt chunk of every layer
    OPS.set_expanded_expert_budget(EXPANDED_EXPERT_BYTES)
    tg = GEN.TokenGenerator(model, context=DECODE_PROMPT + DECODE_NEW, batch_size=batch)
    gen = torch.Generator().manual_seed(1239 + 7919 * rank + batch)
    prompts = torch.randint(0, model.config.vocab_size, (batch, DECODE_PROMPT), generator=gen).to(dev)
    for cache in tg.caches:
        cache.reset()
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    model.prefill(prompts[:, :-1], tg.caches)
    p1.record()
    tg.input_token.copy_(prompts[:, -1:])
    out = torch.empty((batch, DECODE_NEW), dtype=torch.int64, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(dev.index if dev.index is not None else 0)   # the step runs for seconds: clocks under load
    sampler.start()
    e0.record()
    for i in range(DECODE_NEW):
        ids = tg._step(True)
        tg.input_token.copy_(ids.view(-1, 1))
        out[:, i].copy_(ids)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    GEN.check_device_status("decode leg")
    assert int(tg.caches[0].offset.item()) == DECODE_PROMPT - 1 + DECODE_NEW
    assert int(out.min()) >= 0 and int(out.max()) < model.config.vocab_size
    ms = e0.elapsed_time(e1) / DECODE_NEW
    nbytes = decode_bytes_per_step(batch, DECODE_PROMPT - 1 + DECODE_NEW // 2)
    del tg
    torch.cuda.empty_cache()
    return {"ms_per_step": ms, "prefill_ms": p0.elapsed_time(p1), "bytes_per_step": nbytes,
            "gbs": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / hbm_peak, "sequences_per_gpu": batch, "clocks": clocks,
            "expanded_expert_bytes_allowed": EXPANDED_EXPERT_BYTES}


HEADSHARD_T = 8192
EXPANDED_EXPERT_BYTES = 48 << 30


def headshard_leg(dev, rank: int, world: int):
    """Optional long-context mode: the attention block of ONE 8192-token sequence with its heads split over the ranks
    (each rank: norm, its slice of QKV + RoPE, its heads' prefill attention; one NCCL all-gather of [T, 4096 / N]
    bf16 per rank; o_proj + residual replicated).  Full-causal layer.  Returns ms per block and the all-gather's part."""
    from tritonllm_b200 import headshard, ops
    gd = torch.Generator(device=dev).manual_seed(77)   # the same weights and input on every rank
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=gd, device=dev) * sc).to(torch.bfloat16)  # noqa: E731
    x = r(1, HEADSHARD_T, 2880)
    gain = torch.ones(2880, device=dev)
    wqkv, bqkv, wo, bo, sinks = r(5120, 2880, sc=0.02), r(5120, sc=0.02), r(2880, 4096, sc=0.02), r(2880, sc=0.02), r(64)
    cos, sin = ops.yarn_cos_sin(HEADSHARD_T, device=dev)
    shard = headshard.shard_attention_weights(wqkv, bqkv, sinks, rank, world)
    for _ in range(3):
        headshard.attention_block_headsharded(x, gain, shard, wo, bo, sin, cos, HEADSHARD_T, SCALE, 0)
    torch.cuda.synchronize()
    total, gather = [], []
    for _ in range(8):
        tm = {}
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        headshard.attention_block_headsharded(x, gain, shard, wo, bo, sin, cos, HEADSHARD_T, SCALE, 0, timings=tm)
        e1.record()
        torch.cuda.synchronize()
        total.append(e0.elapsed_time(e1))
        gather.append(tm["gather_start"].elapsed_time(tm["gather_end"]))
    total.sort(), gather.sort()
    return total[len(total) // 2], gather[len(gather) // 2]


def run_b200(args, rank: int, world: int, local_rank: int):
    from tritonllm_b200 import _lib, ops, sharding
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    _lib.load()
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    hbm_peak, tf_peak, peak_kind = measured_peaks()

    g, q_h, sinks_h = make_inputs(1236 + rank)
    # one K and one V cache per layer (134 MB each), drawn on the device, seeded per rank
    gd = torch.Generator(device=dev).manual_seed(4321 + rank)
    caches = []
    for _ in range(LAYERS):
        k = torch.randn(B, CTX, HKV, D, generator=gd, device=dev, dtype=torch.float32).to(torch.bfloat16)
        v = torch.randn(B, CTX, HKV, D, generator=gd, device=dev, dtype=torch.float32).to(torch.bfloat16)
        caches.append((k, v))
    q = q_h.to(dev)
    sinks = sinks_h.to(dev)
    start_q = torch.tensor([START_Q], dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream()

    def launches(which):
        for layer, (k, v) in enumerate(caches):
            window = WINDOW if layer % 2 == 0 else 0
            if which == "all" or (which == "full") == (window == 0):
                ops.attention_decode(q, k, v, sinks, SCALE, window, start_q)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    launches("all")   # eager once: workspaces and pooled outputs exist before capture
    torch.cuda.synchronize()
    graphs = {}
    for which in ("all", "full", "window"):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            launches(which)
        graphs[which] = gr
    stream = torch.cuda.current_stream()

    def timed(graph, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            graph.replay()
        e1.record(stream)
        return e0, e1

    # warm-up: the W requested steps, then more until ~0.25 s have passed so the clocks have settled
    for _ in range(args.warmup):
        graphs["all"].replay()
    warm_extra, t_w = 0, time.perf_counter()
    torch.cuda.synchronize()
    while time.perf_counter() - t_w < 0.25:
        graphs["all"].replay()
        warm_extra += 1
        if warm_extra % 16 == 0:
            torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    t0, t1 = timed(graphs["all"], args.steps)
    barrier()
    ms_total = t0.elapsed_time(t1)
    # the two mask variants alone, inside the sampled region too: twelve launches per replay
    f0, f1 = timed(graphs["full"], args.steps)
    w0, w1 = timed(graphs["window"], args.steps)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    full_ms = f0.elapsed_time(f1) / (args.steps * (LAYERS // 2))
    window_ms = w0.elapsed_time(w1) / (args.steps * (LAYERS // 2))
    assert _lib.device_status() == 0, "a kernel gave up a bounded wait"

    # ---- end to end through the public op with HOST buffers (pinned): every layer's q, K and V go
    # host -> device inside the timed region and every layer's result comes back.  One pinned
    # K/V pair is the source for all layers (the bytes moved are what count).
    k_pin = caches[1][0].cpu().pin_memory()
    v_pin = caches[1][1].cpu().pin_memory()
    q_pin = q_h.pin_memory()
    o_pin = torch.empty(LAYERS, B, 1, HQ * D, dtype=torch.bfloat16).pin_memory()
    qd = torch.empty_like(q)
    e2e_steps = 3

    def e2e_step():
        for layer, (k, v) in enumerate(caches):
            qd.copy_(q_pin, non_blocking=True)
            k.copy_(k_pin, non_blocking=True)
            v.copy_(v_pin, non_blocking=True)
            o = ops.attention_decode(qd, k, v, sinks, SCALE, WINDOW if layer % 2 == 0 else 0, start_q)
            o_pin[layer].copy_(o, non_blocking=True)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    h2d_strict = LAYERS * (q_pin.numel() + k_pin.numel() + v_pin.numel()) * 2

    # ---- same, with the KV caches resident on the device as the reference's Cache keeps them
    def e2e_resident_step():
        for layer, (k, v) in enumerate(caches):
            qd.copy_(q_pin, non_blocking=True)
            o = ops.attention_decode(qd, k, v, sinks, SCALE, WINDOW if layer % 2 == 0 else 0, start_q)
            o_pin[layer].copy_(o, non_blocking=True)

    e2e_resident_step()
    barrier()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record(stream)
    for _ in range(args.steps):
        e2e_resident_step()
    r1.record(stream)
    barrier()
    res_ms = r0.elapsed_time(r1) / args.steps

    del graphs, k_pin, v_pin
    caches.clear()
    torch.cuda.empty_cache()

    # ---- every kernel of the path alone at its BASELINE size (one GPU only: the scaling runs need no second copy)
    kernels = None
    if world == 1 and not args.no_kernels:
        kernels = kernel_table(hbm_peak, tf_peak, peak_kind)
        assert _lib.device_status() == 0, "a kernel gave up a bounded wait"

    # ---- whole-model decode tokens/s (the second half of the metric)
    decode, decode_err = {}, None
    if not args.no_decode:
        try:
            from tritonllm_b200 import generate as GEN
            cfg = GEN.ModelConfig.gpt_oss_20b()
            model = GEN.Transformer(cfg, GEN.ModelWeights.random(cfg, dev, seed=1239), max_context=4096)
            barrier()
            decode["weak"] = decode_run(model, dev, rank, DECODE_TOTAL, hbm_peak)
            barrier()
            if world > 1:
                lo, hi = sharding.shard_range(DECODE_TOTAL, world, rank)
                decode["strong"] = decode_run(model, dev, rank, hi - lo, hbm_peak)
                barrier()
            del model
        except Exception as exc:  # reported in the line, never hidden
            decode_err = repr(exc)[:300]
        barrier()

    hs_ms, hs_gather, hs_err = 1e30, 1e30, None
    if not args.no_headshard and 8 % world == 0:
        try:
            barrier()
            hs_ms, hs_gather = headshard_leg(dev, rank, world)
        except Exception as exc:
            hs_err = repr(exc)[:300]
        barrier()

    def dms(kind, key):
        v = decode.get(kind, {}).get(key)
        return v if v is not None else 1e30

    ms_total, e2e_ms, res_ms, full_ms, window_ms, dw, dwp, ds, dsp, hs_ms, hs_gather = sharding.max_over_ranks(
        [ms_total, e2e_ms, res_ms, full_ms, window_ms, dms("weak", "ms_per_step"), dms("weak", "prefill_ms"),
         dms("strong", "ms_per_step"), dms("strong", "prefill_ms"), hs_ms, hs_gather], device=dev)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_step = ms_total / args.steps
    achieved = BYTES_FULL / (full_ms * 1e-3) / 1e9
    ach_w = BYTES_WINDOW / (window_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": NCU_TRAFFIC_FULL, "traffic_measured_in_run": False,
                "traffic_source": "recorded constant: ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this "
                                  "kernel on this workload, captured " + NCU_TRAFFIC_RECORDED,
                "peak_kind": f"of {peak_kind}", "kernel": "attn_decode_kernel (full causal)",
                "algorithmic_bytes_per_launch": BYTES_FULL, "us_per_launch": full_ms * 1e3,
                "launches_timed": (LAYERS // 2) * args.steps,
                "how": "a CUDA graph holding only the twelve full-causal launches of the step, replayed `steps` times between CUDA events",
                "window_variant": {"algorithmic_bytes_per_launch": BYTES_WINDOW, "us_per_launch": window_ms * 1e3,
                                   "achieved": ach_w, "frac": ach_w / hbm_peak,
                                   "note": "8.9 MB per launch: bound by launch latency, not by HBM"}}
    if kernels is not None:
        roofline["kernels"] = kernels
    out = {
        "metric": "fused-layer HBM GB/s", "value": BYTES_STEP * world / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "warmup_extra": warm_extra, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(),
        "roofline": roofline,
        "e2e": {"value": BYTES_STEP * world / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": h2d_strict, "d2h_bytes_per_step": o_pin.numel() * 2, "ms_per_step": e2e_ms,
                "steps": e2e_steps, "note": "q, K and V of all 24 layers copied from pinned host memory every step"},
        "e2e_kv_resident": {"value": BYTES_STEP * world / (res_ms * 1e-3) / 1e9, "unit": "GB/s",
                            "h2d_bytes_per_step": LAYERS * q_pin.numel() * 2, "d2h_bytes_per_step": o_pin.numel() * 2,
                            "ms_per_step": res_ms,
                            "note": "KV cache lives on the device (as the reference's Cache does); q in, o out per step"},
        "gpu_launches": LAYERS * args.steps,
        "clocks": clocks,
    }
    if not args.no_decode:
        ok = decode_err is None and dw < 1e29
        dec = {"unit": "tokens/s", "error": decode_err, "gpu_launches_per_step": 24 * 7 + 4,
               "workload": "config 5: gpt-oss-20b shape, whole model (24 layers, 32 experts top-4 MXFP4, vocab 201088), random "
                           f"weights, {DECODE_PROMPT}-token seeded random prompts really ingested, {DECODE_NEW} tokens generated greedily, "
                           "one CUDA graph replay per step, CUDA events, max over ranks",
               "seven_x_refers_to": "weak (256 sequences per GPU): with a full weight replica per GPU a strong split of 256 "
                                    "sequences still streams every weight on every GPU each step"}
        if ok:
            per = decode["weak"]
            dec["weak"] = {"tokens_per_s": DECODE_TOTAL * world / (dw * 1e-3), "ms_per_step": dw, "sequences_per_gpu": DECODE_TOTAL,
                           "total_sequences": DECODE_TOTAL * world, "bytes_per_step_per_gpu": per["bytes_per_step"],
                           "gbs_per_gpu": per["bytes_per_step"] / dw / 1e6, "frac": per["bytes_per_step"] / dw / 1e6 / hbm_peak,
                           "prefill_tokens_per_s": DECODE_TOTAL * world * (DECODE_PROMPT - 1) / (dwp * 1e-3),
                           "clocks": per.get("clocks")}   # rank 0's SM clock during the 256 steps
            if world > 1 and ds < 1e29:
                per = decode["strong"]
                dec["strong"] = {"tokens_per_s": DECODE_TOTAL / (ds * 1e-3), "ms_per_step": ds,
                                 "sequences_per_gpu": per["sequences_per_gpu"], "total_sequences": DECODE_TOTAL,
                                 "bytes_per_step_per_gpu": per["bytes_per_step"], "gbs_per_gpu": per["bytes_per_step"] / ds / 1e6,
                                 "frac": per["bytes_per_step"] / ds / 1e6 / hbm_peak,
                                 "prefill_tokens_per_s": DECODE_TOTAL * (DECODE_PROMPT - 1) / (dsp * 1e-3)}
            else:
                dec["strong"] = dict(dec["weak"], note="one GPU: the strong and the weak split are the same run")
            dec["tokens_per_s"], dec["ms_per_step"] = dec["weak"]["tokens_per_s"], dw
        out["decode"] = dec
    if not args.no_headshard and 8 % world == 0:
        out["prefill_headshard"] = {
            "ms_per_block": hs_ms if hs_ms < 1e29 else None, "ms_all_gather": hs_gather if hs_gather < 1e29 else None,
            "all_gather_share": hs_gather / hs_ms if hs_ms < 1e29 else None, "tokens": HEADSHARD_T, "kv_heads_per_gpu": 8 // world,
            "all_gather_bytes_per_rank": HEADSHARD_T * (4096 // world) * 2 if world > 1 else 0, "error": hs_err,
            "workload": "one full-causal attention block (norm, QKV + RoPE, attention, o_proj + residual) of one "
                        f"{HEADSHARD_T}-token sequence, heads split over the GPUs, one NCCL all-gather before o_proj; max over ranks"}
    if world == 1:
        out["cpu_baseline"] = cpu_baseline_leg()
        if not args.no_interpreter:
            out["cpu_baseline_interpreter"] = interpreter_leg()
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "interpreter-child"])
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode tokens/s leg")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel roofline table")
    ap.add_argument("--no-headshard", action="store_true", help="skip the head-sharded long-context prefill leg")
    ap.add_argument("--no-interpreter", action="store_true", help="skip the Triton-interpreter CPU leg")
    args = ap.parse_args()
    if args.impl == "interpreter-child":
        return interpreter_leg_child()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else max(args.warmup, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_b200(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
