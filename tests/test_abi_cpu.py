"""CPU checks of the drop-in boundary: the shared library loads without a GPU and exports
every symbol the header declares, with the argument counts the ctypes binding uses."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tritonllm_b200.h")


def _declared():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    decls = {}
    for m in re.finditer(r"\b(?:int|size_t|const char\*)\s+(b2_\w+)\s*\(([^;]*?)\)\s*;", src, flags=re.S):
        args = m.group(2).strip()
        decls[m.group(1)] = 0 if args in ("", "void") else len(args.split(","))
    return decls


@pytest.fixture(scope="module")
def lib():
    from tritonllm_b200 import build, _lib
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


def test_header_declares_entry_points():
    d = _declared()
    for name in ("b2_rmsnorm", "b2_add_rmsnorm", "b2_rope_inplace", "b2_qkv_rope_kv_decode",
                 "b2_oproj_residual_decode", "b2_attn_decode", "b2_swiglu", "b2_topk_softmax"):
        assert name in d


def test_library_exports_every_declared_symbol(lib):
    from tritonllm_b200 import _lib
    decls = _declared()
    assert set(decls) == set(_lib.PROTOTYPES), set(decls) ^ set(_lib.PROTOTYPES)
    for name, nargs in decls.items():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert len(_lib.PROTOTYPES[name][1]) == nargs, f"{name}: ctypes binding has the wrong argument count"


def test_exported_symbols_are_only_the_abi(lib):
    from tritonllm_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True).stdout
    syms = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    assert {s for s in syms if s.startswith("b2_")} == set(_declared())


def test_host_side_argument_checks_need_no_gpu(lib):
    # rejected before any CUDA call
    assert lib.b2_version() >= 100
    assert lib.b2_rmsnorm(None, None, None, 4, 2880, 1e-5, None) == -1
    assert lib.b2_rmsnorm(None, None, None, 0, 2880, 1e-5, None) == 0
    assert lib.b2_rmsnorm(16, 16, 16, 4, 2881, 1e-5, None) == -3
    assert lib.b2_rmsnorm(8, 16, 16, 4, 2880, 1e-5, None) == -4
    assert lib.b2_swiglu(16, 4, 16, 8, 2, 8, 1.702, 7.0, None) == -2
    assert lib.b2_topk_softmax(16, 128, 4, 128, 9, 1, 16, 16, None, 0, 0, None, 0, None) == -3
    assert lib.b2_attn_decode(16, 16, 16, None, 0, 16, 2, 8, 8, 128, 64, 1, 1, 1, 0.125, 0, 16, 0, None, 0, None) == -3
    assert lib.b2_status_string(-5) == b"workspace missing or too small"
    assert lib.b2_set_tunable(b"no_such_knob", 1) == -3


def test_ops_refuse_cpu_tensors():
    import torch
    from tritonllm_b200 import ops
    x = torch.zeros(2, 2880, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.rmsnorm_forward(x, torch.ones(2880), 1e-5)


def test_patch_rebinds_reference_names():
    import types
    from tritonllm_b200 import ops
    fake = types.SimpleNamespace(rmsnorm_forward=1, rope_forward=2, attention_decode=3, moe=5, moe_decode=6, unrelated=4)
    done = ops.patch(fake)
    assert set(done) == {"rmsnorm_forward", "rope_forward", "attention_decode", "moe", "moe_decode"}
    assert fake.rmsnorm_forward is ops.rmsnorm_forward and fake.moe_decode is ops.moe_decode and fake.unrelated == 4


def test_shared_position_counter_needs_the_position_to_slide():
    """The reference's loop `for c in caches: c.slide_window()` reads each cache's own counter; with one counter
    shared by all layers only its owner may do that - the others must be told the position."""
    import torch
    from tritonllm_b200.generate import Cache
    first = Cache(1, 8, 2, 4, device=torch.device("cpu"))
    other = Cache(1, 8, 2, 4, device=torch.device("cpu"), offset=first.offset)
    assert first.owns_offset and not other.owns_offset
    with pytest.raises(ValueError, match="pass `current`"):
        other.slide_window()
    assert other.slide_window(current=3) == 3   # below capacity: nothing to move, no kernel needed


def test_pending_moe_detects_a_later_call_on_the_same_workspace():
    import torch
    from tritonllm_b200 import ops
    ws = torch.zeros(16, dtype=torch.uint8)
    p = ops.PendingMoe(ws, 1, 64, 64)
    ops._moe_generation[ws.data_ptr()] = ops._moe_generation.get(ws.data_ptr(), 0) + 1   # what a later expert call does
    with pytest.raises(RuntimeError, match="overwritten"):
        ops.moe_combine_add_rmsnorm(p, torch.zeros(1, 64, dtype=torch.bfloat16), torch.ones(64), 1e-5)


def test_integration_finds_no_reference_in_an_empty_place(tmp_path, monkeypatch):
    from tritonllm_b200 import integration
    monkeypatch.delenv("TRITONLLM_REFERENCE", raising=False)
    assert integration.reference_path(str(tmp_path)) in (None, integration.reference_path())
    (tmp_path / "tritonllm").mkdir()
    assert integration.reference_path(str(tmp_path)) == str(tmp_path)


def test_scratch_pool_returns_stable_buffers():
    import torch
    from tritonllm_b200 import scratch_pool
    a = scratch_pool.get((2, 3), torch.float32, torch.device("cpu"))
    b = scratch_pool.get((2, 3), torch.float32, torch.device("cpu"))
    assert a.data_ptr() == b.data_ptr()
    assert scratch_pool.stats()["num_buffers"] >= 1


def test_tuning_knobs_from_the_environment():
    """TRITONLLM_B200_TUNE is applied when the library is loaded; an unknown knob is an error, not a silent no-op."""
    import subprocess
    import sys
    code = "from tritonllm_b200 import _lib; _lib.load(); print('loaded')"
    env = dict(os.environ, TRITONLLM_B200_TUNE="moe_fp4_persist=2, unembed_tiles=1")
    ok = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT)
    assert ok.returncode == 0 and "loaded" in ok.stdout, ok.stderr
    env["TRITONLLM_B200_TUNE"] = "no_such_knob=1"
    bad = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT)
    assert bad.returncode != 0 and "TRITONLLM_B200_TUNE" in bad.stderr


def test_prompt_sized_moe_takes_over_earlier_with_a_resident_expansion():
    """The grouped-GEMM path has no per-call expansion to amortise once a weight pair keeps its bf16 copy."""
    from tritonllm_b200 import ops
    w1 = ops.ExpertWeightsFp4.__new__(ops.ExpertWeightsFp4)   # the packed weights live on the GPU; the rule reads n and k only
    w1.n = w1.k = 384                                          # multiples of 192
    assert not ops._prefill_moe_ok(ops.PREFILL_MOE_MIN_TOKENS - 1, w1, w1)
    assert ops._prefill_moe_ok(ops.PREFILL_MOE_MIN_TOKENS, w1, w1)
    w1._expanded = (object(), object(), w1)
    assert ops._prefill_moe_ok(ops.PREFILL_MOE_MIN_TOKENS_RESIDENT, w1, w1)
    assert not ops._prefill_moe_ok(ops.PREFILL_MOE_MIN_TOKENS_RESIDENT - 1, w1, w1)
    assert not ops._prefill_moe_ok(10 ** 6, object(), object())   # plain weights: the conversion path only
