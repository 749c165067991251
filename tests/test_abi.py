"""CPU tests of the C-ABI library: it loads, exports every symbol the header declares, and rejects
bad arguments on the host before touching the GPU."""
import ctypes
import os
import re

import pytest

from custom_helper_op_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            names.update(re.findall(r"CHOP_API[^;(]*?\b(chop_\w+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    syms = declared_symbols()
    assert "chop_cost_volume_fwd" in syms and "chop_cost_volume_bwd" in syms
    for s in syms:
        assert hasattr(L, s), s
    assert L.chop_version() >= 100


def test_desc_layout_matches_header():
    # 6 x int32 followed by 10 x int64
    assert ctypes.sizeof(_lib.CvDesc) == 6 * 4 + 10 * 8


def _desc(**kw):
    d = _lib.CvDesc()
    d.kind, d.dtype, d.reduce, d.half_centor, d.groups = 1, 0, 0, 1, 1
    d.B, d.H, d.W, d.C, d.D, d.N, d.Hs, d.Ws = 1, 8, 8, 4, 4, 2, 8, 8
    for k, v in kw.items():
        setattr(d, k, v)
    return d


def _fwd(d, ptr=ctypes.c_void_p(256)):
    return _lib.lib().chop_cost_volume_fwd(ctypes.byref(d), ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, None)


def test_invalid_arguments_are_rejected_on_the_host():
    assert _fwd(_desc(kind=9)) == -3
    assert _fwd(_desc(dtype=7)) == -3
    assert _fwd(_desc(reduce=5)) == -3
    assert _fwd(_desc(B=0)) == -2
    assert _fwd(_desc(Hs=9)) == -2                      # source and reference sizes must agree
    assert _fwd(_desc(kind=2, groups=3)) == -3          # groups must divide C
    assert _fwd(_desc(d_begin=3, d_end=9)) == -7
    assert _fwd(_desc(), ptr=None) == -1
    assert _fwd(_desc(C=33 * 4 + 4)) == -4              # more channels than 32 lanes x 4 can hold
    assert _fwd(_desc(), ptr=ctypes.c_void_p(258)) == -5
    assert _fwd(_desc(d_begin=2, d_end=2)) == 0         # empty depth range: nothing to do
    assert b"NULL" in _lib.lib().chop_status_string(-1)
    assert _lib.lib().chop_set_tuning(b"nope", 1) == -3


def test_unknown_flag_bits_and_unused_descriptor_fields_are_rejected():
    assert _fwd(_desc(flags=4)) == -3                   # a bit this build does not know
    assert _fwd(_desc(flags=0x80000000)) == -3
    L = _lib.lib()
    ptr = ctypes.c_void_p(256)

    def fa(**kw):
        d = _desc(**dict(dict(kind=0, groups=1), **kw))
        return L.chop_feature_aggregate_fwd(ctypes.byref(d), ptr, ptr, ptr, ptr, ptr, ptr, ptr, None)

    assert fa(kind=1) == -3 and fa(reduce=1) == -3 and fa(groups=8) == -3 and fa(flags=1) == -3
    assert fa(d_begin=2, d_end=2) == 0                  # a valid descriptor with an empty depth range: nothing to do


def test_tuning_knobs_are_inert_without_the_opt_in():
    """chop_set_tuning is process-wide, hence refused unless CHOP_ENABLE_TUNING=1 was in the environment when the
    library first looked (the test session sets it in conftest.py; a fresh process without it must be refused)."""
    import subprocess
    import sys
    assert _lib.lib().chop_set_tuning(b"tuned", 1) == 0
    code = ("import ctypes; L = ctypes.CDLL(%r); L.chop_set_tuning.argtypes = [ctypes.c_char_p, ctypes.c_int]; "
            "print(L.chop_set_tuning(b'tuned', 0))" % _lib.LIB_PATH)
    env = {k: v for k, v in os.environ.items() if k != "CHOP_ENABLE_TUNING"}
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
    assert out.stdout.strip() == "-4", out.stdout + out.stderr


def test_wrappers_refuse_to_run_after_a_reported_give_up(monkeypatch):
    """Host logic of the non-synchronising check: the bf16 manifold-convolution wrappers read chop_umma_watch()
    before launching and raise when it reports abandoned waits; other dtypes do not look.  (A fake library stands
    in: without a device the real entry point answers -1, 'no mirror', which the wrappers ignore.)"""
    import contextlib
    import types
    import torch
    from custom_helper_op_b200.python.ops import custom_helper_ops as ops
    assert _lib.lib().chop_umma_watch() in (-1, 0)
    count = {"n": 0}
    fake = types.SimpleNamespace(chop_umma_watch=lambda: count["n"])
    monkeypatch.setattr(ops._lib, "lib", lambda: fake)
    monkeypatch.setattr(torch.cuda, "device", lambda dev: contextlib.nullcontext())
    bf16 = types.SimpleNamespace(dtype=torch.bfloat16, device=torch.device("cuda", 0))
    f32 = types.SimpleNamespace(dtype=torch.float32, device=torch.device("cuda", 0))
    ops._umma_watch(bf16)
    for n in (-1, 0):
        count["n"] = n
        ops._umma_watch(bf16)
    count["n"] = 2
    ops._umma_watch(f32)
    with pytest.raises(RuntimeError, match="2 tensor-core convolution wait"):
        ops._umma_watch(bf16)
