"""CPU-side checks: the C ABI library loads and exports every declared symbol,
host-side validation raises before any device work, fake (meta) kernels give the
right shapes, and the data-parallel gradient exchange works over gloo."""

import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import ctypes
    from residual_stream_burden_b200 import _lib
    header = open(os.path.join(ROOT, "include", "sihc_b200.h")).read()
    body = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(sihc_[a-z0-9_]+)\s*\(", body))
    assert declared, "no declarations parsed"
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(raw, name), f"{name} declared in include/sihc_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert _lib.lib.sihc_version() >= 1
    assert b"null" in _lib.lib.sihc_status_string(-1)


def test_host_validation_needs_no_device():
    import residual_stream_burden_b200 as R
    x = torch.randn(1, 8, 8, 16)
    a = torch.randn(8, 16, 4)
    with pytest.raises(ValueError, match="contiguous|packed"):
        R.sublayer_read(x.transpose(1, 2), a)
    with pytest.raises(ValueError, match="CUDA"):
        R.sublayer_read(x, a)                     # CPU tensors: no fallback
    with pytest.raises(ValueError):
        R.sublayer_read(x, torch.randn(8, 16, 3))
    with pytest.raises(ValueError):
        R.blockwise_triangular(torch.randn(1, 4, 16), [torch.randn(1, 4, 16)] * 12, torch.randn(12, 16))
    with pytest.raises(ValueError):
        R.sihc_read(x, a)                         # single-event API wants [C, S]


def test_workspace_queries_and_argument_errors_without_gpu():
    from residual_stream_burden_b200 import _lib
    lib = _lib.lib
    assert lib.sihc_wgrad_workspace_bytes(1, 4, 16, 3, 3, 768, 1) == 0       # bad cell
    assert lib.sihc_tri_workspace_bytes(0, 1024, 768, 1) == 0                # bad prefix
    assert lib.sihc_read_fwd(None, None, None, 1, 1, 2, 2, 2, 8, 0, 0, None) == -1
    assert lib.sihc_read_fwd(None, None, None, 1, 1, 2, 2, 2, 8, 0, 1, None) == -2  # bf16 weights with fp32 acts
    assert lib.sihc_tune(b"no_such_knob", 1) == -1
    # a slot's offset inside its cell row block is kept in 32 bits by the kernels: geometries whose
    # (kh-1) carrier rows + one cell row reach 2^32 elements are refused, the largest one below is not
    assert lib.sihc_read_fwd(None, None, None, 1, 1, 128, 4, 4, 1 << 22, 1, 1, None) == -5   # (3*128*4+4)*2^22 >= 2^32
    assert lib.sihc_read_fwd(None, None, None, 1, 1, 16, 2, 2, 1 << 24, 1, 1, None) == -1   # fits: next check (null)
    assert lib.sihc_wgrad_workspace_bytes(1, 1, 128, 4, 4, 1 << 22, 1) == 0


def test_fake_kernels_trace_on_meta_device():
    import residual_stream_burden_b200 as R
    x = torch.empty(2, 32, 32, 64, device="meta", dtype=torch.bfloat16)
    a = torch.empty(24, 64, 4, device="meta", dtype=torch.bfloat16)
    outs = R.sublayer_read(x, a)
    assert len(outs) == 24 and outs[0].shape == (2, 256, 64) and outs[0].dtype == torch.bfloat16
    y = R.sublayer_write(x, outs, a)
    assert y.shape == x.shape
    g = torch.empty(3, 64, device="meta", dtype=torch.float32)
    t = R.sublayer_triangular(outs[0], outs[:3], g)
    assert t.shape == outs[0].shape


def test_product_code_never_reaches_the_oracle_or_scratch_scripts():
    """The package must compute on the CUDA library alone: the CPU oracle is a checker for
    the tests, the smoke run and the benchmark's CPU legs, never a fallback."""
    pkg = os.path.join(ROOT, "residual_stream_burden_b200")
    pattern = re.compile(r"^\s*(from|import)\s+(oracle|_work)\b|[\"'](oracle|_work)[/\"']", re.M)
    for folder, _, files in os.walk(pkg):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(folder, name)).read()
                assert not pattern.search(text), f"{name} refers to oracle/ or _work/"
    bench = open(os.path.join(ROOT, "bench.py")).read()
    assert not re.search(r"(^|[^A-Za-z0-9])_work/", bench)
    # the benchmark imports the oracle lazily, inside its CPU legs only
    assert not re.search(r"^(from|import)\s+oracle\b", bench, re.M)
