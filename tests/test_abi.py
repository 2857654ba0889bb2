"""The C-ABI library builds, loads and exports every symbol that include/jvpattn.h declares; its
argument validation answers with the documented codes.  No GPU needed (no compute call succeeds here)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from semicat_b200 import _lib


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.load()


def test_exports_match_header(lib):
    header = open(os.path.join(ROOT, "include", "jvpattn.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(jvpattn_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_struct_layout_matches_header():
    assert ctypes.sizeof(_lib.Tensor4) == 8 + 4 * 8
    assert ctypes.sizeof(_lib.Problem) == 9 * 4
    assert _lib.Problem.scale.offset == 32


def test_strerror_and_version(lib):
    assert lib.jvpattn_abi_version() == 1
    assert lib.jvpattn_strerror(0) == b"ok"
    assert b"head_dim" in lib.jvpattn_strerror(-4)
    assert b"no CPU path" in lib.jvpattn_strerror(-7)


def _prob(**kw):
    base = dict(batch=1, heads=1, len_q=128, len_k=128, head_dim=64, stat_len=128, dtype=0, kernels=0, scale=0.0)
    base.update(kw)
    return _lib.Problem(**base)


@pytest.mark.parametrize("kw,code", [
    (dict(head_dim=8), -4), (dict(head_dim=256), -4), (dict(stat_len=100), -5), (dict(len_q=200), -5),
    (dict(dtype=7), -1), (dict(kernels=9), -1), (dict(len_k=0), -1), (dict(batch=-1), -1),
])
def test_problem_validation_codes(lib, kw, code):
    p = _prob(**kw)
    assert lib.jvpattn_selected_kernels(ctypes.byref(p), 0) == code
    assert lib.jvpattn_bwd_workspace_bytes(ctypes.byref(p)) == 0


def test_null_and_stride_validation_precede_device_checks(lib):
    p = _prob()
    t = _lib.Tensor4(0x1000, (ctypes.c_int64 * 4)(8192, 64, 64, 1))
    bad = _lib.Tensor4(0x1000, (ctypes.c_int64 * 4)(8192, 64, 64, 2))
    r = ctypes.byref
    assert lib.jvpattn_fwd(r(p), None, r(t), r(t), r(t), r(t), r(t), r(t), r(t), 0x1000, 0x1000, None, None) == -1
    assert lib.jvpattn_fwd(r(p), r(bad), r(t), r(t), r(t), r(t), r(t), r(t), r(t), 0x1000, 0x1000, None, None) == -2
    assert lib.jvpattn_fwd(r(p), r(t), r(t), r(t), r(t), r(t), r(t), r(t), r(t), None, 0x1000, None, None) == -1
    # both cotangents missing
    assert lib.jvpattn_bwd(r(p), *[r(t)] * 8, None, None, 0x1000, 0x1000, *[r(t)] * 6, None, 0, None) == -1


def test_no_device_means_earch_not_a_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = _prob()
    t = _lib.Tensor4(0x1000, (ctypes.c_int64 * 4)(8192, 64, 64, 1))
    r = ctypes.byref
    assert lib.jvpattn_fwd(r(p), *[r(t)] * 8, 0x1000, 0x1000, None, None) == -7
    assert lib.jvpattn_launch_count() == 0


@pytest.mark.parametrize("B,H,Lq", [(1, 1, 128), (64, 12, 128), (3, 5, 200), (8, 16, 8192), (2, 2, 1)])
def test_backward_scratch_is_two_row_vectors(lib, B, H, Lq):
    """jvpattn_bwd_static's fixed array and its row limit rely on the workspace being exactly two fp32 vectors of
    batch * heads * stat_len entries (rounded up to 256 bytes): a workspace that grew would silently shrink that limit."""
    stat = (Lq + 127) // 128 * 128
    for D in (16, 64, 128):
        p = _prob(batch=B, heads=H, len_q=Lq, len_k=Lq, head_dim=D, stat_len=stat)
        need = lib.jvpattn_bwd_workspace_bytes(ctypes.byref(p))
        assert need == (8 * B * H * stat + 255) // 256 * 256
    assert 8 * _lib.STATIC_SCRATCH_ROWS == 2 * 1024 * 1024
