"""Torch-tensor front end of the C ABI: marshals (B, H, L, D) CUDA tensors into ``jvpattn_tensor``
structs and launches on the current torch stream.  Outputs are written in place through raw
pointers, so autograd version counters are untouched (the reference relies on the same property
when its Triton kernel fills the tensors that ``SDPAFunction.forward`` handed out earlier,
semicat/jvp_utils/functional.py:218-258).
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from ._lib import KERNELS_AUTO, KERNELS_SIMT, KERNELS_TCGEN05, Problem, Tensor4  # noqa: F401

_DTYPES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16}


def stat_len(len_q: int) -> int:
    """Row-statistic length the reference allocates: len_q rounded up to 128 (functional.py:57, 229)."""
    return ((len_q + 127) // 128) * 128


def _t4(t: torch.Tensor | None, name: str, dtype: torch.dtype, device: torch.device):
    if t is None:
        return None
    if t.dim() != 4:
        raise ValueError(f"{name} must be 4-D (B, H, L, D), got {tuple(t.shape)}")
    if t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")
    if t.dtype != dtype:
        raise TypeError(f"{name} has dtype {t.dtype}, expected {dtype}")
    s = t.stride()
    # a size-1 axis may carry any stride; normalise the innermost one so the library's check holds
    return Tensor4(t.data_ptr(), (ctypes.c_int64 * 4)(s[0], s[1], s[2], 1 if t.shape[3] == 1 else s[3]))


def _problem(q, k, stats_len, scale, kernels) -> Problem:
    if not q.is_cuda:
        raise RuntimeError("jvpattn kernels run on CUDA tensors only (sm_100a); there is no CPU path")
    if q.dtype not in _DTYPES:
        raise TypeError(f"jvpattn supports bfloat16 and float16, got {q.dtype}")
    B, H, Lq, D = q.shape
    return Problem(B, H, Lq, k.shape[2], D, stats_len, _DTYPES[q.dtype], kernels,
                   float(scale) if scale is not None else 0.0)


def _fptr(t: torch.Tensor | None, name: str, shape, device):
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != tuple(shape) or t.device != device:
        raise ValueError(f"{name} must be a contiguous float32 tensor of shape {tuple(shape)} on {device}")
    return t.data_ptr()


def _check_shapes(q, k, others_q, others_k):
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    for n, t in others_q:
        if t is not None and tuple(t.shape) != (B, H, Lq, D):
            raise ValueError(f"{n} shape mismatch: {tuple(t.shape)} vs {(B, H, Lq, D)}")
    for n, t in others_k:
        if t is not None and tuple(t.shape) != (B, H, Lk, D):
            raise ValueError(f"{n} shape mismatch: {tuple(t.shape)} vs {(B, H, Lk, D)}")


class _on_device:
    """Make the tensors' device current for the duration of the call (cheap when it already is)."""

    def __init__(self, device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


def jvp_attention_fwd(q, k, v, tq, tk, tv, o, to, lse, mu, li=None, scale=None, kernels=KERNELS_AUTO):
    """Fill ``o``, ``to``, ``lse``, ``mu`` (and ``li`` if given) in place.  All 4-D tensors are (B, H, L, D).
    With ``tq``, ``tk``, ``tv``, ``to`` (and ``mu``) all ``None`` the call is primal-only attention: ``o`` and
    ``lse`` alone are written."""
    lib = _lib.load()
    if (tq is None) != (tk is None) or (tq is None) != (tv is None) or (tq is None) != (to is None):
        raise ValueError("pass all of tq, tk, tv, to or none of them")
    _check_shapes(q, k, [("tq", tq), ("o", o), ("to", to)], [("k", k), ("v", v), ("tk", tk), ("tv", tv)])
    B, H, Lq, _ = q.shape
    prob = _problem(q, k, lse.shape[-1], scale, kernels)
    dev, dt = q.device, q.dtype
    args = [_t4(t, n, dt, dev) for n, t in
            (("q", q), ("k", k), ("v", v), ("tq", tq), ("tk", tk), ("tv", tv), ("o", o), ("to", to))]
    stat_shape = (B, H, lse.shape[-1])
    with _on_device(dev):
        rc = lib.jvpattn_fwd(ctypes.byref(prob), *[ctypes.byref(a) if a is not None else None for a in args],
                             _fptr(lse, "lse", stat_shape, dev), _fptr(mu, "mu", stat_shape, dev),
                             _fptr(li, "li", stat_shape, dev), torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "jvpattn_fwd")


def bwd_workspace_bytes(q, k, stats_len, kernels=KERNELS_AUTO) -> int:
    prob = _problem(q, k, stats_len, None, kernels)
    return int(_lib.load().jvpattn_bwd_workspace_bytes(ctypes.byref(prob)))


def jvp_attention_bwd(q, k, v, tq, tk, tv, o, to, g_o, g_to, lse, mu, dq, dk, dv, dtq=None, dtk=None, dtv=None,
                      scale=None, kernels=KERNELS_AUTO, workspace=None):
    """Fill the gradient tensors in place.  ``g_o`` or ``g_to`` may be ``None`` (not both)."""
    lib = _lib.load()
    _check_shapes(q, k, [("tq", tq), ("o", o), ("to", to), ("g_o", g_o), ("g_to", g_to), ("dq", dq), ("dtq", dtq)],
                  [("k", k), ("v", v), ("tk", tk), ("tv", tv), ("dk", dk), ("dv", dv), ("dtk", dtk), ("dtv", dtv)])
    B, H, Lq, _ = q.shape
    prob = _problem(q, k, lse.shape[-1], scale, kernels)
    dev, dt = q.device, q.dtype
    names = ("q", "k", "v", "tq", "tk", "tv", "o", "to", "g_o", "g_to")
    ins = [_t4(t, n, dt, dev) for n, t in zip(names, (q, k, v, tq, tk, tv, o, to, g_o, g_to))]
    outs = [_t4(t, n, dt, dev) for n, t in
            zip(("dq", "dk", "dv", "dtq", "dtk", "dtv"), (dq, dk, dv, dtq, dtk, dtv))]
    ref = lambda a: ctypes.byref(a) if a is not None else None
    stat_shape = (B, H, lse.shape[-1])
    with _on_device(dev):
        need = int(lib.jvpattn_bwd_workspace_bytes(ctypes.byref(prob)))
        if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
            workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        ws_ptr = workspace.data_ptr() if workspace is not None else None
        ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
        rc = lib.jvpattn_bwd(ctypes.byref(prob), *[ref(a) for a in ins],
                             _fptr(lse, "lse", stat_shape, dev), _fptr(mu, "mu", stat_shape, dev),
                             *[ref(a) for a in outs], ws_ptr, ws_bytes,
                             torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "jvpattn_bwd")
    return workspace


def jvp_attention_bwd_static(q, k, v, tq, tk, tv, o, to, g_o, g_to, lse, mu, dq, dk, dv, dtq=None, dtk=None, dtv=None,
                             scale=None, kernels=KERNELS_AUTO):
    """Backward through ``jvpattn_bwd_static``: same results as :func:`jvp_attention_bwd`, but the scratch
    comes from a fixed 2 MiB array inside the library, so neither this wrapper nor the library allocates
    device memory.  For hosts that cannot allocate (all memory pre-claimed by their own pool, or no access to
    an allocator at the point of the call).  Limit: ``B * H * stat_len <= _lib.STATIC_SCRATCH_ROWS``; larger
    problems raise ``JvpAttnError`` (code -10).  Calls on one device share the array, so do not let two of
    them overlap on different streams; make the first call on a device outside any stream capture."""
    lib = _lib.load()
    _check_shapes(q, k, [("tq", tq), ("o", o), ("to", to), ("g_o", g_o), ("g_to", g_to), ("dq", dq), ("dtq", dtq)],
                  [("k", k), ("v", v), ("tk", tk), ("tv", tv), ("dk", dk), ("dv", dv), ("dtk", dtk), ("dtv", dtv)])
    prob = _problem(q, k, lse.shape[-1], scale, kernels)
    dev, dt = q.device, q.dtype
    names = ("q", "k", "v", "tq", "tk", "tv", "o", "to", "g_o", "g_to", "dq", "dk", "dv", "dtq", "dtk", "dtv")
    structs = [_t4(t, n, dt, dev) for n, t in zip(names, (q, k, v, tq, tk, tv, o, to, g_o, g_to, dq, dk, dv, dtq, dtk, dtv))]
    ref = lambda a: ctypes.byref(a) if a is not None else None
    with _on_device(dev):
        rc = lib.jvpattn_bwd_static(ctypes.byref(prob), *[ref(a) for a in structs[:10]],
                                    lse.data_ptr(), mu.data_ptr() if mu is not None else None,
                                    *[ref(a) for a in structs[10:]], torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "jvpattn_bwd_static")


class Plan:
    """Pre-marshalled forward + backward on fixed tensors: everything ctypes needs is built once, so a
    launch costs two foreign calls.  The tensors (all (B, H, L, D) views) must stay alive and in place.
    Used where the same buffers are run repeatedly (benchmarks, CUDA-graph capture)."""

    def __init__(self, q, k, v, tq, tk, tv, o, to, lse, mu, g_o=None, g_to=None, grads=None, scale=None,
                 kernels=KERNELS_AUTO):
        self.lib = _lib.load()
        self.device = q.device
        self.keep = [q, k, v, tq, tk, tv, o, to, lse, mu, g_o, g_to, grads]
        dt, dev = q.dtype, q.device
        self.prob = _problem(q, k, lse.shape[-1], scale, kernels)
        byref = lambda t, n: ctypes.byref(self._hold(_t4(t, n, dt, dev))) if t is not None else None
        self._structs = []
        ins = [byref(t, n) for n, t in zip("q k v tq tk tv o to".split(), (q, k, v, tq, tk, tv, o, to))]
        self.fwd_args = [ctypes.byref(self.prob), *ins, lse.data_ptr(), mu.data_ptr(), None]
        self.bwd_args = None
        if grads is not None:
            with _on_device(dev):
                need = int(self.lib.jvpattn_bwd_workspace_bytes(ctypes.byref(self.prob)))
            self.workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
            outs = [byref(t, n) for n, t in zip("dq dk dv dtq dtk dtv".split(), grads)]
            self.bwd_args = [ctypes.byref(self.prob), *ins, byref(g_o, "g_o"), byref(g_to, "g_to"),
                             lse.data_ptr(), mu.data_ptr(), *outs, self.workspace.data_ptr(), self.workspace.numel()]

    def _hold(self, struct):
        self._structs.append(struct)
        return struct

    def forward(self):
        _lib.check(self.lib.jvpattn_fwd(*self.fwd_args, torch.cuda.current_stream(self.device).cuda_stream), "jvpattn_fwd")

    def backward(self):
        _lib.check(self.lib.jvpattn_bwd(*self.bwd_args, torch.cuda.current_stream(self.device).cuda_stream), "jvpattn_bwd")


def selected_kernels(B, H, Lq, Lk, D, dtype=torch.bfloat16, which="fwd") -> int:
    prob = Problem(B, H, Lq, Lk, D, stat_len(Lq), _DTYPES[dtype], KERNELS_AUTO, 0.0)
    return int(_lib.load().jvpattn_selected_kernels(ctypes.byref(prob), 0 if which == "fwd" else 1))


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
