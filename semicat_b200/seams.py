"""The three kernel entry points of the reference, re-implemented on ``libjvpattn``.

``semicat/jvp_utils/functional.py`` reaches its GPU kernels through three host functions that it imports lazily,
inside the autograd Functions (functional.py:23-25, 127-129, 183-185):

* ``semicat.jvp_utils.ryu_triton.flash_attention_jvp_multihead_triton_kernel_wrapper`` (ryu_triton.py:295-422),
* ``semicat.jvp_utils.flash_jvp_backward._flash_attn_backward`` (flash_jvp_backward.py:2293-2714),
* ``semicat.jvp_utils.flash_attn_triton._flash_attn_backward`` (flash_attn_triton.py:974-1093).

The functions below have those signatures and fill the same tensors in place, so the reference's ``functional.py``
runs unchanged on top of them; :func:`install` puts them into the three modules.  This is the narrowest way to drop
the library in (``semicat_b200.hooks`` replaces ``sdpa_jvp`` / ``safe_sdpa_jvp`` instead, one level up).

One piece of information is missing at the second seam.  The library derives the two per-row sums of the backward
from the primal output ``y`` and the tangent output ``t_y`` (d-length dot products) where the reference recomputes
them from the scores.  But functional.py:74-86 passes ``t_y`` in the ``o`` slot and the softmax denominators in ``li``;
``y`` itself does not reach the call.  The forward seam therefore remembers which ``y`` belongs to each ``t_y`` it
produced, and the backward seam looks it up.  A maintainer who can edit functional.py would rather pass both
(``o=y`` and ``t_y`` in place of ``li``) and call ``ops.jvp_attention_bwd`` directly.
"""
from __future__ import annotations

import importlib
import math

import torch

from . import ops

_SEAMS = (
    ("semicat.jvp_utils.ryu_triton", "flash_attention_jvp_multihead_triton_kernel_wrapper"),
    ("semicat.jvp_utils.flash_jvp_backward", "_flash_attn_backward"),
    ("semicat.jvp_utils.flash_attn_triton", "_flash_attn_backward"),
)
_saved: dict = {}
# (data_ptr, shape) of a tangent output -> the primal output computed with it.  An entry is dropped when the backward
# seam consumes it; forwards that never see a backward (evaluation) are bounded by MAX_REMEMBERED, oldest first.
_primal_of: dict = {}
MAX_REMEMBERED = 256


def _unit_stride(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _remember(t_y: torch.Tensor, y: torch.Tensor) -> None:
    key = (t_y.data_ptr(), tuple(t_y.shape))
    _primal_of.pop(key, None)
    _primal_of[key] = y.detach()
    while len(_primal_of) > MAX_REMEMBERED:
        del _primal_of[next(iter(_primal_of))]


def flash_attention_jvp_multihead_triton_kernel_wrapper(Q, K, V, t_Q, t_K, t_V, scale=None, y=None, t_y=None, M=None,
                                                        MU=None, LI=None, return_M=False):
    """Fused forward; (B, H, L, D) tensors.  Fills ``y``, ``M`` (log-sum-exp), ``MU`` and ``LI`` in place and
    returns ``(y, t_y)`` or ``(y, t_y, M, MU, LI)`` like ryu_triton.py:295-422."""
    B, H, L, D = Q.shape
    if D < 16:
        raise ValueError(f"D_head must be >= 16 for efficient Triton kernel, got {D}")  # ryu_triton.py:319-322
    dev = Q.device
    if y is None:
        y = torch.empty((B, H, L, D), dtype=Q.dtype, device=dev)
    if t_y is None:
        t_y = torch.empty((B, H, L, D), dtype=Q.dtype, device=dev)
    rows = ops.stat_len(L)
    stat = lambda fill: torch.full((B, H, rows), fill, dtype=torch.float32, device=dev)
    M = stat(math.log(max(K.shape[-2], 1))) if M is None else M
    MU = stat(0.0) if MU is None else MU
    with torch.no_grad():
        ops.jvp_attention_fwd(*(_unit_stride(t.detach()) for t in (Q, K, V, t_Q, t_K, t_V)), y.detach(), t_y.detach(),
                              M.detach(), MU.detach(), li=LI.detach() if LI is not None else None, scale=scale)
    _remember(t_y, y)
    return (y, t_y, M, MU, LI) if return_M else (y, t_y)


def jvp_flash_attn_backward(dto, q, k, v, o, tq, tk, tv, lse, mu, li, dq, dk, dv, dtq, dtk, dtv, softmax_scale=None):
    """VJP of a cotangent on the tangent output; (B, S, H, D) tensors as in flash_jvp_backward.py:2293-2312.
    ``o`` carries the tangent output (that is what functional.py:74-86 passes there); the primal output is looked
    up from the forward seam's record.  ``li`` is accepted and ignored.  Fills the six gradients in place."""
    f = lambda t: _unit_stride(t).transpose(1, 2)  # (B, S, H, D) -> (B, H, S, D) view
    y = _primal_of.pop((o.data_ptr(), (o.shape[0], o.shape[2], o.shape[1], o.shape[3])), None)
    if y is None:
        raise RuntimeError("jvp backward seam: the primal output that belongs to this tangent output is unknown (the "
                           "forward seam of semicat_b200.seams did not produce it, or more than MAX_REMEMBERED "
                           "forwards ran since)")
    with torch.no_grad():
        ops.jvp_attention_bwd(f(q), f(k), f(v), f(tq), f(tk), f(tv), _unit_stride(y), f(o), None, f(dto), lse, mu,
                              dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2), dtq.transpose(1, 2),
                              dtk.transpose(1, 2), dtv.transpose(1, 2), scale=softmax_scale)


def primal_flash_attn_backward(do, q, k, v, o, lse, dq, dk, dv, bias=None, causal=False, softmax_scale=None):
    """VJP of a cotangent on the primal output; (B, S, H, D) tensors as in flash_attn_triton.py:974-976.
    The reference's JVP path never passes a bias or a causal mask (functional.py:192-205); both are refused."""
    if bias is not None or causal:
        raise NotImplementedError("libjvpattn implements the non-causal, bias-free attention of sdpa_jvp only")
    f = lambda t: _unit_stride(t).transpose(1, 2)
    with torch.no_grad():
        ops.jvp_attention_bwd(f(q), f(k), f(v), None, None, None, f(o), None, f(do), None, lse, None,
                              dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2), scale=softmax_scale)


_REPLACEMENTS = (flash_attention_jvp_multihead_triton_kernel_wrapper, jvp_flash_attn_backward, primal_flash_attn_backward)


def install() -> list[str]:
    """Put the three functions into an importable ``semicat`` package.  Returns the patched module names.
    Raises if one of the three modules cannot be imported (``flash_attn_triton`` needs a CUDA device at import,
    flash_attn_triton.py:695)."""
    patched = []
    for (modname, attr), fn in zip(_SEAMS, _REPLACEMENTS):
        mod = importlib.import_module(modname)
        _saved.setdefault((modname, attr), getattr(mod, attr))
        setattr(mod, attr, fn)
        patched.append(modname)
    return patched


def uninstall() -> None:
    import sys
    for (modname, attr), fn in list(_saved.items()):
        mod = sys.modules.get(modname)
        if mod is not None:
            setattr(mod, attr, fn)
    _saved.clear()
    _primal_of.clear()
