"""Drop-in replacement for ``semicat.jvp_utils.functional``: ``sdpa_jvp`` / ``safe_sdpa_jvp`` with the
same call contract, backed by the sm_100a kernels of ``libjvpattn.so`` instead of Triton.

Contract kept from the reference (semicat/jvp_utils/functional.py):

* ``sdpa_jvp(q, k, v)`` takes (B, H, S, D) fp16/bf16 CUDA tensors and is meant to be called under
  forward-mode AD (``torch.func.jvp`` around the model, semicat/models/semicat.py:132-136, 153-157): the
  output is a dual tensor whose primal is O and whose tangent is the JVP (functional.py:216-258).
* The result is then reverse-mode differentiable with respect to q, k, v AND their tangents: a
  cotangent on the tangent output is the JVP backward (functional.py:71-87, 90-168), a cotangent on
  the primal output the plain attention backward (functional.py:171-213, 260-268).  Outputs that receive no
  cotangent cost nothing (``set_materialize_grads(False)``); a second reverse pass is refused
  (functional.py:166-168, 211-213).
* ``safe_sdpa_jvp(q, k, v)`` takes (B, S, H, D), casts non-half inputs to bfloat16, and returns
  (B, S, H, D) in the caller's dtype (functional.py:310-332).

Differences, all internal.  The reference splits the work over three ``autograd.Function`` s (a ``forward`` that only
hands out buffers, a ``jvp`` that fills them, one backward per cotangent: 1 + 6 + 2 Triton launches).  Here the duals
are unpacked (``torch.autograd.forward_ad.unpack_dual``), ONE node maps (q, k, v, tq, tk, tv) to (y, ty) with one
library call, and the pair is packed into a dual again; reverse mode reaches that node once, with whichever cotangents
exist, and makes one library call (both cotangents go through the merged backward kernels).  The LI buffer (softmax
denominator) of the reference is not produced because no kernel here needs it; the tangent output is not zero-filled
before the kernel writes it.

One extension: when none of q, k, v carries a forward-mode tangent, ``sdpa_jvp`` runs the primal-only instance
of the same kernels (plain attention, reverse-mode differentiable) instead of returning an uninitialised buffer.
The callers' non-JVP attention (the reference uses ``F.scaled_dot_product_attention`` there,
semicat/net/duo.py:143-152) can therefore go through this library too.
"""
from __future__ import annotations

import math

import torch
import torch.autograd.forward_ad as fwAD
from torch.autograd.function import once_differentiable

from . import ops

__all__ = ["sdpa_jvp", "safe_sdpa_jvp", "set_kernel_family"]

_kernels = ops.KERNELS_AUTO


def set_kernel_family(kind: int) -> int:
    """Force a kernel family for subsequent calls (``ops.KERNELS_*``); returns the previous setting."""
    global _kernels
    prev, _kernels = _kernels, int(kind)
    return prev


def _like_input(x: torch.Tensor) -> torch.Tensor:
    """Uninitialised tensor with the memory layout of ``x`` when that layout is dense, else contiguous."""
    out = torch.empty_like(x)
    return out if out.stride(-1) == 1 else torch.empty(x.shape, dtype=x.dtype, device=x.device)


class _AttentionDual(torch.autograd.Function):
    """The fused kernel as ONE autograd node: (q, k, v, tq, tk, tv) -> (y, ty).

    ``sdpa_jvp`` unpacks the forward-mode duals it is given, calls this node on primals and tangents as six ordinary
    tensors, and packs (y, ty) into a dual again.  Reverse mode then sees a single node with two outputs, so a pass that
    brings cotangents for both (the ``ecld`` objective, and every layer of a deep model under ``lag``: the primal output
    feeds the layers above) runs ONE merged backward - the reference needs a call per cotangent
    (functional.py:71-87 and :171-213) and an addition of the two (dq, dk, dv)."""

    @staticmethod
    def forward(q, k, v, tq, tk, tv):
        B, H, S, _ = q.shape
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
        # (B, H, S, D) views of (B, S, H, D)-contiguous memory: the layout the denoiser wants back (duo.py:154-155
        # reshapes the (B, S, H, D) result to (B, S, H*D)), so that reshape stays a view.
        y = torch.empty((B, S, H, v.shape[-1]), dtype=q.dtype, device=q.device).transpose(1, 2)
        ty = torch.empty_like(y)
        rows = ops.stat_len(S)
        lse = torch.empty((B, H, rows), dtype=torch.float32, device=q.device)
        mu = (torch.empty if rows == S else torch.zeros)((B, H, rows), dtype=torch.float32, device=q.device)
        ops.jvp_attention_fwd(fix(q), fix(k), fix(v), fix(tq), fix(tk), fix(tv), y, ty, lse, mu, kernels=_kernels)
        return y, ty, lse, mu

    @staticmethod
    def setup_context(ctx, inputs, output):
        y, ty, lse, mu = output
        ctx.save_for_backward(*inputs, y, ty, lse, mu)
        ctx.mark_non_differentiable(lse, mu)
        ctx.set_materialize_grads(False)

    @staticmethod
    @once_differentiable
    def backward(ctx, g_y, g_ty, _g_lse, _g_mu):
        if g_y is None and g_ty is None:
            return (None,) * 6
        q, k, v, tq, tk, tv, y, ty, lse, mu = ctx.saved_tensors
        fix = lambda t: t if t is None or t.stride(-1) == 1 else t.contiguous()
        q, k, v, tq, tk, tv, g_y, g_ty = map(fix, (q, k, v, tq, tk, tv, g_y, g_ty))
        if g_ty is None:  # only the primal output was used: plain attention backward, the tangents get no gradient
            dq, dk, dv = (_like_input(t) for t in (q, k, v))
            ops.jvp_attention_bwd(q, k, v, None, None, None, y, None, g_y, None, lse, None, dq, dk, dv, kernels=_kernels)
            return dq, dk, dv, None, None, None
        grads = [_like_input(t) for t in (q, k, v, tq, tk, tv)]
        ops.jvp_attention_bwd(q, k, v, tq, tk, tv, y, ty, g_y, g_ty, lse, mu, *grads, kernels=_kernels)
        return tuple(grads)


class _PrimalAttention(torch.autograd.Function):
    """Plain attention through the primal-only kernel instance; used when no input carries a tangent."""

    @staticmethod
    def forward(ctx, q, k, v):
        B, H, S, _ = q.shape
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
        q, k, v = fix(q), fix(k), fix(v)
        y = torch.empty((B, S, H, v.shape[-1]), dtype=q.dtype, device=q.device).transpose(1, 2)
        lse = torch.empty((B, H, ops.stat_len(S)), dtype=torch.float32, device=q.device)
        ops.jvp_attention_fwd(q, k, v, None, None, None, y, None, lse, None, kernels=_kernels)
        ctx.save_for_backward(q, k, v, y, lse)
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, g_y):
        q, k, v, y, lse = ctx.saved_tensors
        g_y = g_y if g_y.stride(-1) == 1 else g_y.contiguous()
        dq, dk, dv = (_like_input(t) for t in (q, k, v))
        ops.jvp_attention_bwd(q, k, v, None, None, None, y, None, g_y, None, lse, None, dq, dk, dv, kernels=_kernels)
        return dq, dk, dv


def _validate(q, k, v):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("sdpa_jvp expects 4-D (B, H, S, D) tensors")
    B, H, S, D = q.shape
    if k.shape[0] != B or k.shape[1] != H or k.shape[3] != D:
        raise ValueError(f"K shape mismatch: {tuple(k.shape)} vs Q {tuple(q.shape)}")
    if tuple(v.shape) != tuple(k.shape):
        raise ValueError(f"V shape mismatch: {tuple(v.shape)} vs K {tuple(k.shape)}")
    if D < 16:
        raise ValueError(f"D_head must be >= 16, got {D}")  # ryu_triton.py:319-322
    if D > 128:
        raise ValueError(f"D_head must be <= 128, got {D}")  # flash_jvp_backward.py:2318
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("sdpa_jvp supports float16 and bfloat16 (use safe_sdpa_jvp for other dtypes)")


@torch._dynamo.disable
def sdpa_jvp(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Fused scaled-dot-product attention that supports forward-mode AD; (B, H, S, D) in and out.

    Use as ``y, ty = torch.func.jvp(sdpa_jvp, (q, k, v), (tq, tk, tv))`` or call it inside a model that
    is itself wrapped in ``torch.func.jvp``.  Without forward-mode AD (no input carries a tangent) the call is
    plain attention through the primal-only kernels, differentiable in reverse mode (the reference returns an
    uninitialised buffer in that case, functional.py:286-287).
    """
    _validate(q, k, v)
    (qp, tq), (kp, tk), (vp, tv) = (fwAD.unpack_dual(t) for t in (q, k, v))
    if tq is None and tk is None and tv is None:
        return _PrimalAttention.apply(q, k, v)
    # an input without a tangent has tangent zero
    tq = torch.zeros_like(qp) if tq is None else tq
    tk = torch.zeros_like(kp) if tk is None else tk
    tv = torch.zeros_like(vp) if tv is None else tv
    y, ty, _, _ = _AttentionDual.apply(qp, kp, vp, tq, tk, tv)
    return fwAD.make_dual(y, ty)


def safe_sdpa_jvp(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """(B, S, H, D) wrapper around :func:`sdpa_jvp` that casts non-half inputs to bfloat16 and the result
    back to the caller's dtype (keyed on ``q.dtype`` alone, like the reference)."""
    orig = q.dtype
    if orig not in (torch.bfloat16, torch.float16):
        q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    y = sdpa_jvp(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    if y.dtype != orig:
        y = y.to(orig)
    return y.transpose(1, 2)
