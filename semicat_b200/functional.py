"""Drop-in replacement for ``semicat.jvp_utils.functional``: ``sdpa_jvp`` / ``safe_sdpa_jvp`` with the
same call contract, backed by the sm_100a kernels of ``libjvpattn.so`` instead of Triton.

Contract kept from the reference (semicat/jvp_utils/functional.py):

* ``sdpa_jvp(q, k, v)`` takes (B, H, S, D) fp16/bf16 CUDA tensors and is meant to be called under
  forward-mode AD (``torch.func.jvp`` around the model, semicat/models/semicat.py:132-136, 153-157).
  The plain ``forward`` only hands out the output buffer and the row-statistic buffer; the fused
  kernel fills both when autograd calls ``jvp`` (functional.py:216-258).
* The result is then reverse-mode differentiable with respect to q, k, v AND their tangents: a
  cotangent on the tangent output runs the JVP backward (functional.py:71-87, 90-168), a cotangent on
  the primal output runs the plain attention backward (functional.py:171-213, 260-268); autograd sums
  the two q/k/v contributions.  A second reverse pass is refused (functional.py:166-168, 211-213).
* ``safe_sdpa_jvp(q, k, v)`` takes (B, S, H, D), casts non-half inputs to bfloat16, and returns
  (B, S, H, D) in the caller's dtype (functional.py:310-332).

Differences, all internal: one library call per pass instead of 1 + 6 + 2 Triton launches; the
LI buffer (softmax denominator) of the reference is not produced because no kernel here needs it;
the tangent output is not zero-filled before the kernel writes it.

One extension: when none of q, k, v carries a forward-mode tangent, ``sdpa_jvp`` runs the primal-only instance
of the same kernels (plain attention, reverse-mode differentiable) instead of returning an uninitialised buffer.
The callers' non-JVP attention (the reference uses ``F.scaled_dot_product_attention`` there,
semicat/net/duo.py:143-152) can therefore go through this library too.

When both outputs receive a cotangent in one reverse pass (the ``ecld`` objective, semicat/models/semicat.py:131-151),
autograd calls the two backward methods below separately, as it does with the reference's two Functions: two
library calls, and autograd adds the two (dq, dk, dv) contributions.  The single merged call that handles both
cotangents at once (``ops.jvp_attention_bwd`` with ``g_o`` and ``g_to``) is available to direct callers only: the
tangent-side gradients must be returned by the node autograd visits first, before the cotangent of the primal output
is known to it.
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


class _AttentionWithTangent(torch.autograd.Function):
    """Tangent half: runs the fused forward kernel.  Inputs (q, k, v, tq, tk, tv, y, lse); fills y and lse
    in place and returns the new tensors (ty, mu).  Its backward is the VJP of a cotangent on ty."""

    @staticmethod
    def forward(q, k, v, tq, tk, tv, y, lse):
        ty = torch.empty_like(y)
        rows = lse.shape[-1]
        alloc = torch.empty if rows == q.shape[2] else torch.zeros
        mu = alloc(lse.shape, dtype=torch.float32, device=q.device)
        # the reference requires unit innermost stride only for the backward; the kernels here need it
        # everywhere, so repack the rare tensor that lacks it
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
        ops.jvp_attention_fwd(fix(q.detach()), fix(k.detach()), fix(v.detach()), fix(tq.detach()),
                              fix(tk.detach()), fix(tv.detach()), y.detach(), ty, lse.detach(), mu,
                              kernels=_kernels)
        return ty, mu

    @staticmethod
    def setup_context(ctx, inputs, output):
        ty, mu = output
        ctx.save_for_backward(*inputs, ty, mu)
        ctx.mark_non_differentiable(mu)
        ctx.set_materialize_grads(False)

    @staticmethod
    @once_differentiable
    def backward(ctx, g_ty, _g_mu):
        if g_ty is None:
            return (None,) * 8
        q, k, v, tq, tk, tv, y, lse, ty, mu = ctx.saved_tensors
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
        q, k, v, tq, tk, tv, g_ty = map(fix, (q, k, v, tq, tk, tv, g_ty))
        grads = [_like_input(t) for t in (q, k, v, tq, tk, tv)]
        ops.jvp_attention_bwd(q, k, v, tq, tk, tv, y, ty, None, g_ty, lse, mu, *grads, kernels=_kernels)
        return (*grads, None, None)


class _Attention(torch.autograd.Function):
    """Primal half: ``forward`` allocates (y, lse) without computing; ``jvp`` triggers the fused kernel."""

    @staticmethod
    def forward(q, k, v):
        B, H, S, _ = q.shape
        # (B, H, S, D) view of (B, S, H, D)-contiguous memory: the layout the denoiser wants back
        # (duo.py:154-155 reshapes the (B, S, H, D) result to (B, S, H*D)), so that reshape stays a view.
        # The reference hands out a (B, H, S, D)-contiguous buffer and pays a copy there; shapes are the same.
        y = torch.empty((B, S, H, v.shape[-1]), dtype=q.dtype, device=q.device).transpose(1, 2)
        # same placeholder value as the reference (log of the key count), overwritten by the kernel
        lse = torch.full((B, H, ops.stat_len(S)), math.log(max(k.shape[-2], 1)), dtype=torch.float32, device=q.device)
        return y, lse

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.save_for_forward(*inputs, *output)
        ctx.save_for_backward(*inputs, *output)
        ctx.set_materialize_grads(False)

    @staticmethod
    def jvp(ctx, tq, tk, tv):
        q, k, v, y, lse = ctx.saved_for_forward
        # an input without a tangent has tangent zero
        tq = torch.zeros_like(q) if tq is None else tq
        tk = torch.zeros_like(k) if tk is None else tk
        tv = torch.zeros_like(v) if tv is None else tv
        ty, _ = _AttentionWithTangent.apply(q, k, v, tq, tk, tv, y, lse)
        # the statistic output carries no meaningful tangent; like the reference (functional.py:258) the
        # buffer itself is handed back rather than spending a kernel on zeros
        return ty, lse

    @staticmethod
    @once_differentiable
    def backward(ctx, g_y, _g_lse):
        if g_y is None:
            return None, None, None
        q, k, v, y, lse = ctx.saved_tensors
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
        q, k, v, g_y = map(fix, (q, k, v, g_y))
        dq, dk, dv = (_like_input(t) for t in (q, k, v))
        ops.jvp_attention_bwd(q, k, v, None, None, None, y, None, g_y, None, lse, None, dq, dk, dv,
                              kernels=_kernels)
        return dq, dk, dv


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


def _carries_tangent(t: torch.Tensor) -> bool:
    return fwAD.unpack_dual(t).tangent is not None


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
    if not (_carries_tangent(q) or _carries_tangent(k) or _carries_tangent(v)):
        return _PrimalAttention.apply(q, k, v)
    y, _ = _Attention.apply(q, k, v)
    return y


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
