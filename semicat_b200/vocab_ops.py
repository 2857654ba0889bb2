"""Vocabulary-side ends of the flow-map training step as fused kernels (``csrc/vocab_loss.cu``).

The reference's step (semicat/models/semicat.py:70-85, 89-110, 112-167, 210-229) handles (batch, length, vocabulary)
fp32 tensors a dozen times per step: the interpolation towards the one-hot token, the cast in front of the embedding
GEMM, the softmax of the flow map and its forward-mode tangent, the softmax of the target pass, the squared error, the
log-softmax of the cross-entropy, and every one of them again in the backward.  At a vocabulary of 30522 each such tensor is
gigabytes.  Here the network's input and output keep ONE layout - 16-bit, rows padded to a multiple of 8 columns so that
the embedding and head GEMMs take them as they are - and everything between the noise and the two scalar losses is
recomputed per element inside five kernels:

* :func:`interpolate_cast` - the interpolated input, straight into the GEMM's layout;
* :func:`flow_map_input` - the flow map x_{s,t} (the input of the no-grad target pass) from the logits;
* :func:`cross_entropy_padded` - cross-entropy of padded logits, forward and backward;
* :func:`sd_lag_loss` - the ``lag`` self-distillation loss from (logits, their t-tangent, target logits, noise), forward
  and backward (gradients with respect to the logits and their tangent, in the GEMM's layout).

CUDA only; callers check :func:`usable` and keep the PyTorch expressions otherwise.
"""
from __future__ import annotations

import torch

from . import _lib

_CODES = {torch.bfloat16: 0, torch.float32: 2}


def padded(V: int) -> int:
    return (V + 7) & ~7


def usable(x0: torch.Tensor, dtype: torch.dtype) -> bool:
    return x0.is_cuda and x0.dim() == 3 and x0.dtype == torch.float32 and x0.stride(-1) == 1 and dtype in _CODES


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _rows(t: torch.Tensor | None):
    """A (B, L, W) tensor with unit innermost stride and uniformly spaced rows, and that row spacing."""
    if t is None:
        return None, 0
    if t.stride(-1) != 1 or t.stride(0) != t.shape[1] * t.stride(1):
        t = t.contiguous()
    return t, t.stride(1)


def _launch(op, V, dtype, B, L, *, l=None, tl=None, lt=None, ld=0, x0=None, ids=None, s=None, t=None, lse=None, stats=None,
            loss=None, g=None, out=None, out2=None, ldo=0, eps=0.0):
    ldx = 0
    if x0 is not None:
        x0, ldx = _rows(x0)
    dev = (l if l is not None else x0).device
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.jvpattn_vocab_op(op, _ptr(l), _ptr(tl), _ptr(lt), ld, _ptr(x0), ldx, _ptr(ids), _ptr(s), _ptr(t), _ptr(lse),
                                  _ptr(stats), _ptr(loss), _ptr(g), _ptr(out), _ptr(out2), ldo, float(eps), B, L, V,
                                  _CODES[dtype], torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "jvpattn_vocab_op")


def _vec(t: torch.Tensor) -> torch.Tensor:
    return t.detach().float().contiguous()


def interpolate_cast(x0: torch.Tensor, ids: torch.Tensor, t: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """``(1 - t) x0 + t onehot(ids)`` (semicat.py:70-85) as a (B, L, padded(V)) tensor of ``dtype``; padding columns are zero."""
    B, L, V = x0.shape
    out = torch.empty(B, L, padded(V), dtype=dtype, device=x0.device)
    _launch(0, V, dtype, B, L, x0=x0, ids=ids.contiguous(), t=_vec(t), out=out, ldo=out.stride(1))
    return out


def flow_map_input(logits_p: torch.Tensor, x0: torch.Tensor, ids: torch.Tensor, s: torch.Tensor, t: torch.Tensor):
    """``xst = xs + dt (softmax(logits) - xs)`` with ``xs = (1 - s) x0 + s onehot(ids)`` and ``dt = (t - s) / (1 - s + 1e-8)``
    (semicat.py:210-229), from padded logits (B, L, padded(V)); returns (xst in the same padded layout, the rows' lse).
    No gradient: the reference detaches xst (semicat.py:158)."""
    B, L, V = x0.shape
    l, ld = _rows(logits_p.detach())
    out = torch.empty(B, L, padded(V), dtype=l.dtype, device=l.device)
    lse = torch.empty(B * L, dtype=torch.float32, device=l.device)
    _launch(1, V, l.dtype, B, L, l=l, ld=ld, x0=x0, ids=ids.contiguous(), s=_vec(s), t=_vec(t), lse=lse, out=out, ldo=out.stride(1))
    return out, lse


class _CrossEntropyPadded(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_p, ids, V, eps):
        B, L, _ = logits_p.shape
        l, ld = _rows(logits_p)
        lse = torch.empty(B * L, dtype=torch.float32, device=l.device)
        loss = torch.empty(B * L, dtype=torch.float32, device=l.device)
        ids = ids.contiguous()
        _launch(2, V, l.dtype, B, L, l=l, ld=ld, ids=ids, lse=lse, loss=loss, eps=eps)
        ctx.save_for_backward(l, ids, lse)
        ctx.V, ctx.eps, ctx.ld = V, eps, ld
        return loss.mean()

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        l, ids, lse = ctx.saved_tensors
        B, L, Vp = l.shape
        dl = torch.empty(B, L, Vp, dtype=l.dtype, device=l.device)
        _launch(3, ctx.V, l.dtype, B, L, l=l, ld=ctx.ld, ids=ids, lse=lse, g=g.float().reshape(1).contiguous(), out=dl, ldo=Vp, eps=ctx.eps)
        return dl, None, None, None


def cross_entropy_padded(logits_p: torch.Tensor, ids: torch.Tensor, V: int, label_smoothing: float = 0.0) -> torch.Tensor:
    """Mean over all tokens of the cross-entropy between the first ``V`` columns of ``logits_p`` (B, L, padded(V)) and
    ``ids`` (B, L): the value of the reference's ``F.cross_entropy(pred.transpose(-1, 1), x1)`` (semicat.py:107-111)."""
    return _CrossEntropyPadded.apply(logits_p, ids, V, float(label_smoothing))


class _SdLagLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits_p, tlogits_p, target_p, x0, ids, s, t, lse):
        B, L, V = x0.shape
        l, tl, lt = logits_p, tlogits_p, target_p
        if not (l.stride() == tl.stride() == lt.stride() and l.stride(-1) == 1 and l.stride(0) == L * l.stride(1)):
            l, tl, lt = l.contiguous(), tl.contiguous(), lt.contiguous()
        ld = l.stride(1)
        stats = torch.empty(B * L, 4, dtype=torch.float32, device=l.device)
        loss = torch.empty(B * L, dtype=torch.float32, device=l.device)
        ids, s, t = ids.contiguous(), _vec(s), _vec(t)
        _launch(4, V, l.dtype, B, L, l=l, tl=tl, lt=lt, ld=ld, x0=x0, ids=ids, s=s, t=t, lse=lse, stats=stats, loss=loss)
        ctx.save_for_backward(l, tl, lt, x0, ids, s, t, lse, stats)
        ctx.V, ctx.ld = V, ld
        return loss.mean()

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        l, tl, lt, x0, ids, s, t, lse, stats = ctx.saved_tensors
        B, L, Vp = l.shape
        dl = torch.empty(B, L, Vp, dtype=l.dtype, device=l.device)
        dtl = torch.empty_like(dl)
        _launch(5, ctx.V, l.dtype, B, L, l=l, tl=tl, lt=lt, ld=ctx.ld, x0=x0, ids=ids, s=s, t=t, lse=lse, stats=stats,
                g=g.float().reshape(1).contiguous(), out=dl, out2=dtl, ldo=Vp)
        return dl, dtl, None, None, None, None, None, None


def sd_lag_loss(logits_p, tlogits_p, target_p, x0, ids, s, t, lse) -> torch.Tensor:
    """The ``lag`` self-distillation loss of semicat.py:153-164: mean over tokens of
    ``sum_v ((1 - t) dv - softmax(target) + xst)^2`` where ``xst`` is the flow map (:func:`flow_map_input`) and ``dv`` its
    derivative in t, ``ddt (p - xs) + dt p (tlogits - sum(p tlogits))``, formed from the logits and their forward-mode
    tangent ``tlogits``.  All three logit tensors are (B, L, padded(V)); ``lse`` is what :func:`flow_map_input` returned.
    Differentiable with respect to ``logits_p`` and ``tlogits_p`` (xst and the target carry no gradient, as in the reference)."""
    return _SdLagLoss.apply(logits_p, tlogits_p, target_p.detach(), x0, ids, s, t, lse)
