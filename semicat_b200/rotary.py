"""Rotary embedding fused with the cast to the attention input type (``jvpattn_rotary_cast``).

Caller-side helper for the blocks that feed ``safe_sdpa_jvp``: the reference rotates q and k in fp32
(semicat/net/duo.py:52-53, ``apply_rotary_emb_torch``, non-interleaved halves) and casts them to bf16 afterwards
(semicat/jvp_utils/functional.py:318-321); under ``torch.func.jvp`` each pointwise step of that chain runs as
separate primal and tangent kernels.  :func:`apply_rotary_cast` does the whole chain in one kernel per tensor and
returns the 16-bit tensor the attention kernels read, so the wrapper's casts disappear as well.

The map is linear in ``x``: the tangent goes through the same kernel, the VJP through its transpose.  Works
under ``torch.func.jvp`` and is reverse-mode differentiable with respect to primal and tangent.  CUDA only.
"""
from __future__ import annotations

import ctypes

import torch
import torch.autograd.forward_ad as fwAD

from . import _lib

_CODES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _launch(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out_dtype: torch.dtype, transpose: bool) -> torch.Tensor:
    if not x.is_cuda:
        raise RuntimeError("apply_rotary_cast runs on CUDA tensors only (no CPU path in this library)")
    if x.dim() != 4 or x.dtype not in _CODES or out_dtype not in _CODES:
        raise ValueError(f"expected a (B, S, H, D) tensor of dtype bf16/fp16/fp32, got {tuple(x.shape)} {x.dtype}")
    B, S, H, D = x.shape
    if D % 16 or cos.shape != (S, D // 2) or sin.shape != (S, D // 2):
        raise ValueError(f"head_dim must be a multiple of 16 and cos/sin (S, D/2); got D={D}, cos {tuple(cos.shape)}")
    if x.stride(3) != 1:
        x = x.contiguous()
    cos = cos.to(device=x.device, dtype=torch.float32).contiguous()
    sin = sin.to(device=x.device, dtype=torch.float32).contiguous()
    y = torch.empty((B, S, H, D), dtype=out_dtype, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.jvpattn_rotary_cast(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), _CODES[x.dtype], y.data_ptr(),
                                     _CODES[out_dtype], cos.data_ptr(), sin.data_ptr(), B, S, H, D, int(transpose),
                                     torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "jvpattn_rotary_cast")
    return y


class _RotaryCast(torch.autograd.Function):
    """y = R x (rounded to ``out_dtype``); jvp: R x_t through the same function, so that the tangent output is itself
    differentiable; backward: R^T g in the dtype of x."""

    @staticmethod
    def forward(x, cos, sin, out_dtype, transpose):
        return _launch(x, cos, sin, out_dtype, transpose)

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, cos, sin, out_dtype, transpose = inputs
        ctx.cos, ctx.sin, ctx.in_dtype, ctx.out_dtype, ctx.transpose = cos, sin, x.dtype, out_dtype, transpose

    @staticmethod
    def backward(ctx, g):
        return _RotaryCast.apply(g, ctx.cos, ctx.sin, ctx.in_dtype, not ctx.transpose), None, None, None, None

    @staticmethod
    def jvp(ctx, x_t, *_):
        return _RotaryCast.apply(x_t, ctx.cos, ctx.sin, ctx.out_dtype, ctx.transpose)


def apply_rotary_cast(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Rotate the halves of the last axis of ``x`` (B, S, H, D) by the angles whose cosines / sines are ``cos``,
    ``sin`` (S, D/2), in fp32, and return the result as a contiguous (B, S, H, D) tensor of ``out_dtype``.
    Equal, bit for bit, to ``torch.cat((x1*cos - x2*sin, x1*sin + x2*cos), -1).to(out_dtype)`` evaluated in fp32."""
    return _RotaryCast.apply(x, cos.detach(), sin.detach(), out_dtype, False)


# ------------------------------------------------------------------------------------------------ q, k, v in one launch
_QKV_CODES = {torch.bfloat16: 0, torch.float32: 2}


def _strides3(t: torch.Tensor):
    return [t.stride(0), t.stride(1), t.stride(2)]


def _launch_qkv(ins, outs, cos, sin, transpose: bool):
    B, S, H, D = ins[0].shape
    P3, S9 = ctypes.c_void_p * 3, ctypes.c_int64 * 9
    lib = _lib.load()
    with torch.cuda.device(ins[0].device):
        rc = lib.jvpattn_rotary_qkv(ctypes.byref(P3(*[t.data_ptr() for t in ins])), ctypes.byref(S9(*sum((_strides3(t) for t in ins), []))),
                                    _QKV_CODES[ins[0].dtype], ctypes.byref(P3(*[t.data_ptr() for t in outs])),
                                    ctypes.byref(S9(*sum((_strides3(t) for t in outs), []))), _QKV_CODES[outs[0].dtype],
                                    cos.data_ptr(), sin.data_ptr(), B, S, H, D, int(transpose),
                                    torch.cuda.current_stream(ins[0].device).cuda_stream)
    _lib.check(rc, "jvpattn_rotary_qkv")


def _split_forward(qkv, cos, sin, out_dtype):
    B, S, _, H, D = qkv.shape
    outs = [torch.empty(B, S, H, D, dtype=out_dtype, device=qkv.device) for _ in range(3)]
    _launch_qkv([qkv[:, :, t] for t in range(3)], outs, cos, sin, False)
    return outs


def _split_backward(grads, shape, like, cos, sin):
    """(dq, dk, dv) -> the gradient of the (B, S, 3, H, D) projection (dtype and device of ``like``), written in place by
    one launch."""
    B, S, _, H, D = shape
    fix = lambda g: torch.zeros(B, S, H, D, dtype=like.dtype, device=like.device) if g is None else (g if g.stride(3) == 1 else g.contiguous())
    gs = [fix(g) for g in grads]
    if len({g.dtype for g in gs}) != 1 or gs[0].dtype not in _QKV_CODES:
        gs = [g.to(like.dtype) for g in gs]
    d = torch.empty(shape, dtype=like.dtype, device=like.device)
    _launch_qkv(gs, [d[:, :, t] for t in range(3)], cos, sin, True)
    return d


class _RotaryQkv(torch.autograd.Function):
    @staticmethod
    def forward(qkv, cos, sin, out_dtype):
        return tuple(_split_forward(qkv, cos, sin, out_dtype))

    @staticmethod
    def setup_context(ctx, inputs, output):
        qkv, cos, sin, _ = inputs
        ctx.cos, ctx.sin, ctx.like, ctx.shape = cos, sin, qkv.new_empty(0), qkv.shape
        ctx.set_materialize_grads(False)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gq, gk, gv):
        if gq is None and gk is None and gv is None:
            return None, None, None, None
        return _split_backward((gq, gk, gv), ctx.shape, ctx.like, ctx.cos, ctx.sin), None, None, None


class _RotaryQkvDual(torch.autograd.Function):
    """(qkv, its tangent) -> (q, k, v, tq, tk, tv): the map is linear, so primal and tangent go through the same kernel,
    and one node receives all six cotangents."""

    @staticmethod
    def forward(qkv, tqkv, cos, sin, out_dtype):
        return tuple(_split_forward(qkv, cos, sin, out_dtype)) + tuple(_split_forward(tqkv, cos, sin, out_dtype))

    @staticmethod
    def setup_context(ctx, inputs, output):
        qkv, _, cos, sin, _ = inputs
        ctx.cos, ctx.sin, ctx.like, ctx.shape = cos, sin, qkv.new_empty(0), qkv.shape
        ctx.set_materialize_grads(False)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gq, gk, gv, gtq, gtk, gtv):
        d = None if (gq is None and gk is None and gv is None) else _split_backward((gq, gk, gv), ctx.shape, ctx.like, ctx.cos, ctx.sin)
        dt = None if (gtq is None and gtk is None and gtv is None) else _split_backward((gtq, gtk, gtv), ctx.shape, ctx.like, ctx.cos, ctx.sin)
        return d, dt, None, None, None


def rotary_qkv(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16):
    """Split a (B, S, 3, H, D) projection into q, k, v (each contiguous (B, S, H, D) of ``out_dtype``) with q and k rotated
    as by :func:`apply_rotary_cast`, in one launch; the backward writes the projection's gradient in place in one launch
    (instead of three tensors that are concatenated afterwards).  Works under forward-mode AD.  Inputs the kernel does not
    take (fp16, unaligned views) go through :func:`apply_rotary_cast` per tensor."""
    p, t = fwAD.unpack_dual(qkv)
    ok = (p.is_cuda and p.dim() == 5 and p.shape[2] == 3 and p.dtype in _QKV_CODES and out_dtype in _QKV_CODES and p.shape[-1] % 16 == 0
          and p.stride(4) == 1 and all(st % 8 == 0 for st in p.stride()[:4]) and (p.storage_offset() * p.element_size()) % 16 == 0)
    if t is not None:
        ok = ok and t.dtype == p.dtype and t.stride() == p.stride() and (t.storage_offset() * t.element_size()) % 16 == 0
    if not ok:
        q, k, v = qkv.unbind(2)
        return apply_rotary_cast(q, cos, sin, out_dtype), apply_rotary_cast(k, cos, sin, out_dtype), v.to(out_dtype)
    cos = cos.detach().to(device=p.device, dtype=torch.float32).contiguous()
    sin = sin.detach().to(device=p.device, dtype=torch.float32).contiguous()
    if t is None:
        return _RotaryQkv.apply(qkv, cos, sin, out_dtype)
    q, k, v, tq, tk, tv = _RotaryQkvDual.apply(p, t, cos, sin, out_dtype)
    return fwAD.make_dual(q, tq), fwAD.make_dual(k, tk), fwAD.make_dual(v, tv)
