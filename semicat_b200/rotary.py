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

import torch

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
