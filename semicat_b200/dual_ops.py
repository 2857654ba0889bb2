"""Fused (primal, tangent) pointwise ops for the denoiser block around the attention.

Callers of ``safe_sdpa_jvp`` run the whole block under ``torch.func.jvp`` (semicat/models/semicat.py:153-157), where
every pointwise op of semicat/net/duo.py:127-166 becomes several small kernels for the primal and several more for the
tangent, and again for each of them in the backward.  Four ops cover most of that chain:

* :func:`ln_modulate` - ``norm(x) * (1 + scale) + shift`` (duo.py:128-135 and :159),
* :func:`gated_residual` - ``dropout(branch * gate) + skip`` (duo.py:157 and :160),
* :func:`gelu_tanh` - the GELU of the block's MLP (duo.py:118-123),
* :func:`linear` - ``F.linear`` with primal and tangent in one node (the GEMMs stay the BLAS library's).

Under forward-mode AD each op unpacks its dual inputs (``torch.autograd.forward_ad.unpack_dual``), runs ONE
``torch.autograd.Function`` that maps primals and tangents to (output, output tangent), and packs the pair into a dual
again.  Reverse mode then meets a single node per op that receives the cotangents of both outputs together, so the
backward is one or two kernels per op with no additions of partial gradients in between.  They work under
``torch.func.jvp`` and are reverse-mode differentiable with respect to the primals AND the tangents.  CUDA only; shapes the kernels do not take (channels other than 256/512/768/1024, mixed
dtypes) fall back to the equivalent PyTorch expression, so callers need no special cases.

``ln_modulate`` differentiates the LayerNorm tangent like PyTorch does by default (``exact=False``): PyTorch's
forward-mode formula for ``native_layer_norm`` reuses the saved mean and rstd, which are not differentiable outputs, so
the reverse pass through the tangent treats them as constants.  ``exact=True`` includes their dependence on ``x``.
"""
from __future__ import annotations

import contextlib
import ctypes

import torch
import torch.autograd.forward_ad as fwAD
import torch.nn.functional as F

from . import _lib

_CODES = {torch.bfloat16: 0, torch.float32: 2}


def _usable(x: torch.Tensor, *others) -> bool:
    if not x.is_cuda or x.dim() != 3 or x.dtype not in _CODES or x.shape[-1] not in (256, 512, 768, 1024):
        return False
    return all(o is None or (o.dtype == x.dtype and o.is_cuda) for o in others)


def _rows(t: torch.Tensor | None, B: int, C: int):
    """A (B, 1, C) or (B, C) modulation tensor as ((B, C) view with unit channel stride, row stride)."""
    if t is None:
        return None, 0
    t = t.reshape(B, C) if t.dim() == 3 and t.is_contiguous() else (t[:, 0] if t.dim() == 3 else t)
    if t.stride(-1) != 1 or t.stride(0) % 8 or t.data_ptr() % 16:
        t = t.contiguous()
    return t, t.stride(0)


def _nz(t):
    """A tangent as ``None`` when it is absent or a symbolic zero (torch.func.jvp hands inputs without a tangent an
    efficient zero tensor)."""
    if t is None or t._is_zerotensor():
        return None
    return t


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _ln_launch(which, x, tx, gamma, beta, shift, scale, tshift, tscale, mean, rstd, out, g, dx, dtx, sums, eps, exact):
    B, S, C = x.shape
    sc, sc_stride = _rows(scale, B, C)
    sh, sh_stride = _rows(shift, B, C)
    tsc, tsc_stride = _rows(tscale, B, C)
    tsh, tsh_stride = _rows(tshift, B, C)
    if sh is not None and sh_stride != sc_stride:
        sh = sh.contiguous()
        sc = sc.contiguous()
        sc_stride = sh_stride = C
    if tsc is not None and tsh is not None and tsc_stride != tsh_stride:
        tsc, tsh = tsc.contiguous(), tsh.contiguous()
        tsc_stride = C
    tstride = tsc_stride if tsc is not None else tsh_stride
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.jvpattn_ln_modulate(which, _ptr(x), _ptr(tx), _ptr(gamma), _ptr(beta), _ptr(sh), _ptr(sc), _ptr(tsh), _ptr(tsc),
                                     sc_stride, tstride, _ptr(mean), _ptr(rstd), _ptr(out), _ptr(g), _ptr(dx), _ptr(dtx), _ptr(sums),
                                     B, S, C, float(eps), int(exact), _CODES[x.dtype], _stream(x))
    _lib.check(rc, "jvpattn_ln_modulate")


def _ln_finalize(sums_y, sums_ty, gamma, beta, scale, tscale, want_tangent_grads, B, C, param_grads):
    """Gradients of (shift, scale, tshift, tscale, gamma, beta) from the column sums of the backward kernels: one launch.
    ``param_grads``: zeroed fp32 (2, C) that receives d_gamma and d_beta."""
    dev, dt = scale.device, scale.dtype
    sc, sc_stride = _rows(scale, B, C)
    tsc, tsc_stride = _rows(tscale, B, C)
    new = lambda: torch.empty(B, C, dtype=dt, device=dev)
    d_shift = new() if sums_y is not None else None
    d_scale = new()
    d_tshift = new() if (sums_ty is not None and want_tangent_grads[0]) else None
    d_tscale = new() if (sums_ty is not None and want_tangent_grads[1]) else None
    d_gamma = param_grads[0]
    d_beta = param_grads[1] if beta is not None else None
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.jvpattn_ln_finalize(_ptr(sums_y), _ptr(sums_ty), _ptr(gamma), _ptr(beta), _ptr(sc), _ptr(tsc), sc_stride, tsc_stride,
                                     _ptr(d_shift), _ptr(d_scale), _ptr(d_tshift), _ptr(d_tscale), _ptr(d_gamma), _ptr(d_beta),
                                     B, C, _CODES[dt], _stream(scale))
    _lib.check(rc, "jvpattn_ln_finalize")
    return d_shift, d_scale, d_tshift, d_tscale, d_gamma, d_beta


class _LnModulateDual(torch.autograd.Function):
    """(x, gamma, beta, shift, scale, tx, tshift, tscale) -> (y, ty) as one autograd node: a reverse pass brings the
    cotangents of both outputs at once, the two backward kernels leave their sum in dx, and one more launch turns
    their column sums into the gradients of the modulation tensors and of the LayerNorm weight and bias."""

    @staticmethod
    def forward(x, gamma, beta, shift, scale, tx, tshift, tscale, eps, exact):
        B, S, C = x.shape
        y, ty = torch.empty_like(x), torch.empty_like(x)
        mean = torch.empty(B * S, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        _ln_launch(0, x, None, gamma, beta, shift, scale, None, None, mean, rstd, y, None, None, None, None, eps, exact)
        tx_ = torch.zeros_like(x) if tx is None else tx.contiguous()
        _ln_launch(1, x, tx_, gamma, beta, None, scale, tshift, tscale, mean, rstd, ty, None, None, None, None, eps, exact)
        return y, ty, mean, rstd

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, gamma, beta, shift, scale, tx, tshift, tscale, eps, exact = inputs
        _, _, mean, rstd = output
        ctx.mark_non_differentiable(mean, rstd)
        ctx.save_for_backward(x, gamma, beta, shift, scale, tx, tshift, tscale, mean, rstd)
        ctx.eps, ctx.exact = eps, exact
        ctx.set_materialize_grads(False)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy, gty, _gm, _gr):
        if gy is None and gty is None:
            return (None,) * 10
        x, gamma, beta, shift, scale, tx, tshift, tscale, mean, rstd = ctx.saved_tensors
        B, S, C = x.shape
        dx = torch.empty_like(x)
        dtx = None
        zeros = torch.zeros(5 * B * C + 2 * C, dtype=torch.float32, device=x.device)  # one fill for everything that is added to
        sums, param_grads = zeros[:5 * B * C].view(5, B, C), zeros[5 * B * C:].view(2, C)
        sums_y = sums[:2] if gy is not None else None
        sums_ty = sums[2:] if gty is not None else None
        if gy is not None:
            _ln_launch(2, x, None, gamma, None, None, scale, None, None, mean, rstd, None, gy.contiguous(), dx, None, sums_y, ctx.eps, ctx.exact)
        if gty is not None:
            tx_ = torch.zeros_like(x) if tx is None else tx.contiguous()
            dtx = torch.empty_like(x)
            flags = int(ctx.exact) | (2 if gy is not None else 0)
            _ln_launch(3, x, tx_, gamma, None, None, scale, None, tscale, mean, rstd, None, gty.contiguous(), dx, dtx, sums_ty, ctx.eps, flags)
        d_shift, d_scale, d_tshift, d_tscale, d_gamma, d_beta = _ln_finalize(
            sums_y, sums_ty, gamma, beta, scale, tscale, (tshift is not None, tscale is not None), B, C, param_grads)
        shaped = lambda v, ref: None if v is None or ref is None else v.reshape(ref.shape)
        return (dx, d_gamma, d_beta, shaped(d_shift, shift), shaped(d_scale, scale), dtx if tx is not None else None,
                shaped(d_tshift, tshift), shaped(d_tscale, tscale), None, None)


class _LnModulate(torch.autograd.Function):
    @staticmethod
    def forward(x, gamma, beta, shift, scale, eps, exact):
        B, S, C = x.shape
        y = torch.empty_like(x)
        mean = torch.empty(B * S, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        _ln_launch(0, x, None, gamma, beta, shift, scale, None, None, mean, rstd, y, None, None, None, None, eps, exact)
        return y, mean, rstd

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, gamma, beta, shift, scale, eps, exact = inputs
        _, mean, rstd = output
        ctx.mark_non_differentiable(mean, rstd)
        ctx.save_for_backward(x, gamma, beta, shift, scale, mean, rstd)
        ctx.eps, ctx.exact = eps, exact

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g, _gm, _gr):
        x, gamma, beta, shift, scale, mean, rstd = ctx.saved_tensors
        B, S, C = x.shape
        dx = torch.empty_like(x)
        zeros = torch.zeros(2 * B * C + 2 * C, dtype=torch.float32, device=x.device)
        sums, param_grads = zeros[:2 * B * C].view(2, B, C), zeros[2 * B * C:].view(2, C)
        _ln_launch(2, x, None, gamma, None, None, scale, None, None, mean, rstd, None, g.contiguous(), dx, None, sums, ctx.eps, ctx.exact)
        d_shift, d_scale, _, _, d_gamma, d_beta = _ln_finalize(sums, None, gamma, beta, scale, None, (False, False), B, C, param_grads)
        return dx, d_gamma, d_beta, d_shift.reshape(shift.shape), d_scale.reshape(scale.shape), None, None


def ln_modulate(x: torch.Tensor, norm: torch.nn.LayerNorm, shift: torch.Tensor, scale: torch.Tensor, exact: bool = False) -> torch.Tensor:
    """``norm(x) * (1 + scale) + shift`` for ``x`` (B, S, C) and per-sample ``shift`` / ``scale`` ((B, 1, C) or (B, C)).
    The result has the dtype of ``x`` (under autocast the reference computes it in fp32 and the next linear layer rounds
    it to bf16: the same values)."""
    if norm.weight is None or not _usable(x, shift, scale) or tuple(norm.normalized_shape) != (x.shape[-1],):
        return norm(x) * (1.0 + scale) + shift
    beta = norm.bias.float() if norm.bias is not None else None
    (xp, tx), (shp, tsh), (scp, tsc) = (fwAD.unpack_dual(t) for t in (x, shift, scale))
    if tx is None and tsh is None and tsc is None:
        y, _, _ = _LnModulate.apply(x.contiguous(), norm.weight.float(), beta, shift, scale, norm.eps, exact)
        return y
    # forward-mode AD is active: one node maps primals and tangents to (y, ty); the LayerNorm weight and bias are
    # parameters and carry no tangent where this is used
    y, ty, _, _ = _LnModulateDual.apply(xp.contiguous(), norm.weight.float(), beta, shp, scp, tx, tsh, tsc, norm.eps, exact)
    return fwAD.make_dual(y, ty)


class _Drop:
    """Where the dropout masks of a training step come from: a 64-bit seed in device memory, drawn once per step by
    :func:`dropout_seed`, and the number of the call within the step.  The kernels regenerate a call's mask from the two
    wherever they need it (forward, tangent, backward) instead of reading a mask tensor."""
    seed: torch.Tensor | None = None
    calls = 0


@contextlib.contextmanager
def dropout_seed(device):
    """Inside this context the dropout of :func:`gated_residual` is generated in its kernels from one fresh device-side
    seed (one tiny random draw instead of a mask tensor per call; under CUDA-graph capture the draw is part of the graph,
    so every replay sees new masks).  Outside it a mask tensor is drawn per call."""
    prev = (_Drop.seed, _Drop.calls)
    _Drop.seed = torch.randint(0, 2 ** 62, (1,), dtype=torch.int64, device=device)
    _Drop.calls = 0
    try:
        yield
    finally:
        _Drop.seed, _Drop.calls = prev


def _drop_struct(drop):
    """``drop`` = (seed tensor, call number, p) or None -> ctypes argument."""
    if drop is None:
        return None
    seed, call, p = drop
    return ctypes.byref(_lib.Dropout(seed.data_ptr(), call, p))


def _gate_launch(x, y, gate, mask, z, drop=None):
    B, S, C = y.shape
    gt, gt_stride = _rows(gate, B, C)
    lib = _lib.load()
    with torch.cuda.device(y.device):
        rc = lib.jvpattn_gated_residual(_ptr(x), _ptr(y), _ptr(gt), _ptr(mask), gt_stride, _ptr(z), B, S, C, _CODES[y.dtype],
                                        _drop_struct(drop), _stream(y))
    _lib.check(rc, "jvpattn_gated_residual")


def _gate_dual_launch(which, x, tx, y, ty, gate, tgate, mask, z, tz, gz, gtz, d_y, d_ty, sums, drop=None):
    B, S, C = y.shape
    gt, gt_stride = _rows(gate, B, C)
    tg, tg_stride = _rows(tgate, B, C)
    lib = _lib.load()
    with torch.cuda.device(y.device):
        rc = lib.jvpattn_gated_residual_dual(which, _ptr(x), _ptr(tx), _ptr(y), _ptr(ty), _ptr(gt), _ptr(tg), _ptr(mask), gt_stride,
                                             tg_stride, _ptr(z), _ptr(tz), _ptr(gz), _ptr(gtz), _ptr(d_y), _ptr(d_ty), _ptr(sums),
                                             B, S, C, _CODES[y.dtype], _drop_struct(drop), _stream(y))
    _lib.check(rc, "jvpattn_gated_residual_dual")


class _GatedResidualDual(torch.autograd.Function):
    """(x, y, gate, mask, tx, ty, tgate) -> (z, tz) = (x + m gate y, tx + m (gate ty + tgate y)) as one autograd node:
    one kernel forward, one kernel for the cotangents of both outputs.  Any of tx, ty, tgate may be absent (zero)."""

    @staticmethod
    def forward(x, y, gate, mask, tx, ty, tgate, drop):
        c = lambda t: None if t is None else t.contiguous()
        z, tz = torch.empty_like(y), torch.empty_like(y)
        _gate_dual_launch(0, x, c(tx), y, c(ty), gate, tgate, mask, z, tz, None, None, None, None, None, drop)
        return z, tz

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, y, gate, mask, tx, ty, tgate, drop = inputs
        ctx.save_for_backward(y, gate, mask, ty, tgate)
        ctx.has_tx, ctx.drop = tx is not None, drop
        ctx.set_materialize_grads(False)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gz, gtz):
        if gz is None and gtz is None:
            return (None,) * 8
        y, gate, mask, ty, tgate = ctx.saved_tensors
        B, S, C = y.shape
        c = lambda t: None if t is None else t.contiguous()
        gz, gtz = c(gz), c(gtz)
        d_y = torch.empty_like(y)
        d_ty = torch.empty_like(y) if gtz is not None else None
        sums = torch.zeros(2, B, C, dtype=torch.float32, device=y.device)
        _gate_dual_launch(1, None, None, y, c(ty), gate, tgate, mask, None, None, gz, gtz, d_y, d_ty, sums, ctx.drop)
        d_gate = sums[0].to(gate.dtype).reshape(gate.shape)
        d_tgate = sums[1].to(tgate.dtype).reshape(tgate.shape) if (tgate is not None and gtz is not None) else None
        return (gz, d_y, d_gate, None, gtz if ctx.has_tx else None, d_ty if ty is not None else None, d_tgate, None)


class _GatedResidual(torch.autograd.Function):
    @staticmethod
    def forward(x, y, gate, mask, drop):
        z = torch.empty_like(y)
        _gate_launch(x, y, gate, mask, z, drop)
        return z

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, y, gate, mask, drop = inputs
        ctx.save_for_backward(y, gate, mask)
        ctx.drop = drop

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        y, gate, mask = ctx.saved_tensors
        B, S, C = y.shape
        g = g.contiguous()
        d_y = torch.empty_like(y)
        sums = torch.zeros(2, B, C, dtype=torch.float32, device=y.device)
        _gate_dual_launch(1, None, None, y, None, gate, None, mask, None, None, g, None, d_y, None, sums, ctx.drop)
        return g, d_y, sums[0].to(gate.dtype).reshape(gate.shape), None, None


def gated_residual(skip: torch.Tensor, branch: torch.Tensor, gate: torch.Tensor, p: float = 0.0, training: bool = False) -> torch.Tensor:
    """``dropout(branch * gate, p) + skip`` with ``gate`` (B, 1, C) or (B, C).  The dropout keep mask (scaled by
    1 / (1 - p)) is shared by primal, tangent and both backward passes: a tensor drawn here, or, inside
    :func:`dropout_seed`, regenerated by each kernel from the step's seed."""
    if not _usable(branch, skip, gate) or skip.shape != branch.shape:
        return F.dropout(branch * gate, p, training) + skip
    (xp, tx), (yp, ty), (gp, tg) = (fwAD.unpack_dual(t) for t in (skip, branch, gate))
    mask = drop = None
    if training and p > 0.0:
        if _Drop.seed is not None and _Drop.seed.device == yp.device:
            drop = (_Drop.seed, _Drop.calls, float(p))  # the kernels generate this call's mask themselves
            _Drop.calls += 1
        else:
            mask = torch.empty_like(yp).bernoulli_(1.0 - p).div_(1.0 - p)
    if tx is None and ty is None and tg is None:
        return _GatedResidual.apply(skip.contiguous(), branch.contiguous(), gate, mask, drop)
    z, tz = _GatedResidualDual.apply(xp.contiguous(), yp.contiguous(), gp, mask, tx, ty, tg, drop)
    return fwAD.make_dual(z, tz)


# ----------------------------------------------------------------------------------------------- linear layer
class _DualLinear(torch.autograd.Function):
    """(x, tx, w, b) -> (x w^T + b, tx w^T) as one autograd node: two GEMMs forward; backward two GEMMs for dx / dtx, two
    for dw (the second accumulating into the first through the GEMM's own epilogue) and one reduction for db - no
    additions of partial gradients and none of the scalings PyTorch's forward-mode formula for ``addmm`` carries."""

    @staticmethod
    def forward(x, tx, w, b):
        return F.linear(x, w, b), F.linear(tx, w)

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, tx, w, b = inputs
        ctx.save_for_backward(x, tx, w)
        ctx.has_bias = b is not None
        ctx.set_materialize_grads(False)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy, gty):
        x, tx, w = ctx.saved_tensors
        need_x, need_tx, need_w, need_b = ctx.needs_input_grad
        K, N = w.shape[1], w.shape[0]
        dx = dtx = dw = db = None
        if gy is not None:
            g2 = gy.reshape(-1, N)
            if need_x:
                dx = (g2 @ w).view(x.shape)
            if need_w:
                dw = g2.t() @ x.reshape(-1, K)
            if need_b and ctx.has_bias:
                db = g2.sum(0)
        if gty is not None:
            t2 = gty.reshape(-1, N)
            if need_tx:
                dtx = (t2 @ w).view(tx.shape)
            if need_w:
                dw = t2.t() @ tx.reshape(-1, K) if dw is None else torch.addmm(dw, t2.t(), tx.reshape(-1, K))
        return dx, dtx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``F.linear`` that keeps primal and tangent in one autograd node under forward-mode AD (weight and bias are
    parameters and carry no tangent where this is used).  Falls back to ``F.linear`` when no tangent is attached or the
    operands' dtypes differ (autocast then does its own casting)."""
    xp, tx = fwAD.unpack_dual(x)
    if tx is None or not x.is_cuda or xp.dtype != weight.dtype or (bias is not None and bias.dtype != weight.dtype):
        return F.linear(x, weight, bias)
    y, ty = _DualLinear.apply(xp, tx.to(xp.dtype), weight, bias)
    return fwAD.make_dual(y, ty)


# ----------------------------------------------------------------------------------------------- GELU (tanh form)
def _gelu_launch(mode, h, v, w, u, out, out2):
    lib = _lib.load()
    with torch.cuda.device(h.device):
        rc = lib.jvpattn_gelu_dual(mode, _ptr(h), _ptr(v), _ptr(w), _ptr(u), _ptr(out), _ptr(out2), h.numel(), _CODES[h.dtype], _stream(h))
    _lib.check(rc, "jvpattn_gelu_dual")


class _GeluDual(torch.autograd.Function):
    """(h, th) -> (gelu(h), gelu'(h) th) as one autograd node; backward: d_h = gelu'(h) gy + gelu''(h) th gty,
    d_th = gelu'(h) gty, one kernel for whichever cotangents arrive."""

    @staticmethod
    def forward(h, th):
        y, ty = torch.empty_like(h), torch.empty_like(h)
        _gelu_launch(3, h, th.contiguous(), None, None, y, ty)
        return y, ty

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(*inputs)
        ctx.set_materialize_grads(False)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy, gty):
        if gy is None and gty is None:
            return None, None
        h, th = ctx.saved_tensors
        d_h = torch.empty_like(h)
        if gty is None:
            _gelu_launch(1, h, gy.contiguous(), None, None, d_h, None)
            return d_h, None
        d_th = torch.empty_like(h)
        if gy is None:
            _gelu_launch(2, h, gty.contiguous(), th.contiguous(), None, d_th, d_h)
        else:
            _gelu_launch(4, h, gy.contiguous(), th.contiguous(), gty.contiguous(), d_h, d_th)
        return d_h, d_th


class _Gelu(torch.autograd.Function):
    @staticmethod
    def forward(h):
        y = torch.empty_like(h)
        _gelu_launch(0, h, None, None, None, y, None)
        return y

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(*inputs)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g):
        (h,) = ctx.saved_tensors
        d_h = torch.empty_like(h)
        _gelu_launch(1, h, g.contiguous(), None, None, d_h, None)
        return d_h


def gelu_tanh(h: torch.Tensor) -> torch.Tensor:
    """``F.gelu(h, approximate="tanh")`` (the MLP of semicat/net/duo.py:118-123) as one kernel for the primal, one for the
    tangent and one per cotangent; fp32 arithmetic, one rounding per output."""
    if not (h.is_cuda and h.dtype in _CODES and h.is_contiguous() and h.numel() % 8 == 0 and (h.storage_offset() * h.element_size()) % 16 == 0):
        return F.gelu(h, approximate="tanh")
    hp, th = fwAD.unpack_dual(h)
    if th is None:
        return _Gelu.apply(h)
    y, ty = _GeluDual.apply(hp, th)
    return fwAD.make_dual(y, ty)


# ----------------------------------------------------------------------------------------------- vocabulary-side head
def _rows3(t: torch.Tensor):
    """A (B, L, V) tensor with unit innermost stride and uniformly spaced rows, and that row spacing."""
    if t.stride(-1) != 1 or t.stride(0) != t.shape[1] * t.stride(1):
        t = t.contiguous()
    return t, t.stride(1)


def _head_launch(which, logits, tlogits, x, dt, ddt, lse, out, g, dl, dtl):
    B, L, V = logits.shape
    logits, ld = _rows3(logits)
    ldt = 0
    if tlogits is not None:
        tlogits, ldt = _rows3(tlogits)
    lib = _lib.load()
    with torch.cuda.device(logits.device):
        rc = lib.jvpattn_flow_map_head(which, _ptr(logits), _ptr(tlogits), ld, ldt, _ptr(x), _ptr(dt), _ptr(ddt), _ptr(lse), _ptr(out),
                                       _ptr(g), _ptr(dl), _ptr(dtl), B, L, V, _CODES[logits.dtype], _stream(logits))
    _lib.check(rc, "jvpattn_flow_map_head")


class _FlowHeadTangent(torch.autograd.Function):
    """dv = ddt (p - x) + dt p o (tlogits - sum(p tlogits)); backward = VJP of a cotangent on dv w.r.t. both logits."""

    @staticmethod
    def forward(logits, tlogits, x, dt, ddt, lse):
        dv = torch.empty(logits.shape, dtype=torch.float32, device=logits.device)
        _head_launch(1, logits, tlogits, x, dt, ddt, lse, dv, None, None, None)
        return dv

    @staticmethod
    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(*inputs)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, h):
        logits, tlogits, x, dt, ddt, lse = ctx.saved_tensors
        dl = torch.empty(logits.shape, dtype=logits.dtype, device=logits.device)
        dtl = torch.empty_like(dl)
        _head_launch(3, logits, tlogits, None, dt, ddt, lse, None, h.float().contiguous(), dl, dtl)
        return dl, dtl, None, None, None, None


class _FlowHead(torch.autograd.Function):
    @staticmethod
    def forward(logits, x, dt):
        B, L, V = logits.shape
        xst = torch.empty((B, L, V), dtype=torch.float32, device=logits.device)
        lse = torch.empty(B * L, dtype=torch.float32, device=logits.device)
        _head_launch(0, logits, None, x, dt, None, lse, xst, None, None, None)
        return xst, lse

    @staticmethod
    def setup_context(ctx, inputs, output):
        logits, x, dt = inputs
        _, lse = output
        ctx.mark_non_differentiable(lse)
        ctx.save_for_backward(logits, dt, lse)
        ctx.save_for_forward(logits, x, dt, lse)

    @staticmethod
    def jvp(ctx, tlogits, _tx, tdt):
        # x is data of the step (the interpolated input) and carries no tangent
        logits, x, dt, lse = ctx.saved_for_forward
        if tdt is None:
            tdt = torch.zeros_like(dt)
        if tlogits is None:
            tlogits = torch.zeros_like(logits)
        return _FlowHeadTangent.apply(logits, tlogits, x, dt, tdt.float().contiguous(), lse), None

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, g, _glse):
        logits, dt, lse = ctx.saved_tensors
        dl = torch.empty(logits.shape, dtype=logits.dtype, device=logits.device)
        _head_launch(2, logits, None, None, dt, None, lse, None, g.float().contiguous(), dl, None)
        return dl, None, None


def flow_map_head(logits: torch.Tensor, x: torch.Tensor, dt: torch.Tensor) -> torch.Tensor:
    """``x + dt[:, None, None] * (softmax(logits, -1) - x)`` in fp32: the flow map of semicat/models/semicat.py:210-229 from
    the denoiser's logits (B, L, V), the interpolated input ``x`` (fp32, treated as data: no tangent, no gradient) and the
    per-sample step ``dt`` (B,) (data as well; its forward-mode tangent is used, no gradient is formed for it).  Works
    under ``torch.func.jvp`` (the tangent is the flow map's derivative) and is reverse-mode differentiable with respect
    to the logits and their tangent."""
    usable = (logits.is_cuda and logits.dim() == 3 and logits.dtype in _CODES and x.dtype == torch.float32 and x.is_contiguous()
              and x.shape == logits.shape and logits.shape[-1] * (4 if logits.dtype == torch.bfloat16 else 8) <= 200 * 1024 - 64)
    if not usable:
        return x + dt.view(-1, 1, 1) * (logits.softmax(dim=-1) - x)
    xst, _ = _FlowHead.apply(logits, x, dt.float().contiguous())
    return xst
