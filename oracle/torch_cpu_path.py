"""The reference's CPU recipe for the path, restated with torch: math attention under
``torch.func.jvp`` for (O, Od) and ``torch.autograd.grad`` for the six VJPs.

TEST INFRASTRUCTURE - see ``oracle/__init__.py``.  Never imported by the product.  It is the
second oracle for the parity tests (autodiff instead of closed-form algebra) and the thing that
``bench.py`` times as the CPU baseline.

Follows semicat/jvp_utils/ryu_triton.py:426-454 (``naive_multihead_attention_jvp``): scores =
Q K^T * scale, softmax over the last axis, times V, pushed through ``torch.func.jvp`` with the
three tangents.  The reference has no CPU backward of its own; differentiating this function with
autograd is what its kernels are derived from, and is what the fixtures under ``tests/golden/``
were generated with.
"""
from __future__ import annotations

import math
import os
import time

import torch


def attention_jvp(q, k, v, tq, tk, tv, scale=None):
    """(O, Od) by forward-mode AD through plain softmax attention.  Differentiable by autograd."""
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale

    def attend(q_, k_, v_):
        return torch.softmax(torch.matmul(q_, k_.transpose(-2, -1)) * scale, dim=-1) @ v_

    return torch.func.jvp(attend, (q, k, v), (tq, tk, tv))


def attention_jvp_with_grads(q, k, v, tq, tk, tv, g_o=None, g_od=None, scale=None):
    """Return (O, Od, [dq, dk, dv, dtq, dtk, dtv]); a ``None`` cotangent is left out of the VJP."""
    leaves = [x.detach().clone().requires_grad_(True) for x in (q, k, v, tq, tk, tv)]
    o, od = attention_jvp(*leaves, scale=scale)
    outs, cots = [], []
    if g_o is not None:
        outs.append(o)
        cots.append(g_o)
    if g_od is not None:
        outs.append(od)
        cots.append(g_od)
    grads = torch.autograd.grad(outs, leaves, cots, allow_unused=True)
    grads = [torch.zeros_like(x) if g is None else g for g, x in zip(grads, leaves)]
    return o.detach(), od.detach(), grads


def make_inputs(B, H, L, d, dtype=torch.float32, seed=0):
    """Seeded inputs with the value distribution of the microbenchmark configuration, as a tuple
    (q, k, v, tq, tk, tv, g_o, g_od)."""
    gen = torch.Generator().manual_seed(seed)
    mk = lambda s=1.0: (torch.randn(B, H, L, d, generator=gen) * s).to(dtype)
    return (mk(1.0 / math.sqrt(d)), mk(), mk(), mk(0.1), mk(0.1), mk(0.1), mk(), mk())


def reference_attention_jvp():
    """The reference's own ``naive_multihead_attention_jvp`` (semicat/jvp_utils/ryu_triton.py:426-454) from the
    copy that ``oracle/make_ref.py`` makes, or ``None`` where that copy (or triton, which the module imports) is
    absent.  Same call signature as :func:`attention_jvp` without ``scale``."""
    import oracle
    if oracle.import_reference() is None:
        return None
    try:
        from semicat.jvp_utils.ryu_triton import naive_multihead_attention_jvp
    except Exception:
        return None
    return naive_multihead_attention_jvp


def fwd_bwd(inputs, attention=None):
    """One forward (O, Od) and one backward (six VJPs, both cotangents) of ``attention`` (default: the
    restatement in this file) on the host."""
    fn = attention or attention_jvp
    leaves = [x.detach().clone().requires_grad_(True) for x in inputs[:6]]
    o, od = fn(*leaves)
    return torch.autograd.grad([o, od], leaves, [inputs[6], inputs[7]])


def time_fwd_bwd(B, H, L, d, dtype=torch.float32, repeats=3, seed=0, threads=None, attention=None):
    """Best-of-``repeats`` wall time in seconds of one fwd+bwd (both cotangents) on the host cores.  The inputs
    are drawn once, outside the timed region."""
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    inputs = make_inputs(B, H, L, d, dtype, seed)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fwd_bwd(inputs, attention)
        best = min(best, time.perf_counter() - t0)
    return best, threads
