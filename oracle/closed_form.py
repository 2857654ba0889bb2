"""Closed-form float64 restatement of the attention JVP and of its VJPs (numpy only).

TEST INFRASTRUCTURE - see ``oracle/__init__.py``.  Never imported by the product.

What the reference computes on this path, per (batch, head), non-causal, ``scale = 1/sqrt(d)``:

forward  (fused kernel, semicat/jvp_utils/ryu_triton.py:198-291)
    s   = scale * Q K^T                      P   = softmax_rows(s)        LSE = logsumexp_rows(s)
    sd  = scale * (Qd K^T + Q Kd^T)          MU  = rowsum(P * sd)
    O   = P V                                Od  = (P * (sd - MU)) V + P Vd

backward for cotangents gO (on O) and G (on Od)
    (semicat/jvp_utils/flash_jvp_backward.py:2012-2290 preprocess rows, :87-281 / :422-620 W1 terms,
     :762-989 dv / dvd, :1141-1433 / :1582-1863 W2 terms; semicat/jvp_utils/flash_attn_triton.py:406-685
     for the gO terms)
    delta0 = rowsum(gO * O)    delta = rowsum(G * O)    deltad = rowsum(G * Od)
    A0 = gO V^T                A = G V^T                Bm = G Vd^T              N = sd - MU
    W0 = scale * P * (A0 - delta0)
    W1 = scale * P * (A - delta)
    W2 = scale * P * ((A - delta) * N + Bm - deltad)
    dQd = W1 K               dKd = W1^T Q              dVd = P^T G
    dQ  = W1 Kd + (W2+W0) K  dK  = W1^T Qd + (W2+W0)^T Q   dV = (P*N)^T G + P^T gO

All functions take arrays shaped (B, H, L, d) (keys/values may use a different L) and compute
in float64 regardless of the input dtype.
"""
from __future__ import annotations

import math

import numpy as np


def _f64(x):
    return None if x is None else np.asarray(x, dtype=np.float64)


def _t(x):
    return np.swapaxes(x, -1, -2)


def forward(q, k, v, tq, tk, tv, scale=None):
    """Return (O, Od, LSE, MU) in float64.  LSE and MU have shape (B, H, Lq)."""
    q, k, v, tq, tk, tv = map(_f64, (q, k, v, tq, tk, tv))
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else float(scale)
    s = scale * (q @ _t(k))
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(axis=-1, keepdims=True)
    p = e / l
    lse = (m + np.log(l))[..., 0]
    sd = scale * (tq @ _t(k) + q @ _t(tk))
    mu = (p * sd).sum(axis=-1, keepdims=True)
    o = p @ v
    od = (p * (sd - mu)) @ v + p @ tv
    return o, od, lse, mu[..., 0]


def backward(q, k, v, tq, tk, tv, g_o=None, g_od=None, scale=None):
    """Return (dq, dk, dv, dtq, dtk, dtv) in float64 for cotangents ``g_o`` on O and ``g_od`` on Od.

    Either cotangent may be ``None`` (treated as zero), matching the three modes of the training
    objective: tangent-output cotangent only, primal-output cotangent only, or both.
    """
    q, k, v, tq, tk, tv, g_o, g_od = map(_f64, (q, k, v, tq, tk, tv, g_o, g_od))
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else float(scale)
    s = scale * (q @ _t(k))
    p = np.exp(s - s.max(axis=-1, keepdims=True))
    p /= p.sum(axis=-1, keepdims=True)
    sd = scale * (tq @ _t(k) + q @ _t(tk))
    mu = (p * sd).sum(axis=-1, keepdims=True)
    n = sd - mu
    pd = p * n
    o = p @ v
    od = pd @ v + p @ tv

    zq = np.zeros_like(q)
    zk = np.zeros_like(k)
    dq, dk, dv, dtq, dtk, dtv = zq.copy(), zk.copy(), zk.copy(), zq.copy(), zk.copy(), zk.copy()
    w_s = np.zeros_like(s)  # cotangent reaching s (times scale), from both outputs
    if g_od is not None:
        a = g_od @ _t(v)
        bm = g_od @ _t(tv)
        delta = (g_od * o).sum(axis=-1, keepdims=True)
        deltad = (g_od * od).sum(axis=-1, keepdims=True)
        w1 = scale * p * (a - delta)
        w_s = w_s + scale * p * ((a - delta) * n + bm - deltad)
        dtq = w1 @ k
        dtk = _t(w1) @ q
        dtv = _t(p) @ g_od
        dq = dq + w1 @ tk
        dk = dk + _t(w1) @ tq
        dv = dv + _t(pd) @ g_od
    if g_o is not None:
        a0 = g_o @ _t(v)
        delta0 = (g_o * o).sum(axis=-1, keepdims=True)
        w_s = w_s + scale * p * (a0 - delta0)
        dv = dv + _t(p) @ g_o
    dq = dq + w_s @ k
    dk = dk + _t(w_s) @ q
    return dq, dk, dv, dtq, dtk, dtv


def flops(B, H, Lq, Lk, d, mode="both"):
    """Algorithmic FLOPs of one pass: GEMM-unit = 2*Lq*Lk*d per head; softmax work not counted.

    fwd = 6 units; bwd = 15 (both cotangents), 13 (cotangent on Od only), 5 (cotangent on O only).
    """
    unit = 2.0 * B * H * Lq * Lk * d
    bwd_units = {"both": 15, "tangent": 13, "primal": 5}[mode]
    return {"fwd": 6 * unit, "bwd": bwd_units * unit, "total": (6 + bwd_units) * unit}
