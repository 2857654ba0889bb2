"""Test-only stand-ins for the two library calls, computed with the CPU oracle.

They let the autograd glue of ``semicat_b200.functional`` be exercised without a GPU: the tests
monkeypatch ``semicat_b200.ops.jvp_attention_fwd`` / ``jvp_attention_bwd`` with these.  They are never
installed by the product; they write results through ``.data`` the way a raw-pointer kernel would,
i.e. without touching autograd version counters.
"""
import torch

from oracle import closed_form


def _np(t):
    return None if t is None else t.detach().double().cpu().numpy()


def _put(dst, arr):
    dst.data.copy_(torch.from_numpy(arr).to(dst.dtype))


def fwd(q, k, v, tq, tk, tv, o, to, lse, mu, li=None, scale=None, kernels=0):
    primal_only = tq is None
    if primal_only:
        tq, tk, tv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    O, Od, LSE, MU = closed_form.forward(*map(_np, (q, k, v, tq, tk, tv)), scale=scale)
    _put(o, O)
    L = q.shape[2]
    lse.data[..., :L] = torch.from_numpy(LSE).float()
    if not primal_only:
        _put(to, Od)
        mu.data[..., :L] = torch.from_numpy(MU).float()


def bwd(q, k, v, tq, tk, tv, o, to, g_o, g_to, lse, mu, dq, dk, dv, dtq=None, dtk=None, dtv=None,
        scale=None, kernels=0, workspace=None):
    if tq is None:
        tq, tk, tv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    grads = closed_form.backward(*map(_np, (q, k, v, tq, tk, tv)), g_o=_np(g_o), g_od=_np(g_to), scale=scale)
    for dst, g in zip((dq, dk, dv, dtq, dtk, dtv), grads):
        if dst is not None:
            _put(dst, g)
