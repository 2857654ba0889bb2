"""Helpers for the GPU parity tests: run the library through its C ABI (via semicat_b200.ops) on torch
CUDA tensors, with canary-guarded outputs, and compare against the CPU oracle."""
import numpy as np
import torch

from oracle import closed_form
from semicat_b200 import ops

IN_NAMES = ("q", "k", "v", "tq", "tk", "tv")
GRAD_NAMES = ("dq", "dk", "dv", "dtq", "dtk", "dtv")
RTOL, ATOL = 2e-2, 1e-2  # bf16/fp16 bar: |x - ref| <= 1e-2 + 2e-2 |ref| against the fp32/fp64 oracle
CANARY = 12288.0  # exactly representable in bf16 and fp16


def assert_close(got, want, what, rtol=RTOL, atol=ATOL):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    err = np.abs(got - want)
    bad = err > atol + rtol * np.abs(want)
    assert not bad.any(), (f"{what}: {int(bad.sum())}/{bad.size} elements out of tolerance, max abs err "
                           f"{err.max():.4g} at {np.unravel_index(err.argmax(), err.shape)}")


def place(x, dtype, layout, device="cuda"):
    """Put a (B,H,L,D) host array on the device as a (B,H,L,D) view with the requested memory layout."""
    t = torch.as_tensor(np.asarray(x), dtype=torch.float32).to(device=device, dtype=dtype)
    if layout == "bhld":
        return t.contiguous()
    if layout == "bshd":  # the model's layout: (B,S,H,D)-contiguous memory viewed as (B,H,S,D)
        return t.transpose(1, 2).contiguous().transpose(1, 2)
    if layout == "padded":  # row pitch larger than D, 16-byte aligned
        B, H, L, D = t.shape
        buf = torch.zeros(B, H, L, D + 8, dtype=dtype, device=device)
        buf[..., :D] = t
        return buf[..., :D]
    raise ValueError(layout)


def guarded_like(t):
    """Output buffer with the strides of ``t`` embedded in a larger canary-filled allocation."""
    n = t.untyped_storage().nbytes() // t.element_size()
    pad = 256
    buf = torch.full((n + 2 * pad,), CANARY, dtype=t.dtype, device=t.device)
    view = buf[pad:pad + n].as_strided(t.shape, t.stride(), pad + t.storage_offset())
    return buf, view, pad, n


def check_canaries(buf, pad, n, what):
    head, tail = buf[:pad].float(), buf[pad + n:].float()
    assert bool((head == CANARY).all()) and bool((tail == CANARY).all()), f"{what}: wrote outside its buffer"


def run(inputs, dtype=torch.bfloat16, kernels=ops.KERNELS_AUTO, layout="bhld", mode="both", scale=None):
    """Forward + backward through the C ABI.  Returns dict of float32 numpy arrays."""
    dev = "cuda"
    t = {n: place(inputs[n], dtype, layout) for n in IN_NAMES}
    B, H, Lq, D = t["q"].shape
    o_buf, o, pad, n_o = guarded_like(t["q"])
    to_buf, to, _, _ = guarded_like(t["q"])
    stat = ops.stat_len(Lq)
    lse = torch.full((B, H, stat), CANARY, dtype=torch.float32, device=dev)
    mu = torch.full((B, H, stat), CANARY, dtype=torch.float32, device=dev)
    ops.jvp_attention_fwd(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], o, to, lse, mu, scale=scale, kernels=kernels)
    out = {"o": o, "to": to, "lse": lse[..., :Lq], "mu": mu[..., :Lq]}
    check_canaries(o_buf, pad, n_o, "o")
    check_canaries(to_buf, pad, n_o, "to")
    if Lq < stat:
        assert bool((lse[..., Lq:] == CANARY).all()) and bool((mu[..., Lq:] == CANARY).all()), "statistics tail overwritten"
    if mode is not None:
        g_o = place(inputs["g_o"], dtype, layout) if mode in ("both", "pri") else None
        g_to = place(inputs["g_od"], dtype, layout) if mode in ("both", "tan") else None
        guards = {}
        for gn, src in zip(GRAD_NAMES, IN_NAMES):
            if mode == "pri" and gn.startswith("dt"):
                guards[gn] = (None, None, 0, 0)
            else:
                guards[gn] = guarded_like(t[src])
        views = [guards[gn][1] for gn in GRAD_NAMES]
        if mode == "pri":
            ops.jvp_attention_bwd(t["q"], t["k"], t["v"], None, None, None, o, None, g_o, None, lse, None,
                                  *views, scale=scale, kernels=kernels)
        else:
            ops.jvp_attention_bwd(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], o, to, g_o, g_to, lse, mu,
                                  *views, scale=scale, kernels=kernels)
        for gn in GRAD_NAMES:
            buf, view, p, n = guards[gn]
            if buf is not None:
                check_canaries(buf, p, n, gn)
                out[gn] = view
    torch.cuda.synchronize()
    return {k_: v_.detach().float().cpu().numpy() for k_, v_ in out.items()}


def rounded(inputs, dtype):
    """The inputs as the kernel sees them: rounded to the compute dtype, back in float32."""
    r = {}
    for n, x in inputs.items():
        r[n] = torch.as_tensor(np.asarray(x), dtype=torch.float32).to(dtype).float().numpy()
    return r


def oracle(inputs, mode="both", scale=None):
    ins = [inputs[n] for n in IN_NAMES]
    o, od, lse, mu = closed_form.forward(*ins, scale=scale)
    out = {"o": o, "to": od, "lse": lse, "mu": mu}
    if mode is not None:
        g = closed_form.backward(*ins, g_o=inputs["g_o"] if mode in ("both", "pri") else None,
                                 g_od=inputs["g_od"] if mode in ("both", "tan") else None, scale=scale)
        out.update(dict(zip(GRAD_NAMES, g)))
    return out


def synth(B, H, Lq, Lk, D, seed=0, q_scale=None, t_scale=0.1):
    """Seeded synthetic inputs with the value distribution of the microbenchmark configuration:
    q ~ N(0,1)/sqrt(D), k, v ~ N(0,1), tangents ~ 0.1 N(0,1), cotangents ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    q_scale = 1.0 / np.sqrt(D) if q_scale is None else q_scale
    f = lambda L, s: (rng.standard_normal((B, H, L, D)) * s).astype(np.float32)
    return {"q": f(Lq, q_scale), "k": f(Lk, 1.0), "v": f(Lk, 1.0), "tq": f(Lq, t_scale), "tk": f(Lk, t_scale),
            "tv": f(Lk, t_scale), "g_o": f(Lq, 1.0), "g_od": f(Lq, 1.0)}


def compare(got, want, mode, label):
    for n in ("o", "to"):
        assert_close(got[n], want[n], f"{label}:{n}")
    assert_close(got["lse"], want["lse"], f"{label}:lse", rtol=1e-3, atol=2e-3)
    assert_close(got["mu"], want["mu"], f"{label}:mu", rtol=2e-2, atol=1e-2)
    if mode is not None:
        for n in GRAD_NAMES:
            if n in got:
                assert_close(got[n], want[n], f"{label}:{n}")


def oracle_rows(inputs, mode="both", scale=None, rows=1024):
    """The fp64 oracle evaluated in chunks of query rows, for sequences whose (L x L) score matrices would not
    fit at once.  Attention rows are independent, so outputs and query-side gradients are per chunk and the
    key-side gradients are sums over chunks."""
    Lq = inputs["q"].shape[2]
    parts = []
    acc = None
    for r0 in range(0, Lq, rows):
        sl = slice(r0, min(r0 + rows, Lq))
        sub = {n: (x[:, :, sl] if n in ("q", "tq", "g_o", "g_od") else x) for n, x in inputs.items()}
        out = oracle(sub, mode, scale)
        parts.append(out)
        if mode is not None:
            ksum = {n: out[n] for n in ("dk", "dv", "dtk", "dtv")}
            acc = ksum if acc is None else {n: acc[n] + ksum[n] for n in acc}
    res = {n: np.concatenate([p[n] for p in parts], axis=2) for n in ("o", "to", "lse", "mu")}
    if mode is not None:
        res.update({n: np.concatenate([p[n] for p in parts], axis=2) for n in ("dq", "dtq")})
        res.update(acc)
    return res
