"""GPU parity of the fused (primal, tangent) pointwise ops (``semicat_b200.dual_ops``) against the PyTorch expressions they
replace (semicat/net/duo.py:128-135, 157-160), evaluated in fp32 under ``torch.func.jvp`` and differentiated in reverse
mode with cotangents on both the primal and the tangent output."""
import types

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from semicat_b200 import _lib, dual_ops


def _manual_ln(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    xc = x - mu
    return xc * ((xc * xc).mean(-1, keepdim=True) + eps).rsqrt() * w + b


def _run(fn, primals, tangents, cots):
    leaves = [p.detach().clone().requires_grad_(True) for p in primals]
    tleaves = [None if t is None else t.detach().clone().requires_grad_(True) for t in tangents]
    idx = [i for i, t in enumerate(tleaves) if t is not None]

    def call(*dual):
        args = list(leaves)
        for i, d in zip(idx, dual):
            args[i] = d
        return fn(*args)

    y, ty = torch.func.jvp(call, tuple(leaves[i] for i in idx), tuple(tleaves[i] for i in idx))
    wrt = leaves + [t for t in tleaves if t is not None]
    grads = torch.autograd.grad([y, ty], wrt, [cots[0].to(y.dtype), cots[1].to(ty.dtype)], allow_unused=True)
    return y, ty, grads


def _close(a, b, what, rtol, atol):
    if a is None or b is None:
        assert a is None and b is None or (b is None and float(a.abs().max()) == 0) or (a is None and float(b.abs().max()) == 0), what
        return
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.3e} (ref max {b.abs().max().item():.3e})"


def _ln_inputs(B, S, C, dtype, seed=0, tx=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x, t = r(B, S, C).to(dtype), (r(B, S, C).to(dtype) if tx else None)
    mod = (r(B, 1, 6 * C) * 0.5).to(dtype)  # chunks of one projection, as in the denoiser: strided (B, 1, C) views
    tmod = (r(B, 1, 6 * C) * 0.5).to(dtype)
    sh, sc = mod[..., :C], mod[..., C:2 * C]
    tsh, tsc = tmod[..., :C], tmod[..., C:2 * C]
    norm = torch.nn.LayerNorm(C).cuda()
    with torch.no_grad():
        norm.weight.copy_(1.0 + 0.3 * r(C))
        norm.bias.copy_(0.2 * r(C))
    cots = (r(B, S, C), r(B, S, C))
    return x, t, sh, sc, tsh, tsc, norm, cots


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("shape", [(3, 40, 768), (2, 17, 256), (1, 128, 1024)])
def test_ln_modulate_fp32_matches_pytorch(shape, exact):
    B, S, C = shape
    x, t, sh, sc, tsh, tsc, norm, cots = _ln_inputs(B, S, C, torch.float32)
    w, b = norm.weight, norm.bias
    if exact:
        ref_fn = lambda x_, sh_, sc_, w_, b_: _manual_ln(x_, w_, b_, norm.eps) * (1.0 + sc_) + sh_
    else:  # PyTorch's own LayerNorm: its forward-mode formula holds mean / rstd constant when differentiated again
        ref_fn = lambda x_, sh_, sc_, w_, b_: F.layer_norm(x_, (C,), w_, b_, norm.eps) * (1.0 + sc_) + sh_

    def fused(x_, sh_, sc_, w_, b_):
        # the public entry point with the LayerNorm weight and bias as differentiable leaves
        stand_in = types.SimpleNamespace(weight=w_, bias=b_, eps=norm.eps, normalized_shape=(C,))
        return dual_ops.ln_modulate(x_, stand_in, sh_, sc_, exact=exact)

    before = _lib.launch_count()
    got = _run(fused, (x, sh, sc, w, b), (t, tsh, tsc, None, None), cots)
    # primal and tangent forward; one backward kernel per cotangent (the second adds to dx); one launch for the
    # gradients of the modulation tensors and the LayerNorm parameters
    assert _lib.launch_count() - before == 5
    want = _run(ref_fn, (x, sh, sc, w, b), (t, tsh, tsc, None, None), cots)
    _close(got[0], want[0], "y", 1e-4, 1e-4)
    _close(got[1], want[1], "ty", 1e-4, 1e-4)
    for name, a, r in zip(("dx", "dshift", "dscale", "dgamma", "dbeta", "dtx", "dtshift", "dtscale"), got[2], want[2]):
        _close(a, r, f"{name} (exact={exact})", 2e-3, 2e-3 * float(r.abs().max()))


def test_ln_modulate_bf16_and_missing_tangent_on_x():
    """bf16 tensors as under autocast; the first block of the denoiser sees a tangent on the modulation only."""
    B, S, C = 4, 64, 768
    for tx in (True, False):
        x, t, sh, sc, tsh, tsc, norm, cots = _ln_inputs(B, S, C, torch.bfloat16, seed=3, tx=tx)
        fused = lambda x_, sh_, sc_: dual_ops.ln_modulate(x_, norm, sh_, sc_)
        ref_fn = lambda x_, sh_, sc_: F.layer_norm(x_.float(), (C,), norm.weight, norm.bias, norm.eps) * (1.0 + sc_.float()) + sh_.float()
        got = _run(fused, (x, sh, sc), (t, tsh, tsc), cots)
        want = _run(ref_fn, (x, sh, sc), (t, tsh, tsc), cots)
        assert got[0].dtype == torch.bfloat16
        _close(got[0], want[0], "y", 2e-2, 2e-2)
        _close(got[1], want[1], "ty", 2e-2, 4e-2)
        for name, a, r in zip(("dx", "dshift", "dscale", "dtx", "dtshift", "dtscale") if tx else ("dx", "dshift", "dscale", "dtshift", "dtscale"),
                              got[2], want[2]):
            _close(a, r, f"{name} (tx={tx})", 3e-2, 3e-2 * float(r.float().abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_residual_matches_pytorch(dtype):
    B, S, C = 3, 50, 768
    g = torch.Generator(device="cuda").manual_seed(5)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g).to(dtype)
    x, y, tx, ty = r(B, S, C), r(B, S, C), r(B, S, C), r(B, S, C)
    gates, tgates = r(B, 1, 6 * C), r(B, 1, 6 * C)
    gate, tgate = gates[..., 2 * C:3 * C], tgates[..., 2 * C:3 * C]
    cots = (torch.randn(B, S, C, device="cuda", generator=g), torch.randn(B, S, C, device="cuda", generator=g))
    fused = lambda x_, y_, g_: dual_ops.gated_residual(x_, y_, g_, p=0.1, training=False)
    ref_fn = lambda x_, y_, g_: y_.float() * g_.float() + x_.float()
    before = _lib.launch_count()
    got = _run(fused, (x, y, gate), (tx, ty, tgate), cots)
    assert _lib.launch_count() - before == 2  # one kernel for (z, tz), one for both cotangents
    want = _run(ref_fn, (x, y, gate), (tx, ty, tgate), cots)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    _close(got[0], want[0], "z", tol, tol)
    _close(got[1], want[1], "tz", tol, 2 * tol)
    for name, a, rr in zip(("dx", "dy", "dgate", "dtx", "dty", "dtgate"), got[2], want[2]):
        _close(a, rr, name, tol, tol * float(rr.float().abs().max()) + 1e-6)


def test_gated_residual_dropout_uses_one_mask_for_primal_and_tangent():
    B, S, C = 2, 64, 512
    g = torch.Generator(device="cuda").manual_seed(9)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x, y, tx, ty, gate = r(B, S, C), r(B, S, C), r(B, S, C), r(B, S, C), r(B, 1, C)
    z, tz = torch.func.jvp(lambda x_, y_: dual_ops.gated_residual(x_, y_, gate, p=0.25, training=True), (x, y), (tx, ty))
    kept = (z - x) != 0
    frac = kept.float().mean().item()
    assert 0.70 < frac < 0.80, frac
    assert torch.allclose((z - x)[kept], (y * gate / 0.75)[kept], rtol=1e-5, atol=1e-6)
    assert torch.equal((tz - tx) != 0, kept)  # same mask
    assert torch.allclose((tz - tx)[kept], (ty * gate / 0.75)[kept], rtol=1e-5, atol=1e-6)


def test_unsupported_shapes_fall_back_to_pytorch():
    x = torch.randn(2, 8, 96, device="cuda")
    norm = torch.nn.LayerNorm(96).cuda()
    sh, sc = torch.randn(2, 1, 96, device="cuda"), torch.randn(2, 1, 96, device="cuda")
    before = _lib.launch_count()
    y = dual_ops.ln_modulate(x, norm, sh, sc)
    assert _lib.launch_count() == before
    assert torch.allclose(y, norm(x) * (1 + sc) + sh)
    z = dual_ops.gated_residual(x, x, sc)
    assert torch.allclose(z, x * sc + x)


@pytest.mark.parametrize("dtype,V,pad", [(torch.float32, 27, 0), (torch.bfloat16, 30522, 6), (torch.float32, 1000, 0)])
def test_flow_map_head_matches_pytorch(dtype, V, pad):
    """xst = x + dt (softmax(l) - x) and its derivative in t, with cotangents on both, against the PyTorch expression in
    fp32; the 30522-wide case reads the logits as a view of a padded (…, 30528) projection output, as the denoiser does."""
    B, L = 3, 5
    g = torch.Generator(device="cuda").manual_seed(2)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    lfull, tlfull = (2.0 * r(B, L, V + pad)).to(dtype), r(B, L, V + pad).to(dtype)
    l, tl = lfull[..., :V], tlfull[..., :V]
    x = r(B, L, V)
    t = torch.rand(B, device="cuda", generator=g) * 0.8 + 0.1
    s = torch.rand(B, device="cuda", generator=g) * t
    cots = (r(B, L, V), r(B, L, V))

    def run(fn):
        ll, tll = l.detach().clone().requires_grad_(True), tl.detach().clone().requires_grad_(True)
        tt = t.clone()

        def f(l_, t_):
            dt = (t_ - s) / (1.0 - s + 1e-8)
            return fn(l_, x, dt)

        xst, dv = torch.func.jvp(f, (ll, tt), (tll, torch.ones_like(tt)))
        grads = torch.autograd.grad([xst, dv], [ll, tll], list(cots))
        return xst, dv, grads

    before = _lib.launch_count()
    got = run(dual_ops.flow_map_head)
    assert _lib.launch_count() - before == 4
    want = run(lambda l_, x_, dt: x_ + dt.view(-1, 1, 1) * (l_.float().softmax(dim=-1) - x_))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    _close(got[0], want[0], "xst", tol, 1e-5)
    _close(got[1], want[1], "dv", tol, 1e-4 if dtype == torch.float32 else 1e-3)
    for name, a, b in zip(("dlogits", "dtlogits"), got[2], want[2]):
        _close(a, b, name, tol, (1e-5 if dtype == torch.float32 else 2e-2) * float(b.float().abs().max()))


def test_generated_dropout_masks_are_consistent_between_passes_and_have_the_right_rate():
    """Inside ``dropout_seed`` the kernels regenerate each call's keep mask from (seed, call number): forward, tangent and
    backward of one call must see the same mask, different calls and different steps different ones."""
    B, S, C, p = 4, 64, 768, 0.25
    dev = "cuda"
    x = torch.zeros(B, S, C, device=dev)
    ones = torch.ones(B, S, C, device=dev)
    gate = torch.ones(B, 1, C, device=dev)
    masks = []
    for _ in range(2):  # two "steps"
        with dual_ops.dropout_seed(torch.device(dev)):
            # call 0: primal-only path; z = mask, and d z / d y = mask
            y = ones.clone().requires_grad_(True)
            z = dual_ops.gated_residual(x, y, gate, p, True)
            (gy,) = torch.autograd.grad(z, y, ones)
            assert torch.equal(z.detach(), gy)
            # call 1: (primal, tangent) path with tangent 1 on the branch only: z = tz = mask, gradients = mask
            y2, t2 = ones.clone().requires_grad_(True), ones.clone().requires_grad_(True)
            z2, tz2 = torch.func.jvp(lambda y_: dual_ops.gated_residual(x, y_, gate, p, True), (y2,), (t2,))
            assert torch.equal(z2.detach(), tz2.detach())
            g_y2, g_t2 = torch.autograd.grad([z2, tz2], [y2, t2], [ones, ones])
            assert torch.equal(g_y2, z2.detach()) and torch.equal(g_t2, z2.detach())
            masks += [z.detach(), z2.detach()]
    for m in masks:
        kept = m != 0
        assert torch.allclose(m[kept], torch.full_like(m[kept], 1.0 / (1.0 - p)))
        assert abs(float((~kept).float().mean()) - p) < 0.01  # 196608 draws: sigma = 0.001
    for i in range(4):
        for j in range(i + 1, 4):
            assert not torch.equal(masks[i], masks[j])
    assert _lib.device_status() == 0
