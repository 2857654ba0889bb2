"""GPU parity of the fused vocabulary-side kernels (``semicat_b200.vocab_ops``) and of the dual-number GELU against the
PyTorch expressions of the reference's training step (semicat/models/semicat.py:70-85, 89-110, 112-167, 210-229;
semicat/net/duo.py:118-123), evaluated in fp32 on the same 16-bit inputs."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from semicat_b200 import _lib, dual_ops, train_step, vocab_ops


def _case(V, B=3, L=5, dtype=torch.bfloat16, seed=0, padded_noise=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    Vp = vocab_ops.padded(V)
    width = Vp if padded_noise else V
    x0 = torch.randn(B, L, width, device="cuda", generator=g)[..., :V]
    ids = torch.randint(0, V, (B, L), device="cuda", generator=g)
    t = torch.rand(B, device="cuda", generator=g)
    s = torch.rand(B, device="cuda", generator=g) * t
    mk = lambda scale: (torch.randn(B, L, Vp, device="cuda", generator=g) * scale).to(dtype)
    # the padding columns of the GEMM output hold zeros in the model; make them loud here so that a kernel that read
    # them would fail
    l, tl, lt = mk(2.0), mk(1.0), mk(2.0)
    for z in (l, tl, lt):
        z[..., V:] = 7.0
    return x0, ids, s, t, l, tl, lt


def _onehot_mix(x0, ids, w):
    return (1.0 - w.view(-1, 1, 1)) * x0 + w.view(-1, 1, 1) * F.one_hot(ids, x0.shape[-1]).float()


@pytest.mark.parametrize("V,padded_noise", [(1003, True), (1003, False), (1024, True), (30522, True)])
def test_interpolate_cast(V, padded_noise):
    x0, ids, s, t, *_ = _case(V, padded_noise=padded_noise)
    out = vocab_ops.interpolate_cast(x0, ids, t)
    assert out.shape[-1] == vocab_ops.padded(V) and out.dtype == torch.bfloat16
    want = _onehot_mix(x0, ids, t)
    assert float(out[..., V:].abs().max()) == 0.0 if out.shape[-1] > V else True
    assert torch.allclose(out[..., :V].float(), want, rtol=2 ** -7, atol=1e-6)


@pytest.mark.parametrize("V,dtype", [(1003, torch.bfloat16), (30522, torch.bfloat16), (777, torch.float32)])
def test_flow_map_input(V, dtype):
    x0, ids, s, t, l, *_ = _case(V, dtype=dtype)
    xst, lse = vocab_ops.flow_map_input(l, x0, ids, s, t)
    lf = l[..., :V].float()
    xs = _onehot_mix(x0, ids, s)
    dt = ((t - s) / (1.0 - s + 1e-8)).view(-1, 1, 1)
    want = xs + dt * (lf.softmax(-1) - xs)
    tol = 2 ** -7 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(xst[..., :V].float(), want, rtol=tol, atol=1e-5)
    assert torch.allclose(lse.view(l.shape[:2]), lf.logsumexp(-1), rtol=1e-5, atol=1e-5)
    if xst.shape[-1] > V:
        assert float(xst[..., V:].abs().max()) == 0.0


@pytest.mark.parametrize("V,eps", [(1003, 0.0), (1003, 0.1), (30522, 0.0)])
def test_cross_entropy_padded(V, eps):
    _, ids, _, _, l, *_ = _case(V)
    lp = l.clone().requires_grad_(True)
    loss = vocab_ops.cross_entropy_padded(lp, ids, V, eps)
    (g,) = torch.autograd.grad(loss * 3.0, lp)
    lf = l[..., :V].float().requires_grad_(True)
    want = F.cross_entropy(lf.reshape(-1, V), ids.reshape(-1), label_smoothing=eps)
    (gw,) = torch.autograd.grad(want * 3.0, lf)
    assert abs(loss.item() - want.item()) <= 1e-5 * abs(want.item()) + 1e-6
    assert torch.allclose(g[..., :V].float(), gw, rtol=2 ** -7, atol=1e-7)
    if g.shape[-1] > V:
        assert float(g[..., V:].abs().max()) == 0.0


def _sd_loss_reference(l, tl, lt, x0, ids, s, t):
    """The reference's expressions: flow map, its t-derivative by the product rule, squared error (fp32)."""
    p = l.softmax(-1)
    xs = _onehot_mix(x0, ids, s)
    dt = ((t - s) / (1.0 - s + 1e-8)).view(-1, 1, 1)
    ddt = (1.0 / (1.0 - s + 1e-8)).view(-1, 1, 1)
    xst = (xs + dt * (p - xs)).detach()
    dv = ddt * (p - xs) + dt * p * (tl - (p * tl).sum(-1, keepdim=True))
    return ((1.0 - t).view(-1, 1, 1) * dv - lt.softmax(-1) + xst).pow(2).sum(-1).mean()


@pytest.mark.parametrize("V,dtype", [(1003, torch.bfloat16), (30522, torch.bfloat16), (777, torch.float32)])
def test_sd_lag_loss_value_and_gradients(V, dtype):
    x0, ids, s, t, l, tl, lt = _case(V, dtype=dtype)
    lp, tlp = l.clone().requires_grad_(True), tl.clone().requires_grad_(True)
    _, lse = vocab_ops.flow_map_input(lp, x0, ids, s, t)
    loss = vocab_ops.sd_lag_loss(lp, tlp, lt, x0, ids, s, t, lse)
    g_l, g_tl = torch.autograd.grad(loss * 2.0, [lp, tlp])
    lf, tlf = l[..., :V].float().requires_grad_(True), tl[..., :V].float().requires_grad_(True)
    want = _sd_loss_reference(lf, tlf, lt[..., :V].float(), x0, ids, s, t)
    w_l, w_tl = torch.autograd.grad(want * 2.0, [lf, tlf])
    assert abs(loss.item() - want.item()) <= 1e-4 * abs(want.item()) + 1e-6
    rt = 2 ** -7 if dtype == torch.bfloat16 else 1e-4
    for got, ref, name in ((g_l, w_l, "d logits"), (g_tl, w_tl, "d tlogits")):
        scale = float(ref.abs().max())
        assert torch.allclose(got[..., :V].float(), ref, rtol=rt, atol=rt * scale * 0.05 + 1e-9), name
        if got.shape[-1] > V:
            assert float(got[..., V:].abs().max()) == 0.0
    assert _lib.device_status() == 0


def test_sd_lag_loss_agrees_with_jvp_of_the_flow_map():
    """The kernel's dv is the forward-mode derivative of the flow map: check against torch.func.jvp of the reference's
    expression with logits that depend on t."""
    V = 523
    x0, ids, s, t, l, tl, lt = _case(V, dtype=torch.float32)
    lf, tlf, ltf = l[..., :V], tl[..., :V], lt[..., :V]

    def flow(_t):
        logits = lf + (_t - t).view(-1, 1, 1) * tlf  # d logits / d t = tlf at _t = t
        dt = ((_t - s) / (1.0 - s + 1e-8)).view(-1, 1, 1)
        xs = _onehot_mix(x0, ids, s)
        return xs + dt * (logits.softmax(-1) - xs)

    xst, dv = torch.func.jvp(flow, (t,), (torch.ones_like(t),))
    want = ((1.0 - t).view(-1, 1, 1) * dv - ltf.softmax(-1) + xst).pow(2).sum(-1).mean()
    _, lse = vocab_ops.flow_map_input(l, x0, ids, s, t)
    got = vocab_ops.sd_lag_loss(l, tl, lt, x0, ids, s, t, lse)
    assert abs(got.item() - want.item()) <= 1e-4 * abs(want.item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gelu_tanh_dual(dtype):
    g = torch.Generator(device="cuda").manual_seed(3)
    h = (torch.randn(4, 33, 256, device="cuda", generator=g) * 2.0).to(dtype)
    th = torch.randn(4, 33, 256, device="cuda", generator=g).to(dtype)
    gy, gty = (torch.randn(4, 33, 256, device="cuda", generator=g).to(dtype) for _ in range(2))

    def run(fn, hh, tt, cast):
        hh, tt = hh.detach().clone().requires_grad_(True), tt.detach().clone().requires_grad_(True)
        y, ty = torch.func.jvp(fn, (hh,), (tt,))
        grads = torch.autograd.grad([y, ty], [hh, tt], [gy.to(cast), gty.to(cast)])
        return y, ty, grads

    before = _lib.launch_count()
    y, ty, (d_h, d_th) = run(dual_ops.gelu_tanh, h, th, dtype)
    assert _lib.launch_count() - before == 2  # one kernel for (y, ty), one for both cotangents
    ry, rty, (rd_h, rd_th) = run(lambda z: F.gelu(z, approximate="tanh"), h.double(), th.double(), torch.float64)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    for got, ref, name in ((y, ry, "y"), (ty, rty, "ty"), (d_h, rd_h, "d h"), (d_th, rd_th, "d th")):
        assert torch.allclose(got.double(), ref, rtol=tol, atol=tol), name


@pytest.mark.parametrize("autocast", [None, torch.bfloat16])
def test_training_step_with_fused_vocabulary_side_matches_plain_path(autocast):
    """Model level: vocabulary large enough for the fused kernels (and not a multiple of 8), against the plain-formula path."""
    torch.manual_seed(0)
    vocab, B, L = 1003, 8, 128
    net = train_step.DiT(vocab, hidden_size=128, cond_dim=32, n_blocks=2, n_heads=2, dropout=0.0, length=L).cuda()
    train_step.randomise_zero_init(net)
    g = torch.Generator(device="cuda").manual_seed(1)
    x1 = torch.randint(0, vocab, (B, L), device="cuda", generator=g)
    noise = train_step.draw_noise(x1, vocab, generator=g)

    def step(attention):
        net.zero_grad(set_to_none=True)
        vf, sd = train_step.model_step(net, x1, noise, sd_prop=0.25, jvp_attention=attention, autocast_dtype=autocast,
                                       primal_attention="lib" if attention != "math" else "math")
        (vf + sd).backward()
        return vf.detach(), sd.detach(), torch.cat([p.grad.flatten() for p in net.parameters() if p.grad is not None])

    before = _lib.launch_count()
    vf_k, sd_k, grad_k = step("jvp")
    assert _lib.launch_count() - before > 20
    vf_m, sd_m, grad_m = step("math")
    tol = 2e-2 if autocast is None else 5e-2
    assert abs(vf_k.item() - vf_m.item()) <= tol * abs(vf_m.item())
    assert abs(sd_k.item() - sd_m.item()) <= tol * abs(sd_m.item()) + 1e-4
    rel = (grad_k - grad_m).norm() / grad_m.norm()
    assert rel < (3e-2 if autocast is None else 8e-2), f"gradient relative L2 error {rel:.3e}"
    assert _lib.device_status() == 0
