"""GPU, model level, with the REFERENCE's own denoiser in the loop: the unmodified ``semicat.net.duo.DIT``
(semicat/net/duo.py:299-360) from the copy that ``oracle/make_ref.py`` makes, with ``hooks.install()`` putting this
library behind its ``safe_sdpa_jvp`` call (duo.py:141).  A self-distillation step (forward-mode JVP through the net,
semicat/models/semicat.py:112-167) is compared, loss and parameter gradients, with the same model running its
non-JVP branch (duo.py:143-152) under PyTorch's math attention, which supports forward-mode AD natively.

``lag``: the primal output is detached, only the cotangent of the tangent output flows (semicat.py:153-164).
``ecld``: the primal output takes a gradient too (semicat.py:131-151), so both backward paths of the attention run."""
import pytest
import torch
from torch.nn.attention import SDPBackend, sdpa_kernel

import oracle

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(oracle.reference_root() is None, reason="no copy of the reference package (oracle/make_ref.py)")]

if torch.cuda.is_available():
    from semicat_b200 import _lib, hooks, train_step


@pytest.fixture
def reference_dit():
    oracle.import_reference()
    duo = pytest.importorskip("semicat.net.duo")
    patched = hooks.install(strict=True)
    assert "semicat.net.duo" in patched
    yield duo
    hooks.uninstall()


def _flow_map(net, x, s, t, jvp_attention):
    """semicat/models/semicat.py:210-229"""
    dt = (t - s) / (1.0 - s + 1e-8)
    return x + dt.view(-1, 1, 1) * (net(x, s, t, jvp_attention=jvp_attention).softmax(dim=-1) - x)


def _step(net, xs, s, t, kind, jvp_attention):
    net.zero_grad(set_to_none=True)
    xst, dv = torch.func.jvp(lambda t_: _flow_map(net, xs, s, t_, jvp_attention), (t,), (torch.ones_like(t),))
    if kind == "lag":
        xst = xst.detach()
        with torch.no_grad():
            target = net(xst, t, t).softmax(dim=-1)
        loss = ((1.0 - t).view(-1, 1, 1) * dv - target + xst).pow(2).sum(dim=-1).mean()
    else:  # both outputs of every attention layer receive a cotangent
        loss = (xst + (1.0 - t).view(-1, 1, 1) * dv).clamp_min(1e-4).log().pow(2).sum(dim=-1).mean() + dv.pow(2).sum(dim=-1).mean()
    loss.backward()
    grads = torch.cat([p.grad.flatten() for p in net.parameters() if p.grad is not None])
    return loss.detach(), grads


@pytest.mark.parametrize("kind", ["lag", "ecld"])
def test_step_of_the_reference_denoiser_matches_math_attention(reference_dit, kind):
    torch.manual_seed(0)
    vocab, L, B = 48, 128, 6
    net = reference_dit.DIT(vocab_size=vocab, hidden_size=256, cond_dim=64, n_blocks=3, n_heads=4, dropout=0.0,
                            length=L).cuda()
    train_step.randomise_zero_init(net)  # zero-initialised gates would multiply every attention branch by zero
    g = torch.Generator(device="cuda").manual_seed(1)
    x1 = torch.randint(0, vocab, (B, L), device="cuda", generator=g)
    t = torch.rand(B, device="cuda", generator=g) * 0.8 + 0.1
    s = torch.rand(B, device="cuda", generator=g) * t
    xs = train_step.interpolate(torch.randn(B, L, vocab, device="cuda", generator=g), x1, s.view(-1, 1, 1))
    before = _lib.launch_count()
    loss_k, grad_k = _step(net, xs, s, t, kind, jvp_attention=True)
    launched = _lib.launch_count() - before
    assert launched >= 3 * 4, f"the reference's JVP branch did not reach the library ({launched} launches)"
    with sdpa_kernel([SDPBackend.MATH]):
        loss_m, grad_m = _step(net, xs, s, t, kind, jvp_attention=False)
    assert torch.isfinite(loss_k) and torch.isfinite(grad_k).all()
    assert abs(loss_k.item() - loss_m.item()) <= 2e-2 * abs(loss_m.item()) + 1e-4, (loss_k.item(), loss_m.item())
    rel = ((grad_k - grad_m).norm() / grad_m.norm()).item()
    assert rel < 3e-2, f"gradient relative L2 error {rel:.3e}"  # q, k, v pass through bf16 inside safe_sdpa_jvp
    assert _lib.device_status() == 0


def test_restated_denoiser_equals_the_reference_denoiser_on_the_gpu(reference_dit):
    """Same weights in ``train_step.DiT`` and in the reference ``DIT``, both through this library's kernels:
    the restatement that the training benchmark times is the reference's architecture."""
    torch.manual_seed(3)
    vocab, L, B = 40, 128, 4
    ref = reference_dit.DIT(vocab_size=vocab, hidden_size=128, cond_dim=32, n_blocks=2, n_heads=2, dropout=0.0, length=L).cuda()
    train_step.randomise_zero_init(ref)
    ours = train_step.DiT(vocab, hidden_size=128, cond_dim=32, n_blocks=2, n_heads=2, dropout=0.0, length=L).cuda()
    train_step.load_reference_state(ours, ref.state_dict())
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(B, L, vocab, device="cuda", generator=g)
    t = torch.rand(B, device="cuda", generator=g)
    s = torch.rand(B, device="cuda", generator=g) * t
    ones = torch.ones_like(t)
    want, want_t = torch.func.jvp(lambda t_: ref(x, s, t_, jvp_attention=True), (t,), (ones,))
    got, got_t = torch.func.jvp(lambda t_: ours(x, s, t_, attention="jvp"), (t,), (ones,))
    # identical kernels and weights; the restated block rotates and rounds q, k in one fused kernel where the reference
    # rotates in fp32 and rounds inside safe_sdpa_jvp (same values), and hands v over in bf16 either way
    assert torch.allclose(got, want, rtol=2e-3, atol=2e-3), (got - want).abs().max()
    assert torch.allclose(got_t, want_t, rtol=2e-2, atol=2e-2), (got_t - want_t).abs().max()
