"""GPU, model level: the DiT flow-map ("lag") training step with the JVP-attention kernels against the same
step with plain-formula attention (which supports forward-mode AD natively) on the same weights and noise."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from semicat_b200 import _lib, train_step


def _setup(seed=0, B=8, L=128, vocab=37):
    torch.manual_seed(seed)
    net = train_step.DiT(vocab, hidden_size=128, cond_dim=32, n_blocks=2, n_heads=2, dropout=0.0, length=L).cuda()
    train_step.randomise_zero_init(net)  # a fresh DiT multiplies its attention branch by zero gates
    g = torch.Generator(device="cuda").manual_seed(seed + 1)
    x1 = torch.randint(0, vocab, (B, L), device="cuda", generator=g)
    noise = train_step.draw_noise(x1, vocab, generator=g)
    return net, x1, noise


def _step(net, x1, noise, attention, sd_prop):
    net.zero_grad(set_to_none=True)
    vf, sd = train_step.model_step(net, x1, noise, sd_prop=sd_prop, jvp_attention=attention, autocast_dtype=None)
    loss = train_step.total_loss(vf, sd)
    loss.backward()
    flat = torch.cat([p.grad.flatten() for p in net.parameters() if p.grad is not None])
    return loss.detach(), flat


@pytest.mark.parametrize("sd_prop", [0.25, 1.0])
def test_lag_step_matches_plain_attention(sd_prop):
    net, x1, noise = _setup()
    before = _lib.launch_count()
    loss_k, grad_k = _step(net, x1, noise, "jvp", sd_prop)
    assert _lib.launch_count() - before >= 2 * 4, "the JVP branch did not go through the library"
    loss_m, grad_m = _step(net, x1, noise, "math", sd_prop)
    assert torch.isfinite(loss_k) and torch.isfinite(grad_k).all()
    assert abs(loss_k.item() - loss_m.item()) <= 2e-2 * abs(loss_m.item()) + 1e-4
    rel = (grad_k - grad_m).norm() / grad_m.norm()
    assert rel < 3e-2, f"gradient relative L2 error {rel:.3e}"  # q, k, v pass through bf16 inside safe_sdpa_jvp
    assert _lib.device_status() == 0


def test_attention_output_comes_back_in_the_models_layout():
    from semicat_b200 import safe_sdpa_jvp
    q = torch.randn(2, 128, 4, 64, device="cuda")
    o, to = torch.func.jvp(safe_sdpa_jvp, (q, q, q), (q, q, q))
    assert o.shape == q.shape and o.is_contiguous() and to.is_contiguous()  # (B, S, H, D): reshape to (B, S, H*D) is a view
