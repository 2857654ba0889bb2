"""The restated denoiser (semicat_b200/train_step.py) against the reference's own ``DIT`` (semicat/net/duo.py:299-360)
on identical weights, on the CPU: forward values and the forward-mode tangent with respect to ``t``.

Needs the unmodified copy of the reference package that ``oracle/make_ref.py`` makes; skipped where it is absent."""
import pytest
import torch
from torch.nn.attention import SDPBackend, sdpa_kernel

import oracle
from semicat_b200 import train_step

pytestmark = pytest.mark.skipif(oracle.reference_root() is None, reason="no copy of the reference package (oracle/make_ref.py)")


def _pair(embed_type, vocab, seed=0):
    oracle.import_reference()
    duo = pytest.importorskip("semicat.net.duo")
    torch.manual_seed(seed)
    ref = duo.DIT(vocab_size=vocab, hidden_size=64, cond_dim=32, n_blocks=2, n_heads=2, dropout=0.0, length=16,
                  embed_type=embed_type)
    train_step.randomise_zero_init(ref, seed=seed)  # zero-initialised gates would hide every attention branch
    ours = train_step.DiT(vocab, hidden_size=64, cond_dim=32, n_blocks=2, n_heads=2, dropout=0.0, length=16,
                          embed_type=embed_type)
    train_step.load_reference_state(ours, ref.state_dict())
    return ref.eval(), ours.eval()


def _inputs(vocab, B=3, L=16, seed=1):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, L, vocab, generator=g)
    t = torch.rand(B, generator=g)
    s = torch.rand(B, generator=g) * t
    return x, s, t


@pytest.mark.parametrize("embed_type,vocab", [("naive", 50), ("rms", 27)])
def test_forward_equals_the_reference_model(embed_type, vocab):
    ref, ours = _pair(embed_type, vocab)
    x, s, t = _inputs(vocab)
    with torch.no_grad():
        want = ref(x, s, t, jvp_attention=False)
        got_sdpa = ours(x, s, t, attention="sdpa")
        got_math = ours(x, s, t, attention="math")
    assert torch.allclose(got_sdpa, want, rtol=1e-4, atol=1e-5), (got_sdpa - want).abs().max()
    assert torch.allclose(got_math, want, rtol=1e-4, atol=1e-5), (got_math - want).abs().max()


@pytest.mark.parametrize("embed_type,vocab", [("naive", 50), ("rms", 27)])
def test_tangent_in_t_equals_the_reference_model(embed_type, vocab):
    """d/dt of the network output by forward-mode AD, the derivative the self-distillation step takes
    (semicat/models/semicat.py:153-157).  The reference side runs its non-JVP branch under the math SDPA backend,
    the one PyTorch attention implementation that supports forward-mode AD on the CPU."""
    ref, ours = _pair(embed_type, vocab)
    x, s, t = _inputs(vocab)
    ones = torch.ones_like(t)
    with sdpa_kernel([SDPBackend.MATH]):
        want, want_t = torch.func.jvp(lambda t_: ref(x, s, t_, jvp_attention=False), (t,), (ones,))
    got, got_t = torch.func.jvp(lambda t_: ours(x, s, t_, attention="math"), (t,), (ones,))
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    assert torch.allclose(got_t, want_t, rtol=1e-3, atol=1e-4), (got_t - want_t).abs().max()


def test_state_mapping_rejects_a_different_architecture():
    ref, _ = _pair("naive", 50)
    other = train_step.DiT(50, hidden_size=64, cond_dim=32, n_blocks=3, n_heads=2, dropout=0.0, length=16)
    with pytest.raises(KeyError):
        train_step.load_reference_state(other, ref.state_dict())
