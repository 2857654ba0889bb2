"""The autograd / forward-AD contract of semicat_b200.functional, exercised on CPU with oracle stand-ins
in place of the two library calls (see tests/standin.py)."""
import numpy as np
import pytest
import torch

import standin
from conftest import GRAD_NAMES, load_golden
from semicat_b200 import functional, ops


@pytest.fixture(autouse=True)
def _standins(monkeypatch):
    monkeypatch.setattr(ops, "jvp_attention_fwd", standin.fwd)
    monkeypatch.setattr(ops, "jvp_attention_bwd", standin.bwd)
    # fp32 on CPU is outside the product's dtype contract; the glue itself is dtype-agnostic
    monkeypatch.setattr(functional, "_validate", lambda q, k, v: None)


def _leaves(g, dtype=torch.float32):
    return [torch.from_numpy(g[n]).to(dtype).requires_grad_(True) for n in ("q", "k", "v", "tq", "tk", "tv")]


@pytest.mark.parametrize("case", ["c1_fp32", "ragged_bf16"])
@pytest.mark.parametrize("mode", ["both", "tan", "pri"])
def test_jvp_then_backward_matches_reference(case, mode):
    g = load_golden(case)
    leaves = _leaves(g)
    o, to = torch.func.jvp(functional.sdpa_jvp, tuple(leaves[:3]), tuple(leaves[3:]))
    np.testing.assert_allclose(o.detach().numpy(), g["o"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(to.detach().numpy(), g["od"], rtol=1e-4, atol=1e-4)
    outs, cots = [], []
    if mode in ("both", "pri"):
        outs.append(o); cots.append(torch.from_numpy(g["g_o"]))
    if mode in ("both", "tan"):
        outs.append(to); cots.append(torch.from_numpy(g["g_od"]))
    grads = torch.autograd.grad(outs, leaves, cots, allow_unused=True)
    for n, got in zip(GRAD_NAMES, grads):
        want = g[f"{n}_{mode}"]
        if got is None:
            assert np.abs(want).max() == 0
        else:
            np.testing.assert_allclose(got.numpy(), want, rtol=1e-4, atol=1e-4)


def test_safe_wrapper_layout_and_dtype():
    g = load_golden("c2_small_bf16")
    q, k, v, tq, tk, tv = (torch.from_numpy(g[n]).transpose(1, 2).contiguous() for n in ("q", "k", "v", "tq", "tk", "tv"))
    o, to = torch.func.jvp(functional.safe_sdpa_jvp, (q, k, v), (tq, tk, tv))
    assert o.shape == q.shape and o.dtype == torch.float32  # (B, S, H, D), caller's dtype
    # inputs are exactly representable in bf16, outputs were rounded to bf16 on the way back
    np.testing.assert_allclose(o.transpose(1, 2).numpy(), g["o"], rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(to.transpose(1, 2).numpy(), g["od"], rtol=2e-2, atol=1e-2)


def test_missing_tangent_is_zero():
    g = load_golden("selftest_1")
    q, k, v, tq, tk, tv = _leaves(g)
    f = lambda q_: functional.sdpa_jvp(q_, k.detach(), v.detach())
    o, to = torch.func.jvp(f, (q.detach(),), (tq.detach(),))
    f3 = functional.sdpa_jvp
    o3, to3 = torch.func.jvp(f3, (q.detach(), k.detach(), v.detach()),
                             (tq.detach(), torch.zeros_like(k), torch.zeros_like(v)))
    assert torch.allclose(o, o3) and torch.allclose(to, to3)


def test_double_backward_is_refused():
    g = load_golden("selftest_0")
    leaves = _leaves(g)
    o, to = torch.func.jvp(functional.sdpa_jvp, tuple(leaves[:3]), tuple(leaves[3:]))
    (dq,) = torch.autograd.grad(to.sum(), leaves[0], create_graph=True)
    with pytest.raises(RuntimeError):
        torch.autograd.grad(dq.sum(), leaves[1])


def test_no_cotangent_on_primal_output_skips_primal_backward(monkeypatch):
    calls = []
    real = standin.bwd
    monkeypatch.setattr(ops, "jvp_attention_bwd", lambda *a, **kw: (calls.append(a[8] is not None), real(*a, **kw))[1])
    g = load_golden("selftest_1")
    leaves = _leaves(g)
    o, to = torch.func.jvp(functional.sdpa_jvp, tuple(leaves[:3]), tuple(leaves[3:]))
    torch.autograd.grad(to.square().sum(), leaves)
    assert calls == [False]  # one launch, tangent cotangent only ("lag" objective)


def test_validate_messages(monkeypatch):
    monkeypatch.undo()  # the real _validate and the real library binding for this test
    q = torch.zeros(1, 1, 8, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="D_head must be >= 16"):
        functional.sdpa_jvp(q, q, q)
    q = torch.zeros(1, 1, 8, 32)
    with pytest.raises(TypeError):
        functional.sdpa_jvp(q, q, q)
    q = torch.zeros(1, 1, 8, 32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        torch.func.jvp(functional.sdpa_jvp, (q, q, q), (q, q, q))


def test_without_tangents_the_call_is_plain_attention():
    """No input carries a forward-mode tangent: the primal-only path runs (the reference hands back an
    uninitialised buffer there) and is reverse-mode differentiable."""
    g = load_golden("c1_fp32")
    q, k, v = (torch.from_numpy(g[n]).requires_grad_(True) for n in ("q", "k", "v"))
    o = functional.sdpa_jvp(q, k, v)
    np.testing.assert_allclose(o.detach().numpy(), g["o"], rtol=1e-4, atol=1e-4)
    grads = torch.autograd.grad(o, (q, k, v), torch.from_numpy(g["g_o"]))
    for n, got in zip(("dq", "dk", "dv"), grads):
        np.testing.assert_allclose(got.numpy(), g[f"{n}_pri"], rtol=1e-4, atol=1e-4)
    # the safe wrapper takes the same route, in the (B, S, H, D) layout (fp32 inputs pass through bf16 there)
    o2 = functional.safe_sdpa_jvp(*(t.detach().transpose(1, 2).contiguous() for t in (q, k, v)))
    assert o2.dtype == torch.float32
    np.testing.assert_allclose(o2.transpose(1, 2).numpy(), g["o"], rtol=2e-2, atol=2e-2)


def test_tangent_on_one_input_only_takes_the_jvp_path():
    g = load_golden("selftest_1")
    q, k, v, tq, tk, tv = _leaves(g)
    o, to = torch.func.jvp(lambda v_: functional.sdpa_jvp(q.detach(), k.detach(), v_), (v.detach(),), (tv.detach(),))
    o3, to3 = torch.func.jvp(functional.sdpa_jvp, (q.detach(), k.detach(), v.detach()),
                             (torch.zeros_like(q), torch.zeros_like(k), tv.detach()))
    assert torch.allclose(o, o3) and torch.allclose(to, to3)
