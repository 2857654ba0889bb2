"""GPU: the public PyTorch entry points (sdpa_jvp / safe_sdpa_jvp under torch.func.jvp, then reverse
mode), the way the DiT denoiser calls them."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as G
    from semicat_b200 import _lib, safe_sdpa_jvp, sdpa_jvp


@pytest.mark.parametrize("mode", ["both", "tan", "pri"])
def test_sdpa_jvp_forward_ad_then_backward(mode):
    ins = G.rounded(G.synth(2, 4, 128, 128, 64, seed=3), torch.bfloat16)
    leaves = [torch.as_tensor(ins[n]).to("cuda", torch.bfloat16).requires_grad_(True) for n in G.IN_NAMES]
    before = _lib.launch_count()
    o, to = torch.func.jvp(sdpa_jvp, tuple(leaves[:3]), tuple(leaves[3:]))
    assert _lib.launch_count() - before == 1  # the fused forward
    outs, cots = [], []
    if mode in ("both", "pri"):
        outs.append(o); cots.append(torch.as_tensor(ins["g_o"]).to("cuda", torch.bfloat16))
    if mode in ("both", "tan"):
        outs.append(to); cots.append(torch.as_tensor(ins["g_od"]).to("cuda", torch.bfloat16))
    before = _lib.launch_count()
    grads = torch.autograd.grad(outs, leaves, cots, allow_unused=True)
    # one autograd node for (o, to): whichever cotangents arrive go through ONE backward call (row dots, query owner,
    # key owner), also when both do
    assert _lib.launch_count() - before == 3
    want = G.oracle(ins, mode)
    G.assert_close(o.detach().float().cpu().numpy(), want["o"], "o")
    G.assert_close(to.detach().float().cpu().numpy(), want["to"], "to")
    for n, g in zip(G.GRAD_NAMES, grads):
        if g is None:
            assert np.abs(want[n]).max() == 0
        else:
            G.assert_close(g.float().cpu().numpy(), want[n], n)
    assert _lib.device_status() == 0


def test_safe_wrapper_fp32_bshd_like_the_denoiser():
    """q, k arrive fp32 (rotary promotes), v bf16, all (B,S,H,D); result comes back fp32 (B,S,H,D)."""
    ins = G.rounded(G.synth(2, 4, 128, 128, 64, seed=4), torch.bfloat16)
    bshd = lambda n, dt: torch.as_tensor(ins[n]).transpose(1, 2).contiguous().to("cuda", dt).requires_grad_(True)
    q, k, tq, tk = (bshd(n, torch.float32) for n in ("q", "k", "tq", "tk"))
    v, tv = bshd("v", torch.bfloat16), bshd("tv", torch.bfloat16)
    o, to = torch.func.jvp(safe_sdpa_jvp, (q, k, v), (tq, tk, tv))
    assert o.dtype == torch.float32 and o.shape == q.shape
    want = G.oracle(ins, "tan")
    G.assert_close(o.detach().transpose(1, 2).float().cpu().numpy(), want["o"], "o")
    G.assert_close(to.detach().transpose(1, 2).float().cpu().numpy(), want["to"], "to")
    g_to = torch.as_tensor(ins["g_od"]).transpose(1, 2).contiguous().to("cuda", torch.float32)
    grads = torch.autograd.grad([to], [q, k, v, tq, tk, tv], [g_to])
    for n, g in zip(G.GRAD_NAMES, grads):
        G.assert_close(g.transpose(1, 2).float().cpu().numpy(), want[n], n)
    assert grads[0].dtype == torch.float32 and grads[2].dtype == torch.bfloat16


def test_output_buffers_keep_their_autograd_version():
    """The kernels fill tensors that autograd already handed out; they must do so without bumping the
    version counter, or the later backward would refuse to run."""
    ins = G.rounded(G.synth(1, 2, 128, 128, 64, seed=6), torch.bfloat16)
    leaves = [torch.as_tensor(ins[n]).to("cuda", torch.bfloat16).requires_grad_(True) for n in G.IN_NAMES]
    o, to = torch.func.jvp(sdpa_jvp, tuple(leaves[:3]), tuple(leaves[3:]))
    (o.float().square().sum() + to.float().square().sum()).backward()
    assert all(t.grad is not None and torch.isfinite(t.grad).all() for t in leaves)


def test_without_tangents_the_public_entry_points_run_plain_attention():
    """No forward-mode tangent on any input: sdpa_jvp / safe_sdpa_jvp go through the primal-only kernels and are
    reverse-mode differentiable (the reference returns an uninitialised buffer here, functional.py:286-287)."""
    ins = G.rounded(G.synth(2, 3, 256, 256, 64, seed=8), torch.bfloat16)
    q, k, v = (torch.as_tensor(ins[n]).to("cuda", torch.bfloat16).requires_grad_(True) for n in ("q", "k", "v"))
    before = _lib.launch_count()
    o = sdpa_jvp(q, k, v)
    assert _lib.launch_count() == before + 1
    want = G.oracle(ins, "pri")
    G.assert_close(o.detach().float().cpu().numpy(), want["o"], "o")
    grads = torch.autograd.grad(o, (q, k, v), torch.as_tensor(ins["g_o"]).to("cuda", torch.bfloat16))
    for n, g in zip(("dq", "dk", "dv"), grads):
        G.assert_close(g.float().cpu().numpy(), want[n], n)
    # (B, S, H, D) wrapper with fp32 inputs
    q2, k2, v2 = (t.detach().float().transpose(1, 2).contiguous() for t in (q, k, v))
    o2 = safe_sdpa_jvp(q2, k2, v2)
    assert o2.dtype == torch.float32 and o2.shape == q2.shape
    G.assert_close(o2.transpose(1, 2).cpu().numpy(), want["o"], "o (safe wrapper)")
    # a tangent on a single input still takes the fused path
    o3, to3 = torch.func.jvp(lambda v_: sdpa_jvp(q.detach(), k.detach(), v_), (v.detach(),), (v.detach(),))
    assert torch.equal(o3, o.detach())  # zero tangents on q, k; P V with tv = v gives Od = O
    G.assert_close(to3.float().cpu().numpy(), want["o"], "Od with tv = v equals O")
