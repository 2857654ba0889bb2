"""GPU parity of the fused rotary + cast helper (``jvpattn_rotary_cast`` through ``semicat_b200.rotary``).

Oracle: the function the reference itself calls, ``flash_attn.layers.rotary.apply_rotary_emb_torch`` (flash_attn
2.8, pure PyTorch; call sites semicat/net/duo.py:52-53), applied to the 16-bit or fp32 input with fp32 tables exactly
as the reference does (the product promotes to fp32), then rounded once to the output type.  The kernel rounds every
product and sum separately, so forward values, tangents and VJPs must agree bit for bit."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from semicat_b200 import _lib
    from semicat_b200.rotary import apply_rotary_cast


def _tables(S, D, device):
    ang = torch.arange(S, device=device)[:, None] * (1.0 / (10000 ** (torch.arange(0, D, 2, device=device) / D)))[None]
    return ang.cos().float(), ang.sin().float()


def _formula(x, cos, sin):
    from flash_attn.layers.rotary import apply_rotary_emb_torch
    return apply_rotary_emb_torch(x, cos, sin).float()


@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shape", [(2, 128, 12, 64), (1, 33, 3, 128), (3, 7, 1, 16)])
def test_forward_is_the_fp32_formula_rounded_once(shape, in_dtype, out_dtype):
    B, S, H, D = shape
    g = torch.Generator(device="cuda").manual_seed(7)
    # a strided view, as the qkv projection hands it over: (B, S, 3, H, D).unbind(2)
    qkv = torch.randn(B, S, 3, H, D, device="cuda", generator=g).to(in_dtype)
    x = qkv.unbind(2)[1]
    cos, sin = _tables(S, D, "cuda")
    before = _lib.launch_count()
    y = apply_rotary_cast(x, cos, sin, out_dtype)
    assert _lib.launch_count() == before + 1
    assert y.dtype == out_dtype and y.is_contiguous() and y.shape == x.shape
    assert torch.equal(y, _formula(x, cos, sin).to(out_dtype))


@pytest.mark.parametrize("leaf_dtype", [torch.float32, torch.bfloat16])
def test_tangent_and_gradients_match_autograd_of_the_formula(leaf_dtype):
    B, S, H, D = 2, 64, 4, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(B, S, H, D, device="cuda", generator=g).to(leaf_dtype)
    t = torch.randn(B, S, H, D, device="cuda", generator=g).to(leaf_dtype)
    gy = torch.randn(B, S, H, D, device="cuda", generator=g)
    gt = torch.randn(B, S, H, D, device="cuda", generator=g)
    cos, sin = _tables(S, D, "cuda")

    def run(fn):
        xl, tl = x.clone().requires_grad_(True), t.clone().requires_grad_(True)
        y, ty = torch.func.jvp(fn, (xl,), (tl,))
        gx, gtl = torch.autograd.grad([y, ty], [xl, tl], [gy.to(y.dtype), gt.to(ty.dtype)])
        return y, ty, gx, gtl

    fused = run(lambda z: apply_rotary_cast(z, cos, sin, torch.float32))
    plain = run(lambda z: _formula(z, cos, sin))
    for name, a, b in zip(("y", "ty", "dx", "dt"), fused, plain):
        assert a.dtype == b.dtype, name
        if leaf_dtype == torch.float32 or name in ("y", "ty"):
            assert torch.equal(a, b), f"{name}: max diff {(a.float() - b.float()).abs().max().item()}"
        else:
            # with 16-bit leaves autograd rounds the two terms of each gradient element to 16 bits before adding
            # them (one rounding per product, one for the sum); the kernel adds in fp32 and rounds once
            assert torch.allclose(a.float(), b.float(), rtol=2.0 ** -7, atol=2.0 ** -7 * b.float().abs().max().item())


def test_rejects_what_it_cannot_run():
    cos, sin = _tables(8, 64, "cuda")
    with pytest.raises(RuntimeError):
        apply_rotary_cast(torch.zeros(1, 8, 1, 64), cos.cpu(), sin.cpu())
    with pytest.raises(ValueError):
        apply_rotary_cast(torch.zeros(1, 8, 1, 24, device="cuda"), cos, sin)
    assert math.isfinite(float(apply_rotary_cast(torch.zeros(0, 8, 1, 64, device="cuda"), cos, sin).sum()))


def test_unaligned_views_take_the_scalar_path():
    B, S, H, D = 2, 9, 3, 32
    g = torch.Generator(device="cuda").manual_seed(11)
    buf = torch.randn(B, S, H, D + 3, device="cuda", generator=g).bfloat16()
    x = buf[..., 1:D + 1]  # row starts 2 bytes off a 16-byte boundary, row pitch not a multiple of 8 elements
    cos, sin = _tables(S, D, "cuda")
    assert torch.equal(apply_rotary_cast(x, cos, sin, torch.bfloat16), _formula(x, cos, sin).bfloat16())


@pytest.mark.parametrize("leaf_dtype", [torch.bfloat16, torch.float32])
def test_rotary_qkv_equals_the_per_tensor_path_under_forward_and_reverse_mode(leaf_dtype):
    """q, k, v of one (B, S, 3, H, D) projection in one launch: outputs bit-equal to apply_rotary_cast per tensor (and a
    plain cast for v); the gradient of the projection, written in place by one launch, equal to what autograd assembles
    from the three per-tensor gradients."""
    from semicat_b200 import _lib
    from semicat_b200.rotary import rotary_qkv
    B, S, H, D = 2, 37, 3, 64
    g = torch.Generator(device="cuda").manual_seed(17)
    qkv = torch.randn(B, S, 3, H, D, device="cuda", generator=g).to(leaf_dtype)
    tqkv = torch.randn(B, S, 3, H, D, device="cuda", generator=g).to(leaf_dtype)
    cots = [torch.randn(B, S, H, D, device="cuda", generator=g).bfloat16() for _ in range(6)]
    cos, sin = _tables(S, D, "cuda")

    def per_tensor(z):
        q, k, v = z.unbind(2)
        return apply_rotary_cast(q, cos, sin, torch.bfloat16), apply_rotary_cast(k, cos, sin, torch.bfloat16), v.to(torch.bfloat16)

    def run(fn):
        xl, tl = qkv.clone().requires_grad_(True), tqkv.clone().requires_grad_(True)
        outs, touts = torch.func.jvp(fn, (xl,), (tl,))
        grads = torch.autograd.grad(list(outs) + list(touts), [xl, tl], cots)
        return list(outs) + list(touts) + list(grads)

    before = _lib.launch_count()
    fused = run(lambda z: rotary_qkv(z, cos, sin, torch.bfloat16))
    assert _lib.launch_count() - before == 4  # primal and tangent forward, one launch per gradient tensor
    plain = run(per_tensor)
    names = ["q", "k", "v", "tq", "tk", "tv", "d qkv", "d tqkv"]
    for name, a, b in zip(names, fused, plain):
        assert a.dtype == b.dtype and a.shape == b.shape, name
        assert torch.equal(a, b), f"{name}: max diff {(a.float() - b.float()).abs().max().item()}"
    # without a tangent: one launch each way
    xl = qkv.clone().requires_grad_(True)
    before = _lib.launch_count()
    q, k, v = rotary_qkv(xl, cos, sin, torch.bfloat16)
    (dx,) = torch.autograd.grad([q, k, v], [xl], cots[:3])
    assert _lib.launch_count() - before == 2
    xl2 = qkv.clone().requires_grad_(True)
    (want,) = torch.autograd.grad(list(per_tensor(xl2)), [xl2], cots[:3])
    assert torch.equal(dx, want)
