"""GPU parity at the shapes of the long-sequence sweep (H = 16, d in {64, 128}, L up to 8192, N(0,1) primals and
tangents): the CUDA kernels through the C ABI against the fp64 oracle.

Each launch holds enough (batch, head) pairs that every persistent CTA of the backward walks several work items
(more than two 128-row items per SM), so the item loops, the barrier-phase wrap-around over hundreds of streamed
tiles and the cross-item prefetch all run; the oracle, evaluated in chunks of query rows, checks a sample of heads.
Tolerance as everywhere: |x - ref| <= 1e-2 + 2e-2 |ref|."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as G
    from semicat_b200 import _lib

SM_COUNT = 148
# (L, D, batch * heads in the launch): items = BH * L / 128 > 2 * SM_COUNT
SHAPES = [(4096, 64, 10), (8192, 64, 5), (2048, 128, 20), (4096, 128, 10), (8192, 128, 5)]


def _device_inputs(BH, L, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda: torch.randn(1, L, BH, D, device="cuda", generator=g).bfloat16().transpose(1, 2)  # (1, BH, L, D) view
    return {n: mk() for n in (*G.IN_NAMES, "g_o", "g_od")}


@pytest.mark.parametrize("mode", ["both", "tan", "pri"])
@pytest.mark.parametrize("L,D,BH", SHAPES)
def test_sweep_shapes_against_the_oracle(L, D, BH, mode):
    from semicat_b200 import ops
    assert BH * (L // 128) > 2 * SM_COUNT
    t = _device_inputs(BH, L, D, seed=L + D)
    like = lambda: torch.empty(1, L, BH, D, dtype=torch.bfloat16, device="cuda").transpose(1, 2)
    o, to = like(), like()
    lse = torch.empty(1, BH, ops.stat_len(L), dtype=torch.float32, device="cuda")
    mu = torch.empty_like(lse)
    ops.jvp_attention_fwd(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], o, to, lse, mu)
    grads = [like() for _ in range(6)]
    g_o = t["g_o"] if mode in ("both", "pri") else None
    g_to = t["g_od"] if mode in ("both", "tan") else None
    if mode == "pri":
        ops.jvp_attention_bwd(t["q"], t["k"], t["v"], None, None, None, o, None, g_o, None, lse, None, *grads[:3])
    else:
        ops.jvp_attention_bwd(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], o, to, g_o, g_to, lse, mu, *grads)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert ops.selected_kernels(1, BH, L, L, D) == ops.KERNELS_TCGEN05
    # every head must at least be finite; a sample of heads (first, and one that a later work item of a CTA covers)
    # is compared with the oracle
    for x in (o, to, *(grads if mode != "pri" else grads[:3])):
        assert bool(torch.isfinite(x).all())
    heads = [0, BH - 1] if mode == "both" else [BH // 2]
    for h in heads:
        ins = {n: x[:, h:h + 1].float().cpu().numpy() for n, x in t.items()}
        want = G.oracle_rows(ins, mode)
        got = {"o": o, "to": to, "lse": lse[..., :L], "mu": mu[..., :L]}
        got.update(dict(zip(G.GRAD_NAMES, grads)) if mode != "pri" else dict(zip(G.GRAD_NAMES[:3], grads[:3])))
        got = {n: x[:, h:h + 1].float().cpu().numpy() for n, x in got.items()}
        G.compare(got, want, mode, f"L{L} d{D} head {h} {mode}")
