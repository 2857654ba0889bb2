"""GPU test of ``jvpattn_bwd_static``, the backward entry point for callers that cannot allocate device
memory (a plug-in that is only handed pointers, a process whose pool already owns all of HBM).  It keeps
its scratch in a fixed array inside the library instead of asking for a workspace.

Checked here, through the C ABI: two calls in a row (different data, so whatever the first call left in
the shared scratch must not leak into the second) give the same gradients as the workspace-taking entry
point ``jvpattn_bwd`` within the bf16 bar of the other GPU tests, the call really allocates nothing on the
torch side, and a problem beyond the built-in limit is refused with its own error code.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as G
    from semicat_b200 import _lib, ops


def _device_problem(seed, B=2, H=3, L=256, D=64):
    ins = G.rounded(G.synth(B, H, L, L, D, seed=seed), torch.bfloat16)
    t = {n: G.place(ins[n], torch.bfloat16, "bshd") for n in (*G.IN_NAMES, "g_o", "g_od")}
    o, to = torch.empty_like(t["q"]), torch.empty_like(t["q"])
    lse = torch.empty(B, H, ops.stat_len(L), dtype=torch.float32, device="cuda")
    mu = torch.empty_like(lse)
    ops.jvp_attention_fwd(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], o, to, lse, mu)
    return ins, t, o, to, lse, mu


def _grads_like(t):
    return [torch.full_like(t[n], float("nan")) for n in G.IN_NAMES]


@pytest.mark.parametrize("mode", ["both", "tan", "pri"])
def test_static_scratch_backward_matches_workspace_backward_twice(mode):
    for call, seed in enumerate((21, 22)):  # two calls in a row on the shared scratch
        ins, t, o, to, lse, mu = _device_problem(seed)
        g_o = t["g_o"] if mode in ("both", "pri") else None
        g_to = t["g_od"] if mode in ("both", "tan") else None
        tang = (t["tq"], t["tk"], t["tv"]) if g_to is not None else (None, None, None)
        to_arg, mu_arg = (to, mu) if g_to is not None else (None, None)
        n_out = 6 if g_to is not None else 3
        want = _grads_like(t)[:n_out]
        got = _grads_like(t)[:n_out]
        ops.jvp_attention_bwd(t["q"], t["k"], t["v"], *tang, o, to_arg, g_o, g_to, lse, mu_arg, *want)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        ops.jvp_attention_bwd_static(t["q"], t["k"], t["v"], *tang, o, to_arg, g_o, g_to, lse, mu_arg, *got)
        assert torch.cuda.memory_allocated() == before, "the allocation-free entry point allocated through torch"
        torch.cuda.synchronize()
        ref = G.oracle(ins, mode)
        for name, a, b in zip(G.GRAD_NAMES, got, want):
            a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
            G.assert_close(a, b, f"call {call} {mode}:{name} static vs workspace")
            G.assert_close(a, ref[name], f"call {call} {mode}:{name} static vs oracle")
    assert _lib.device_status() == 0


def test_problem_beyond_the_builtin_scratch_is_refused():
    B, H, L, D = 33, 64, 128, 64  # 33 * 64 * 128 rows > 262144
    assert B * H * ops.stat_len(L) > _lib.STATIC_SCRATCH_ROWS
    z = torch.zeros(B, H, L, D, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(B, H, ops.stat_len(L), dtype=torch.float32, device="cuda")
    launches = _lib.launch_count()
    with pytest.raises(_lib.JvpAttnError) as e:
        ops.jvp_attention_bwd_static(z, z, z, z, z, z, z, z, z, z, lse, lse, z, z, z, z, z, z)
    assert e.value.code == -10 and "jvpattn_bwd_static" in str(e.value)
    assert _lib.launch_count() == launches
