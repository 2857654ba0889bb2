"""Pin both CPU oracles against the fixtures generated from the reference's own CPU path."""
import numpy as np
import pytest
import torch

from oracle import closed_form, torch_cpu_path
from conftest import GRAD_NAMES

MODES = {"both": (True, True), "tan": (False, True), "pri": (True, False)}


def _close(a, b, tol):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape
    err = np.abs(a - b)
    assert np.all(err <= tol + tol * np.abs(b)), f"max err {err.max():.3e}"


def test_closed_form_forward_matches_reference(golden):
    _, g = golden
    o, od, lse, mu = closed_form.forward(*(g[n] for n in ("q", "k", "v", "tq", "tk", "tv")))
    # fixtures are fp32 evaluations; 1e-4 is the fp32 bar of the spec
    _close(o, g["o"], 1e-4)
    _close(od, g["od"], 1e-4)
    _close(lse, g["lse"], 1e-5)
    _close(mu, g["mu"], 1e-5)


@pytest.mark.parametrize("mode", list(MODES))
def test_closed_form_backward_matches_reference(golden, mode):
    _, g = golden
    use_o, use_od = MODES[mode]
    grads = closed_form.backward(
        *(g[n] for n in ("q", "k", "v", "tq", "tk", "tv")),
        g_o=g["g_o"] if use_o else None, g_od=g["g_od"] if use_od else None)
    for n, val in zip(GRAD_NAMES, grads):
        _close(val, g[f"{n}_{mode}"], 1e-4)


@pytest.mark.parametrize("mode", list(MODES))
def test_torch_cpu_path_matches_reference(golden, mode):
    _, g = golden
    use_o, use_od = MODES[mode]
    t = lambda n: torch.from_numpy(g[n])
    o, od, grads = torch_cpu_path.attention_jvp_with_grads(
        t("q"), t("k"), t("v"), t("tq"), t("tk"), t("tv"),
        t("g_o") if use_o else None, t("g_od") if use_od else None)
    _close(o.numpy(), g["o"], 1e-5)
    _close(od.numpy(), g["od"], 1e-5)
    for n, val in zip(GRAD_NAMES, grads):
        _close(val.numpy(), g[f"{n}_{mode}"], 1e-5)


def test_two_oracles_agree_in_float64():
    rng = np.random.default_rng(7)
    shp_q, shp_k = (2, 2, 24, 16), (2, 2, 40, 16)
    q, tq, g_o, g_od = (rng.standard_normal(shp_q) for _ in range(4))
    k, v, tk, tv = (rng.standard_normal(shp_k) for _ in range(4))
    o, od, _, _ = closed_form.forward(q, k, v, tq, tk, tv)
    grads = closed_form.backward(q, k, v, tq, tk, tv, g_o, g_od)
    T = torch.from_numpy
    o2, od2, grads2 = torch_cpu_path.attention_jvp_with_grads(*map(T, (q, k, v, tq, tk, tv, g_o, g_od)))
    assert np.abs(o - o2.numpy()).max() < 1e-12
    assert np.abs(od - od2.numpy()).max() < 1e-12
    for a, b in zip(grads, grads2):
        assert np.abs(a - b.numpy()).max() < 1e-11


def test_tangent_linearity_of_closed_form():
    """Od is linear in the tangents: a size-independent property also used at full size on the GPU."""
    rng = np.random.default_rng(1)
    shp = (1, 2, 32, 16)
    q, k, v, a1, a2, a3, b1, b2, b3 = (rng.standard_normal(shp) for _ in range(9))
    f = lambda x, y, z: closed_form.forward(q, k, v, x, y, z)[1]
    lhs = f(2 * a1 + 3 * b1, 2 * a2 + 3 * b2, 2 * a3 + 3 * b3)
    rhs = 2 * f(a1, a2, a3) + 3 * f(b1, b2, b3)
    assert np.abs(lhs - rhs).max() < 1e-10


def test_flop_model():
    f = closed_form.flops(64, 12, 128, 128, 64)
    assert abs(f["total"] - 42 * 64 * 12 * 128 * 128 * 64) < 1
    assert abs(f["fwd"] / 1e9 - 9.66) < 0.01
