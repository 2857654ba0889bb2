"""GPU: the reference's autograd glue, byte for byte, on top of this library.

``semicat/jvp_utils/functional.py`` of the reference copy (``oracle/make_ref.py``) is used unchanged; only the three
kernel wrappers it imports lazily are replaced (``semicat_b200.seams.install()``):
ryu_triton.flash_attention_jvp_multihead_triton_kernel_wrapper, flash_jvp_backward._flash_attn_backward and
flash_attn_triton._flash_attn_backward.  O, Od and the six gradients must match the CPU oracle within the bf16 bar."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(oracle.reference_root() is None, reason="no copy of the reference package (oracle/make_ref.py)")]

if torch.cuda.is_available():
    import gpu_util as G
    from semicat_b200 import _lib, seams


@pytest.fixture
def reference_functional():
    oracle.import_reference()
    try:
        patched = seams.install()
    except Exception as e:  # the reference's Triton modules need triton and a CUDA device at import
        pytest.skip(f"reference kernel modules not importable here: {type(e).__name__}: {e}")
    assert len(patched) == 3
    import semicat.jvp_utils.functional as functional
    assert functional.__file__.startswith(oracle.reference_root())
    yield functional
    seams.uninstall()


@pytest.mark.parametrize("mode", ["both", "tan", "pri"])
@pytest.mark.parametrize("shape", [(2, 3, 256, 64), (1, 2, 200, 32), (1, 2, 384, 128)])
def test_reference_glue_on_library_kernels_matches_the_oracle(reference_functional, shape, mode):
    B, H, L, D = shape
    ins = G.rounded(G.synth(B, H, L, L, D, seed=21), torch.bfloat16)
    dev = "cuda"
    leaves = [torch.as_tensor(ins[n]).to(dev, torch.bfloat16).requires_grad_(True) for n in G.IN_NAMES]
    before = _lib.launch_count()
    o, to = torch.func.jvp(reference_functional.sdpa_jvp, tuple(leaves[:3]), tuple(leaves[3:]))
    outs, cots = [], []
    if mode in ("both", "pri"):
        outs.append(o); cots.append(torch.as_tensor(ins["g_o"]).to(dev, torch.bfloat16))
    if mode in ("both", "tan"):
        outs.append(to); cots.append(torch.as_tensor(ins["g_od"]).to(dev, torch.bfloat16))
    grads = torch.autograd.grad(outs, leaves, cots, allow_unused=True)
    torch.cuda.synchronize()
    assert _lib.launch_count() > before and _lib.device_status() == 0
    want = G.oracle(ins, mode)
    G.assert_close(o.detach().float().cpu().numpy(), want["o"], f"{shape}/{mode}:o")
    G.assert_close(to.detach().float().cpu().numpy(), want["to"], f"{shape}/{mode}:to")
    for name, g in zip(G.GRAD_NAMES, grads):
        if g is None:
            assert mode == "pri" and name.startswith("dt"), name
            assert not np.any(want[name]), name
            continue
        G.assert_close(g.float().cpu().numpy(), want[name], f"{shape}/{mode}:{name}")
