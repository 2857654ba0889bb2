"""GPU: many back-to-back forward + backward calls replayed from a CUDA graph, at the shape the training step gives the
library (128 samples x 12 heads, length 128, head dimension 64), in the three cotangent modes.

With several MMA-issuing threads per CTA the roles of a kernel run ahead of one another by whole tiles; a wait that is
only correct while the waiter stays within one barrier phase of the signaller then fails rarely and only under
back-to-back launches (it did: the thread that issues the output products fell two tiles behind and misread a phase
parity).  The test replays a few thousand kernels without a host synchronisation in between and requires a clean device
status and results that are bit-identical to the first call's."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from semicat_b200 import _lib, ops


@pytest.mark.parametrize("mode", ["tan", "both", "pri"])
def test_graph_replays_back_to_back(mode):
    B, H, L, D = 128, 12, 128, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    mk = lambda: torch.randn(B, L, H, D, device="cuda", generator=g).bfloat16().transpose(1, 2)
    q, k, v, tq, tk, tv, go, gto = (mk() for _ in range(8))
    o, to = torch.empty_like(q), torch.empty_like(q)
    lse = torch.empty(B, H, ops.stat_len(L), dtype=torch.float32, device="cuda")
    mu = torch.empty_like(lse)
    grads = [torch.empty_like(q) for _ in range(6)]
    n_out = 3 if mode == "pri" else 6
    ws = [None]

    def step():
        ops.jvp_attention_fwd(q, k, v, tq, tk, tv, o, to, lse, mu)
        if mode == "pri":
            ws[0] = ops.jvp_attention_bwd(q, k, v, None, None, None, o, None, go, None, lse, None, *grads[:3], workspace=ws[0])
        else:
            ws[0] = ops.jvp_attention_bwd(q, k, v, tq, tk, tv, o, to, go if mode == "both" else None, gto, lse, mu, *grads,
                                          workspace=ws[0])

    step()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    first = [x.clone() for x in (o, to, *grads[:n_out])]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(12):
                step()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(60):
        graph.replay()
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a bounded wait inside a kernel ran out"
    for name, a, b in zip(("o", "to", "dq", "dk", "dv", "dtq", "dtk", "dtv"), (o, to, *grads[:n_out]), first):
        assert torch.equal(a, b), name
