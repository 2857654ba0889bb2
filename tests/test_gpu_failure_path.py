"""GPU: the failure path of the bounded device-side waits, exercised without hanging or faulting anything.

Every wait inside the tcgen05 kernels gives up after a budget of clock cycles, records a code in the library's device
status word and lets the CTA leave through its normal teardown.  The test shortens the budget to about a millisecond
(``jvpattn_debug_set``) and makes one barrier of the next forward launch expect bytes that never arrive (a flag that
nothing sets): the kernel must end by itself, ``jvpattn_stream_check`` must answer JVPATTN_EDEVICE,
``jvpattn_device_status`` must name a forward wait, and the next ordinary call must be correct."""
import pytest
import torch

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import gpu_util as G
    from semicat_b200 import _lib, ops


def test_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    dt = torch.bfloat16
    ins = G.rounded(G.synth(1, 2, 256, 256, 64, seed=4), dt)
    t = {n: G.place(ins[n], dt, "bshd") for n in G.IN_NAMES}
    o, to = torch.zeros_like(t["q"]), torch.zeros_like(t["q"])
    lse = torch.zeros(1, 2, 256, dtype=torch.float32, device="cuda")
    mu = torch.zeros_like(lse)
    assert ops.selected_kernels(1, 2, 256, 256, 64) == ops.KERNELS_TCGEN05
    assert _lib.device_status() == 0
    _lib.debug_set(_lib.DEBUG_WAIT_CYCLES, 2_000_000)  # about 1 ms at B200 clocks
    try:
        _lib.debug_set(_lib.DEBUG_STALL_NEXT_FWD, 1)
        ops.jvp_attention_fwd(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], o, to, lse, mu)
        with pytest.raises(_lib.JvpAttnError) as err:
            _lib.stream_check(torch.cuda.current_stream().cuda_stream)
        assert err.value.code == -9
        code = _lib.device_status()
        assert 101 <= code <= 107, code
        assert _lib.device_status() == 0  # reading clears the word
    finally:
        _lib.debug_set(_lib.DEBUG_STALL_NEXT_FWD, 0)
        _lib.debug_set(_lib.DEBUG_WAIT_CYCLES, 0)
    # the hook was one-shot and the context is intact: an ordinary forward + backward is correct
    got = G.run(ins, mode="both", layout="bshd")
    G.compare(got, G.oracle(ins, "both"), "both", "after a failed wait")
    _lib.stream_check(torch.cuda.current_stream().cuda_stream)
    assert _lib.device_status() == 0


def test_unknown_debug_knob_is_refused():
    with pytest.raises(_lib.JvpAttnError) as err:
        _lib.debug_set(17, 1)
    assert err.value.code == -1
