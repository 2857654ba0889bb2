"""Host-side logic of the training caller, on CPU: the DiT restatement steps under torch.func.jvp, the
gradient all-reduce over 2 gloo ranks reproduces the single-process gradients of the concatenated batch,
and a rank that fails before the collective is reported on the host (no GPU involved)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from semicat_b200 import ddp, train_step

VOCAB, L = 11, 16


def _net(seed=0):
    torch.manual_seed(seed)
    net = train_step.DiT(VOCAB, hidden_size=32, cond_dim=16, n_blocks=2, n_heads=2, dropout=0.0, length=L)
    train_step.randomise_zero_init(net)
    return net


def _data(B, seed=1):
    g = torch.Generator().manual_seed(seed)
    x1 = torch.randint(0, VOCAB, (B, L), generator=g)
    return x1, train_step.draw_noise(x1, VOCAB, generator=g)


def _loss(net, x1, noise, sd_prop=0.5):
    vf, sd = train_step.model_step(net, x1, noise, sd_prop=sd_prop, jvp_attention="math", autocast_dtype=None)
    return train_step.total_loss(vf, sd)


def test_model_step_has_gradients_through_the_jvp_branch():
    net = _net()
    x1, noise = _data(4)
    loss = _loss(net, x1, noise)
    loss.backward()
    g = net.blocks[0].attn_qkv.weight.grad
    assert torch.isfinite(loss) and g is not None and g.abs().sum() > 0


def test_shard_bounds_cover_the_batch():
    for world in (1, 2, 3, 8):
        spans = [ddp.shard_bounds(10, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == 10
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fail_rank, out, buckets=0):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(1)
    import datetime
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20))
    try:
        net = _net()
        flat = ddp.FlatGradients(net.parameters())
        if buckets:
            assert flat.overlap_buckets(buckets) == buckets
            flat.zero()
        x1, noise = _data(4)
        # each rank takes every world-th sample so that both ranks have a JVP part and a VFM part
        idx = torch.arange(rank, 4, world)
        sub = {k: v[idx] for k, v in noise.items()}
        if rank == fail_rank:
            raise RuntimeError("injected failure before the collective")
        _loss(net, x1[idx], sub).backward()
        flat.all_reduce_mean()
        out[rank] = flat.flat.clone()
    except Exception as e:  # the surviving rank must see an error from the collective, not hang
        out[rank] = f"{type(e).__name__}: {e}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _spawn(world, fail_rank=-1, buckets=0):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), fail_rank, out, buckets), nprocs=world, join=True)
    return dict(out)


@pytest.mark.timeout(180)
def test_two_rank_gloo_allreduce_matches_single_process():
    out = _spawn(2)
    assert all(torch.is_tensor(v) for v in out.values()), out
    assert torch.equal(out[0], out[1])
    # single process: mean over the two shards' losses == what the averaged gradients correspond to
    net = _net()
    flat = ddp.FlatGradients(net.parameters())
    x1, noise = _data(4)
    total = 0
    for r in range(2):
        idx = torch.arange(r, 4, 2)
        total = total + _loss(net, x1[idx], {k: v[idx] for k, v in noise.items()}) / 2
    total.backward()
    assert torch.allclose(flat.flat, out[0], rtol=1e-4, atol=1e-6)


@pytest.mark.timeout(180)
def test_bucketed_allreduce_during_backward_gives_the_same_gradients():
    """The exchange split into buckets that leave from autograd hooks while backward() is still running must end with
    the same averaged gradients as one all-reduce after it."""
    plain, bucketed = _spawn(2), _spawn(2, buckets=3)
    assert all(torch.is_tensor(v) for v in bucketed.values()), bucketed
    assert torch.equal(bucketed[0], bucketed[1])
    assert torch.allclose(bucketed[0], plain[0], rtol=1e-6, atol=1e-8)


@pytest.mark.timeout(180)
def test_rank_failure_before_the_collective_is_reported_not_hung():
    out = _spawn(2, fail_rank=1)
    assert isinstance(out[1], str) and "injected failure" in out[1]
    assert isinstance(out[0], str), "the surviving rank should get an error from the all-reduce"


@pytest.mark.parametrize("sd_prop", [0.0, 0.5])
def test_noise_release_is_reported_once_and_buffers_refill_in_place(sd_prop):
    """A training loop refills the noise buffers for the next step as soon as model_step says they are no longer read."""
    net = _net()
    x1, noise = _data(4)
    calls = []
    vf, sd = train_step.model_step(net, x1, noise, sd_prop=sd_prop, jvp_attention="math", autocast_dtype=None,
                                   noise_released=lambda: calls.append(1))
    train_step.total_loss(vf, sd).backward()
    assert calls == [1]
    before, ptr = noise["x0"].clone(), noise["x0"].data_ptr()
    again = train_step.draw_noise(x1, VOCAB, out=noise)
    assert again is noise and noise["x0"].data_ptr() == ptr and not torch.equal(noise["x0"], before)
    assert noise["x0"].shape == before.shape and float(noise["t_vfm"].min()) >= 0.0 and float(noise["t_vfm"].max()) <= 1.0
