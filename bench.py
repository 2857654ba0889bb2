#!/usr/bin/env python
"""Benchmark of the JVP-attention hot path: fused forward + backward TFLOP/s on synthetic data.

    python bench.py --gpus N --steps K --warmup W            # this library on N GPUs of one node
    python bench.py --impl reference --steps K --warmup W     # the CPU path on the host cores

Workload (BASELINE config 2): bf16, non-causal, B=64, H=12, L=128, d=64; q ~ N(0,1)/sqrt(d), k, v ~ N(0,1),
tangents ~ 0.1 N(0,1), cotangents on O and Od ~ N(0,1); tensors are (B,H,L,D) views of (B,S,H,D) memory,
the layout the denoiser hands over.  One step = one forward (O, Od, lse, mu) + one backward (all six
VJPs, both cotangents) over one batch.  With N > 1 every rank runs that batch on its own GPU (the
(batch, head) problems are independent: no data-path collective, weak scaling).

FLOP model: GEMM-unit = 2 L^2 d per head; forward 6 units, backward 15, total 42 B H L^2 d per step.
Recomputation inside the kernels is not counted.  Byte model: T = 2 B H L d; forward 8T, backward 16T.

One JSON line is printed by rank 0; see the keys at the bottom of `main`.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, L, D, value distribution)
    "config2": dict(B=64, H=12, L=128, D=64, q_scale=None, t_scale=0.1),
    "L2048_d64": dict(B=32, H=16, L=2048, D=64, q_scale=1.0, t_scale=1.0),
    # a slice of the long-sequence sweep small enough for an ncu capture (268 MB resident per set)
    "L2048_d64_small": dict(B=4, H=16, L=2048, D=64, q_scale=1.0, t_scale=1.0),
    "L2048_d128_small": dict(B=2, H=16, L=2048, D=128, q_scale=1.0, t_scale=1.0),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
# The same `config` object is printed by the GPU arm and by `--impl reference`, so that the two lines can be matched.
TIMING_NOTE = ("GPU arm: rotating over >= 4 resident input/output sets (> 400 MB) so that no step finds its data in the "
               "126 MB L2, one CUDA graph per set (eager launches where capture is unavailable; see launch_mode); "
               "CPU arm: inputs drawn once outside the timed region")


def ncu_traffic(workload, kernel):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel`, from the ncu capture recorded in
    profiles/ncu_traffic.json (written when a capture is taken); None where no capture covers it."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            return json.load(f).get(workload, {}).get(kernel)
    except Exception:
        return None


def flops_per_step(B, H, L, D):
    return 42.0 * B * H * L * L * D


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS, source="fallback")


# ----------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while a region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------- inputs
def host_inputs(cfg, seed):
    import torch
    B, H, L, D = cfg["B"], cfg["H"], cfg["L"], cfg["D"]
    g = torch.Generator().manual_seed(seed)
    qs = 1.0 / math.sqrt(D) if cfg["q_scale"] is None else cfg["q_scale"]
    # generated directly in the model's (B,S,H,D) memory order
    mk = lambda s: (torch.randn(B, L, H, D, generator=g) * s).to(torch.bfloat16)
    t = cfg["t_scale"]
    return {"q": mk(qs), "k": mk(1.0), "v": mk(1.0), "tq": mk(t), "tk": mk(t), "tv": mk(t), "g_o": mk(1.0), "g_to": mk(1.0)}


class DeviceSet:
    """One resident set of inputs, outputs and gradients plus its pre-marshalled launch plan."""

    def __init__(self, host, device):
        import torch
        from semicat_b200 import ops
        self.t = {n: x.to(device).transpose(1, 2) for n, x in host.items()}  # (B,H,L,D) views
        q = self.t["q"]
        B, H, L, D = q.shape
        like = lambda: torch.empty(B, L, H, D, dtype=q.dtype, device=device).transpose(1, 2)
        self.o, self.to = like(), like()
        self.lse = torch.empty(B, H, ops.stat_len(L), dtype=torch.float32, device=device)
        self.mu = torch.empty_like(self.lse)
        self.grads = [like() for _ in range(6)]
        t = self.t
        self.plan = ops.Plan(t["q"], t["k"], t["v"], t["tq"], t["tk"], t["tv"], self.o, self.to, self.lse, self.mu,
                             g_o=t["g_o"], g_to=t["g_to"], grads=self.grads)

    def step(self):
        self.plan.forward()
        self.plan.backward()

    def nbytes(self):
        return sum(x.numel() * x.element_size() for x in (*self.t.values(), self.o, self.to, *self.grads))


# ----------------------------------------------------------------------------------------------- GPU arm
def run_device(cfg, sets, steps, warmup, dist, sampler, use_graph=True):
    """Device-resident timing: CUDA events on the launching stream around exactly `steps` steps."""
    import torch
    from semicat_b200 import _lib
    count0 = _lib.launch_count()
    for i in range(max(warmup, 3)):
        sets[i % len(sets)].step()
    torch.cuda.synchronize()
    per_step = (_lib.launch_count() - count0) // max(warmup, 3)  # kernels of this library per step
    graphs, mode = [], "eager"
    try:  # one CUDA graph per input set: the steps are launch-bound at this size
        if not use_graph:
            raise RuntimeError("disabled by --profile-mode")
        for s in sets:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                s.step()
            graphs.append(g)
        mode = "cuda_graph"
        for g in graphs:
            g.replay()
        torch.cuda.synchronize()
    except Exception as e:  # pragma: no cover - depends on the driver
        print(f"[bench] CUDA graph capture unavailable ({type(e).__name__}: {e}); timing eager launches", file=sys.stderr)
        graphs, mode = [], "eager"
        torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = _lib.launch_count()
    with sampler:
        start.record()
        for i in range(steps):
            if graphs:
                graphs[i % len(graphs)].replay()
            else:
                sets[i % len(sets)].step()
        end.record()
        end.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    launched = (_lib.launch_count() - launches0) if not graphs else per_step * steps
    return ms, launched, mode


def run_profile(sets, steps):
    """Per-kernel device time from CUDA events recorded by the library around each launch."""
    import torch
    from semicat_b200 import _lib
    torch.cuda.synchronize()
    _lib.profile_begin()
    for i in range(steps):
        sets[i % len(sets)].step()
    return _lib.profile_end()


def run_e2e(cfg, host_sets, steps, warmup, device, dist, sampler):
    """End to end through the public API with HOST buffers: per step, pinned host -> device copies of the
    eight inputs, sdpa_jvp under torch.func.jvp, reverse mode for both cotangents, and the eight results
    copied back to pinned host memory."""
    import torch
    from semicat_b200 import sdpa_jvp
    pinned = [{n: x.pin_memory() for n, x in hs.items()} for hs in host_sets]
    B, H, L, D = cfg["B"], cfg["H"], cfg["L"], cfg["D"]
    # two steps in flight on two streams, so one step's result copy overlaps the next step's input copy
    # (PCIe is full duplex); each stream has its own pinned result buffers
    streams = [torch.cuda.Stream(device=device) for _ in range(2)]
    out_host = [[torch.empty(B, H, L, D, dtype=torch.bfloat16).pin_memory() for _ in range(8)] for _ in range(2)]
    names = ("q", "k", "v", "tq", "tk", "tv")

    def step(i):
        src = pinned[i % len(pinned)]
        with torch.cuda.stream(streams[i % 2]):
            dev = {n: x.to(device, non_blocking=True) for n, x in src.items()}
            leaves = [dev[n].transpose(1, 2).requires_grad_(True) for n in names]
            o, to = torch.func.jvp(sdpa_jvp, tuple(leaves[:3]), tuple(leaves[3:]))
            grads = torch.autograd.grad([o, to], leaves, [dev["g_o"].transpose(1, 2), dev["g_to"].transpose(1, 2)])
            for dst, src_t in zip(out_host[i % 2], (o.detach(), to.detach(), *grads)):
                dst.copy_(src_t, non_blocking=True)

    def fork():
        for st in streams:
            st.wait_stream(torch.cuda.current_stream())

    def join():
        for st in streams:
            torch.cuda.current_stream().wait_stream(st)

    fork()
    for i in range(max(warmup, 3)):
        step(i)
    join()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with sampler:
        t0 = time.perf_counter()
        start.record()
        fork()
        for i in range(steps):
            step(i)
        join()
        end.record()
        end.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
    if dist is not None:
        dist.barrier()
    ms = max(start.elapsed_time(end), wall_ms)  # device time and host wall agree unless the host is the bottleneck
    per_tensor = B * H * L * D * 2
    return ms, 8 * per_tensor, 8 * per_tensor


# ----------------------------------------------------------------------------------------------- DiT training
TRAIN_CONFIGS = {
    # BASELINE configs 3 and 4: 12 layers, hidden 768, 12 heads (d = 64), MLP 3072, adaLN, bf16 autocast
    "dit_lm1b": dict(vocab=30522, length=128, global_batch=512, embed="naive"),
    "dit_text8": dict(vocab=27, length=256, global_batch=256, embed="rms"),
}


def attention_jvp_flops(batch, heads, length, head_dim, layers, mode="lag"):
    """Algorithmic FLOPs of the library's attention calls in one self-distillation step: forward 6 GEMM-units,
    backward 13 with the cotangent of the tangent output alone (`lag`), 15 with both."""
    units = 6 + (13 if mode == "lag" else 15)
    return float(units) * 2.0 * batch * heads * length * length * head_dim * layers


def count_step_flops(body, attn_flops):
    """FLOPs of one eager training step: what torch.utils.flop_counter sees (matmuls and library attention of the
    torch ops, primal and tangent passes, forward and backward) plus the algorithmic FLOPs of this library's own
    attention kernels, which the counter cannot see."""
    from torch.utils.flop_counter import FlopCounterMode
    with FlopCounterMode(display=False) as fc:
        body()
    return float(fc.get_total_flops()) + attn_flops


def run_train(name, steps, warmup, device, rank, world, dist, sampler, sd_prop=0.25, attention="jvp", use_graph=True,
              primal_attention="lib", global_batch=0, overlap=True):
    """Flow-map training steps of the DiT (semicat_b200/train_step.py) on uniform random tokens: global batch
    sharded over the ranks, forward-mode JVP through every attention layer for the first `sd_prop` of each
    shard, AdamW, one flat gradient all-reduce per step.  Every step copies its token ids from pinned host memory
    and writes its loss back to the host.  Returns a dict (times in ms, max over ranks)."""
    import torch
    from semicat_b200 import ddp, train_step
    tc = dict(TRAIN_CONFIGS[name])
    if global_batch:
        tc["global_batch"] = global_batch
    torch.manual_seed(1234)  # same initial weights on every rank
    net = train_step.DiT(tc["vocab"], 768, 128, 12, 12, dropout=0.1, length=tc["length"], embed_type=tc["embed"]).to(device)
    flat = ddp.FlatGradients(net.parameters())
    buckets = flat.overlap_buckets(4) if (dist is not None and overlap) else 0  # exchange overlapped with the backward
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, weight_decay=0.0, fused=True, capturable=True)
    lo, hi = ddp.shard_bounds(tc["global_batch"], rank, world)
    gen = torch.Generator().manual_seed(99 + rank)
    # a ring of pinned token batches that the host never rewrites: the copy of step i cannot race with anything
    host_tokens = [torch.randint(0, tc["vocab"], (hi - lo, tc["length"]), generator=gen).pin_memory() for _ in range(4)]
    torch.cuda.manual_seed(7 + rank)  # per-rank noise from the default CUDA generator (graph-capturable)
    loss_host = torch.zeros((), dtype=torch.float32).pin_memory()
    x1 = torch.empty(hi - lo, tc["length"], dtype=torch.long, device=device)

    # The noise of step i + 1 is drawn while step i is still running: the last kernel that reads the noise is the first
    # node of the backward (the self-distillation loss), after which a second stream refills the buffers in place under
    # the rest of the backward (an 8 GB write at the lm1b shape, hidden under GEMMs that do not use the memory system).
    noise = train_step.draw_noise(x1, tc["vocab"])
    noise_stream = torch.cuda.Stream(device) if overlap else None

    def refill():
        if noise_stream is None:
            train_step.draw_noise(x1, tc["vocab"], out=noise)
            return
        noise_stream.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(noise_stream):
            train_step.draw_noise(x1, tc["vocab"], out=noise)

    def body():
        flat.zero()
        vf, sd = train_step.model_step(net, x1, noise, sd_prop=sd_prop, jvp_attention=attention,
                                       primal_attention=primal_attention, overlap_branches=overlap, noise_released=refill)
        loss = train_step.total_loss(vf, sd)
        loss.backward()
        flat.all_reduce_mean()
        opt.step()
        loss_host.copy_(loss.detach(), non_blocking=True)
        if noise_stream is not None:
            torch.cuda.current_stream(device).wait_stream(noise_stream)

    graph = None

    def step(i):
        x1.copy_(host_tokens[i % 4], non_blocking=True)  # stream-ordered before the (graph of the) step
        if graph is not None:
            graph.replay()
        else:
            body()

    x1.copy_(host_tokens[0])
    n_sd = int(sd_prop * (hi - lo))
    step_flops = count_step_flops(body, attention_jvp_flops(n_sd, 12, tc["length"], 64, 12) if attention == "jvp" else 0.0)
    for i in range(max(warmup - 1, 2)):
        step(i)
    torch.cuda.synchronize()
    mode = "eager"
    if use_graph:
        # The step is launch-bound on the host (thousands of small kernels under forward-mode AD), so the whole
        # step - noise, forward/JVP, backward, gradient all-reduce, AdamW, D2H of the loss - is captured once into
        # a CUDA graph and replayed; the H2D copy of the tokens is enqueued in front of every replay.
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                body()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                body()
            graph = g
            mode = "cuda_graph"
            step(0)
            torch.cuda.synchronize()
        except Exception as e:  # pragma: no cover - depends on driver / NCCL support for capture
            print(f"[bench] training-step graph capture unavailable ({type(e).__name__}: {str(e)[:200]}); running eagerly",
                  file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    with sampler:
        marks[0].record()
        for i in range(steps):
            step(i)
            marks[i + 1].record()
        marks[-1].synchronize()
    if dist is not None:
        dist.barrier()
    per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    ms = marks[0].elapsed_time(marks[-1]) / steps
    med = statistics.median(per_step)
    last_loss = float(loss_host)
    # the gradient all-reduce alone (the only collective of the step), on the same flat buffer
    ar = []
    if dist is not None:
        for _ in range(7):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            a.record()
            dist.all_reduce(flat.flat)  # the whole buffer as one message, whatever the step itself does
            flat.flat.div_(world)
            b.record()
            b.synchronize()
            ar.append(a.elapsed_time(b))
    ar_ms = statistics.median(ar[2:]) if ar else 0.0
    if dist is not None:
        t = torch.tensor([ms, med, ar_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, med, ar_ms = float(t[0]), float(t[1]), float(t[2])
        f = torch.tensor([step_flops], device=device, dtype=torch.float64)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
        step_flops = float(f[0])
    peak_gb = torch.cuda.max_memory_allocated() / 1e9
    graph = None
    nbytes = flat.nbytes()
    from semicat_b200 import _lib
    status = _lib.device_status()  # non-zero: a bounded wait inside one of the library's kernels ran out
    del net, opt, flat
    torch.cuda.empty_cache()
    return {"ms_per_step": ms, "ms_per_step_median": med, "tokens_per_step": tc["global_batch"] * tc["length"],
            "loss": last_loss, "peak_mem_gb": peak_gb, "launch": mode, "allreduce_ms": ar_ms, "allreduce_bytes": nbytes, "allreduce_buckets": buckets,
            "flops_per_step": step_flops, "steps": steps, "warmup": max(warmup, 3), "primal_attention": primal_attention,
            "device_status": status, "ms_per_step_max": max(per_step), "ms_per_step_min": min(per_step)}


def train_block(r, world, pk, label):
    """The `train` object of the JSON line from run_train's result."""
    tps = r["tokens_per_step"] / (r["ms_per_step"] * 1e-3)
    tf = r["flops_per_step"] / (r["ms_per_step"] * 1e-3) / 1e12
    return {"workload": label, "scaling": "strong", "ms_per_step": r["ms_per_step"], "ms_per_step_median": r["ms_per_step_median"],
            "tokens_per_s": tps, "tokens_per_s_median": r["tokens_per_step"] / (r["ms_per_step_median"] * 1e-3),
            "steps": r["steps"], "warmup": r["warmup"], "loss": r["loss"], "launch": r["launch"], "peak_mem_gb": r["peak_mem_gb"],
            "primal_attention": r["primal_attention"], "device_status": r["device_status"],
            "ms_per_step_min": r["ms_per_step_min"], "ms_per_step_max": r["ms_per_step_max"],
            "allreduce_ms": r["allreduce_ms"], "allreduce_bytes": r["allreduce_bytes"],
            "allreduce_in_step": (f"{r['allreduce_buckets']} buckets, each sent on a second stream when its last gradient is accumulated"
                                  if r["allreduce_buckets"] else "one message after the backward"),
            "flops_per_step": r["flops_per_step"], "flops_source": "torch.utils.flop_counter over one eager step + algorithmic "
            "FLOPs of the library's attention calls", "tflops": tf, "frac_of_bf16_peak": tf / (world * pk["bf16_tflops"])}


# ----------------------------------------------------------------------------------------------- CPU arm
def cpu_arm():
    """The CPU implementation of the path that the CPU legs time: the reference's own
    naive_multihead_attention_jvp (semicat/jvp_utils/ryu_triton.py:426-454) differentiated by autograd when the copy of
    the reference package made by oracle/make_ref.py is present ("reference"), else its restatement in
    oracle/torch_cpu_path.py ("port").  Returns (callable or None for the port, kind)."""
    from oracle import torch_cpu_path
    fn = torch_cpu_path.reference_attention_jvp()
    return fn, ("reference" if fn is not None else "port")


def cpu_path(cfg, repeats, threads=None):
    """Best-of-`repeats` seconds of one fwd+bwd of the CPU arm over the full workload in fp32, on all host threads."""
    from oracle import torch_cpu_path
    fn, kind = cpu_arm()
    best, used = torch_cpu_path.time_fwd_bwd(cfg["B"], cfg["H"], cfg["L"], cfg["D"], repeats=repeats, threads=threads,
                                             attention=fn)
    return best, used, kind


def run_triton_comparator(args):
    """`--impl reference_triton`: the reference's own GPU path (its Triton kernels behind semicat.jvp_utils.functional.sdpa_jvp,
    JIT-compiled by the installed Triton for this GPU) timed with the same inputs and the same CUDA-event harness, forward
    and backward separately, on config 2 and on a B4 H16 L2048 d64 slice of the long-sequence sweep.  A comparator and a
    second parity opinion only; needs the copy of the reference package made by oracle/make_ref.py.  Any failure to
    import, compile or run is reported as text in the JSON line instead of a number."""
    import torch
    import oracle
    out = {"impl": "reference_triton", "metric": "jvp_attn_fwd_bwd_tflops", "unit": "TFLOP/s", "rows": []}
    try:
        if oracle.import_reference() is None:
            raise RuntimeError("no copy of the reference package (run oracle/make_ref.py where the reference checkout is)")
        import triton
        from semicat.jvp_utils import functional as ref_functional
        out["triton"] = triton.__version__
    except Exception as e:
        out["unavailable"] = f"{type(e).__name__}: {e}"[:400]
        print(json.dumps(out))
        return
    from semicat_b200 import functional as ours
    dev = torch.device("cuda", 0)
    for name in ("config2", "L2048_d64_small"):
        cfg = WORKLOADS[name]
        B, H, L, D = cfg["B"], cfg["H"], cfg["L"], cfg["D"]
        host = host_inputs(cfg, seed=0)
        t = {n: x.to(dev).transpose(1, 2) for n, x in host.items()}  # (B,H,L,D) views of (B,S,H,D) memory
        row = {"workload": name, "shape": [B, H, L, D]}
        for label, fn in (("reference_triton", ref_functional.sdpa_jvp), ("this_library", ours.sdpa_jvp)):
            try:
                leaves = [t[n].detach().requires_grad_(True) for n in ("q", "k", "v", "tq", "tk", "tv")]

                def fwd():
                    return torch.func.jvp(fn, tuple(leaves[:3]), tuple(leaves[3:]))

                def time_it(f, reps):
                    for _ in range(3):
                        r = f()
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(reps):
                        r = f()
                    b.record()
                    b.synchronize()
                    return a.elapsed_time(b) / reps, r

                reps = 20 if name == "config2" else 5
                f_ms, (o, to) = time_it(fwd, reps)
                both_ms, _ = time_it(lambda: torch.autograd.grad(list(fwd()), leaves, [t["g_o"], t["g_to"]]), reps)
                row[label] = {"fwd_ms": f_ms, "fwd_bwd_ms": both_ms, "bwd_ms": both_ms - f_ms,
                              "fwd_bwd_tflops": flops_per_step(B, H, L, D) / (both_ms * 1e-3) / 1e12}
                if label == "reference_triton":
                    ref_out = (o.detach().float(), to.detach().float())
                else:
                    row["max_abs_diff_vs_reference"] = {"o": float((o.detach().float() - ref_out[0]).abs().max()),
                                                        "to": float((to.detach().float() - ref_out[1]).abs().max())}
            except Exception as e:  # one attempt: the message is the record
                row[label] = {"error": f"{type(e).__name__}: {e}"[:600]}
                ref_out = None
        out["rows"].append(row)
    out["note"] = ("through the PyTorch entry point (autograd glue included on both sides), eager launches, both cotangents; "
                   "the reference runs its tangent and primal backward as two kernel-wrapper calls, this library one merged call (one autograd node for both outputs)")
    print(json.dumps(out))


def _claim_stdout():
    """Libraries (NCCL among them) print banners on stdout; the contract is ONE JSON line there.  Point fd 1 at
    stderr for the rest of the process and hand back a file object on the real stdout for the final line."""
    sys.stdout.flush()
    real = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    return real


def main():
    global print
    _out = _claim_stdout()
    _print = print

    def print(*a, **kw):  # noqa: A001 - route only this module's prints
        if "file" in kw:
            return _print(*a, **kw)
        _print(*a, file=_out, **kw)
        _out.flush()

    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "reference_triton"])
    ap.add_argument("--workload", default="config2", choices=list(WORKLOADS) + list(TRAIN_CONFIGS) + ["sweep5"])
    ap.add_argument("--sd-prop", type=float, default=0.25, help="share of each batch that takes the JVP step (training workloads)")
    ap.add_argument("--primal-attention", default="lib", choices=["sdpa", "lib"],
                    help="attention of the passes without tangents in the training workloads: torch SDPA or this library")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="training workloads: override the configuration's global batch (e.g. 64 = one rank's share of an 8-GPU run)")
    ap.add_argument("--no-overlap", action="store_true",
                    help="training workloads: one stream for both branches of the objective and one all-reduce after the backward")
    ap.add_argument("--kernel-mix", action="store_true",
                    help="training workloads: profile one eager step and print the device time by kernel family and operator")
    ap.add_argument("--no-extras", action="store_true", help="skip the long-sequence point and the CPU baseline")
    ap.add_argument("--profile-mode", action="store_true",
                    help="for runs under ncu: eager launches (no CUDA graph), no end-to-end leg, no extras")
    args = ap.parse_args()
    if args.impl == "reference_triton":
        return run_triton_comparator(args)
    if args.workload in TRAIN_CONFIGS:
        return main_train(args)
    if args.workload == "sweep5":
        return main_sweep(args)
    cfg = WORKLOADS[args.workload]
    B, H, L, D = cfg["B"], cfg["H"], cfg["L"], cfg["D"]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    flops = flops_per_step(B, H, L, D)
    config = {"workload": f"{args.workload}: JVP attention fwd+bwd, bf16, non-causal, B{B} H{H} L{L} d{D}, "
                          "both cotangents, (B,S,H,D) memory layout",
              "flop_model": "42*B*H*L^2*d per step (6 fwd + 15 bwd GEMM-units)", "l2": TIMING_NOTE}

    if args.impl == "reference":
        if rank != 0:
            return
        import torch
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        from oracle import torch_cpu_path
        fn, kind = cpu_arm()
        inputs = torch_cpu_path.make_inputs(B, H, L, D, torch.float32, seed=0)  # drawn once, outside the timed region
        for _ in range(max(min(args.warmup, 3), 1)):
            torch_cpu_path.fwd_bwd(inputs, fn)
        times = []
        for _ in range(max(args.steps, 1)):
            t0 = time.perf_counter()
            torch_cpu_path.fwd_bwd(inputs, fn)
            times.append((time.perf_counter() - t0) * 1e3)
        ms = sum(times) / len(times)
        val = flops / (ms * 1e-3) / 1e12
        what = ("the reference's naive_multihead_attention_jvp + torch.autograd.grad" if kind == "reference"
                else "restatement of the reference's naive_multihead_attention_jvp + torch.autograd.grad")
        print(json.dumps({
            "impl": "reference", "metric": "jvp_attn_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "ms_per_step_median": statistics.median(times),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": kind,
                             "sample": f"the full workload per step (one batch of B{B} H{H} L{L} d{D}), fp32, {what}; "
                                       "rank 0 only"},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
        return

    import torch
    from semicat_b200 import _lib
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path (use --impl reference for the CPU arm)")
    _lib.load()
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=device)
        dist = dist_mod

    # rotate over enough resident input sets that consecutive steps never find their data in the 126 MB L2
    host_sets = [host_inputs(cfg, seed=1000 * rank + i) for i in range(4)]
    sets = [DeviceSet(hs, device) for hs in host_sets]
    resident_mb = sum(s.nbytes() for s in sets) / 1e6
    while resident_mb < 400 and len(sets) < 16:
        host_sets.append(host_inputs(cfg, seed=1000 * rank + len(sets)))
        sets.append(DeviceSet(host_sets[-1], device))
        resident_mb = sum(s.nbytes() for s in sets) / 1e6
    resident_note = f"{len(sets)} resident input/output sets, {resident_mb:.0f} MB"

    sampler = ClockSampler(local_rank)
    ms, launched, mode = run_device(cfg, sets, args.steps, args.warmup, dist, sampler, use_graph=not args.profile_mode)
    e2e_steps = max(3, min(args.steps, 20))
    if args.profile_mode:
        args.no_extras = True
        e2e_ms, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_ms, h2d, d2h = run_e2e(cfg, host_sets, e2e_steps, min(args.warmup, 3), device, dist, sampler)
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    ms_per_step = ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    e2e_value = world * flops / (e2e_ms / e2e_steps * 1e-3) / 1e12

    line = {
        "metric": "jvp_attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "api": "sdpa_jvp under torch.func.jvp + torch.autograd.grad, pinned host buffers, two steps in flight on two streams"},
        "gpu_launches": int(launched), "launch_mode": mode, "resident": resident_note,
    }

    if rank == 0:
        pk = peaks()
        T = 2.0 * B * H * L * D
        stat = 4.0 * B * H * L
        # algorithmic bytes / FLOPs of each kernel: the tensors it must read and write once
        model = {
            "sm100_fwd_kernel": (8 * T + 2 * stat, 6),
            "row_dots_kernel": (4 * T + 2 * stat, 0),
            "sm100_bwd_kernel<query owner>": (10 * T + 4 * stat, 9),
            "sm100_bwd_kernel<key owner>": (12 * T + 4 * stat, 12),
        }
        with sampler:
            prof = run_profile(sets, max(8, min(args.steps, 40)))
        total = sum(v[0] for v in prof.values()) or 1.0
        unit_flops = 2.0 * B * H * L * L * D
        kernels = []
        for name, (tot_ms, n) in sorted(prof.items(), key=lambda kv: -kv[1][0]):
            by, units = model.get(name, (0.0, 0))
            avg = tot_ms / n
            kernels.append({"kernel": name, "launches": n, "avg_ms": avg, "share": tot_ms / total,
                            "gb_s": by / (avg * 1e-3) / 1e9, "executed_tflops": units * unit_flops / (avg * 1e-3) / 1e12})
        line["kernels"] = kernels
        intensity = flops / (24 * T)
        bound = "hbm" if intensity < pk["bf16_tflops"] * 1e12 / (pk["hbm_gbs"] * 1e9) else "tensor"
        top = kernels[0]
        if bound == "hbm":
            line["roofline"] = {"bound": "hbm", "kernel": top["kernel"], "achieved": top["gb_s"], "peak": pk["hbm_gbs"],
                                "unit": "GB/s", "frac": top["gb_s"] / pk["hbm_gbs"],
                                "traffic": ncu_traffic(args.workload, top["kernel"]),
                                "peak_source": pk["source"]}
        else:
            line["roofline"] = {"bound": "tensor", "kernel": top["kernel"], "achieved": top["executed_tflops"],
                                "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": top["executed_tflops"] / pk["bf16_tflops"],
                                "traffic": None, "peak_source": pk["source"]}
        # whole-step view against the binding ceiling: max(FLOPs / tensor peak, bytes / HBM peak)
        t_roof = max(flops / (pk["bf16_tflops"] * 1e12), (24 * T + 6 * stat) / (pk["hbm_gbs"] * 1e9))
        line["step_roofline"] = {"t_roof_ms": t_roof * 1e3, "frac_of_t_roof": t_roof * 1e3 / ms_per_step,
                                 "frac_of_bf16_peak": value / world / pk["bf16_tflops"]}
        if not args.no_extras and world == 1:
            del sets, host_sets
            torch.cuda.empty_cache()
            big = WORKLOADS["L2048_d64"]
            bsets = [DeviceSet(host_inputs(big, seed=7 + i), device) for i in range(2)]
            with sampler:
                bms, _, _ = run_device(big, bsets, 6, 3, None, ClockSampler(local_rank))
                bprof = run_profile(bsets, 4)
            bf = flops_per_step(big["B"], big["H"], big["L"], big["D"])
            tf = bf / (bms / 6 * 1e-3) / 1e12
            line["long_sequence"] = {"workload": "B32 H16 L2048 d64 bf16, N(0,1) primals and tangents", "ms_per_step": bms / 6,
                                     "tflops": tf, "frac_of_bf16_peak": tf / pk["bf16_tflops"],
                                     "kernel_ms": {k_: v_[0] / v_[1] for k_, v_ in bprof.items()}}
            del bsets
            cpu_s, cores, cpu_kind = cpu_path(cfg, repeats=3)
            line["cpu_baseline"] = {"value": flops / cpu_s / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": cpu_kind,
                                    "sample": "the full config-2 workload, fp32, best of 3 "
                                              f"({cpu_s * 1e3:.0f} ms per fwd+bwd)"}
    if not args.no_extras:
        # DiT flow-map training (BASELINE config 3) at the same N: fixed global batch 512, sharded over the ranks
        try:
            sets = host_sets = None  # release the attention buffers before the model is built
            torch.cuda.empty_cache()
            tr = run_train("dit_lm1b", max(args.steps, 20) if args.steps >= 20 else args.steps, max(args.warmup, 5) if args.steps >= 20 else max(args.warmup, 3),
                           device, rank, world, dist, ClockSampler(local_rank), sd_prop=0.25)
            line["train"] = train_block(tr, world, peaks(), "DiT 12x768, 12 heads, vocab 30522, seq 128, global batch 512, "
                                        "sd_prop 0.25 (lag), bf16 autocast, AdamW, uniform random tokens")
        except Exception as e:  # the attention line above stands on its own
            line["train"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0:
        line["clocks"] = sampler.summary()
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main_sweep(args):
    """`--workload sweep5`: BASELINE config 5, the long-sequence sweep (H=16, d in {64,128}, L in {1024..8192},
    B*L = 65536, N(0,1) primals and tangents), fused fwd+bwd TFLOP/s per shape on one GPU.  One JSON line."""
    import torch
    from semicat_b200 import _lib
    _lib.load()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    pk = peaks()
    rows = []
    for D in (64, 128):
        for L in (1024, 2048, 4096, 8192):
            cfg = dict(B=65536 // L, H=16, L=L, D=D, q_scale=1.0, t_scale=1.0)
            sets = [DeviceSet(host_inputs(cfg, seed=i), device) for i in range(2)]
            ms, _, _ = run_device(cfg, sets, max(2, min(args.steps, 6)), 3, None, ClockSampler(0), use_graph=False)
            prof = run_profile(sets, 2)
            steps = max(2, min(args.steps, 6))
            fl = flops_per_step(cfg["B"], 16, L, D)
            tf = fl / (ms / steps * 1e-3) / 1e12
            rows.append({"L": L, "d": D, "B": cfg["B"], "ms_per_step": ms / steps, "tflops": tf,
                         "frac_of_bf16_peak": tf / pk["bf16_tflops"],
                         "kernel_ms": {k_: v_[0] / v_[1] for k_, v_ in prof.items()}})
            del sets
            torch.cuda.empty_cache()
    print(json.dumps({"metric": "jvp_attn_fwd_bwd_tflops", "unit": "TFLOP/s", "workload": "config 5 sweep, bf16, H16, B*L=65536",
                      "peak": pk, "sweep": rows}))


def kernel_mix(args):
    """`--kernel-mix` with a training workload: one eager step under the torch profiler (after three warm-up steps), one
    GPU; prints where the device time of the step goes, by kernel family and by operator.  Not a timing of the step (the
    profiler serialises the launches); the timed numbers come from the plain run."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from semicat_b200 import _lib, train_step
    _lib.load()
    device = torch.device("cuda", 0)
    tc = dict(TRAIN_CONFIGS[args.workload])
    B = args.global_batch or tc["global_batch"]
    torch.manual_seed(1234)
    net = train_step.DiT(tc["vocab"], 768, 128, 12, 12, dropout=0.1, length=tc["length"], embed_type=tc["embed"]).to(device)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, weight_decay=0.0, fused=True)
    x1 = torch.randint(0, tc["vocab"], (B, tc["length"]), device=device)

    def step():
        noise = train_step.draw_noise(x1, tc["vocab"])
        vf, sd = train_step.model_step(net, x1, noise, sd_prop=args.sd_prop, jvp_attention="jvp",
                                       primal_attention=args.primal_attention, overlap_branches=not args.no_overlap)
        opt.zero_grad(set_to_none=True)
        train_step.total_loss(vf, sd).backward()
        opt.step()

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        step()
        torch.cuda.synchronize()
    rows = prof.key_averages()
    kernels = [r for r in rows if r.device_type.name == "CUDA"]
    ops = [r for r in rows if r.device_type.name != "CUDA" and r.self_device_time_total > 0]

    def family(name):
        if "nvjet" in name or "gemm" in name.lower() or "cutlass" in name:
            return "library GEMM"
        if "jvpattn" in name:
            return "this library: attention" if ("sm100_" in name or "row_dots" in name or "simt_" in name) else "this library: other"
        if "Optimizer" in name or "multi_tensor" in name:
            return "optimizer"
        if "Memcpy" in name or "Memset" in name:
            return "memcpy / memset"
        return "PyTorch elementwise / reduction / copy"

    fam = {}
    for r in kernels:
        if r.key.startswith("Optimizer.step"):
            continue  # the profiler's own range around the optimizer, not a kernel
        f = fam.setdefault(family(r.key), [0.0, 0])
        f[0] += r.self_device_time_total
        f[1] += r.count
    total = sum(v[0] for v in fam.values())
    print(json.dumps({
        "workload": f"{args.workload}, batch {B} on one GPU, sd_prop {args.sd_prop}, one eager step under torch.profiler",
        "device_ms_summed_over_kernels": total / 1e3, "kernels": sum(v[1] for v in fam.values()),
        "by_family_ms": {k: {"ms": v[0] / 1e3, "launches": v[1]} for k, v in sorted(fam.items(), key=lambda kv: -kv[1][0])},
        "top_operators_ms": [{"op": r.key, "ms": r.self_device_time_total / 1e3, "calls": r.count}
                             for r in sorted(ops, key=lambda r: -r.self_device_time_total)[:30]]}))


def main_train(args):
    """`--workload dit_lm1b | dit_text8`: the training step is the benchmark step; metric = tokens/s."""
    import torch
    from semicat_b200 import _lib, ddp
    if args.kernel_mix:
        return kernel_mix(args)
    _lib.load()
    rank, world, local_rank = ddp.init_from_env("nccl")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    import torch.distributed as dist_mod
    dist = dist_mod if world > 1 else None
    sampler = ClockSampler(local_rank)
    launches0 = _lib.launch_count()
    tr = run_train(args.workload, args.steps, max(args.warmup, 3), device, rank, world, dist,
                   sampler, sd_prop=args.sd_prop, use_graph=not args.profile_mode, primal_attention=args.primal_attention,
                   global_batch=args.global_batch, overlap=not args.no_overlap)
    ms, tokens, loss, peak_gb, mode = tr["ms_per_step"], tr["tokens_per_step"], tr["loss"], tr["peak_mem_gb"], tr["launch"]
    launched = _lib.launch_count() - launches0
    tc = dict(TRAIN_CONFIGS[args.workload])
    if args.global_batch:
        tc["global_batch"] = args.global_batch
    if rank == 0:
        val = tokens / (ms * 1e-3)
        print(json.dumps({
            "metric": "dit_jvp_train_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: DiT 12x768/12 heads, vocab {tc['vocab']}, seq {tc['length']}, global batch "
                                   f"{tc['global_batch']}, sd_prop {args.sd_prop} (lag), AdamW", "parallelism": f"dp{world}",
                       "l2": "activations per step far exceed the 126 MB L2", "launch": mode},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": tokens * 8 // world, "d2h_bytes_per_step": 4,
                    "note": "token ids come from pinned host memory and the loss goes back to the host every step"},
            "gpu_launches": int(launched), "loss": loss, "peak_mem_gb": peak_gb, "clocks": sampler.summary(),
            "train": train_block(tr, world, peaks(), args.workload),
        }))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
