"""Generate the golden fixtures in this folder by running the REFERENCE's own CPU implementation.

Run once, in a container where the reference checkout is mounted (it is not needed afterwards;
the ``.npz`` files are committed and nothing at test time reads the reference):

    python tests/golden/make_golden.py /path/to/reference

Source of truth: ``semicat.jvp_utils.ryu_triton.naive_multihead_attention_jvp``
(semicat/jvp_utils/ryu_triton.py:426-454) for (O, Od), differentiated with
``torch.autograd.grad`` for the six VJPs (the reference has no CPU backward; its Triton backward
kernels are the hand-derived form of exactly this derivative).  LSE and MU, the two row
statistics the reference's fused kernel stores (ryu_triton.py:271, 286-291), are recomputed from
their definitions with torch in float64.

Cases
  c1_fp32               BASELINE config 1: fp32, B2 H4 L64 d32, seed 0, N(0,1) inputs and cotangents.
  selftest_{0..4}       the five fp16 shapes of the reference's ``test_multihead_correctness``
                        (ryu_triton.py:504-510), seed 42, tangents x0.1, inputs rounded to fp16,
                        evaluated in fp32 from the rounded values.
  c2_small_bf16         the config-2 value distribution (q ~ N(0,1)/sqrt(d), tangents x0.1) on
                        B1 H2 L128 d64, inputs rounded to bf16, evaluated in fp32.
  ragged_bf16           Lq=80, Lk=200, d=64: tails in both sequence axes and Lq != Lk.
"""
from __future__ import annotations

import math
import os
import sys

import numpy as np
import torch


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from semicat.jvp_utils.ryu_triton import naive_multihead_attention_jvp

    here = os.path.dirname(os.path.abspath(__file__))

    def evaluate(name, q, k, v, tq, tk, tv, g_o, g_od):
        ins = [x.float().clone().requires_grad_(True) for x in (q, k, v, tq, tk, tv)]
        o, od = naive_multihead_attention_jvp(*ins)
        grads_both = torch.autograd.grad([o, od], ins, [g_o.float(), g_od.float()], retain_graph=True)
        grads_tan = torch.autograd.grad([od], ins, [g_od.float()], retain_graph=True)
        grads_pri = torch.autograd.grad([o], ins, [g_o.float()], allow_unused=True)
        grads_pri = [torch.zeros_like(x) if g is None else g for g, x in zip(grads_pri, ins)]
        q64, k64, tq64, tk64 = (x.double() for x in (q, k, tq, tk))
        scale = 1.0 / math.sqrt(q.shape[-1])
        s = q64 @ k64.transpose(-1, -2) * scale
        p = s.softmax(-1)
        sd = (tq64 @ k64.transpose(-1, -2) + q64 @ tk64.transpose(-1, -2)) * scale
        out = {
            "q": q, "k": k, "v": v, "tq": tq, "tk": tk, "tv": tv, "g_o": g_o, "g_od": g_od,
            "o": o, "od": od, "lse": torch.logsumexp(s, -1), "mu": (p * sd).sum(-1),
        }
        for tag, gs in (("both", grads_both), ("tan", grads_tan), ("pri", grads_pri)):
            for n, g in zip(("dq", "dk", "dv", "dtq", "dtk", "dtv"), gs):
                out[f"{n}_{tag}"] = g
        np.savez_compressed(
            os.path.join(here, name + ".npz"),
            **{n: x.detach().float().numpy() for n, x in out.items()},
        )
        print(name, {n: tuple(x.shape) for n, x in out.items() if n in ("q", "k")})

    # BASELINE config 1
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)
    shp = (2, 4, 64, 32)
    evaluate("c1_fp32", *(r(*shp) for _ in range(8)))

    # the reference's own five self-test shapes, generated the way its test does (one seed, in order)
    torch.manual_seed(42)
    for i, (B, H, L, D) in enumerate([(1, 1, 8, 16), (2, 2, 16, 32), (1, 4, 32, 32), (1, 1, 64, 64), (2, 3, 128, 16)]):
        h = lambda s=1.0: (torch.randn(B, H, L, D, dtype=torch.float16) * s).float()
        q, k, v = h(), h(), h()
        tq, tk, tv = h(0.1), h(0.1), h(0.1)
        evaluate(f"selftest_{i}", q, k, v, tq, tk, tv, h(), h())

    g = torch.Generator().manual_seed(2)
    b = lambda s, *shape: (torch.randn(*shape, generator=g) * s).bfloat16().float()
    shp = (1, 2, 128, 64)
    evaluate("c2_small_bf16", b(1 / 8.0, *shp), b(1, *shp), b(1, *shp), b(.1, *shp), b(.1, *shp), b(.1, *shp),
             b(1, *shp), b(1, *shp))

    g = torch.Generator().manual_seed(3)
    sq, sk = (1, 2, 80, 64), (1, 2, 200, 64)
    evaluate("ragged_bf16", b(1 / 8.0, *sq), b(1, *sk), b(1, *sk), b(.1, *sq), b(.1, *sk), b(.1, *sk),
             b(1, *sq), b(1, *sq))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
