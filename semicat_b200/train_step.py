"""The caller of the hot path, restated for measurement: the adaLN DiT denoiser and the flow-map training
step that pushes ``torch.func.jvp`` through it.

This is NOT part of the kernel library; it exists so that ``bench.py`` can report DiT JVP-training
tokens/s on the reference's architecture without depending on the reference package, Lightning or Hydra.
:func:`load_reference_state` copies the parameters of a reference ``DIT`` into this restatement (the tests use it
to check the two models against each other).  Architecture and objective follow the reference:

* denoiser: semicat/net/duo.py:299-360 (``DIT``), blocks :101-166 (LayerNorm, adaLN modulation with
  zero-initialised projection, bias-free qkv, rotary on q and k in fp32, attention through
  ``safe_sdpa_jvp`` when ``jvp_attention`` else ``F.scaled_dot_product_attention``, 4x GELU-tanh MLP, gates),
  timestep embedders :69-93 on ``s`` and ``t - s``, dense (B, L, V) input embedding :169-180 / :205-296,
  zero-initialised adaLN output layer :183-202;
* objective: semicat/models/semicat.py:169-191 (``model_step``: the first ``sd_prop`` of the batch takes the
  self-distillation step, the rest the cross-entropy step), :89-110 (VFM step), :112-167 (``lag``
  self-distillation: ``torch.func.jvp`` of the flow map x_{s,t} with respect to t, squared error against
  a no-grad target), :210-229 (flow map), :70-85 (interpolation towards the one-hot token).
"""
from __future__ import annotations

import contextlib
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import vocab_ops
from .dual_ops import dropout_seed, flow_map_head, gated_residual, gelu_tanh, ln_modulate
from .dual_ops import linear as dual_linear
from .functional import safe_sdpa_jvp
from .rotary import apply_rotary_cast, rotary_qkv


def _rotate(x, cos, sin):
    """Non-interleaved rotary embedding on (B, S, H, D); cos/sin are (S, D/2) fp32, so the result is fp32
    (the reference's q and k reach the attention in fp32 under bf16 autocast for the same reason)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    cos, sin = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1)


def _prepare_aligned(lin: nn.Linear, in_scale: float, dtype):
    """Weight and bias of a vocabulary-sized ``nn.Linear`` scaled, cast and zero-padded to multiples of 8 once."""
    w, b = lin.weight, lin.bias
    if in_scale != 1.0:
        w = w * in_scale
    n_out, n_in = w.shape
    pad_in, pad_out = (-n_in) % 8, (-n_out) % 8
    if dtype is not None:
        w = w.to(dtype)
        b = b.to(dtype) if b is not None else None
    if pad_in:
        w = F.pad(w, (0, pad_in))
    if pad_out:
        w = F.pad(w, (0, 0, 0, pad_out))
        b = F.pad(b, (0, pad_out)) if b is not None else None
    return w, b


def _aligned_linear(x, lin: nn.Linear, in_scale: float = 1.0, keep_padding: bool = False):
    """``lin(x * in_scale)`` with the vocabulary-sized dimension padded to a multiple of 8 elements.  ``x`` may already be
    in the padded layout (``vocab_ops.interpolate_cast``); with ``keep_padding`` the padded output columns (zeros) stay.

    30522 is not a multiple of 8, so the operand rows of the embedding and head GEMMs are only 4-byte aligned and
    the BLAS library falls back to its pre-Hopper kernels for them (17 % of the step).  Zero columns / rows change
    nothing in the products; ``in_scale`` is folded into the weight instead of a pass over the (B, L, V) input.
    ``model_step`` prepares the padded weight once per step (``lin._prepared``) for its three passes."""
    if not x.is_cuda:
        w = lin.weight * in_scale if in_scale != 1.0 else lin.weight
        return F.linear(x, w, lin.bias)
    n_out, n_in = lin.weight.shape
    pad_in, pad_out = (-n_in) % 8, (-n_out) % 8
    dt = torch.get_autocast_dtype("cuda") if torch.is_autocast_enabled("cuda") else None
    prepared = getattr(lin, "_prepared", None)
    w, b = prepared if prepared is not None else _prepare_aligned(lin, in_scale, dt if pad_in else None)
    if pad_in and x.shape[-1] != n_in + pad_in:
        x = F.pad(x.to(w.dtype), (0, pad_in))
    y = dual_linear(x, w, b)
    return y[..., :n_out] if pad_out and not keep_padding else y


class TimeEmbed(nn.Module):
    def __init__(self, dim, n_freq=256, max_period=10000):
        super().__init__()
        self.mlp = nn.Sequential(nn.Linear(n_freq, dim), nn.SiLU(), nn.Linear(dim, dim))
        half = n_freq // 2
        self.register_buffer("freqs", torch.exp(-math.log(max_period) * torch.arange(half) / half))

    def forward(self, t):
        a = t[:, None] * self.freqs[None]
        return self.mlp(torch.cat((a.cos(), a.sin()), dim=-1))


class Block(nn.Module):
    def __init__(self, dim, heads, cond_dim, dropout):
        super().__init__()
        self.heads, self.dim = heads, dim
        self.norm1, self.norm2 = nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.attn_qkv = nn.Linear(dim, 3 * dim, bias=False)
        self.attn_out = nn.Linear(dim, dim, bias=False)
        self.mlp = nn.Sequential(nn.Linear(dim, 4 * dim), nn.GELU(approximate="tanh"), nn.Linear(4 * dim, dim))
        self.drop = nn.Dropout(dropout)
        self.ada = nn.Linear(cond_dim, 6 * dim)
        nn.init.zeros_(self.ada.weight)
        nn.init.zeros_(self.ada.bias)

    def forward(self, x, cos, sin, c, attention):
        B, S, _ = x.shape
        # On the GPU the pointwise chain around the attention runs as fused (primal, tangent) kernels (dual_ops); the
        # plain-formula path ("math") keeps the PyTorch expressions and serves as the independent check.
        fused = x.is_cuda and attention != "math"
        mod = dual_linear(c, self.ada.weight, self.ada.bias) if fused else self.ada(c)
        sh1, sc1, g1, sh2, sc2, g2 = mod[:, None].chunk(6, dim=2)
        h = ln_modulate(x, self.norm1, sh1, sc1) if fused else self.norm1(x) * (1.0 + sc1) + sh1
        lin = (lambda m, z: dual_linear(z, m.weight, m.bias)) if fused else (lambda m, z: m(z))
        qkv = lin(self.attn_qkv, h).reshape(B, S, 3, self.heads, self.dim // self.heads)
        if x.is_cuda and attention != "math":
            # one kernel for the split, the rotation of q and k and the cast of all three (and one for their gradients,
            # which lands in the projection's gradient directly) instead of the fp32 pointwise chain plus the casts to bf16
            rot_dtype = qkv.dtype if qkv.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16
            q, k, v = rotary_qkv(qkv, cos, sin, rot_dtype)
        else:
            q, k, v = qkv.unbind(2)
            q, k = _rotate(q, cos, sin), _rotate(k, cos, sin)
        if attention in ("jvp", "lib"):
            # the library's kernels: fused JVP attention where the inputs carry forward-mode tangents, the primal-only
            # instance of the same kernels where they do not ("lib" names that use in the non-JVP passes)
            a = safe_sdpa_jvp(q, k, v)
        elif attention == "math":  # plain formula: supports forward-mode AD anywhere (used by the CPU tests)
            qh, kh, vh = (z.transpose(1, 2).float() for z in (q, k, v))
            w = torch.softmax(qh @ kh.transpose(-1, -2) / math.sqrt(qh.shape[-1]), dim=-1)
            a = (w @ vh).transpose(1, 2).to(x.dtype)
        else:
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2).to(q.dtype)).transpose(1, 2)
        if fused:
            x = gated_residual(x, lin(self.attn_out, a.reshape(B, S, self.dim).to(h.dtype)), g1, self.drop.p, self.training)
            m = lin(self.mlp[2], gelu_tanh(lin(self.mlp[0], ln_modulate(x, self.norm2, sh2, sc2))))
            return gated_residual(x, m, g2, self.drop.p, self.training)
        x = self.drop(self.attn_out(a.reshape(B, S, self.dim).to(h.dtype)) * g1) + x
        return self.drop(self.mlp(self.norm2(x) * (1.0 + sc2) + sh2) * g2) + x


class RmsEmbed(nn.Module):
    """duo.py:205-296: RMS time scaling, projection, small residual MLP, FiLM on the condition, RMSNorm."""

    def __init__(self, vocab, dim, cond_dim, residual_scale=0.1, eps=1e-6):
        super().__init__()
        self.vocab, self.eps, self.res = vocab, eps, residual_scale
        self.proj = nn.Linear(vocab, dim)
        self.mlp = nn.Sequential(nn.Linear(dim, 2 * dim), nn.GELU(approximate="tanh"), nn.Linear(2 * dim, dim))
        self.gamma, self.beta = nn.Linear(cond_dim, dim), nn.Linear(cond_dim, dim)
        self.norm = nn.RMSNorm(dim, eps=1e-8)
        for lin in (self.gamma, self.beta):
            nn.init.zeros_(lin.weight)
            nn.init.zeros_(lin.bias)

    def forward(self, x, t, cond):
        scale = torch.rsqrt(t ** 2 + (1.0 - t) ** 2 * self.vocab + self.eps).view(-1, 1, 1)
        h = self.proj(x * scale)
        h = h + self.res * self.mlp(h)
        return self.norm((1.0 + self.gamma(cond).unsqueeze(1)) * h + self.beta(cond).unsqueeze(1))


class NaiveEmbed(nn.Module):
    def __init__(self, vocab, dim):
        super().__init__()
        self.seq = nn.Linear(vocab, dim)
        self.coeff = vocab ** 0.5

    def forward(self, x, t, cond):
        return _aligned_linear(x, self.seq, 1.0 / self.coeff)


class DiT(nn.Module):
    def __init__(self, vocab_size, hidden_size=768, cond_dim=128, n_blocks=12, n_heads=12, dropout=0.1, length=128,
                 embed_type="naive"):
        super().__init__()
        self.embed = NaiveEmbed(vocab_size, hidden_size) if embed_type == "naive" else RmsEmbed(vocab_size, hidden_size, cond_dim)
        self.s_map, self.t_map = TimeEmbed(cond_dim), TimeEmbed(cond_dim)
        d = hidden_size // n_heads
        ang = torch.arange(length)[:, None] * (1.0 / (10000 ** (torch.arange(0, d, 2) / d)))[None]
        self.register_buffer("cos", ang.cos())
        self.register_buffer("sin", ang.sin())
        self.blocks = nn.ModuleList(Block(hidden_size, n_heads, cond_dim, dropout) for _ in range(n_blocks))
        self.norm_out = nn.LayerNorm(hidden_size)
        self.ada_out = nn.Linear(cond_dim, 2 * hidden_size)
        self.head = nn.Linear(hidden_size, vocab_size)
        for lin in (self.ada_out, self.head):
            nn.init.zeros_(lin.weight)
            nn.init.zeros_(lin.bias)

    def forward(self, x, s, t, attention="sdpa", padded_logits=False):
        """``x``: (B, L, V) as the reference passes it, or (B, L, padded V) 16-bit from ``vocab_ops.interpolate_cast``.
        ``padded_logits`` keeps the head GEMM's padded output columns (zeros) for the fused vocabulary-side losses."""
        cond = F.silu(self.s_map(s)) + F.silu(self.t_map(t - s))
        h = self.embed(x, s, cond)
        for blk in self.blocks:
            h = blk(h, self.cos, self.sin, cond, attention)
        fused = h.is_cuda and attention != "math"
        mod = dual_linear(cond, self.ada_out.weight, self.ada_out.bias) if fused else self.ada_out(cond)
        shift, scale = mod[:, None].chunk(2, dim=2)
        out = ln_modulate(h, self.norm_out, shift, scale) if fused else self.norm_out(h) * (1.0 + scale) + shift
        return _aligned_linear(out, self.head, keep_padding=padded_logits)


_REFERENCE_NAMES = (  # prefix in semicat/net/duo.py's DIT -> prefix here
    ("vocab_embed.film_gamma.", "embed.gamma."), ("vocab_embed.film_beta.", "embed.beta."),
    ("vocab_embed.final_norm.", "embed.norm."), ("vocab_embed.", "embed."),
    ("output_layer.norm_final.", "norm_out."), ("output_layer.adaLN_modulation.", "ada_out."),
    ("output_layer.linear.", "head."), (".adaLN_modulation.", ".ada."),
)


def load_reference_state(net: "DiT", reference_state: dict) -> None:
    """Copy the parameters of a reference ``semicat.net.duo.DIT`` (its ``state_dict()``) into ``net``.
    The rotary tables are buffers computed from the shape on both sides and are not copied."""
    mapped = {}
    for name, value in reference_state.items():
        if name.startswith("rotary_emb."):
            continue
        for old, new in _REFERENCE_NAMES:
            if old in name:
                name = name.replace(old, new)
                break
        mapped[name] = value
    own = net.state_dict()
    missing = [k for k in own if k not in mapped and k not in ("cos", "sin")]
    extra = [k for k in mapped if k not in own]
    if missing or extra:
        raise KeyError(f"reference state does not match: missing {missing}, unexpected {extra}")
    net.load_state_dict(mapped, strict=False)


def randomise_zero_init(net: nn.Module, std=0.05, seed=0):
    """A freshly built DiT multiplies its attention branch by zero gates; parity tests un-zero them first."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in net.parameters():
            if p.numel() and not p.any():
                p.copy_(torch.randn(p.shape, generator=g).to(p) * std)


def interpolate(x0, x1, t):
    """(1 - t) x0 + t onehot(x1) without materialising the one-hot (semicat.py:70-85)."""
    xt = x0 * (1.0 - t)
    xt.scatter_add_(-1, x1[..., None], t.expand_as(xt[..., :1]).to(xt.dtype))
    return xt


def flow_map(net, x, s, t, attention):
    dt = (t - s) / (1.0 - s + 1e-8)
    logits = net(x, s, t, attention=attention)
    if logits.is_cuda and attention != "math":  # one fused pass over the vocabulary axis (primal, tangent and their VJPs)
        return flow_map_head(logits, x, dt)
    diff = logits.softmax(dim=-1) - x
    return x + dt.view(-1, 1, 1) * diff


def draw_noise(x1, vocab, generator=None, out=None):
    """The random draws of one step, separated out so that tests can inject the same draws everywhere.  On the GPU the
    noise rows are spaced a multiple of 8 columns apart (16-byte aligned rows for the fused vocabulary-side kernels);
    ``x0`` is the (B, L, vocab) view of that buffer.  With ``out`` (a dict this function returned) the same buffers are
    refilled in place, which lets a training loop draw the next step's noise while the current step is still running
    (see ``model_step(noise_released=...)``)."""
    B = x1.shape[0]
    dev = x1.device
    if out is not None:
        out["x0_buffer"].normal_(generator=generator)
        for k in ("t_vfm", "t_sd", "u_sd"):
            out[k].uniform_(generator=generator)
        return out
    width = vocab_ops.padded(vocab) if dev.type == "cuda" else vocab
    buf = torch.randn(B, x1.shape[1], width, device=dev, generator=generator)
    return {"x0": buf[..., :vocab], "x0_buffer": buf,
            "t_vfm": torch.rand(B, device=dev, generator=generator), "t_sd": torch.rand(B, device=dev, generator=generator),
            "u_sd": torch.rand(B, device=dev, generator=generator)}


def _fused_vocabulary_side(net, x0, attention, dtype) -> bool:
    """The fused vocabulary-side kernels serve the dense ("naive") embedding on the GPU at vocabularies where a row is
    worth a CTA; the plain-formula path ("math") keeps the PyTorch expressions and serves as the independent check."""
    return (attention != "math" and isinstance(net.embed, NaiveEmbed) and x0.shape[-1] >= 512 and vocab_ops.usable(x0, dtype))


_SIDE_STREAMS: dict = {}


def _side_stream(device):
    if device not in _SIDE_STREAMS:
        _SIDE_STREAMS[device] = torch.cuda.Stream(device)
        # a parameter's gradient now arrives from two streams; autograd synchronises them itself and only warns about it
        torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
    return _SIDE_STREAMS[device]


def _model_step_fused(net, x1, noise, split, jvp_attention, primal_attention, dtype, label_smoothing, overlap=True,
                      noise_released=None):
    """``model_step`` with the (B, L, V) tensors kept in one 16-bit padded layout between the noise and the two scalar
    losses (vocab_ops): same objective, same rounding points at the network's boundary (input and logits in ``dtype``).

    The cross-entropy branch and the self-distillation branch share nothing but the weights, so with ``overlap`` the
    first runs on a second stream (forward here; autograd runs each backward node on its forward's stream): at a few
    dozen samples per GPU a single branch's kernels do not fill 148 SMs.  Captured into a CUDA graph the two streams become
    two parallel branches of the graph."""
    B = x1.shape[0]
    x0 = noise["x0"]
    V = x0.shape[-1]
    vf_loss = sd_loss = None
    both = 0 < split < B
    main = torch.cuda.current_stream(x1.device)
    side = _side_stream(x1.device) if (overlap and both) else main
    if split < B:
        side.wait_stream(main)
        with torch.cuda.stream(side):
            t = noise["t_vfm"][split:]
            xt = vocab_ops.interpolate_cast(x0[split:], x1[split:], t, dtype)
            pred = net(xt, t, t, attention=primal_attention, padded_logits=True)
            vf_loss = vocab_ops.cross_entropy_padded(pred, x1[split:], V, label_smoothing)
            del xt, pred
    if split > 0:
        t = noise["t_sd"][:split]
        s = noise["u_sd"][:split] * t
        xs = vocab_ops.interpolate_cast(x0[:split], x1[:split], s, dtype)
        logits, tlogits = torch.func.jvp(lambda _t: net(xs, s, _t, attention=jvp_attention, padded_logits=True), (t,), (torch.ones_like(t),))
        xst, lse = vocab_ops.flow_map_input(logits, x0[:split], x1[:split], s, t)
        with torch.no_grad():
            target = net(xst, t, t, attention=primal_attention, padded_logits=True)
        sd_loss = vocab_ops.sd_lag_loss(logits, tlogits, target, x0[:split], x1[:split], s, t, lse)
        if noise_released is not None:
            # the last reader of the noise is the backward kernel of this loss, the first node of the reverse pass: the
            # gradient of the logits exists as soon as it has been enqueued
            logits.register_hook(lambda _g: noise_released())
    elif noise_released is not None:
        noise_released()
    main.wait_stream(side)
    return vf_loss, sd_loss


class _CastParams(torch.autograd.Function):
    """All 16-bit copies of a step in one node: the casts run as a few multi-tensor launches into one flat buffer instead of
    one kernel per parameter, and so do the casts of their gradients back to fp32 in the backward."""

    @staticmethod
    def forward(ctx, dtype, *params):
        flat = torch.empty(sum(p.numel() for p in params), dtype=dtype, device=params[0].device)
        outs, off = [], 0
        for p in params:
            outs.append(flat[off:off + p.numel()].view(p.shape))
            off += p.numel()
        torch._foreach_copy_(outs, [p.detach() for p in params])
        ctx.shapes = [p.shape for p in params]
        ctx.param_dtype = params[0].dtype
        return tuple(outs)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, *grads):
        live = [i for i, g in enumerate(grads) if g is not None]
        if not live:
            return (None,) * (1 + len(grads))
        flat = torch.empty(sum(grads[i].numel() for i in live), dtype=ctx.param_dtype, device=grads[live[0]].device)
        outs, off = [None] * len(grads), 0
        for i in live:
            n = grads[i].numel()
            outs[i] = flat[off:off + n].view(ctx.shapes[i])
            off += n
        torch._foreach_copy_([outs[i] for i in live], [grads[i] for i in live])
        return (None, *outs)


class _StepCasts:
    """The 16-bit copies of the ``nn.Linear`` parameters for one objective evaluation, made once and shared by its three
    passes.  Autocast keeps such a cache itself, but not inside ``torch.func.jvp`` (wrapped tensors are not leaves), where
    every use of a weight was cast again: five casts per parameter and step.  The casts are one differentiable node
    (``_CastParams``), so a weight's gradients from the passes are summed in 16 bits and cast back to fp32 once."""

    def __init__(self, net, dtype):
        self.net, self.params, self.aligned = net, {}, []
        if dtype is None or not next(net.parameters()).is_cuda:
            return
        vocab_sized = {id(net.head): 1.0}
        if isinstance(net.embed, NaiveEmbed):
            vocab_sized[id(net.embed.seq)] = 1.0 / net.embed.coeff
        names, tensors = [], []
        for mname, m in net.named_modules():
            if not isinstance(m, nn.Linear):
                continue
            if id(m) in vocab_sized:
                m._prepared = _prepare_aligned(m, vocab_sized[id(m)], dtype)
                self.aligned.append(m)
            else:
                for pname, p in m.named_parameters(recurse=False):
                    names.append(f"{mname}.{pname}")
                    tensors.append(p)
        # A few nodes rather than one: a node's backward runs when the gradients of ALL its outputs exist, and a
        # data-parallel caller wants the late layers' gradients early (to exchange them under the rest of the backward).
        total, groups, start, acc = sum(t.numel() for t in tensors), 4, 0, 0
        for i, t in enumerate(tensors):
            acc += t.numel()
            if acc >= total / groups or i == len(tensors) - 1:
                cast = _CastParams.apply(dtype, *tensors[start:i + 1])
                self.params.update(zip(names[start:i + 1], cast))
                start, acc = i + 1, 0

    def __call__(self, *args, **kwargs):
        if not self.params:
            return self.net(*args, **kwargs)
        return torch.func.functional_call(self.net, self.params, args, kwargs)

    def close(self):
        for m in self.aligned:
            m._prepared = None


def model_step(net, x1, noise, sd_prop=0.25, jvp_attention="jvp", autocast_dtype=torch.bfloat16, label_smoothing=0.0,
               primal_attention="sdpa", overlap_branches=True, noise_released=None):
    """One training objective evaluation: returns (vfm_loss, sd_loss or None).  ``x1`` are token ids (B, L).
    ``jvp_attention`` selects the attention of the forward-mode pass, ``primal_attention`` that of the passes without
    tangents (the cross-entropy step and the no-grad target): "sdpa" is ``F.scaled_dot_product_attention`` as in the
    reference (semicat/net/duo.py:143-152), "lib" this library's primal-only kernels, "math" the plain formula.
    ``noise_released``: optional callable, invoked on the host as soon as the last kernel that reads ``noise`` has been
    enqueued (during ``backward()`` when the self-distillation loss reads the noise again, else before this returns); the
    stream that is current at that moment is the one the reader was enqueued on.  A training loop uses it to refill the
    noise buffers for the next step on another stream under the rest of the backward."""
    B = x1.shape[0]
    split = int(sd_prop * B)
    dev_type = x1.device.type
    x0 = noise["x0"]
    # One autocast region for the whole objective: the bf16 copies of the weights that autocast makes are cached per
    # region, so the cross-entropy pass, the forward-mode pass and the no-grad target pass share one set of casts.
    model = net
    net = _StepCasts(model, autocast_dtype)  # called like the model; shares one set of 16-bit weights between the passes
    # one device-side seed for every dropout mask of the step (the fused kernels regenerate the masks from it)
    seeded = dropout_seed(x1.device) if x1.is_cuda and jvp_attention != "math" else contextlib.nullcontext()
    try:
        with seeded:
            return _model_step(model, net, x1, noise, split, jvp_attention, autocast_dtype, label_smoothing, primal_attention,
                               overlap_branches, noise_released)
    finally:
        net.close()


def _model_step(model, net, x1, noise, split, jvp_attention, autocast_dtype, label_smoothing, primal_attention, overlap_branches,
                noise_released=None):
    B = x1.shape[0]
    dev_type = x1.device.type
    x0 = noise["x0"]
    with torch.autocast(dev_type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
        io_dtype = autocast_dtype if autocast_dtype is not None else torch.float32
        if _fused_vocabulary_side(model, x0, jvp_attention, io_dtype) and primal_attention != "math":
            return _model_step_fused(net, x1, noise, split, jvp_attention, primal_attention, io_dtype, label_smoothing,
                                     overlap_branches, noise_released)
        # VFM step on the tail of the batch
        vf_loss = None
        if split < B:
            t = noise["t_vfm"][split:]
            xt = interpolate(x0[split:], x1[split:], t.view(-1, 1, 1))
            pred = net(xt, t, t, attention=primal_attention)
            # Same value as the reference's F.cross_entropy(pred.transpose(-1, 1), x1) (semicat.py:107-111): mean over all
            # tokens.  With the classes innermost the log-softmax over the 30522-entry vocabulary runs as a row softmax;
            # in the transposed (B, V, L) layout it is a strided "spatial" softmax that took a third of the whole step.
            vf_loss = F.cross_entropy(pred.float().reshape(-1, pred.shape[-1]), x1[split:].reshape(-1), label_smoothing=label_smoothing)
        if split == 0:
            if noise_released is not None:
                noise_released()
            return vf_loss, None
        # self-distillation ("lag") step on the head of the batch: d/dt of the flow map by forward-mode AD
        t = noise["t_sd"][:split]
        s = noise["u_sd"][:split] * t
        xs = interpolate(x0[:split], x1[:split], s.view(-1, 1, 1))
        xst, dv = torch.func.jvp(lambda _t: flow_map(net, xs, s, _t, jvp_attention), (t,), (torch.ones_like(t),))
        xst = xst.detach()
        with torch.no_grad():
            target = net(xst, t, t, attention=primal_attention).softmax(dim=-1)
    sd_loss = ((1.0 - t).view(-1, 1, 1) * dv - target + xst).pow(2).sum(dim=-1).mean()
    if noise_released is not None:
        noise_released()  # this path reads the noise in the forward only (the interpolated inputs are tensors of their own)
    return vf_loss, sd_loss


def total_loss(vf_loss, sd_loss):
    if vf_loss is None:
        return sd_loss
    return vf_loss if sd_loss is None else vf_loss + sd_loss
