"""Mixers that carry a fixed-size state per sequence instead of a growing cache, and mixers made of two.

Each asks the cache for a row of 32-bit state per sequence (``StateRequest``), zero when a sequence
starts; a step reads the row, walks the step's tokens of that sequence and writes it back, so whole
prompts, pieces of prompts and single tokens give the same result.  The projections run as one
product per mixer over joined weights; gates, decays, step sizes, unit norms and the state are
32-bit in the kernels (csrc/recurrent.cu).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import ops
from ..config.specs import MixerSpec
from .base import Mixer, ParamSpec, StateRequest, build_mixer, build_position, register_mixer


def _pad8(n: int) -> int:
    return (n + 7) & ~7


def _joined(weights, biases, dtype_like: torch.Tensor):
    """Rows of several projections as one matrix (padded with zero rows to a multiple of 8 columns of
    output, so that the product's output rows are whole 16-byte units) and one float32 bias."""
    ws = list(weights)
    if len({w.dtype for w in ws}) > 1:
        ws = [w.float() for w in ws]
    n = sum(w.shape[0] for w in ws)
    pad = _pad8(n) - n
    if pad:
        ws.append(torch.zeros((pad, ws[0].shape[1]), dtype=ws[0].dtype, device=ws[0].device))
    w = torch.cat(ws, 0).contiguous()
    bias = None
    if any(b is not None for b in biases):
        bias = torch.zeros(n + pad, dtype=torch.float32, device=w.device)
        at = 0
        for wi, b in zip(weights, biases):
            if b is not None:
                bias[at:at + wi.shape[0]] = b.float()
            at += wi.shape[0]
    return w, bias


def _finish(o, w, add: Sequence, out: Optional[torch.Tensor]) -> torch.Tensor:
    """The last product of a mixer: out = o . w^T + sum(add) in float32."""
    if len(add) > 2:
        raise ValueError("at most two tensors can be added in the projection's epilogue")
    add = [a() if callable(a) else a for a in add]
    a0 = add[0] if len(add) > 0 else None
    a1 = add[1] if len(add) > 1 else None
    return ops.linear(o, w, None, add0=a0, add1=a1, out_dtype=torch.float32, out=out)


class MatrixLstm(Mixer):
    """The matrix memory of xLSTM (mLSTM).  Per head: q = W_q h / sqrt(dim), k, v; log input gate
    gi = cap tanh((W_i h + b_i) / cap), log forget gate gf = logsigmoid(cap tanh((W_f h + b_f) / cap));
    with a running maximum m (from 0): m' = max(gf + m, gi), S' = e^(gf+m-m') S + e^(gi-m') k v^T, the
    normaliser n' likewise with k alone, o = S'^T q / (max(|n'.q|, e^(-m')) + 1e-6).  Each head's o is
    brought to unit root mean square, the heads are joined, scaled by a weight, gated by sigmoid(W_g h)
    and projected.  Options: ``gate_cap``, ``norm_eps``."""
    capturable = True
    launches_only = True
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.H, self.D, self.V = spec.num_heads, spec.head_dim, spec.value_dim or spec.head_dim
        self.cap = float(spec.option("gate_cap", 0.0))
        self.eps = float(spec.option("norm_eps", 1e-6))
        if not self.cap > 0:
            raise ValueError("mlstm needs a positive gate_cap")
        self.state_size = ops.memory_state_size(ops.MEMORY_GATED, self.H, self.D, self.V)
        self.w_in = self.b_in = self.w_o = self.norm = None

    def parameters(self) -> Dict[str, ParamSpec]:
        H, D, V, W = self.H, self.D, self.V, self.spec.hidden
        return {"q.weight": ParamSpec((H * D, W)), "k.weight": ParamSpec((H * D, W)),
                "v.weight": ParamSpec((H * V, W)), "g.weight": ParamSpec((H * V, W)),
                "o.weight": ParamSpec((W, H * V)), "norm.weight": ParamSpec((H * V,), "vector", "gamma"),
                "i.weight": ParamSpec((H, W)), "i.bias": ParamSpec((H,), "vector", "wide"),
                "f.weight": ParamSpec((H, W)), "f.bias": ParamSpec((H,), "vector", "wide")}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        names = ("q", "k", "v", "g", "i", "f")
        self.w_in, self.b_in = _joined([t[n + ".weight"] for n in names],
                                       [t.get(n + ".bias") for n in names], t["q.weight"])
        self.w_o, self.norm = t["o.weight"], t["norm.weight"]
        H, D, V = self.H, self.D, self.V
        self.off = dict(q=0, k=H * D, v=2 * H * D, g=2 * H * D + H * V, i=2 * H * D + 2 * H * V,
                        f=2 * H * D + 2 * H * V + H)

    def cache_request(self):
        return StateRequest((self.state_size,))

    def products(self):
        return [("in", self.w_in, self.b_in, None), ("o", self.w_o, None, None)]

    def until_last(self, xn, ctx, cache, first=None):
        proj = first if first is not None else ops.linear(xn, self.w_in, self.b_in, out_dtype=ctx.act_dtype)
        o = self.off
        mem = ops.memory_scan(ops.MEMORY_GATED, proj, cache.rows, ctx, self.H, self.D, self.V,
                              o["q"], o["k"], o["v"], o["i"], o["f"], cap=self.cap, q_scale=self.spec.q_scale)
        y = ops.head_norm_gate(mem, self.norm, self.H, self.V, self.eps, ctx.act_dtype, gate=proj, gate_off=o["g"])
        return y, self.w_o, None

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y, w, _ = self.until_last(xn, ctx, cache)
        return _finish(y, w, add, out)


class GatedLinearMemory(Mixer):
    """HGRN2: linear attention whose forget gate also decides what is written.  q = silu(W_q h), v = W_v h;
    per head and row f = l + (1 - l) sigmoid(W_f h + b_f) with a learned lower bound l; S' = diag(f) S +
    (1 - f) v^T, o = S'^T q; each head's o is RMS-normed over its values with one weight shared by the
    heads, the heads are joined and projected.  Option: ``norm_eps``."""
    capturable = True
    launches_only = True
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.H, self.D, self.V = spec.num_heads, spec.head_dim, spec.value_dim or spec.head_dim
        self.eps = float(spec.option("norm_eps", 1e-6))
        self.state_size = ops.memory_state_size(ops.MEMORY_BOUNDED_FORGET, self.H, self.D, self.V)
        self.w_in = self.b_in = self.w_o = self.norm = self.lower = None

    def parameters(self) -> Dict[str, ParamSpec]:
        H, D, V, W = self.H, self.D, self.V, self.spec.hidden
        return {"q.weight": ParamSpec((H * D, W)), "f.weight": ParamSpec((H * D, W)),
                "f.bias": ParamSpec((H * D,), "vector", "wide"), "lower": ParamSpec((H * D,), "vector", "unit"),
                "v.weight": ParamSpec((H * V, W)), "norm.weight": ParamSpec((V,), "vector", "gamma"),
                "o.weight": ParamSpec((W, H * V))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        names = ("q", "f", "v")
        self.w_in, self.b_in = _joined([t[n + ".weight"] for n in names],
                                       [t.get(n + ".bias") for n in names], t["q.weight"])
        self.w_o, self.norm, self.lower = t["o.weight"], t["norm.weight"], t["lower"]
        self.off = dict(q=0, f=self.H * self.D, v=2 * self.H * self.D)

    def cache_request(self):
        return StateRequest((self.state_size,))

    def products(self):
        return [("in", self.w_in, self.b_in, None), ("o", self.w_o, None, None)]

    def until_last(self, xn, ctx, cache, first=None):
        proj = first if first is not None else ops.linear(xn, self.w_in, self.b_in, out_dtype=ctx.act_dtype)
        o = self.off
        mem = ops.memory_scan(ops.MEMORY_BOUNDED_FORGET, proj, cache.rows, ctx, self.H, self.D, self.V,
                              o["q"], 0, o["v"], 0, o["f"], lower=self.lower)
        y = ops.head_norm_gate(mem, self.norm, self.H, self.V, self.eps, ctx.act_dtype)
        return y, self.w_o, None

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y, w, _ = self.until_last(xn, ctx, cache)
        return _finish(y, w, add, out)


class SelectiveScan(Mixer):
    """Mamba: W_in h = [x | z]; x through a causal convolution per channel (``conv`` taps, bias) and silu;
    W_x x = [dt | B | C]; dt = softplus(W_dt dt + b_dt) per channel; A = -exp(A_log);
    S[c, n] <- e^(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c; y silu(z), projected.
    The state row holds S [inner, state] and the convolution's last taps-1 inputs.
    Options: ``inner``, ``state``, ``dt_rank``, ``conv``."""
    capturable = True
    launches_only = True
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.C, self.N = int(spec.option("inner")), int(spec.option("state"))
        self.R, self.taps = int(spec.option("dt_rank")), int(spec.option("conv"))
        if self.N > ops.SCAN_MAX_STATE:
            raise ValueError(f"mamba1: state {self.N} exceeds what the scan takes ({ops.SCAN_MAX_STATE})")
        self.tail_off = self.C * self.N
        self.state_size = self.C * self.N + self.C * (self.taps - 1)
        self.w_in = self.conv_w = self.conv_b = self.w_xdt = self.w_xbc = None
        self.w_dt = self.b_dt = self.a_log = self.d_skip = self.w_o = None

    def parameters(self) -> Dict[str, ParamSpec]:
        C, N, R, W = self.C, self.N, self.R, self.spec.hidden
        return {"in.weight": ParamSpec((2 * C, W)), "conv.weight": ParamSpec((C, self.taps), "vector", "wide"),
                "conv.bias": ParamSpec((C,), "vector", "bias"), "x.weight": ParamSpec((R + 2 * N, C)),
                "dt.weight": ParamSpec((C, R)), "dt.bias": ParamSpec((C,), "vector", "wide"),
                "A_log": ParamSpec((C, N), "vector", "wide"), "D": ParamSpec((C,), "vector", "gamma"),
                "o.weight": ParamSpec((W, C))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_in, self.conv_w, self.conv_b = t["in.weight"], t["conv.weight"], t["conv.bias"]
        self.w_xdt = t["x.weight"][:self.R].contiguous()        # the products' outputs stay whole tensors
        self.w_xbc = t["x.weight"][self.R:].contiguous()
        self.w_dt, self.b_dt = t["dt.weight"], t["dt.bias"]
        self.a_log, self.d_skip, self.w_o = t["A_log"], t["D"], t["o.weight"]

    def cache_request(self):
        return StateRequest((self.state_size,))

    def products(self):
        return [("in", self.w_in, None, None), ("x_dt", self.w_xdt, None, None), ("x_bc", self.w_xbc, None, None),
                ("dt", self.w_dt, self.b_dt, None), ("o", self.w_o, None, None)]

    def until_last(self, xn, ctx, cache, first=None):
        xz = first if first is not None else ops.linear(xn, self.w_in, None, out_dtype=ctx.act_dtype)
        xc = ops.conv_silu(xz, self.conv_w, self.conv_b, cache.rows, self.tail_off, ctx, x_off=0)
        low = ops.linear(xc, self.w_xdt, None, out_dtype=ctx.act_dtype)
        bc = ops.linear(xc, self.w_xbc, None, out_dtype=ctx.act_dtype)
        dtp = ops.linear(low, self.w_dt, self.b_dt, out_dtype=torch.float32)
        y = ops.selective_scan(xc, dtp, bc, xz, self.C, self.a_log, self.d_skip, cache.rows, ctx)
        return y, self.w_o, None

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y, w, _ = self.until_last(xn, ctx, cache)
        return _finish(y, w, add, out)


class GatedDeltaRule(Mixer):
    """The gated delta rule: a matrix memory per head that, before it writes, takes back what it already
    holds under the same key.  q and k have ``num_kv_heads`` heads of ``head_dim`` (each read by
    heads / kv_heads heads), v has ``num_heads`` heads of ``value_dim``; no biases.  q, k and v each pass a
    causal convolution per channel (``conv`` taps, the last is the current token's, no bias) and silu; q and k
    are then brought to unit length, x / sqrt(sum x^2 + 1e-6), q times q_scale.  Per head beta = sigmoid(W_b h)
    and a decay g = exp(-exp(A_log) softplus(W_a h + dt_bias));
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
    Each head's o is divided by its root mean square (``norm_eps``), times a weight [value_dim] shared by the
    heads, times silu(W_g h); then the output projection.  The state row holds S [heads, head_dim, value_dim]
    and the convolution's last taps - 1 inputs.  Options: ``conv``, ``norm_eps``."""
    capturable = True
    launches_only = True
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.H, self.G = spec.num_heads, spec.num_kv_heads or spec.num_heads
        self.D, self.V = spec.head_dim, spec.value_dim or spec.head_dim
        self.taps = int(spec.option("conv", 1))
        self.eps = float(spec.option("norm_eps", 1e-6))
        if self.H % self.G:
            raise ValueError(f"gated_delta: {self.H} heads are not a multiple of {self.G} heads of q and k")
        if self.taps < 1:
            raise ValueError("gated_delta: the convolution has at least one tap")
        self.C = 2 * self.G * self.D + self.H * self.V                  # convolved channels: q, k, v
        self.tail_off = ops.memory_state_size(ops.MEMORY_DELTA, self.H, self.D, self.V)
        self.state_size = self.tail_off + self.C * (self.taps - 1)
        self.w_in = self.conv_w = self.w_o = self.norm = self.a_log = self.dt_bias = None

    def parameters(self) -> Dict[str, ParamSpec]:
        H, G, D, V, W = self.H, self.G, self.D, self.V, self.spec.hidden
        return {"q.weight": ParamSpec((G * D, W)), "q.conv": ParamSpec((G * D, self.taps), "vector", "wide"),
                "k.weight": ParamSpec((G * D, W)), "k.conv": ParamSpec((G * D, self.taps), "vector", "wide"),
                "v.weight": ParamSpec((H * V, W)), "v.conv": ParamSpec((H * V, self.taps), "vector", "wide"),
                "b.weight": ParamSpec((H, W)), "a.weight": ParamSpec((H, W)),
                "A_log": ParamSpec((H,), "vector", "bias"), "dt_bias": ParamSpec((H,), "vector", "wide"),
                "g.weight": ParamSpec((H * V, W)), "norm.weight": ParamSpec((V,), "vector", "gamma"),
                "o.weight": ParamSpec((W, H * V))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        names = ("q", "k", "v", "g", "b", "a")
        self.w_in, _ = _joined([t[n + ".weight"] for n in names], [None] * len(names), t["q.weight"])
        self.conv_w = torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], 0).contiguous()
        self.w_o, self.norm = t["o.weight"], t["norm.weight"]
        self.a_log, self.dt_bias = t["A_log"], t["dt_bias"]
        G, D, H, V = self.G, self.D, self.H, self.V
        self.off = dict(q=0, k=G * D, v=2 * G * D, g=self.C, b=self.C + H * V, a=self.C + H * V + H)

    def cache_request(self):
        return StateRequest((self.state_size,))

    def first_product(self):
        return self.w_in, None, None

    def products(self):
        return [("in", self.w_in, None, None), ("o", self.w_o, None, None)]

    def until_last(self, xn, ctx, cache, first=None):
        proj = first if first is not None else ops.linear(xn, self.w_in, None, out_dtype=ctx.act_dtype)
        o = self.off
        xc = ops.conv_silu(proj, self.conv_w, None, cache.rows, self.tail_off, ctx, x_off=0)
        mem = ops.memory_scan(ops.MEMORY_DELTA, xc, cache.rows, ctx, self.H, self.D, self.V,
                              o["q"], o["k"], o["v"], o["b"], o["a"], q_scale=self.spec.q_scale,
                              gates=proj, a_log=self.a_log, dt_bias=self.dt_bias, kv_heads=self.G)
        y = ops.head_norm_gate(mem, self.norm, self.H, self.V, self.eps, ctx.act_dtype, gate=proj, gate_off=o["g"],
                               gate_act="silu")
        return y, self.w_o, None

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y, w, _ = self.until_last(xn, ctx, cache)
        return _finish(y, w, add, out)


class NormedPair(Mixer):
    """Two mixers side by side on the same input: each output is RMS-normed over the model width with
    a weight of its own, and the result is ``weight`` times their sum.  The children are whole mixer
    specs (options ``left`` and ``right``); their cache needs travel together as a pair.
    Options: ``left``, ``right``, ``norm_eps``, ``weight``."""
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.left, self.right = build_mixer(spec.option("left")), build_mixer(spec.option("right"))
        self.eps = float(spec.option("norm_eps", 1e-6))
        self.weight = float(spec.option("weight", 0.5))
        self.w_left = self.w_right = None

    @property
    def capturable(self):
        return self.left.capturable and self.right.capturable

    @property
    def launches_only(self):
        return self.left.launches_only and self.right.launches_only

    def parameters(self) -> Dict[str, ParamSpec]:
        p = {f"left.{k}": v for k, v in self.left.parameters().items()}
        p.update({f"right.{k}": v for k, v in self.right.parameters().items()})
        W = self.spec.hidden
        p["left.out.weight"] = ParamSpec((W,), "vector", "gamma")
        p["right.out.weight"] = ParamSpec((W,), "vector", "gamma")
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        own = ("left.out.weight", "right.out.weight")
        self.left.load({k[len("left."):]: v for k, v in t.items() if k.startswith("left.") and k not in own})
        self.right.load({k[len("right."):]: v for k, v in t.items() if k.startswith("right.") and k not in own})
        self.w_left, self.w_right = t[own[0]], t[own[1]]

    def cache_request(self):
        return (self.left.cache_request(), self.right.cache_request())

    def products(self):
        return ([("left." + n, w, b, a) for n, w, b, a in self.left.products()]
                + [("right." + n, w, b, a) for n, w, b, a in self.right.products()])

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if len(add) > 2:
            raise ValueError("at most two tensors can be added to a pair's result")
        yl = self.left.forward(xn, ctx, cache[0], (), None)
        yr = self.right.forward(xn, ctx, cache[1], (), None)
        add = [a() if callable(a) else a for a in add]
        return ops.rms_scale_add(yl, self.w_left, self.eps, self.weight, adds=add, out=out,
                                 second=(yr, self.w_right))


class Retention(Mixer):
    """Linear attention with a fixed decay per head and neither softmax nor denominator.  q = W_q h, k = W_k h
    (heads of ``head_dim``), v = W_v h (heads of ``value_dim``), no biases; q and k pass the mixer's position
    encoding (rotation of the first dims of every head), k is then multiplied by head_dim^(-1/2);
        S <- decay_h S + k v^T;  o = S^T q
    per head, from a zero state.  Each head's o is divided by its root mean square (``norm_eps``, no weight), the
    heads are joined, multiplied by silu(W_g h) and projected.  The rotation, the scale, the decay and the state
    are 32-bit.  Options: ``decay`` (one factor per head), ``norm_eps``."""
    capturable = True
    launches_only = True
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.H, self.D, self.V = spec.num_heads, spec.head_dim, spec.value_dim or spec.head_dim
        self.eps = float(spec.option("norm_eps", 1e-6))
        decay = spec.option("decay")
        if decay is None or len(decay) != self.H or not all(0.0 < float(d) <= 1.0 for d in decay):
            raise ValueError(f"retention: one decay in (0, 1] for each of the {self.H} heads expected, got {decay!r}")
        self.decay_values = tuple(float(d) for d in decay)
        self.position = build_position(spec.position)
        self.state_size = ops.memory_state_size(ops.MEMORY_DECAY, self.H, self.D, self.V)
        self.w_in = self.w_o = self.decay = None

    def parameters(self) -> Dict[str, ParamSpec]:
        H, D, V, W = self.H, self.D, self.V, self.spec.hidden
        return {"q.weight": ParamSpec((H * D, W)), "k.weight": ParamSpec((H * D, W)),
                "v.weight": ParamSpec((H * V, W)), "g.weight": ParamSpec((H * V, W)),
                "o.weight": ParamSpec((W, H * V))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        names = ("q", "k", "v", "g")
        self.w_in, _ = _joined([t[n + ".weight"] for n in names], [None] * len(names), t["q.weight"])
        self.w_o = t["o.weight"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(self.w_in.device)
        H, D, V = self.H, self.D, self.V
        self.off = dict(q=0, k=H * D, v=2 * H * D, g=2 * H * D + H * V)

    def cache_request(self):
        return StateRequest((self.state_size,))

    def first_product(self):
        return self.w_in, None, None

    def products(self):
        return [("in", self.w_in, None, None), ("o", self.w_o, None, None)]

    def until_last(self, xn, ctx, cache, first=None):
        proj = first if first is not None else ops.linear(xn, self.w_in, None, out_dtype=ctx.act_dtype)
        o = self.off
        tables = self.position.tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        mem = ops.memory_scan(ops.MEMORY_DECAY, proj, cache.rows, ctx, self.H, self.D, self.V,
                              o["q"], o["k"], o["v"], 0, 0, q_scale=1.0, k_scale=float(self.D) ** -0.5,
                              decay=self.decay, cos=cos, sin=sin)
        y = ops.head_norm_gate(mem, None, self.H, self.V, self.eps, ctx.act_dtype, gate=proj, gate_off=o["g"],
                               gate_act="silu")
        return y, self.w_o, None

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y, w, _ = self.until_last(xn, ctx, cache)
        return _finish(y, w, add, out)


class StateSpaceDual(Mixer):
    """Mamba-2: a state-space layer whose decay is one number per head and token, so that a head is a matrix
    memory S [state, value_dim] with keys B, values x and queries C.  With inner = heads * value_dim and
    ``groups`` groups of B and C (head h reads group h / (heads / groups)):
        W_in h = [z: inner | x: inner | B: groups * state | C: groups * state | dt: heads];
        x, B and C together pass a causal convolution per channel (``conv`` taps, bias, the last tap is the current
        token's, zeros before the start) and silu;
        dt = softplus(dt + dt_bias);  S <- exp(-exp(A_log_h) dt) S + dt B x^T;  y = S^T C + D_h x;
        y silu(z) is RMS-normed in ``norm_groups`` equal parts, each by its own root mean square (``norm_eps``),
        times a weight [inner], and projected.
    The state row holds S [heads, state, value_dim] and the convolution's last taps - 1 inputs; step sizes,
    decays and the state are 32-bit.  Options: ``state``, ``groups``, ``conv``, ``norm_groups``, ``norm_eps``."""
    capturable = True
    launches_only = True
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.H, self.P = spec.num_heads, spec.value_dim or spec.head_dim
        self.N, self.G = int(spec.option("state")), int(spec.option("groups", 1))
        self.taps, self.parts = int(spec.option("conv", 1)), int(spec.option("norm_groups", 1))
        self.eps = float(spec.option("norm_eps", 1e-6))
        self.inner = self.H * self.P
        if self.G < 1 or self.H % self.G:
            raise ValueError(f"mamba2: {self.H} heads do not form {self.G} equal groups")
        if self.parts < 1 or self.inner % self.parts:
            raise ValueError(f"mamba2: {self.inner} channels do not form {self.parts} equal parts for the norm")
        if self.taps < 1:
            raise ValueError("mamba2: the convolution has at least one tap")
        self.C = self.inner + 2 * self.G * self.N                       # convolved channels: x, B, C
        self.tail_off = ops.memory_state_size(ops.MEMORY_DECAY, self.H, self.N, self.P)
        self.state_size = self.tail_off + self.C * (self.taps - 1)
        self.w_in = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm = self.w_o = None

    def parameters(self) -> Dict[str, ParamSpec]:
        W = self.spec.hidden
        return {"in.weight": ParamSpec((2 * self.inner + 2 * self.G * self.N + self.H, W)),
                "conv.weight": ParamSpec((self.C, self.taps), "vector", "wide"),
                "conv.bias": ParamSpec((self.C,), "vector", "bias"),
                "dt_bias": ParamSpec((self.H,), "vector", "wide"), "A_log": ParamSpec((self.H,), "vector", "bias"),
                "D": ParamSpec((self.H,), "vector", "gamma"), "norm.weight": ParamSpec((self.inner,), "vector", "gamma"),
                "o.weight": ParamSpec((W, self.inner))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_in, _ = _joined([t["in.weight"]], [None], t["in.weight"])
        self.conv_w, self.conv_b = t["conv.weight"], t["conv.bias"]
        self.dt_bias, self.a_log, self.d_skip = t["dt_bias"], t["A_log"], t["D"]
        self.norm, self.w_o = t["norm.weight"], t["o.weight"]

    def cache_request(self):
        return StateRequest((self.state_size,))

    def first_product(self):
        return self.w_in, None, None

    def products(self):
        return [("in", self.w_in, None, None), ("o", self.w_o, None, None)]

    def until_last(self, xn, ctx, cache, first=None):
        proj = first if first is not None else ops.linear(xn, self.w_in, None, out_dtype=ctx.act_dtype)
        inner, GN = self.inner, self.G * self.N
        xbc = ops.conv_silu(proj, self.conv_w, self.conv_b, cache.rows, self.tail_off, ctx, x_off=inner)
        # keys B, values x, queries C; the step sizes are still in the projection
        mem = ops.memory_scan(ops.MEMORY_DECAY, xbc, cache.rows, ctx, self.H, self.N, self.P,
                              inner + GN, inner, 0, 0, 2 * inner + 2 * GN, gates=proj, a_log=self.a_log,
                              dt_bias=self.dt_bias, kv_heads=self.G, skip=self.d_skip)
        y = ops.head_norm_gate(mem, self.norm, self.parts, inner // self.parts, self.eps, ctx.act_dtype, gate=proj,
                               gate_off=0, gate_act="silu", gate_first=True)
        return y, self.w_o, None

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y, w, _ = self.until_last(xn, ctx, cache)
        return _finish(y, w, add, out)


class ScaledPair(Mixer):
    """Two mixers side by side on the same input, summed with a factor each: left_scale * left(h) +
    right_scale * right(h).  The children are whole mixer specs (options ``left`` and ``right``); their cache
    needs travel together as a pair.  ``branches`` hands a block the two outputs and their factors unsummed, so
    that it can sum them in the pass that norms the result.  Options: ``left``, ``right``, ``left_scale``,
    ``right_scale``."""
    deferred_add = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.left, self.right = build_mixer(spec.option("left")), build_mixer(spec.option("right"))
        self.left_scale, self.right_scale = float(spec.option("left_scale", 1.0)), float(spec.option("right_scale", 1.0))

    @property
    def capturable(self):
        return self.left.capturable and self.right.capturable

    @property
    def launches_only(self):
        return self.left.launches_only and self.right.launches_only

    def parameters(self) -> Dict[str, ParamSpec]:
        p = {f"left.{k}": v for k, v in self.left.parameters().items()}
        p.update({f"right.{k}": v for k, v in self.right.parameters().items()})
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.left.load({k[len("left."):]: v for k, v in t.items() if k.startswith("left.")})
        self.right.load({k[len("right."):]: v for k, v in t.items() if k.startswith("right.")})

    def cache_request(self):
        return (self.left.cache_request(), self.right.cache_request())

    def products(self):
        return ([("left." + n, w, b, a) for n, w, b, a in self.left.products()]
                + [("right." + n, w, b, a) for n, w, b, a in self.right.products()])

    def branches(self, xn, ctx, cache):
        """[(float32 output, factor)] of the two children."""
        return [(self.left.forward(xn, ctx, cache[0], (), None), self.left_scale),
                (self.right.forward(xn, ctx, cache[1], (), None), self.right_scale)]

    def forward(self, xn, ctx, cache, add: Sequence, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        (yl, sl), (yr, sr) = self.branches(xn, ctx, cache)
        add = [a() if callable(a) else a for a in add]
        return ops.scaled_sum(yl, sl, yr, sr, adds=add, out=out)


register_mixer("mlstm", MatrixLstm)
register_mixer("hgrn2", GatedLinearMemory)
register_mixer("mamba1", SelectiveScan)
register_mixer("normed_pair", NormedPair)
register_mixer("gated_delta", GatedDeltaRule)
register_mixer("retention", Retention)
register_mixer("mamba2", StateSpaceDual)
register_mixer("scaled_pair", ScaledPair)
