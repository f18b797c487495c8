"""Softmax attention over the paged key/value cache."""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from .. import ops
from ..config.specs import MixerSpec
from .base import KVRequest, Mixer, ParamSpec, build_norm, build_position, register_mixer


class Attention(Mixer):
    """q, k, v projections (one fused product, rows ordered Q, K, V as the
    reference's fused matrix is, model.go:2222-2227), optional per-head norm of
    q and k, position encoding, query scale, cache write, attention over the
    cache, output projection.  Grouped-query attention when num_kv_heads <
    num_heads (query head h reads group h / (nH/nKV), model.go:2828)."""

    deferred_add = True
    capturable = True
    launches_only = True

    def __init__(self, spec: MixerSpec):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim > 256:
            raise ValueError(f"head size {spec.head_dim} exceeds what the attention kernels take (256)")
        self.spec = spec
        self.position = build_position(spec.position)
        self.q_norm = build_norm(spec.qk_norm) if spec.qk_norm else None
        self.k_norm = build_norm(spec.qk_norm) if spec.qk_norm else None
        self.w_qkv = self.b_qkv = self.w_out = self.b_out = None

    # -- parameters -----------------------------------------------------
    def parameters(self) -> Dict[str, ParamSpec]:
        s = self.spec
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        p = {"q.weight": ParamSpec((q, s.hidden)), "k.weight": ParamSpec((kv, s.hidden)),
             "v.weight": ParamSpec((kv, s.hidden)), "out.weight": ParamSpec((s.hidden, q))}
        if s.bias:
            p.update({"q.bias": ParamSpec((q,), "vector", "bias"),
                      "k.bias": ParamSpec((kv,), "vector", "bias"),
                      "v.bias": ParamSpec((kv,), "vector", "bias"),
                      "out.bias": ParamSpec((s.hidden,), "vector", "bias")})
        if self.q_norm is not None:
            for name, n in (("q_norm", self.q_norm), ("k_norm", self.k_norm)):
                for k, v in n.parameters().items():
                    p[f"{name}.{k}"] = v
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        ws = [t["q.weight"], t["k.weight"], t["v.weight"]]
        if len({w.dtype for w in ws}) > 1:           # mixed storage: widen to the widest
            ws = [w.float() for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        self.w_out = t["out.weight"]
        if self.spec.bias:
            self.b_qkv = torch.cat([t["q.bias"], t["k.bias"], t["v.bias"]]).contiguous()
            self.b_out = t["out.bias"]
        if self.q_norm is not None:
            self.q_norm.load({k[len("q_norm."):]: v for k, v in t.items() if k.startswith("q_norm.")})
            self.k_norm.load({k[len("k_norm."):]: v for k, v in t.items() if k.startswith("k_norm.")})

    def cache_request(self):
        s = self.spec
        return KVRequest(s.num_kv_heads, s.head_dim, s.window)

    # -- compute ----------------------------------------------------------
    def forward(self, xn, ctx, cache, add: Sequence[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        if len(add) > 2:
            raise ValueError("at most two tensors can be added in the projection's epilogue")
        o, w, b = self.until_last(xn, ctx, cache)
        add = [a() if callable(a) else a for a in add]
        a0 = add[0] if len(add) > 0 else None
        a1 = add[1] if len(add) > 1 else None
        return ops.linear(o, w, b, add0=a0, add1=a1, out=out)

    def first_product(self):
        return self.w_qkv, self.b_qkv, None

    def products(self):
        return [("qkv", self.w_qkv, self.b_qkv, None), ("out", self.w_out, self.b_out, None)]

    def decode_fusable(self, ctx, cache):
        if not ctx.is_decode or cache is None:
            return None
        s = self.spec
        tables = self.position.tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        return dict(w_qkv=self.w_qkv, b_qkv=self.b_qkv, w_out=self.w_out, b_out=self.b_out,
                    num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, q_scale=s.q_scale,
                    window=s.window, cos=cos, sin=sin, interleaved=s.position.interleaved,
                    head_norm=self.q_norm is not None, k=cache.k, v=cache.v, pages=ctx.pages[cache.group],
                    writes=cache.writes)

    def until_last(self, xn, ctx, cache, first=None):
        """Everything but the output projection: the attention output [T, heads * head size] with the
        projection's weight and bias.  ``first``: the joined q, k, v projection if the caller made it."""
        s = self.spec
        T = xn.shape[0]
        qkv = first if first is not None else ops.linear(xn, self.w_qkv, self.b_qkv, out_dtype=ctx.act_dtype)
        tables = self.position.tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        pages = ctx.pages[cache.group]
        group = s.num_heads // s.num_kv_heads
        if (ctx.is_decode and group <= ops.DECODE_MAX_GROUP
                and ops.decode_takes_qkv(qkv.dtype, cache.k.dtype, s.head_dim, 0 if cos is None else cos.shape[1],
                                         s.position.interleaved, self.q_norm is not None)):
            # one token a sequence: attention reads the projection's output itself (rotation, query scale
            # and the cache write happen inside it), one kernel less between two products
            o = ops.empty((T, s.num_heads * s.head_dim), ctx.act_dtype, xn.device)
            splits = ops.decode_splits(ctx.n_seqs, s.num_kv_heads, ctx.max_len, xn.device, s.head_dim, group)
            ops.attention_decode(None, o, cache.k, cache.v, ctx.seq_ctx, pages, s.num_heads, s.num_kv_heads,
                                 s.head_dim, splits, s.window, qkv=qkv, cos=cos, sin=sin, q_scale=s.q_scale,
                                 write_kv=cache.writes)
            return o, self.w_out, self.b_out
        q = ops.empty((T, s.num_heads * s.head_dim), ctx.act_dtype, xn.device)
        qn = kn = None
        eps, rms = 0.0, False
        if self.q_norm is not None:
            qn, kn = (self.q_norm.weight, self.q_norm.bias), (self.k_norm.weight, self.k_norm.bias)
            eps, rms = s.qk_norm.eps, self.q_norm.rms
        ops.qkv_to_cache(qkv, q, cache.k, cache.v, ctx.tok_seq, ctx.tok_pos, pages,
                         s.num_heads, s.num_kv_heads, s.head_dim, s.q_scale, cos, sin,
                         interleaved=s.position.interleaved, q_norm=qn, k_norm=kn,
                         norm_eps=eps, norm_rms=rms, write_kv=cache.writes)
        o = ops.empty(q.shape, q.dtype, q.device)
        ops.attention(q, o, cache.k, cache.v, ctx, pages, s.num_heads, s.num_kv_heads,
                      s.head_dim, window=s.window)
        return o, self.w_out, self.b_out



class MixedHeadAttention(Mixer):
    """Softmax attention whose heads talk to one another after the softmax, over the paged cache.

    q, k, v projections without bias (one product; values of size ``value_dim`` per head); with option
    ``qk_norm`` = "projection" the whole q row and the whole k row of a token are RMS-normed (weights of
    the rows' sizes, option ``norm_eps``) before the heads are split; position encoding on q and k; score
    = (q . k) * q_scale; causal softmax per head; with option ``talk`` a learned table M [heads, heads] mixes
    the heads' weights, w_h = sum_g M[h, g] p_g, and head h applies w_h to the values of its own key/value
    head; output projection.  The sum over keys is linear, so the kernel computes every pair (query head's
    weights, value head) once and mixes the results (csrc/attention_mixed.cu).

    Further options, all off by default.  ``spec.bias``: q, k and v have biases (the output projection has
    none).  ``q_temp`` = (coef, every): the query at position p is multiplied by
    1 + coef * ln(floor((p + 1) / every) + 1).  ``score_scale``: the score is (q . k) * score_scale, applied to
    the 32-bit score (``q_scale`` multiplies q before it is rounded).  ``softcap`` c > 0: score <- c tanh(score / c).
    ``distance_bias`` x > 0: head h's score loses slope_h * (i - j) for the key at position j <= i, slope_h =
    2^(-x (h + 1) / heads).  ``shared_kv``: the mixer has no key and value projections; it reads the cache
    entry another mixer with the same head counts and sizes wrote.  ``qk_norm`` = "head_unit": after the
    rotation every head of q and of k is divided by its own root mean square (``norm_eps`` inside the root, no
    weight).  ``sink``: a learned score per head ("sink" [heads]) whose exponential joins the softmax's
    denominator once, with no key and no value, unscaled.  ``out_bias``: the output projection has a bias.
    ``spec.window`` w > 0: a query sees itself and the w - 1 positions before it."""

    deferred_add = True
    capturable = True
    launches_only = True

    def __init__(self, spec: MixerSpec):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.vdim = spec.value_dim or spec.head_dim
        if spec.head_dim > 256 or self.vdim > 256:
            raise ValueError(f"head sizes {spec.head_dim}/{self.vdim} exceed what the attention kernels take (256)")
        scope = spec.option("qk_norm", None)
        if scope not in (None, "projection", "head_unit"):
            raise ValueError(f"qk_norm {scope!r}: this mixer norms over the whole projection, every head to unit "
                             f"root mean square after the rotation, or not at all")
        self.row_norm = scope == "projection"
        self.head_unit = scope == "head_unit"
        self.sink = bool(spec.option("sink", False))
        self.out_bias = bool(spec.option("out_bias", False))
        self.talk = bool(spec.option("talk", False))
        self.eps = float(spec.option("norm_eps", 1e-6))
        self.position = build_position(spec.position)
        self.shared_kv = bool(spec.option("shared_kv", False))
        self.q_temp = spec.option("q_temp", None)
        self.score_scale = float(spec.option("score_scale", 1.0))
        self.softcap = float(spec.option("softcap", 0.0) or 0.0)
        self.distance_bias = float(spec.option("distance_bias", 0.0) or 0.0)
        if self.q_temp is not None:
            self.q_temp = (float(self.q_temp[0]), float(self.q_temp[1]))
            if not self.q_temp[1] > 0:
                raise ValueError("q_temp: the period must be positive")
        if self.softcap < 0 or self.distance_bias < 0:
            raise ValueError("softcap and distance_bias must not be negative")
        if self.shared_kv and (self.row_norm or self.head_unit):
            raise ValueError("a mixer that reads another one's keys has no key norm of its own")
        self.w_qkv = self.b_qkv = self.w_out = self.q_gamma = self.k_gamma = self.mix = self.slopes = None
        self.b_out = self.sinks = None

    def parameters(self) -> Dict[str, ParamSpec]:
        s = self.spec
        q, kv, vv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * self.vdim
        p = {"q.weight": ParamSpec((q, s.hidden)), "k.weight": ParamSpec((kv, s.hidden)),
             "v.weight": ParamSpec((vv, s.hidden)), "o.weight": ParamSpec((s.hidden, s.num_heads * self.vdim))}
        if s.bias:
            p.update({"q.bias": ParamSpec((q,), "vector", "bias"), "k.bias": ParamSpec((kv,), "vector", "bias"),
                      "v.bias": ParamSpec((vv,), "vector", "bias")})
        if self.shared_kv:
            for k in ("k.weight", "v.weight", "k.bias", "v.bias"):
                p.pop(k, None)
        if self.row_norm:
            p["q_norm.weight"] = ParamSpec((q,), "vector", "gamma")
            p["k_norm.weight"] = ParamSpec((kv,), "vector", "gamma")
        if self.talk:
            p["talk"] = ParamSpec((s.num_heads, s.num_heads), "vector", "wide")
        if self.sink:
            p["sink"] = ParamSpec((s.num_heads,), "vector", "wide")
        if self.out_bias:
            p["o.bias"] = ParamSpec((s.hidden,), "vector", "bias")
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        names = ("q",) if self.shared_kv else ("q", "k", "v")
        ws = [t[n + ".weight"] for n in names]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        n = sum(w.shape[0] for w in ws)
        pad = (8 - n % 8) % 8                           # output rows of whole 16-byte units
        if pad:
            ws.append(torch.zeros((pad, ws[0].shape[1]), dtype=ws[0].dtype, device=ws[0].device))
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        if self.spec.bias:
            bs = [t[n + ".bias"].float() for n in names]
            if pad:
                bs.append(torch.zeros(pad, dtype=torch.float32, device=bs[0].device))
            self.b_qkv = torch.cat(bs).contiguous()
        if self.distance_bias > 0:
            H = self.spec.num_heads
            self.slopes = torch.tensor([2.0 ** (-self.distance_bias * (h + 1) / H) for h in range(H)],
                                       dtype=torch.float64).to(torch.float32).to(self.w_qkv.device)
        self.w_out = t["o.weight"]
        self.q_gamma, self.k_gamma = t.get("q_norm.weight"), t.get("k_norm.weight")
        self.mix = t.get("talk")
        self.sinks, self.b_out = t.get("sink"), t.get("o.bias")

    def cache_request(self):
        s = self.spec
        return KVRequest(s.num_kv_heads, s.head_dim, s.window, value_dim=0 if self.vdim == s.head_dim else self.vdim)

    def products(self):
        return [("qkv", self.w_qkv, self.b_qkv, None), ("o", self.w_out, self.b_out, None)]

    def first_product(self):
        return self.w_qkv, self.b_qkv, None

    def until_last(self, xn, ctx, cache, first=None):
        s = self.spec
        if self.shared_kv and cache.writes:
            raise ValueError("a mixer without key and value projections cannot be the writer of its cache entry")
        qkv = first if first is not None else ops.linear(xn, self.w_qkv, self.b_qkv, out_dtype=ctx.act_dtype)
        tables = self.position.tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        pages = ctx.pages[cache.group]
        q = ops.qkv_rownorm_to_cache(qkv, cache.k, cache.v, ctx, pages, s.num_heads, s.num_kv_heads, s.head_dim,
                                     self.vdim, s.q_scale, cos, sin, s.position.interleaved,
                                     self.q_gamma, self.k_gamma, self.eps, write_kv=cache.writes,
                                     q_temp=self.q_temp, q_only=self.shared_kv, head_unit=self.head_unit)
        o = ops.attention_mixed(q, cache.k, cache.v, ctx, pages, s.num_heads, s.num_kv_heads, s.head_dim, self.vdim,
                                mix=self.mix, window=s.window, score_scale=self.score_scale, softcap=self.softcap,
                                slopes=self.slopes, sinks=self.sinks)
        return o, self.w_out, self.b_out

    def forward(self, xn, ctx, cache, add: Sequence[torch.Tensor], out=None) -> torch.Tensor:
        if len(add) > 2:
            raise ValueError("at most two tensors can be added in the projection's epilogue")
        o, w, b = self.until_last(xn, ctx, cache)
        add = [a() if callable(a) else a for a in add]
        a0 = add[0] if len(add) > 0 else None
        a1 = add[1] if len(add) > 1 else None
        return ops.linear(o, w, b, add0=a0, add1=a1, out_dtype=torch.float32, out=out)


register_mixer("attention", Attention)
register_mixer("attention_mixed", MixedHeadAttention)
