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
    ``spec.window`` w > 0: a query sees itself and the w - 1 positions before it.
    ``talk_scores``: a learned table T ("talk" [heads, heads]) mixes the heads' SCORES before the softmax,
    s'_h = sum_g T[h, g] s_g, and head h applies its own softmax of s'_h to the values of its own key/value head.
    The sum is taken on the queries: with q'_h,c = sum of T[h, g] q_g over the query heads g of key head c,
    s'_h(i, j) = sum_c q'_h,c(i) . k_c(j), one product of a row of kv_heads * head_dim numbers with the position's key
    heads side by side.  The cache entry of such a mixer holds one key row of that length and kv_heads value rows
    per position, and attention runs as ``heads`` query heads on one wide key head; the mixing costs no pass over
    the scores and runs where the score products run."""

    deferred_add = True
    capturable = True
    launches_only = True

    def __init__(self, spec: MixerSpec):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.spec = spec
        self.vdim = spec.value_dim or spec.head_dim
        self.talk_scores = bool(spec.option("talk_scores", False))
        if self.talk_scores:
            if spec.head_dim * spec.num_kv_heads > 1024 or self.vdim > 256:
                raise ValueError(f"{spec.num_kv_heads} key heads of {spec.head_dim} side by side exceed what the attention "
                                 f"kernels take (1024), or values of {self.vdim} do (256)")
            if spec.option("talk", False):
                raise ValueError("a table mixes the heads' scores or their softmax weights, not both")
        elif spec.head_dim > 256 or self.vdim > 256:
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
        if self.shared_kv and self.row_norm:
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
        if self.talk or self.talk_scores:
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
        if self.talk_scores:
            wide = s.num_kv_heads * s.head_dim
            return KVRequest(1, wide, s.window, value_dim=0 if self.vdim == wide else self.vdim,
                             value_heads=0 if s.num_kv_heads == 1 else s.num_kv_heads)
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
        if self.talk_scores:
            q = ops.qkv_rownorm_to_cache(qkv, cache.k, cache.v, ctx, pages, s.num_heads, s.num_kv_heads, s.head_dim,
                                         self.vdim, s.q_scale, cos, sin, s.position.interleaved,
                                         self.q_gamma, self.k_gamma, self.eps, write_kv=cache.writes,
                                         q_temp=self.q_temp, q_only=self.shared_kv, head_unit=self.head_unit,
                                         talk=self.mix, k_joined=True)
            o = ops.attention_mixed(q, cache.k, cache.v, ctx, pages, s.num_heads, 1, s.num_kv_heads * s.head_dim,
                                    self.vdim, mix=None, window=s.window, score_scale=self.score_scale,
                                    softcap=self.softcap, slopes=self.slopes, sinks=self.sinks,
                                    value_heads=s.num_kv_heads)
            return o, self.w_out, self.b_out
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


class LatentAttention(Mixer):
    """Softmax attention whose keys and values are read out of a small latent per position.

    c_q = rms(W_dq x) * g_q;  q = W_uq c_q, per head [``head_dim`` plain | ``rot`` rotated] columns;
    W_dkv x = [c' | k_r]: c = rms(c') * g_c (``kv_rank`` numbers), k_r (``rot`` numbers, rotated) one key part for
    all heads; per head k = [W_uk,h c | k_r], v = W_uv,h c (``value_dim``); score = q . k * ``score_scale``; window
    and sink as in the other mixers; option ``gate``: head h's output times sigmoid(w_g,h . x); output projection.

    Keys and values are never built.  (W_uk,h^T q_h) . c = q_h . (W_uk,h c), and sum_j p_j W_uv,h c_j =
    W_uv,h sum_j p_j c_j, so the cache holds the row [c | k_r] per position and nothing else (the values are its first columns),
    every query head becomes a row [W_uk,h^T q_h | its rotated part] of kv_rank + rot numbers, attention runs as
    ``num_heads`` query heads on ONE key head with values of size kv_rank, and W_uv,h is applied to a head's result.
    The three down projections (query latent, [c' | k_r], gates) are one product; the per-head products are
    csrc/latent.cu's.  Options: ``q_rank``, ``kv_rank``, ``rot`` (the position encoding's rotary size),
    ``score_scale``, ``norm_eps``, ``sink``, ``gate``."""

    deferred_add = True
    capturable = True
    launches_only = True

    def __init__(self, spec: MixerSpec):
        self.spec = spec
        self.q_rank, self.kv_rank = int(spec.option("q_rank")), int(spec.option("kv_rank"))
        self.rot = int(spec.option("rot", 0))
        self.vdim = spec.value_dim or spec.head_dim
        if min(self.q_rank, self.kv_rank, spec.num_heads, spec.head_dim, self.vdim) < 1 or self.rot < 0 or self.rot % 2:
            raise ValueError("latent attention: ranks, heads and head sizes are positive, the rotated part is even")
        if spec.position.kind != "none" and spec.position.rotary_dim != self.rot:
            raise ValueError("latent attention: the rotation covers the rotated part exactly")
        if self.kv_rank + self.rot > 1024 or self.kv_rank > 256:
            raise ValueError(f"a latent of {self.kv_rank} + {self.rot} exceeds what the attention kernels take (256 + 768)")
        self.sink = bool(spec.option("sink", False))
        self.gate = bool(spec.option("gate", False))
        self.eps = float(spec.option("norm_eps", 1e-6))
        self.score_scale = float(spec.option("score_scale", 1.0))
        self.position = build_position(spec.position)
        self.w_down = self.w_uq = self.w_uk_t = self.w_uv = self.w_out = None
        self.q_gamma = self.kv_gamma = self.sinks = None

    def parameters(self) -> Dict[str, ParamSpec]:
        s, H = self.spec, self.spec.num_heads
        p = {"dq.weight": ParamSpec((self.q_rank, s.hidden)), "dq.norm.weight": ParamSpec((self.q_rank,), "vector", "gamma"),
             "uq.weight": ParamSpec((H * (s.head_dim + self.rot), self.q_rank)),
             "dkv.weight": ParamSpec((self.kv_rank + self.rot, s.hidden)),
             "dkv.norm.weight": ParamSpec((self.kv_rank,), "vector", "gamma"),
             "uk.weight": ParamSpec((H * s.head_dim, self.kv_rank)), "uv.weight": ParamSpec((H * self.vdim, self.kv_rank)),
             "o.weight": ParamSpec((s.hidden, H * self.vdim))}
        if self.sink:
            p["sink"] = ParamSpec((H,), "vector", "wide")
        if self.gate:
            p["g.weight"] = ParamSpec((H, s.hidden))
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        s, H = self.spec, self.spec.num_heads
        ws = [t["dq.weight"], t["dkv.weight"]] + ([t["g.weight"]] if self.gate else [])
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        n = sum(w.shape[0] for w in ws)
        pad = (8 - n % 8) % 8                           # output rows of whole 16-byte units
        if pad:
            ws.append(torch.zeros((pad, ws[0].shape[1]), dtype=ws[0].dtype, device=ws[0].device))
        self.w_down = torch.cat(ws, dim=0).contiguous()
        self.w_uq = t["uq.weight"]
        # W_uk,h^T as a product's weight [out = kv_rank, in = head_dim], head by head
        self.w_uk_t = t["uk.weight"].view(H, s.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = t["uv.weight"].view(H, self.vdim, self.kv_rank).contiguous()
        self.w_out = t["o.weight"]
        self.q_gamma, self.kv_gamma = t["dq.norm.weight"], t["dkv.norm.weight"]
        self.sinks = t.get("sink")

    def cache_request(self):
        return KVRequest(1, self.kv_rank + self.rot, self.spec.window, value_dim=self.kv_rank, values_in_keys=True)

    def products(self):
        return [("down", self.w_down, None, None), ("uq", self.w_uq, None, None), ("o", self.w_out, None, None)]

    def first_product(self):
        return self.w_down, None, None

    def until_last(self, xn, ctx, cache, first=None):
        s, H = self.spec, self.spec.num_heads
        proj = first if first is not None else ops.linear(xn, self.w_down, None, out_dtype=ctx.act_dtype)
        tables = self.position.tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        pages = ctx.pages[cache.group]
        cq = ops.latent_prepare(proj, cache.k, cache.v, ctx, pages, self.q_rank, self.kv_rank, self.rot, self.q_gamma,
                                self.kv_gamma, self.eps, cos, sin, s.position.interleaved, write_kv=cache.writes)
        q = ops.linear(cq, self.w_uq, None, out_dtype=ctx.act_dtype)
        wide = ops.head_linear(q, self.w_uk_t, s.head_dim + self.rot, tail=self.rot, cos=cos, sin=sin,
                               interleaved=s.position.interleaved)
        mixed = ops.attention_mixed(wide, cache.k, cache.v, ctx, pages, H, 1, self.kv_rank + self.rot, self.kv_rank,
                                    window=s.window, score_scale=self.score_scale, sinks=self.sinks, values_in_keys=True)
        o = ops.head_linear(mixed, self.w_uv, self.kv_rank, gate=proj if self.gate else None,
                            gate_off=self.q_rank + self.kv_rank + self.rot)
        return o, self.w_out, None

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
register_mixer("latent_attention", LatentAttention)
