"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from .. import ops
from ..config.specs import FeedForwardSpec
from .base import FeedForward, ParamSpec, register_feed_forward


class DenseFeedForward(FeedForward):
    """down(act(up(x))) with biases: the plain, ungated MLP (model.go:2758-2772,
    forward_batch.go:537-581).  The activation runs in the first product's
    epilogue, the additions to the residual in the second's.

    Activation ``xielu`` has two learned numbers p, q (tensor "act" [2]): above zero softplus(p) z^2 + z / 2, at and
    below zero (1/2 + softplus(q)) (e^z - 1 - z) + z / 2.  The two factors are taken once, when the weights are loaded,
    and travel with the activation into the first product's epilogue, like the activations without numbers."""
    capturable = True
    launches_only = True

    def __init__(self, spec: FeedForwardSpec):
        self.learned = spec.activation == "xielu"
        if not self.learned and spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} unknown")
        self.spec = spec
        self.w_up = self.b_up = self.w_down = self.b_down = None
        self.act_up = self.act_down = 0.0
        if self.learned:
            self.fusable = None                      # no block runs this feed-forward inside a fused layer
            self.first_product = None                # ... or its first product beside another branch's

    def parameters(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"up.weight": ParamSpec((s.intermediate, s.hidden)),
             "down.weight": ParamSpec((s.hidden, s.intermediate))}
        if s.bias:
            p["up.bias"] = ParamSpec((s.intermediate,), "vector", "bias")
            p["down.bias"] = ParamSpec((s.hidden,), "vector", "bias")
        if self.learned:
            p["act"] = ParamSpec((2,), "vector", "wide")
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = t["up.weight"], t["down.weight"]
        self.b_up, self.b_down = t.get("up.bias"), t.get("down.bias")
        if self.learned:
            soft = torch.nn.functional.softplus(t["act"].double().cpu())
            self.act_up, self.act_down = float(soft[0]), 0.5 + float(soft[1])

    def _first_activation(self):
        return ("xielu", self.act_up, self.act_down) if self.learned else self.spec.activation

    def first_product(self):
        return self.w_up, self.b_up, self._first_activation()

    def fusable(self):
        return self.w_up, self.b_up, self.spec.activation, self.w_down, self.b_down

    def products(self):
        return [("up", self.w_up, self.b_up, self._first_activation()), ("down", self.w_down, self.b_down, None)]

    def until_last(self, xn, ctx, first=None):
        h = first if first is not None else ops.linear(xn, self.w_up, self.b_up, act=self._first_activation(),
                                                       out_dtype=ctx.act_dtype)
        return h, self.w_down, self.b_down

    def forward(self, xn, ctx, add: Sequence[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        if len(add) > 2:
            raise ValueError("at most two tensors can be added in the projection's epilogue")
        h, _, _ = self.until_last(xn, ctx)
        a0 = add[0] if len(add) > 0 else None
        a1 = add[1] if len(add) > 1 else None
        return ops.linear(h, self.w_down, self.b_down, add0=a0, add1=a1, out_dtype=torch.float32, out=out)


class GatedFeedForward(FeedForward):
    """down(act(gate(x)) * up(x)), biases optional: the gate's and the up projection's rows are one
    product, the activation and the multiplication one pass between the products (32-bit arithmetic,
    one rounding), the additions to the residual in the last product's epilogue."""
    capturable = True
    launches_only = True

    def __init__(self, spec: FeedForwardSpec):
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} unknown")
        self.spec = spec
        self.w_gu = self.b_gu = self.w_down = self.b_down = None

    def parameters(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"gate.weight": ParamSpec((s.intermediate, s.hidden)), "up.weight": ParamSpec((s.intermediate, s.hidden)),
             "down.weight": ParamSpec((s.hidden, s.intermediate))}
        if s.bias:
            p["gate.bias"] = ParamSpec((s.intermediate,), "vector", "bias")
            p["up.bias"] = ParamSpec((s.intermediate,), "vector", "bias")
            p["down.bias"] = ParamSpec((s.hidden,), "vector", "bias")
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        ws = [t["gate.weight"], t["up.weight"]]
        if ws[0].dtype != ws[1].dtype:
            ws = [w.float() for w in ws]
        self.w_gu = torch.cat(ws, 0).contiguous()
        self.w_down = t["down.weight"]
        if self.spec.bias:
            self.b_gu = torch.cat([t["gate.bias"], t["up.bias"]]).contiguous()
            self.b_down = t["down.bias"]

    def products(self):
        return [("gate_up", self.w_gu, self.b_gu, None), ("down", self.w_down, self.b_down, None)]

    def until_last(self, xn, ctx, first=None):
        gu = first if first is not None else ops.linear(xn, self.w_gu, self.b_gu, out_dtype=ctx.act_dtype)
        return ops.gated_act(gu, self.spec.activation), self.w_down, self.b_down

    def forward(self, xn, ctx, add: Sequence[torch.Tensor], out=None) -> torch.Tensor:
        if len(add) > 2:
            raise ValueError("at most two tensors can be added in the projection's epilogue")
        h, w, b = self.until_last(xn, ctx)
        a0 = add[0] if len(add) > 0 else None
        a1 = add[1] if len(add) > 1 else None
        return ops.linear(h, w, b, add0=a0, add1=a1, out_dtype=torch.float32, out=out)


class MixtureOfExperts(FeedForward):
    """A mixture of small gated feed-forwards, down(silu(gate(x)) * up(x)) without biases, of which every
    token uses ``top``.  The router's logits z = W_router x and its scores sigmoid(z) are 32-bit.  The experts
    form ``groups`` equal groups of neighbours; a group's score is the sum of its two largest scores, and only
    experts of the best ``keep`` groups can be chosen (one group: every expert can).  The chosen experts'
    outputs are summed with weights score / (sum of the chosen scores + 1e-20) * ``router_scale``.  A shared
    expert of the same form (``shared`` > 0: its inner size) runs for every token and is added.
    With ``router`` = "table" there is no router: a table of integers [``vocab``, top] names every token id's
    experts (the entries of a row differ), and each counts 1 / top.
    With ``weights`` = "softmax_chosen" the ``top`` largest logits are chosen and weighted by the softmax over those
    alone (one group); ``router_bias``: a learned vector is added to the logits.  ``shared_gate``: the shared expert's
    output is multiplied, token by token, by sigmoid(w_sg . x) ("shared.sg.weight" [1, hidden]); the row rides in the
    shared expert's first product and the share is applied before its last product, which is linear.
    Options: ``experts``, ``top``, ``groups``, ``keep``, ``router_scale``, ``shared``, ``router``, ``vocab``,
    ``weights``, ``router_bias``, ``shared_gate``; ``intermediate`` is an expert's inner size."""
    capturable = True
    launches_only = True

    def __init__(self, spec: FeedForwardSpec):
        self.spec = spec
        self.E, self.top = int(spec.option("experts")), int(spec.option("top"))
        self.groups, self.keep = int(spec.option("groups", 1)), int(spec.option("keep", 1))
        self.scale = float(spec.option("router_scale", 1.0))
        self.shared = int(spec.option("shared", 0))
        self.router = str(spec.option("router", "scores"))
        self.vocab = int(spec.option("vocab", 0))
        if self.router not in ("scores", "table"):
            raise ValueError(f"moe: router {self.router!r} is neither scores nor table")
        self.weights_by = str(spec.option("weights", "scores"))
        self.router_bias = bool(spec.option("router_bias", False))
        self.shared_gate = bool(spec.option("shared_gate", False))
        if self.weights_by not in ("scores", "softmax_chosen"):
            raise ValueError(f"moe: weights {self.weights_by!r} are neither scores nor softmax_chosen")
        if self.router == "table" and (self.weights_by != "scores" or self.router_bias):
            raise ValueError("moe: a table of experts has neither logits nor a bias")
        if self.weights_by == "softmax_chosen" and self.groups != 1:
            raise ValueError("moe: the softmax over the chosen logits takes one group of experts")
        if self.shared_gate and not self.shared:
            raise ValueError("moe: a gate on the shared expert needs a shared expert")
        if self.router == "table" and self.vocab < 1:
            raise ValueError("moe: a table of experts by token id needs the vocabulary's size")
        if spec.activation != "silu":
            raise ValueError("the experts' activation is silu")
        if not (0 < self.top <= self.E and self.groups >= 1 and self.E % self.groups == 0
                and 1 <= self.keep <= self.groups and self.keep * (self.E // self.groups) >= self.top):
            raise ValueError(f"moe: top {self.top} of {self.E} experts in {self.groups} groups of which "
                             f"{self.keep} stay is not possible")
        self.w_router = self.w_router_16 = self.w_gu = self.w_down = self.ws_gu = self.ws_down = self.table = None
        self.b_router = None

    def parameters(self) -> Dict[str, ParamSpec]:
        s, F = self.spec, self.spec.intermediate
        if self.router == "table":
            p = {"table": ParamSpec((self.vocab, self.top), "table_int", f"distinct:{self.E}")}
        else:
            p = {"router.weight": ParamSpec((self.E, s.hidden), "vector", "wide")}
            if self.router_bias:
                p["router.bias"] = ParamSpec((self.E,), "vector", "bias")
        for e in range(self.E):
            p[f"e{e}.gate.weight"] = ParamSpec((F, s.hidden))
            p[f"e{e}.up.weight"] = ParamSpec((F, s.hidden))
            p[f"e{e}.down.weight"] = ParamSpec((s.hidden, F))
        if self.shared:
            p["shared.gate.weight"] = ParamSpec((self.shared, s.hidden))
            p["shared.up.weight"] = ParamSpec((self.shared, s.hidden))
            p["shared.down.weight"] = ParamSpec((s.hidden, self.shared))
            if self.shared_gate:
                p["shared.sg.weight"] = ParamSpec((1, s.hidden))
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        if self.router == "table":
            self.table = t["table"]
            if int(self.table.min()) < 0 or int(self.table.max()) >= self.E:
                raise ValueError(f"moe: the table names experts outside 0..{self.E - 1}")
        else:
            self.w_router = t["router.weight"]
            self.b_router = t.get("router.bias")
            # Router weights whose values bfloat16 holds exactly (a 16-bit checkpoint's are) may go through the
            # tensor cores: the products are then exact and the sums 32-bit, which is what "32-bit logits" asks for.
            as16 = self.w_router.to(torch.bfloat16)
            self.w_router_16 = as16.contiguous() if bool((as16.float() == self.w_router).all()) else None
        mats = [t[f"e{e}.{n}.weight"] for e in range(self.E) for n in ("gate", "up", "down")]
        if len({m.dtype for m in mats}) > 1:
            t = dict(t)
            for k in list(t):
                if k not in ("router.weight", "router.bias", "table"):
                    t[k] = t[k].float()
        # every expert's gate rows, then its up rows: [E, 2F, hidden]; the down weights [E, hidden, F]
        self.w_gu = torch.stack([torch.cat([t[f"e{e}.gate.weight"], t[f"e{e}.up.weight"]], 0)
                                 for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down.weight"] for e in range(self.E)]).contiguous()
        if self.shared:
            rows = [t["shared.gate.weight"], t["shared.up.weight"]]
            if self.shared_gate:
                # the share's row behind the up projection's, then rows of zeros up to whole 16-byte output rows
                rows.append(t["shared.sg.weight"].to(rows[0].dtype))
                pad = (8 - (2 * self.shared + 1) % 8) % 8
                if pad:
                    rows.append(torch.zeros((pad, rows[0].shape[1]), dtype=rows[0].dtype, device=rows[0].device))
            self.ws_gu = torch.cat(rows, 0).contiguous()
            self.ws_down = t["shared.down.weight"]

    def products(self):
        out = [("router", self.w_router, None, None)] if self.router != "table" else []
        if self.shared:
            out += [("shared.gate_up", self.ws_gu, None, None), ("shared.down", self.ws_down, None, None)]
        return out

    def route(self, xn, ctx=None):
        """(experts int32 [T, top], weights float32 [T, top]) of the step's tokens."""
        if self.router == "table":
            return ops.moe_route_table(ctx.tokens, self.table, self.E)
        if xn.dtype == torch.bfloat16 and self.w_router_16 is not None and xn.shape[1] % 8 == 0:
            logits = ops.linear(xn, self.w_router_16, None, out_dtype=torch.float32)
            return ops.moe_route(logits, self.top, self.groups, self.keep, self.scale, self.b_router,
                                 self.weights_by == "softmax_chosen")
        return ops.moe_route_from(xn, self.w_router, self.top, self.groups, self.keep, self.scale, self.b_router,
                                  self.weights_by == "softmax_chosen")

    def forward(self, xn, ctx, add: Sequence[torch.Tensor], out=None) -> torch.Tensor:
        if len(add) > (2 if self.shared else 1):
            raise ValueError("more tensors to add than this feed-forward's kernels take")
        side = getattr(ctx, "side_stream", None)
        if self.shared and side is not None and len(add) <= 1 and torch.cuda.current_stream() != side:
            # few tokens: every kernel is short, and the shared expert's three do not depend on the router.  They run on
            # a second stream beside the routing and the chosen experts' products and join in the kernel that sums a
            # token's experts (the same sums in another order: (shared + what is to be added) + experts).
            main = torch.cuda.current_stream()
            ys = ops.empty((xn.shape[0], self.spec.hidden), torch.float32, xn.device)
            fork, join = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            with torch.cuda.stream(side):
                gu = ops.linear(xn, self.ws_gu, None, out_dtype=ctx.act_dtype)
                hs = (ops.gated_act(gu, "silu", inner=self.shared, row_gate=2 * self.shared) if self.shared_gate
                      else ops.gated_act(gu, "silu"))
                ops.linear(hs, self.ws_down, None, add0=add[0] if len(add) > 0 else None, out_dtype=torch.float32, out=ys)
                join.record(side)

            def shared():
                main.wait_event(join)
                return ys

            ids, weights = self.route(xn, ctx)
            return ops.moe_experts(xn, ids, weights, self.w_gu, self.w_down, add=shared, out=out)
        ids, weights = self.route(xn, ctx)
        out = ops.moe_experts(xn, ids, weights, self.w_gu, self.w_down, add=add[0] if len(add) > 0 else None, out=out)
        if self.shared:
            gu = ops.linear(xn, self.ws_gu, None, out_dtype=ctx.act_dtype)
            hs = (ops.gated_act(gu, "silu", inner=self.shared, row_gate=2 * self.shared) if self.shared_gate
                  else ops.gated_act(gu, "silu"))
            ops.linear(hs, self.ws_down, None, add0=out, add1=add[1] if len(add) > 1 else None,
                       out_dtype=torch.float32, out=out)
        return out


register_feed_forward("dense", DenseFeedForward)
register_feed_forward("moe", MixtureOfExperts)
register_feed_forward("gated", GatedFeedForward)
