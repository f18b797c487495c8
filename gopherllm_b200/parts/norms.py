"""Normalisation parts: LayerNorm and RMSNorm over the last axis."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.specs import NormSpec
from .base import Norm, ParamSpec, register_norm


class LayerNorm(Norm):
    """y = (x - mean) * rsqrt(var + eps) * weight + bias, biased variance, in
    32-bit with the reciprocal square root in 64-bit (bert.go:748-776)."""
    capturable = True
    launches_only = True
    rms = False

    def __init__(self, spec: NormSpec):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        # (a weight stored as its distance from weight_offset is drawn around zero in the random-weights mode)
        shape = () if self.spec.single_weight else (self.spec.dim,)
        p = {"weight": ParamSpec(shape, "vector", "bias" if self.spec.weight_offset else "gamma")}
        if self.spec.bias:
            p["bias"] = ParamSpec((self.spec.dim,), "vector", "beta")
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]
        if self.spec.single_weight:                  # one number for all coordinates: the kernels take a vector
            self.weight = self.weight.reshape(1).expand(self.spec.dim).contiguous()
        if self.spec.weight_offset:
            self.weight = (self.weight + float(self.spec.weight_offset)).contiguous()
        self.bias = tensors.get("bias")

    def fusable(self):
        return self.weight, self.bias, self.spec.eps, self.rms

    def forward(self, x, out_dtype, rows=None):
        return ops.norm(x, self.weight, self.bias, self.spec.eps, out_dtype, rms=self.rms, rows=rows)


class RMSNorm(LayerNorm):
    """y = x * rsqrt(mean(x²) + eps) * weight (model.go:2949-2981)."""
    rms = True


register_norm("layernorm", LayerNorm)
register_norm("rmsnorm", RMSNorm)
