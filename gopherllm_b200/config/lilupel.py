"""The Lilupel design: a decoder whose layers mix tokens by a state-space layer with a scalar decay per head, or by
a windowed softmax attention and a retention side by side, and whose feed-forwards are mixtures of experts chosen
by token id.

config.json lists the layers one by one: ``layers[i].type`` is ``mamba2`` or ``parallel``, ``layers[i].mixer``
the mixer's sizes and constants, ``layers[i].mlp`` a mixture of experts or null.  A layer with ``weights_of: j``
has no tensors of its own: it runs layer j's mixer, feed-forward and norms on a cache entry and state of its own.
A layer norms what a sublayer returns, not what it reads:

    x <- x + norm1(mixer(x));  x <- x + norm2(ff(x)),   norm(y) = y / sqrt(mean(y^2) + eps) * (1 + w).

  mamba2    see parts/recurrent.py (StateSpaceDual)
  parallel  left_scale * left(x) + right_scale * right(x).  left: grouped-query attention with biases on q, k, v and
            the output; the first rot.dims dims of every head rotated, then every head of q and k divided by its
            root mean square; score = q . k * scale; a window of the last mask.size positions; a sink per head in the
            softmax's denominator.  right: retention, a matrix memory with a fixed decay per head, rotated q and k,
            k / sqrt(dim), per-head unit norm, a silu gate.
  moe       a table [vocab, top] names every token id's experts; each counts 1 / top; experts are gated silu
            feed-forwards without biases.

The embedding is tied to the head; the final norm has the same (1 + w) form.  Every size and every constant that
differs between models comes from config.json.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Optional

from .registry import Architecture, register_architecture
from .specs import BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry

# the design sets no longest sequence; the cache's size bounds one
UNBOUNDED_POSITIONS = 1 << 20


def _int(where: str, d: dict, key: str, least: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ValueError(f"config.json: {where}.{key} must be an integer of at least {least}, is {v!r}")
    return v


def _number(where: str, d: dict, key: str, positive: bool = True) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or (positive and not v > 0):
        raise ValueError(f"config.json: {where}.{key} must be a {'positive ' if positive else ''}number, is {v!r}")
    return float(v)


def _object(where: str, d: dict, key: str) -> dict:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ValueError(f"config.json: {where}.{key} must be an object")
    return v


@dataclass
class LilupelConfig:
    """Typed view of a Lilupel config.json (key names are the file's own)."""
    vocab: int
    width: int
    layers: list
    norm_eps: float
    architecture: str = "Lilupel"
    torch_dtype: str = "bfloat16"
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, d: dict) -> "LilupelConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in d]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        if not isinstance(d["norm"], dict):
            raise ValueError("config.json: norm must be an object with eps")
        cfg = cls(vocab=_int("config", d, "vocab"), width=_int("config", d, "width"),
                  layers=copy.deepcopy(d["layers"]), norm_eps=_number("norm", d["norm"], "eps"),
                  architecture=str(d.get("architecture", "Lilupel")),
                  torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
                  initializer_range=float(d.get("initializer_range", 0.05)))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
                "torch_dtype": self.torch_dtype, "initializer_range": self.initializer_range}

    def validate(self) -> None:
        if not isinstance(self.layers, list) or not self.layers:
            raise ValueError("config.json: layers must be a non-empty list")
        lilupel_model_spec(self)            # raises on anything a part or the schedule cannot take


def _rotation(where: str, m: dict, dim: int) -> PositionSpec:
    rot = m.get("rot")
    if rot is None:
        return PositionSpec("none")
    if not isinstance(rot, dict):
        raise ValueError(f"config.json: {where}.rot must be an object")
    dims = rot.get("dims", 0)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ValueError(f"config.json: {where}.rot.dims must be even and at most dim, is {dims!r}")
    if dims == 0:
        return PositionSpec("none")
    return PositionSpec("rope", dims, _number(where + ".rot", rot, "base"), interleaved=False,
                        extra=(("exact_angles", True),))


def _window_attention(cfg: LilupelConfig, m: dict, where: str) -> MixerSpec:
    heads, kv = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv:
        raise ValueError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv}")
    dim = _int(where, m, "dim")
    window = _int(where + ".mask", _object(where, m, "mask"), "size") if m.get("mask") is not None else 0
    return MixerSpec(kind="attention_mixed", hidden=cfg.width, num_heads=heads, num_kv_heads=kv, head_dim=dim,
                     value_dim=_int(where, m, "vdim"), window=window, q_scale=1.0, bias=True,
                     position=_rotation(where, m, dim),
                     extra=(("score_scale", _number(where, m, "scale")), ("qk_norm", "head_unit"),
                            ("norm_eps", cfg.norm_eps), ("sink", True), ("out_bias", True)))


def _retention(cfg: LilupelConfig, m: dict, where: str) -> MixerSpec:
    heads, dim = _int(where, m, "heads"), _int(where, m, "dim")
    decay = m.get("decay")
    if (not isinstance(decay, list) or len(decay) != heads
            or any(isinstance(d, bool) or not isinstance(d, (int, float)) or not 0.0 < d <= 1.0 for d in decay)):
        raise ValueError(f"config.json: {where}.decay must list one factor in (0, 1] for each of the {heads} heads")
    return MixerSpec(kind="retention", hidden=cfg.width, num_heads=heads, num_kv_heads=heads, head_dim=dim,
                     value_dim=_int(where, m, "vdim"), bias=False, position=_rotation(where, m, dim),
                     extra=(("decay", tuple(float(d) for d in decay)), ("norm_eps", cfg.norm_eps)))


def _parallel(cfg: LilupelConfig, m: dict, where: str) -> MixerSpec:
    return MixerSpec(kind="scaled_pair", hidden=cfg.width, bias=False,
                     extra=(("left", _window_attention(cfg, _object(where, m, "left"), where + ".left")),
                            ("right", _retention(cfg, _object(where, m, "right"), where + ".right")),
                            ("left_scale", _number(where, m, "left_scale", positive=False)),
                            ("right_scale", _number(where, m, "right_scale", positive=False))))


def _mamba2(cfg: LilupelConfig, m: dict, where: str) -> MixerSpec:
    heads, groups = _int(where, m, "heads"), _int(where, m, "groups")
    if heads % groups:
        raise ValueError(f"config.json: {where}.heads {heads} is not a multiple of groups {groups}")
    vdim, parts = _int(where, m, "vdim"), _int(where, m, "norm_groups")
    if (heads * vdim) % parts:
        raise ValueError(f"config.json: {where}: {heads * vdim} channels do not form {parts} equal parts for the norm")
    return MixerSpec(kind="mamba2", hidden=cfg.width, num_heads=heads, value_dim=vdim, bias=False,
                     extra=(("state", _int(where, m, "state")), ("groups", groups), ("conv", _int(where, m, "conv")),
                            ("norm_groups", parts), ("norm_eps", cfg.norm_eps)))


_MIXERS = {"parallel": _parallel, "mamba2": _mamba2}


def _feed_forward(cfg: LilupelConfig, mlp: Optional[dict], where: str) -> Optional[FeedForwardSpec]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind", "moe") != "moe":
        raise ValueError(f"config.json: {where} must be a mixture of experts (kind moe) or null")
    r, ex = _object(where, mlp, "router"), _object(where, mlp, "expert")
    experts, top = _int(where + ".router", r, "experts"), _int(where + ".router", r, "top")
    if top > experts:
        raise ValueError(f"config.json: {where}.router: top {top} of {experts} experts is not possible")
    return FeedForwardSpec(kind="moe", hidden=cfg.width, intermediate=_int(where + ".expert", ex, "ff"),
                           activation="silu", bias=False,
                           extra=(("experts", experts), ("top", top), ("router", "table"), ("vocab", cfg.vocab)))


def own_layers(cfg: LilupelConfig) -> list:
    """Indices (in config.json's list) of the layers that have tensors of their own, in order."""
    return [i for i, L in enumerate(cfg.layers) if not (isinstance(L, dict) and L.get("weights_of") is not None)]


def lilupel_model_spec(cfg: LilupelConfig) -> ModelSpec:
    norm = NormSpec("rmsnorm", cfg.width, cfg.norm_eps, bias=False, weight_offset=1.0)
    layers, schedule = [], []
    block_of = {}                    # layer of the file -> index of its block
    n = len(cfg.layers)
    for i, L in enumerate(cfg.layers):
        where = f"layers[{i}]"
        if not isinstance(L, dict) or L.get("type") not in _MIXERS:
            raise ValueError(f"config.json: {where}.type must be one of {', '.join(sorted(_MIXERS))}")
        if L.get("weights_of") is not None:
            continue
        mixer = _MIXERS[L["type"]](cfg, _object(where, L, "mixer"), where + ".mixer")
        ffn = _feed_forward(cfg, L.get("mlp"), where + ".mlp")
        block_of[i] = len(layers)
        layers.append(BlockSpec(arrangement="post_norm", norm=norm, mixer=mixer, ffn=ffn,
                                norm2=norm if ffn is not None else None))
    for i, L in enumerate(cfg.layers):
        where = f"layers[{i}]"
        source, hops = i, 0
        while cfg.layers[source].get("weights_of") is not None:       # a layer may name one that names another
            nxt = cfg.layers[source]["weights_of"]
            hops += 1
            if isinstance(nxt, bool) or not isinstance(nxt, int) or not 0 <= nxt < n or nxt == source or hops > n:
                raise ValueError(f"config.json: {where}.weights_of must lead to a layer with tensors of its own, "
                                 f"is {L.get('weights_of')!r}")
            source = nxt
        if source != i:
            theirs = cfg.layers[source]
            if any(theirs.get(k) != L.get(k) for k in ("type", "mixer", "mlp")):
                raise ValueError(f"config.json: {where} runs on layer {source}'s weights but its entry differs")
        schedule.append(ScheduleEntry(layer=block_of[source], cache=i))
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, max_positions=UNBOUNDED_POSITIONS, layers=tuple(layers),
                     schedule=tuple(schedule), final_norm=norm, tie_embeddings=True, head_bias=False)


class LilupelTensorNames:
    """Names of the tensors in a Lilupel safetensors file: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``,
    ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, with i the layer's place in config.json's list (a layer that
    runs on another's weights has none); a linear layer's weight carries no suffix, its bias ``.b``, a
    convolution's taps ``.conv`` and their bias ``.conv.b``."""
    _top = {"embedding": "embed", "final_norm/weight": "final.norm"}
    _slots = {"norm": "norm1", "norm2": "norm2", "mixer": "mix", "ffn": "mlp"}

    def __init__(self, cfg: LilupelConfig):
        self.cfg = cfg
        self.file_index = own_layers(cfg)

    def top(self, key: str) -> str:
        return self._top[key]

    def layer(self, i: int, slot: str, key: str) -> str:
        """Parts spell a parameter "left.q.weight", "left.q.bias", "conv.bias", "norm.weight", "e3.gate.weight";
        the file spells them "left.q", "left.q.b", "conv.b", "norm", "e3.gate"."""
        base = f"l{self.file_index[i]}.{self._slots[slot]}"
        if slot in ("norm", "norm2"):
            return base
        words = key.split(".")
        if words[-1] == "weight":
            words = words[:-1]
        elif words[-1] == "bias":
            words[-1] = "b"
        return ".".join([base] + words)


register_architecture(
    Architecture(name="lilupel", config_class=LilupelConfig, build_spec=lilupel_model_spec,
                 tensor_names=LilupelTensorNames),
)
