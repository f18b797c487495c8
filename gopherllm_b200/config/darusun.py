"""The Darusun design: a decoder whose layers mix tokens by grouped softmax attention whose heads' scores are mixed by
a learned table before the softmax, or by attention through a latent with a window, a sink and a gate per head; with
dense feed-forwards whose activation has two learned numbers, or mixtures of experts with a softmax over the chosen
logits and a gated shared expert.

config.json lists the layers one by one: ``layers[i].type`` is ``attention`` or ``latent_attention``,
``layers[i].mixer`` the mixer's sizes and constants, ``layers[i].mlp`` a feed-forward (``kind`` dense or moe) or null.
A layer norms what a sublayer returns, not what it reads, with ONE number as the norm's weight, and adds it times a
factor the whole model shares:

    x <- x + m * norm1(mixer(x));  x <- x + m * norm2(ff(x)),   norm(y) = y / sqrt(mean(y^2) + eps) * g,  m = residual_mult.

  attention         H query heads on G key/value heads (key size dim, value size vdim), no biases; the first rot.dims
                    dims of every head of q and k rotated (dim i with dim i + dims/2), then every head divided by its
                    root mean square; score = q . k * scale; the heads' scores mixed by a table [H, H]; causal softmax.
                    With ``kv_from: j`` the layer has no key and value projections and reads layer j's cache entry.
  latent_attention  see parts/attention.py (LatentAttention): query latent q_rank, key/value latent kv_rank, per head dim
                    plain and rot_dim rotated dims (dim 2i with dim 2i + 1), values vdim, a window of mask.size
                    positions, a sink per head, a sigmoid gate per head.
  dense             W_down act(W_up x), act = xielu with the two numbers of tensor ``act``.
  moe               logits W_router x + b; the ``top`` largest chosen, weights the softmax over those; experts
                    W_down (silu(W_gate x) * W_up x); a shared expert of the same form times sigmoid(w_sg . x).

The head has weights of its own and no bias; the final norm has the one-number form.  Every size and every constant
that differs between models comes from config.json.
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
class DarusunConfig:
    """Typed view of a Darusun config.json (key names are the file's own)."""
    vocab: int
    width: int
    layers: list
    norm_eps: float
    residual_mult: float
    architecture: str = "Darusun"
    torch_dtype: str = "bfloat16"
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, d: dict) -> "DarusunConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "residual_mult") if k not in d]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        if not isinstance(d["norm"], dict):
            raise ValueError("config.json: norm must be an object with eps")
        cfg = cls(vocab=_int("config", d, "vocab"), width=_int("config", d, "width"),
                  layers=copy.deepcopy(d["layers"]), norm_eps=_number("norm", d["norm"], "eps"),
                  residual_mult=_number("config", d, "residual_mult", positive=False),
                  architecture=str(d.get("architecture", "Darusun")),
                  torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
                  initializer_range=float(d.get("initializer_range", 0.05)))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "torch_dtype": self.torch_dtype,
                "initializer_range": self.initializer_range}

    def validate(self) -> None:
        if not isinstance(self.layers, list) or not self.layers:
            raise ValueError("config.json: layers must be a non-empty list")
        darusun_model_spec(self)            # raises on anything a part or the schedule cannot take


def _rotation(where: str, m: dict, dim: int, interleaved: bool) -> PositionSpec:
    rot = m.get("rot")
    if rot is None:
        return PositionSpec("none")
    if not isinstance(rot, dict):
        raise ValueError(f"config.json: {where}.rot must be an object")
    dims = rot.get("dims", 0)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ValueError(f"config.json: {where}.rot.dims must be even and at most {dim}, is {dims!r}")
    if dims == 0:
        return PositionSpec("none")
    return PositionSpec("rope", dims, _number(where + ".rot", rot, "base"), interleaved=interleaved,
                        extra=(("exact_angles", True),))


def _window(where: str, m: dict) -> int:
    return _int(where + ".mask", _object(where, m, "mask"), "size") if m.get("mask") is not None else 0


def _attention(cfg: DarusunConfig, m: dict, where: str) -> MixerSpec:
    heads, kv = _int(where, m, "heads"), _int(where, m, "kv_heads")
    if heads % kv:
        raise ValueError(f"config.json: {where}.heads {heads} is not a multiple of kv_heads {kv}")
    dim = _int(where, m, "dim")
    extra = [("score_scale", _number(where, m, "scale")), ("qk_norm", "head_unit"), ("norm_eps", cfg.norm_eps),
             ("talk_scores", True)]
    if m.get("kv_from") is not None:
        extra.append(("shared_kv", True))
    return MixerSpec(kind="attention_mixed", hidden=cfg.width, num_heads=heads, num_kv_heads=kv, head_dim=dim,
                     value_dim=_int(where, m, "vdim"), window=_window(where, m), q_scale=1.0, bias=False,
                     position=_rotation(where, m, dim, interleaved=False), extra=tuple(extra))


def _latent_attention(cfg: DarusunConfig, m: dict, where: str) -> MixerSpec:
    rot_dim = _int(where, m, "rot_dim", least=0)
    if rot_dim % 2:
        raise ValueError(f"config.json: {where}.rot_dim must be even, is {rot_dim}")
    position = _rotation(where, m, rot_dim, interleaved=True)
    if rot_dim and (position.kind == "none" or position.rotary_dim != rot_dim):
        raise ValueError(f"config.json: {where}.rot.dims must equal rot_dim {rot_dim}")
    return MixerSpec(kind="latent_attention", hidden=cfg.width, num_heads=_int(where, m, "heads"),
                     num_kv_heads=1, head_dim=_int(where, m, "dim"), value_dim=_int(where, m, "vdim"),
                     window=_window(where, m), q_scale=1.0, bias=False, position=position,
                     extra=(("q_rank", _int(where, m, "q_rank")), ("kv_rank", _int(where, m, "kv_rank")),
                            ("rot", rot_dim), ("score_scale", _number(where, m, "scale")),
                            ("norm_eps", cfg.norm_eps), ("sink", True), ("gate", True)))


_MIXERS = {"attention": _attention, "latent_attention": _latent_attention}


def _feed_forward(cfg: DarusunConfig, mlp: Optional[dict], where: str) -> Optional[FeedForwardSpec]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ValueError(f"config.json: {where} must be a feed-forward of kind dense or moe, or null")
    if mlp["kind"] == "dense":
        return FeedForwardSpec(kind="dense", hidden=cfg.width, intermediate=_int(where, mlp, "ff"),
                               activation="xielu", bias=False)
    r, ex = _object(where, mlp, "router"), _object(where, mlp, "expert")
    experts, top = _int(where + ".router", r, "experts"), _int(where + ".router", r, "top")
    if top > experts:
        raise ValueError(f"config.json: {where}.router: top {top} of {experts} experts is not possible")
    extra = [("experts", experts), ("top", top), ("weights", "softmax_chosen"), ("router_bias", True)]
    if mlp.get("shared") is not None:
        extra += [("shared", _int(where + ".shared", _object(where, mlp, "shared"), "ff")), ("shared_gate", True)]
    return FeedForwardSpec(kind="moe", hidden=cfg.width, intermediate=_int(where + ".expert", ex, "ff"),
                           activation="silu", bias=False, extra=tuple(extra))


def darusun_model_spec(cfg: DarusunConfig) -> ModelSpec:
    norm = NormSpec("rmsnorm", cfg.width, cfg.norm_eps, bias=False, single_weight=True)
    layers, schedule = [], []
    n = len(cfg.layers)
    for i, L in enumerate(cfg.layers):
        where = f"layers[{i}]"
        if not isinstance(L, dict) or L.get("type") not in _MIXERS:
            raise ValueError(f"config.json: {where}.type must be one of {', '.join(sorted(_MIXERS))}")
        m = _object(where, L, "mixer")
        mixer = _MIXERS[L["type"]](cfg, m, where + ".mixer")
        ffn = _feed_forward(cfg, L.get("mlp"), where + ".mlp")
        layers.append(BlockSpec(arrangement="post_norm", norm=norm, mixer=mixer, ffn=ffn,
                                norm2=norm if ffn is not None else None,
                                extra=(("branch_scale", cfg.residual_mult), ("hand_on_rounded", True))))
        source = m.get("kv_from") if L["type"] == "attention" else None
        if source is None:
            schedule.append(ScheduleEntry(layer=i, cache=i))
            continue
        if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
            raise ValueError(f"config.json: {where}.mixer.kv_from must name an earlier layer, is {source!r}")
        theirs = cfg.layers[source]
        tm = theirs.get("mixer") if isinstance(theirs, dict) else None
        if (not isinstance(tm, dict) or theirs.get("type") != "attention" or tm.get("kv_from") is not None
                or any(tm.get(k) != m.get(k) for k in ("heads", "kv_heads", "dim", "vdim", "rot", "mask"))):
            raise ValueError(f"config.json: {where}.mixer.kv_from names layer {source}, which is not an attention "
                             f"layer with key and value projections of the same head counts, sizes and rotation")
        schedule.append(ScheduleEntry(layer=i, cache=source, writes=False))
    return ModelSpec(hidden=cfg.width, vocab=cfg.vocab, max_positions=UNBOUNDED_POSITIONS, layers=tuple(layers),
                     schedule=tuple(schedule), final_norm=norm, tie_embeddings=False, head_bias=False)


class DarusunTensorNames:
    """Names of the tensors in a Darusun safetensors file: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``,
    ``l<i>.mlp.*``, ``final.norm``, ``head``; a linear layer's weight carries no suffix, a bias ``.b``."""
    _top = {"embedding": "embed", "final_norm/weight": "final.norm", "head/weight": "head"}
    _slots = {"norm": "norm1", "norm2": "norm2", "mixer": "mix", "ffn": "mlp"}

    def __init__(self, cfg: DarusunConfig):
        self.cfg = cfg

    def top(self, key: str) -> str:
        return self._top[key]

    def layer(self, i: int, slot: str, key: str) -> str:
        """Parts spell a parameter "q.weight", "dq.norm.weight", "router.bias", "e3.gate.weight", "talk"; the file
        spells them "q", "dq.norm", "router.b", "e3.gate", "talk"."""
        base = f"l{i}.{self._slots[slot]}"
        if slot in ("norm", "norm2"):
            return base
        words = key.split(".")
        if words[-1] == "weight":
            words = words[:-1]
        elif words[-1] == "bias":
            words[-1] = "b"
        return ".".join([base] + words)


register_architecture(
    Architecture(name="darusun", config_class=DarusunConfig, build_spec=darusun_model_spec,
                 tensor_names=DarusunTensorNames),
)
