"""Small Darusun configurations for the tests, with weights made by the tests themselves.

The tensors are drawn here by name (the design's naming rules, restated), written with the library's container
writer and read back by the library and by the plain implementation, so a wrong name or shape on either side shows.
The configurations differ in every respect: widths (one a multiple of nothing), head counts (one head, as many
key/value heads as query heads, six query heads on one key/value head), key sizes that are no multiples of 16, value
sizes other than key sizes, latents of other sizes than the heads they feed, query latents smaller and larger than
the key/value latents, rotations of a part of a head, of the whole head and of nothing, windows shorter than a page,
longer than two pages and of one position, one to three experts a token (all of them, one of them), mixtures with and
without a shared expert, layers without a feed-forward, layers on an earlier layer's keys (a neighbour's and a distant
one's, once and twice), either kind of layer first, factors on the sublayers of one and other than one.
"""
import json
import os
import tempfile

import torch

ALPHA = dict(
    architecture="Darusun", vocab=300, width=64, norm={"eps": 1e-6}, residual_mult=0.5,
    layers=[
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3, "rot": {"dims": 8, "base": 10000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 16}}},
        {"type": "latent_attention",
         "mixer": {"heads": 4, "dim": 16, "rot_dim": 8, "vdim": 24, "q_rank": 32, "kv_rank": 40, "scale": 0.2,
                   "mask": {"size": 20}, "rot": {"dims": 8, "base": 500.0}},
         "mlp": {"kind": "dense", "ff": 48}},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3, "rot": {"dims": 8, "base": 10000.0},
                   "kv_from": 0},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 2, "dim": 8, "rot_dim": 16, "vdim": 16, "q_rank": 24, "kv_rank": 32, "scale": 0.25,
                   "mask": {"size": 70}, "rot": {"dims": 16, "base": 10000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 3, "top": 1}}},
    ])

BETA = dict(
    architecture="Darusun", vocab=257, width=96, norm={"eps": 1e-5}, residual_mult=1.0,
    layers=[
        {"type": "latent_attention",
         "mixer": {"heads": 3, "dim": 32, "rot_dim": 4, "vdim": 16, "q_rank": 20, "kv_rank": 64, "scale": 0.15,
                   "mask": {"size": 130}, "rot": {"dims": 4, "base": 3000.0}},
         "mlp": {"kind": "dense", "ff": 80}},
        {"type": "attention",
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "rot": {"dims": 32, "base": 3000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 4, "top": 3}, "shared": {"ff": 40}}},
        {"type": "attention",
         "mixer": {"heads": 6, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25},
         "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 1}}},
        {"type": "attention",
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "rot": {"dims": 32, "base": 3000.0},
                   "kv_from": 1},
         "mlp": {"kind": "dense", "ff": 24}},
        {"type": "attention",
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "rot": {"dims": 32, "base": 3000.0},
                   "kv_from": 1},
         "mlp": None},
    ])

# sizes that are multiples of nothing convenient
GAMMA = dict(
    architecture="Darusun", vocab=91, width=36, norm={"eps": 3e-6}, residual_mult=1.3,
    layers=[
        {"type": "attention",
         "mixer": {"heads": 6, "kv_heads": 3, "dim": 6, "vdim": 10, "scale": 0.4, "rot": {"dims": 2, "base": 7.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 5}, "router": {"experts": 2, "top": 2}, "shared": {"ff": 3}}},
        {"type": "latent_attention",
         "mixer": {"heads": 1, "dim": 5, "rot_dim": 2, "vdim": 7, "q_rank": 9, "kv_rank": 11, "scale": 0.5,
                   "mask": {"size": 3}, "rot": {"dims": 2, "base": 100.0}},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 5, "dim": 4, "rot_dim": 6, "vdim": 3, "q_rank": 12, "kv_rank": 10, "scale": 0.3,
                   "mask": {"size": 1}, "rot": {"dims": 6, "base": 50.0}},
         "mlp": {"kind": "dense", "ff": 13}},
    ])


def only(cfg, index, mlp=True):
    """A model of one layer of ``cfg`` (a mechanism alone), with or without its feed-forward."""
    layer = json.loads(json.dumps(cfg["layers"][index]))
    layer["mixer"].pop("kv_from", None)
    if not mlp:
        layer["mlp"] = None
    out = {k: v for k, v in cfg.items() if k != "layers"}
    out["layers"] = [layer]
    return out


def tensor_shapes(cfg):
    """name -> (shape, how it is drawn)."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": ((V, W), "embed"), "final.norm": ((), "one"), "head": ((V, W), "matrix")}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = ((), "one")
        if L["type"] == "attention":
            H, G, D, Vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": ((H * D, W), "query"), p + "mix.talk": ((H, H), "talk"), p + "mix.o": ((W, H * Vd), "matrix")})
            if m.get("kv_from") is None:
                s.update({p + "mix.k": ((G * D, W), "query"), p + "mix.v": ((G * Vd, W), "matrix")})
        else:
            H, D, R, Vd, Q, K = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            s.update({p + "mix.dq": ((Q, W), "matrix"), p + "mix.dq.norm": ((Q,), "gamma"), p + "mix.uq": ((H * (D + R), Q), "query"),
                      p + "mix.dkv": ((K + R, W), "matrix"), p + "mix.dkv.norm": ((K,), "gamma"),
                      p + "mix.uk": ((H * D, K), "query"), p + "mix.uv": ((H * Vd, K), "matrix"), p + "mix.sink": ((H,), "sink"),
                      p + "mix.g": ((H, W), "matrix"), p + "mix.o": ((W, H * Vd), "matrix")})
        mlp = L.get("mlp")
        if not mlp:
            continue
        s[p + "norm2"] = ((), "one")
        if mlp["kind"] == "dense":
            s.update({p + "mlp.up": ((mlp["ff"], W), "matrix"), p + "mlp.down": ((W, mlp["ff"]), "matrix"),
                      p + "mlp.act": ((2,), "sink")})
            continue
        F = mlp["expert"]["ff"]
        s.update({p + "mlp.router": ((mlp["router"]["experts"], W), "router"), p + "mlp.router.b": ((mlp["router"]["experts"],), "small")})
        for e in range(mlp["router"]["experts"]):
            s.update({f"{p}mlp.e{e}.gate": ((F, W), "matrix"), f"{p}mlp.e{e}.up": ((F, W), "matrix"),
                      f"{p}mlp.e{e}.down": ((W, F), "matrix")})
        if mlp.get("shared"):
            Fs = mlp["shared"]["ff"]
            s.update({p + "mlp.shared.gate": ((Fs, W), "matrix"), p + "mlp.shared.up": ((Fs, W), "matrix"),
                      p + "mlp.shared.down": ((W, Fs), "matrix"), p + "mlp.shared.sg": ((1, W), "matrix")})
    return s


def draw(cfg, seed, sharp=1.0):
    """Random bfloat16 tensors for ``cfg``.  ``sharp``: factor on the weights that make queries and keys (heads that
    are brought to unit length afterwards do not feel it; the latent attention's do)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, kind) in sorted(tensor_shapes(cfg).items()):
        z = torch.randn(shape, generator=g)
        if kind == "matrix":
            t = z * (1.0 / shape[-1] ** 0.5)
        elif kind == "query":
            t = z * (sharp / shape[-1] ** 0.5)
        elif kind == "router":
            t = z * (3.0 / shape[-1] ** 0.5)          # logits a few apart: few close calls
        elif kind == "embed":
            t = z
        elif kind == "gamma":
            t = 1.0 + 0.1 * z
        elif kind == "one":
            t = 1.0 + 0.2 * z
        elif kind == "small":
            t = 0.3 * z
        elif kind == "sink":
            t = z
        elif kind == "talk":
            t = torch.eye(shape[0]) + 0.3 * z
        else:
            raise ValueError(kind)
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(cfg, tensors, folder=None):
    from gopherllm_b200.weights.safetensors_io import write_file
    folder = folder or tempfile.mkdtemp(prefix="gl_darusun_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(folder, "model.safetensors"), sorted(tensors.items()), metadata={"format": "pt"})
    return folder


def read_folder(folder):
    """(config dict, name -> 64-bit tensor) with a reader of the tests' own: 8 bytes of length, a JSON header, the data."""
    import struct
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    raw = open(os.path.join(folder, "model.safetensors"), "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
    tensors = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a:8 + n + b]), dtype=kinds[e["dtype"]]).reshape(e["shape"])
        tensors[name] = t.to(torch.float64)
    return cfg, tensors
