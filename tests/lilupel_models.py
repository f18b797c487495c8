"""Small Lilupel configurations for the tests, with weights made by the tests themselves.

The tensors are drawn here by name (the design's naming rules, restated), written with the library's
container writer and read back by the library and by the plain implementation, so a wrong name or shape
on either side shows.  The configurations differ in every respect: widths (one a multiple of nothing),
head counts (one head, as many key/value heads as query heads, six query heads on one key/value head),
key sizes that are no multiples of 16, value sizes other than key sizes, rotations of a part of a head, of the
whole head and of nothing, windows shorter than a page, longer than a page and of one position, one group and
several groups of B and C, norms in one part and in several, filters of one to four taps, one to three experts
a token, layers without a feed-forward, layers that run on an earlier layer's weights (a neighbour's and a
distant one's, once and twice), either kind of layer first.
"""
import json
import os
import tempfile

import torch

ALPHA = dict(
    architecture="Lilupel", vocab=300, width=64, norm={"eps": 1e-5},
    layers=[
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 8, "state": 16, "groups": 2, "conv": 3, "norm_groups": 2},
         "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3, "mask": {"size": 20},
                            "rot": {"dims": 8, "base": 10000.0}},
                   "right": {"heads": 2, "dim": 16, "vdim": 24, "decay": [0.9, 0.99], "rot": {"dims": 16, "base": 500.0}},
                   "left_scale": 0.7, "right_scale": 1.3},
         "mlp": {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 3, "top": 1}}},
        {"type": "mamba2", "mixer": {"heads": 2, "vdim": 24, "state": 8, "groups": 1, "conv": 2, "norm_groups": 1},
         "mlp": None},
        {"type": "parallel",
         "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3, "mask": {"size": 20},
                            "rot": {"dims": 8, "base": 10000.0}},
                   "right": {"heads": 2, "dim": 16, "vdim": 24, "decay": [0.9, 0.99], "rot": {"dims": 16, "base": 500.0}},
                   "left_scale": 0.7, "right_scale": 1.3},
         "mlp": {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 3, "top": 1}}, "weights_of": 1},
    ])

BETA = dict(
    architecture="Lilupel", vocab=257, width=96, norm={"eps": 1e-6},
    layers=[
        {"type": "parallel",
         "mixer": {"left": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "mask": {"size": 70},
                            "rot": {"dims": 32, "base": 3000.0}},
                   "right": {"heads": 1, "dim": 48, "vdim": 40, "decay": [0.995]},
                   "left_scale": 1.0, "right_scale": 0.5},
         "mlp": None},
        {"type": "mamba2", "mixer": {"heads": 3, "vdim": 32, "state": 40, "groups": 1, "conv": 4, "norm_groups": 1},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 4, "top": 3}}},
        {"type": "mamba2", "mixer": {"heads": 3, "vdim": 32, "state": 40, "groups": 1, "conv": 4, "norm_groups": 1},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 4, "top": 3}}, "weights_of": 1},
        {"type": "parallel",
         "mixer": {"left": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "mask": {"size": 70},
                            "rot": {"dims": 32, "base": 3000.0}},
                   "right": {"heads": 1, "dim": 48, "vdim": 40, "decay": [0.995]},
                   "left_scale": 1.0, "right_scale": 0.5},
         "mlp": None, "weights_of": 0},
        {"type": "mamba2", "mixer": {"heads": 3, "vdim": 32, "state": 40, "groups": 1, "conv": 4, "norm_groups": 1},
         "mlp": {"kind": "moe", "expert": {"ff": 32}, "router": {"experts": 4, "top": 3}}, "weights_of": 1},
    ])

# sizes that are multiples of nothing convenient
GAMMA = dict(
    architecture="Lilupel", vocab=91, width=36, norm={"eps": 3e-6},
    layers=[
        {"type": "mamba2", "mixer": {"heads": 3, "vdim": 5, "state": 7, "groups": 3, "conv": 1, "norm_groups": 3},
         "mlp": {"kind": "moe", "expert": {"ff": 11}, "router": {"experts": 4, "top": 3}}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 6, "kv_heads": 1, "dim": 6, "vdim": 10, "scale": 0.4, "mask": {"size": 3},
                            "rot": {"dims": 2, "base": 7.0}},
                   "right": {"heads": 2, "dim": 10, "vdim": 6, "decay": [1.0, 0.5], "rot": {"dims": 4, "base": 100.0}},
                   "left_scale": -0.5, "right_scale": 2.0},
         "mlp": {"kind": "moe", "expert": {"ff": 5}, "router": {"experts": 2, "top": 2}}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.25, "mask": {"size": 1},
                            "rot": {"dims": 16, "base": 50.0}},
                   "right": {"heads": 2, "dim": 8, "vdim": 20, "decay": [0.75, 0.875], "rot": {"dims": 8, "base": 20.0}},
                   "left_scale": 1.0, "right_scale": 1.0},
         "mlp": None},
    ])


def only(cfg, index, mlp=True):
    """A model of one layer of ``cfg`` (a mechanism alone), with or without a feed-forward."""
    layer = json.loads(json.dumps(cfg["layers"][index]))
    layer.pop("weights_of", None)
    if not mlp:
        layer["mlp"] = None
    elif layer["mlp"] is None:
        layer["mlp"] = {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 2}}
    out = {k: v for k, v in cfg.items() if k != "layers"}
    out["layers"] = [layer]
    return out


def tensor_shapes(cfg):
    """name -> (shape, how it is drawn)."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": ((V, W), "embed"), "final.norm": ((W,), "offset")}
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = ((W,), "offset")
        if L["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            s.update({p + "mix.in": ((2 * inner + 2 * G * N + H, W), "matrix"), p + "mix.conv": ((ch, m["conv"]), "taps"),
                      p + "mix.conv.b": ((ch,), "small"), p + "mix.dt_bias": ((H,), "step"), p + "mix.A_log": ((H,), "decay"),
                      p + "mix.D": ((H,), "gamma"), p + "mix.norm": ((inner,), "gamma"), p + "mix.o": ((W, inner), "matrix")})
        else:
            a, r = m["left"], m["right"]
            H, G, D, Vd = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            s.update({p + "mix.left.q": ((H * D, W), "query"), p + "mix.left.q.b": ((H * D,), "small"),
                      p + "mix.left.k": ((G * D, W), "query"), p + "mix.left.k.b": ((G * D,), "small"),
                      p + "mix.left.v": ((G * Vd, W), "matrix"), p + "mix.left.v.b": ((G * Vd,), "small"),
                      p + "mix.left.o": ((W, H * Vd), "matrix"), p + "mix.left.o.b": ((W,), "small"),
                      p + "mix.left.sink": ((H,), "sink")})
            H, D, Vd = r["heads"], r["dim"], r["vdim"]
            s.update({p + "mix.right.q": ((H * D, W), "matrix"), p + "mix.right.k": ((H * D, W), "matrix"),
                      p + "mix.right.v": ((H * Vd, W), "matrix"), p + "mix.right.g": ((H * Vd, W), "matrix"),
                      p + "mix.right.o": ((W, H * Vd), "matrix")})
        mlp = L.get("mlp")
        if mlp:
            s[p + "norm2"] = ((W,), "offset")
            F = mlp["expert"]["ff"]
            s[p + "mlp.table"] = ((V, mlp["router"]["top"]), f"table:{mlp['router']['experts']}")
            for e in range(mlp["router"]["experts"]):
                s.update({f"{p}mlp.e{e}.gate": ((F, W), "matrix"), f"{p}mlp.e{e}.up": ((F, W), "matrix"),
                          f"{p}mlp.e{e}.down": ((W, F), "matrix")})
    return s


def draw(cfg, seed, long_memory=False, sharp=1.0):
    """Random tensors (bfloat16, tables int32) for ``cfg``.  ``long_memory``: state-space decays near one, so that
    a state still holds tokens from hundreds of positions back.  ``sharp``: factor on the attention's query and key
    weights (the heads are brought to unit length afterwards, so it only outweighs the biases) ."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, kind) in sorted(tensor_shapes(cfg).items()):
        if kind.startswith("table:"):
            E = int(kind.split(":")[1])
            out[name] = torch.stack([torch.randperm(E, generator=g)[:shape[1]] for _ in range(shape[0])]).to(torch.int32)
            continue
        z = torch.randn(shape, generator=g)
        if kind == "matrix":
            t = z * (1.0 / shape[-1] ** 0.5)
        elif kind == "query":
            t = z * (sharp / shape[-1] ** 0.5)
        elif kind == "embed":
            t = z
        elif kind == "gamma":
            t = 1.0 + 0.1 * z
        elif kind == "offset":
            t = 0.2 * z
        elif kind == "small":
            t = 0.1 * z
        elif kind == "sink":
            t = z
        elif kind == "taps":
            t = 0.6 * z
        elif kind == "decay":
            t = 0.5 * z - (4.0 if long_memory else 0.0)
        elif kind == "step":
            t = z - (2.0 if long_memory else 0.0)
        else:
            raise ValueError(kind)
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(cfg, tensors, folder=None):
    from gopherllm_b200.weights.safetensors_io import write_file
    folder = folder or tempfile.mkdtemp(prefix="gl_lilupel_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(folder, "model.safetensors"), sorted(tensors.items()), metadata={"format": "pt"})
    return folder


def read_folder(folder):
    """(config dict, name -> 64-bit tensor, integer tables as int64) with a reader of the tests' own: 8 bytes of
    length, a JSON header, the data."""
    import struct
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    raw = open(os.path.join(folder, "model.safetensors"), "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}
    tensors = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a:8 + n + b]), dtype=kinds[e["dtype"]]).reshape(e["shape"])
        tensors[name] = t.to(torch.int64) if e["dtype"] == "I32" else t.to(torch.float64)
    return cfg, tensors
