"""The Lilupel design on the CPU: its configuration, tensor names, schedule and cache needs in the library,
and the plain implementation's own sanity."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import lilupel_models as lm
import plain_lilupel as pl
from gopherllm_b200.api import build_model
from gopherllm_b200.cache.sequence_cache import KVView, SequenceCache, StateView
from gopherllm_b200.config.registry import architecture_from_config
from gopherllm_b200.parts.base import KVRequest, StateRequest
from gopherllm_b200.weights.loader import check_folder, tensor_table


def build(cfg):
    arch = architecture_from_config(cfg)
    typed = arch.config_class.from_dict(cfg)
    return arch, typed, build_model(arch, typed)


@pytest.mark.parametrize("cfg", [lm.ALPHA, lm.BETA, lm.GAMMA], ids=["ALPHA", "BETA", "GAMMA"])
def test_declared_tensors_are_the_files_tensors(cfg):
    arch, typed, model = build(cfg)
    assert arch.name == "lilupel"
    table = tensor_table(model.parameters(), arch.tensor_names(typed))
    want = lm.tensor_shapes(cfg)
    assert set(table) == set(want)
    for name, (shape, _) in want.items():
        assert tuple(table[name][1].shape) == tuple(shape), name
    assert table["l0.mlp.table" if cfg is not lm.BETA else "l1.mlp.table"][1].kind == "table_int"


def test_every_constant_of_the_file_reaches_the_spec():
    _, typed, model = build(lm.ALPHA)
    spec = model.spec
    assert spec.tie_embeddings and not spec.head_bias and spec.final_norm.eps == 1e-5 and spec.final_norm.weight_offset == 1.0
    assert len(spec.layers) == 3 and all(b.arrangement == "post_norm" for b in spec.layers)
    ssd, pair, bare = (b.mixer for b in spec.layers)
    assert (ssd.kind, ssd.num_heads, ssd.value_dim) == ("mamba2", 4, 8)
    assert [ssd.option(k) for k in ("state", "groups", "conv", "norm_groups", "norm_eps")] == [16, 2, 3, 2, 1e-5]
    assert pair.kind == "scaled_pair" and (pair.option("left_scale"), pair.option("right_scale")) == (0.7, 1.3)
    left, right = pair.option("left"), pair.option("right")
    assert (left.kind, left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim, left.window) == ("attention_mixed", 4, 2, 16, 32, 20)
    assert left.option("score_scale") == 0.3 and left.option("qk_norm") == "head_unit" and left.option("sink") and left.bias
    assert (left.position.kind, left.position.rotary_dim, left.position.theta, left.position.interleaved) == ("rope", 8, 10000.0, False)
    assert (right.kind, right.num_heads, right.head_dim, right.value_dim) == ("retention", 2, 16, 24)
    assert right.option("decay") == (0.9, 0.99) and right.position.rotary_dim == 16 and right.position.theta == 500.0
    moe = spec.layers[1].ffn
    assert moe.kind == "moe" and moe.intermediate == 40
    assert [moe.option(k) for k in ("experts", "top", "router", "vocab")] == [3, 1, "table", 300]
    assert spec.layers[2].ffn is None and spec.layers[2].norm2 is None and bare.option("groups") == 1
    assert typed.to_dict()["layers"] == lm.ALPHA["layers"]
    # a retention without rotation
    _, _, other = build(lm.BETA)
    assert other.spec.layers[0].mixer.option("right").position.kind == "none"


def test_layers_that_run_on_another_layers_weights():
    arch, typed, model = build(lm.BETA)
    runs = model.spec.schedule
    assert [(e.layer, e.cache, e.writes) for e in runs] == [(0, 0, True), (1, 1, True), (1, 2, True), (0, 3, True), (1, 4, True)]
    assert len(model.blocks) == 2
    names = arch.tensor_names(typed)
    assert names.layer(1, "mixer", "conv.bias") == "l1.mix.conv.b" and names.layer(0, "mixer", "left.o.bias") == "l0.mix.left.o.b"
    _, typed_a, model_a = build(lm.ALPHA)
    assert [(e.layer, e.cache) for e in model_a.spec.schedule] == [(0, 0), (1, 1), (2, 2), (1, 3)]
    assert architecture_from_config(lm.ALPHA).tensor_names(typed_a).layer(2, "norm", "weight") == "l2.norm1"
    reqs = model.cache_requests()
    assert len(reqs) == 5
    # the pair keeps pages of keys (a window of 70) and values of another size, and the retention's memory
    assert reqs[0] == (KVRequest(3, 32, 70, value_dim=16), StateRequest((1 * 48 * 40,))) and reqs[3] == reqs[0]
    # the state-space layer keeps S [heads, state, vdim] and three taps back of its 96 + 2 x 40 convolved channels
    assert reqs[1] == StateRequest((3 * 40 * 32 + (96 + 80) * 3,)) and reqs[2] == reqs[1] == reqs[4]
    cache = SequenceCache(reqs, max_tokens=256, max_positions=256, dtype=torch.float32, device="cpu", max_slots=2)
    kv, state = cache.view(3)
    assert isinstance(kv, KVView) and isinstance(state, StateView) and isinstance(cache.view(2), StateView)
    assert tuple(kv.k.shape[1:]) == (3, 64, 32) and tuple(kv.v.shape[1:]) == (3, 64, 16)
    assert cache.view(0)[0].k.data_ptr() != kv.k.data_ptr() and cache.view(1).rows.data_ptr() != cache.view(2).rows.data_ptr()
    s = cache.open()
    cache.view(2).rows[s].fill_(7.0)
    cache.close(s)
    assert cache.open() == s and float(cache.view(2).rows[s].abs().max()) == 0.0


def test_weights_of_a_later_layer_and_of_a_layer_that_names_another():
    cfg = copy.deepcopy(lm.ALPHA)
    del cfg["layers"][3]["weights_of"]
    cfg["layers"][1]["weights_of"] = 3                 # the owner comes after its user
    arch, typed, model = build(cfg)
    assert [(e.layer, e.cache) for e in model.spec.schedule] == [(0, 0), (2, 1), (1, 2), (2, 3)]
    names = arch.tensor_names(typed)
    assert names.layer(2, "norm", "weight") == "l3.norm1" and names.layer(1, "mixer", "in.weight") == "l2.mix.in"
    cfg["layers"].append(dict(copy.deepcopy(cfg["layers"][1]), weights_of=1))     # 4 -> 1 -> 3
    _, _, chained = build(cfg)
    assert [(e.layer, e.cache) for e in chained.spec.schedule][-1] == (2, 4)
    cfg["layers"][3]["weights_of"] = 4                 # 3 -> 4 -> 1 -> 3: nobody has the tensors
    with pytest.raises(ValueError):
        build(cfg)


def _with(cfg, path, value):
    out = copy.deepcopy(cfg)
    at = out
    for k in path[:-1]:
        at = at[k]
    if value is KeyError:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return out


@pytest.mark.parametrize("path,value", [
    (("layers", 3, "weights_of"), 3), (("layers", 3, "weights_of"), 0), (("layers", 3, "weights_of"), 5),
    (("layers", 3, "mixer", "left_scale"), 0.8), (("layers", 1, "mixer", "left", "kv_heads"), 3),
    (("layers", 1, "mixer", "left", "scale"), KeyError), (("layers", 1, "mixer", "left", "rot", "dims"), 7),
    (("layers", 1, "mixer", "left", "rot", "dims"), 18), (("layers", 1, "mixer", "right", "decay"), [0.9]),
    (("layers", 1, "mixer", "right", "decay"), [0.9, 1.5]), (("layers", 1, "mixer", "left", "mask", "size"), 0),
    (("layers", 0, "mixer", "groups"), 3), (("layers", 0, "mixer", "norm_groups"), 3), (("layers", 0, "mixer", "conv"), 0),
    (("layers", 0, "mlp", "router", "top"), 6), (("layers", 0, "mlp", "kind"), "dense"), (("layers", 0, "type"), "mamba"),
    (("norm", "eps"), 0.0), (("width",), KeyError)])
def test_configurations_that_are_refused(path, value):
    with pytest.raises((ValueError, KeyError)):
        build(_with(lm.ALPHA, path, value))


def test_plain_layers_do_not_look_ahead():
    for cfg in (lm.ALPHA, lm.GAMMA):
        t = {k: (v.double() if v.dtype != torch.int32 else v.long()) for k, v in lm.draw(cfg, 2).items()}
        toks = [int(x) for x in np.random.default_rng(0).integers(0, cfg["vocab"], size=12)]
        a = pl.forward(toks, t, cfg)
        b = pl.forward(toks[:7], t, cfg)
        assert torch.allclose(a[:7], b, atol=1e-10)


def test_plain_rotation_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64).repeat(3, 1, 1)      # [T=3, 1 head, 6]
    y = pl.rotate(x, {"dims": 4, "base": 100.0})
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 4:], x[:, :, 4:])                         # position 0; the unrotated rest
    for p in (1, 2):
        for i, f in enumerate((1.0, 100.0 ** -0.5)):                                               # pairs (0, 2) and (1, 3)
            u, v = float(x[p, 0, i]), float(x[p, 0, i + 2])
            assert math.isclose(float(y[p, 0, i]), u * math.cos(p * f) - v * math.sin(p * f), abs_tol=1e-12)
            assert math.isclose(float(y[p, 0, i + 2]), v * math.cos(p * f) + u * math.sin(p * f), abs_tol=1e-12)
    assert torch.equal(pl.rotate(x, {"dims": 0, "base": 2.0}), x)


def test_plain_window_and_sink_by_hand():
    """One head, keys of unit length that all equal the query: every visible score is scale * dim (unit root mean
    square), so the weights are equal and the sink's share can be written down."""
    T, W, D, window, sink, scale = 7, 4, 4, 3, 0.7, 0.5
    w = {"q": torch.zeros(D, W), "q.b": torch.ones(D), "k": torch.zeros(D, W), "k.b": torch.ones(D),
         "v": torch.eye(D, W), "v.b": torch.zeros(D), "o": torch.eye(W, D), "o.b": torch.zeros(W), "sink": torch.tensor([sink])}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": scale, "mask": {"size": window}, "rot": {"dims": 0, "base": 10.0}}
    got = pl.window_attention(h, w, "", m, 0.0)
    score = scale * D                               # q . k of two all-ones heads brought to unit root mean square
    for t in range(T):
        seen = list(range(max(0, t - window + 1), t + 1))
        share = math.exp(score) / (len(seen) * math.exp(score) + math.exp(sink))
        assert torch.allclose(got[t], share * h[seen].sum(0), atol=1e-12)


def test_plain_retention_by_hand():
    """o_t = sum_j decay^(t-j) (q_t . k_j / sqrt(dim)) v_j before the unit norm and the gate."""
    torch.manual_seed(1)
    T, W, D, V, decay = 6, 5, 4, 3, 0.8
    w = {k: torch.randn(s, dtype=torch.float64) for k, s in (("q", (D, W)), ("k", (D, W)), ("v", (V, W)), ("g", (V, W)))}
    w["o"] = torch.eye(V, dtype=torch.float64)
    h = torch.randn(T, W, dtype=torch.float64)
    m = {"heads": 1, "dim": D, "vdim": V, "decay": [decay], "rot": {"dims": 0, "base": 10.0}}
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    o = torch.stack([sum(decay ** (t - j) * float(q[t] @ k[j]) / math.sqrt(D) * v[j] for j in range(t + 1)) for t in range(T)])
    gate = h @ w["g"].T
    want = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-6) * gate * torch.sigmoid(gate)
    assert torch.allclose(pl.retention(h, w, "", m, 1e-6), want, atol=1e-10)


def test_plain_state_space_layer_by_hand():
    """One head, one tap: y_t = sum_j exp(-rate (dt_{j+1} + .. + dt_t)) dt_j (C_t . B_j) x_j + D x_t, then gate and norm."""
    torch.manual_seed(2)
    T, W, P, N = 5, 6, 3, 4
    rows = 2 * P + 2 * N + 1
    w = {"in": torch.randn(rows, W), "conv": torch.ones(P + 2 * N, 1), "conv.b": torch.zeros(P + 2 * N), "dt_bias": torch.tensor([0.3]),
         "A_log": torch.tensor([-0.5]), "D": torch.tensor([1.5]), "norm": torch.randn(P), "o": torch.eye(P)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    m = {"heads": 1, "vdim": P, "state": N, "groups": 1, "conv": 1, "norm_groups": 1}
    u = h @ w["in"].T
    silu = lambda z: z * torch.sigmoid(z)
    z, x, B, C = u[:, :P], silu(u[:, P:2 * P]), silu(u[:, 2 * P:2 * P + N]), silu(u[:, 2 * P + N:2 * P + 2 * N])
    dt = torch.log1p(torch.exp(u[:, -1] + 0.3))
    rate = math.exp(-0.5)
    y = torch.zeros(T, P, dtype=torch.float64)
    for t in range(T):
        for j in range(t + 1):
            y[t] += math.exp(-rate * float(dt[j + 1:t + 1].sum())) * dt[j] * float(C[t] @ B[j]) * x[j]
        y[t] += 1.5 * x[t]
    y = y * silu(z)
    want = y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-6) * w["norm"]
    assert torch.allclose(pl.mamba2_mixer(h, w, "", m, 1e-6), want, atol=1e-10)


def test_plain_experts_by_token_id():
    cfg = lm.only(lm.ALPHA, 0)
    t = {k: (v.double() if v.dtype != torch.int32 else v.long()) for k, v in lm.draw(cfg, 4).items()}
    h = torch.randn(3, cfg["width"], dtype=torch.float64)
    toks = torch.tensor([7, 7, 250])
    out = pl.table_moe(h, toks, t, "l0.mlp.", cfg["layers"][0]["mlp"])
    e0, e1 = t["l0.mlp.table"][7].tolist()
    assert e0 != e1
    want = 0.5 * (pl.expert_ff(h[1:2], t, f"l0.mlp.e{e0}.") + pl.expert_ff(h[1:2], t, f"l0.mlp.e{e1}."))[0]
    assert torch.allclose(out[1], want, atol=1e-12)


def test_command_line_inspects_and_writes_a_random_folder(tmp_path, capsys):
    from gopherllm_b200.cli import main
    cfg_file = tmp_path / "c.json"
    cfg_file.write_text(json.dumps(lm.GAMMA))
    folder = str(tmp_path / "m")
    assert main([folder, "--random-config", str(cfg_file), "--seed", "3"]) == 0
    arch, typed, model = build(lm.GAMMA)
    check_folder(folder, tensor_table(model.parameters(), arch.tensor_names(typed)))
    capsys.readouterr()
    assert main([folder, "--inspect"]) == 0
    out = capsys.readouterr().out
    assert "architecture: Lilupel" in out and "supported: true" in out
    cfg, t = lm.read_folder(folder)
    table = t["l0.mlp.table"]
    assert table.min() >= 0 and table.max() < 4 and all(len(set(r.tolist())) == 3 for r in table)      # a row's experts differ
    assert torch.isfinite(pl.forward([1, 2, 3, 4, 5], t, cfg)).all()
