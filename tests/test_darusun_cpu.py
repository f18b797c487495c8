"""The Darusun design on the CPU: its configuration, tensor names, schedule and cache needs in the library,
and the plain implementation's own sanity."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import darusun_models as dm
import plain_darusun as pd
from gopherllm_b200.api import build_model
from gopherllm_b200.cache.sequence_cache import KVView, SequenceCache
from gopherllm_b200.config.registry import architecture_from_config
from gopherllm_b200.parts.base import KVRequest
from gopherllm_b200.weights.loader import tensor_table


def build(cfg):
    arch = architecture_from_config(cfg)
    typed = arch.config_class.from_dict(cfg)
    return arch, typed, build_model(arch, typed)


@pytest.mark.parametrize("cfg", [dm.ALPHA, dm.BETA, dm.GAMMA], ids=["ALPHA", "BETA", "GAMMA"])
def test_declared_tensors_are_the_files_tensors(cfg):
    arch, typed, model = build(cfg)
    assert arch.name == "darusun"
    table = tensor_table(model.parameters(), arch.tensor_names(typed))
    want = dm.tensor_shapes(cfg)
    assert set(table) == set(want)
    for name, (shape, _) in want.items():
        assert tuple(table[name][1].shape) == tuple(shape), name
    assert table["final.norm"][1].shape == () and table["l0.norm1"][1].kind == "vector"


def test_every_constant_of_the_file_reaches_the_spec():
    _, typed, model = build(dm.ALPHA)
    spec = model.spec
    assert not spec.tie_embeddings and not spec.head_bias and spec.final_norm.eps == 1e-6 and spec.final_norm.single_weight
    assert len(spec.layers) == 4 and all(b.arrangement == "post_norm" and b.option("branch_scale") == 0.5 for b in spec.layers)
    talk, latent, shared, second = (b.mixer for b in spec.layers)
    assert (talk.kind, talk.num_heads, talk.num_kv_heads, talk.head_dim, talk.value_dim, talk.window) == ("attention_mixed", 4, 2, 16, 32, 0)
    assert talk.option("score_scale") == 0.3 and talk.option("qk_norm") == "head_unit" and talk.option("talk_scores") and not talk.bias
    assert (talk.position.kind, talk.position.rotary_dim, talk.position.theta, talk.position.interleaved) == ("rope", 8, 10000.0, False)
    assert shared.option("shared_kv") and not talk.option("shared_kv", False)
    assert (latent.kind, latent.num_heads, latent.head_dim, latent.value_dim, latent.window) == ("latent_attention", 4, 16, 24, 20)
    assert [latent.option(k) for k in ("q_rank", "kv_rank", "rot", "score_scale", "norm_eps", "sink", "gate")] == [32, 40, 8, 0.2, 1e-6, True, True]
    assert (latent.position.rotary_dim, latent.position.theta, latent.position.interleaved) == (8, 500.0, True)
    assert second.window == 70 and second.option("kv_rank") == 32
    moe, dense, none, top1 = (b.ffn for b in spec.layers)
    assert moe.kind == "moe" and moe.intermediate == 24
    assert [moe.option(k) for k in ("experts", "top", "weights", "router_bias", "shared", "shared_gate")] == [5, 2, "softmax_chosen", True, 16, True]
    assert (dense.kind, dense.intermediate, dense.activation, dense.bias) == ("dense", 48, "xielu", False)
    assert none is None and spec.layers[2].norm2 is None
    assert top1.option("shared", 0) == 0 and not top1.option("shared_gate", False)
    assert typed.to_dict()["layers"] == dm.ALPHA["layers"] and typed.to_dict()["residual_mult"] == 0.5


def test_layers_that_read_another_layers_keys():
    arch, typed, model = build(dm.BETA)
    assert [(e.layer, e.cache, e.writes) for e in model.spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (1 + 2, 1, False), (4, 1, False)]
    names = arch.tensor_names(typed)
    assert names.layer(1, "ffn", "router.bias") == "l1.mlp.router.b" and names.layer(0, "mixer", "dq.norm.weight") == "l0.mix.dq.norm"
    assert names.layer(3, "norm2", "weight") == "l3.norm2" and names.layer(1, "ffn", "shared.sg.weight") == "l1.mlp.shared.sg"
    reqs = model.cache_requests()
    # the latent: one row of kv_rank + rot_dim numbers, values of kv_rank, a window; three key heads side by side with
    # three rows of values; six heads on one key head
    assert reqs[0] == KVRequest(1, 68, 130, value_dim=64, values_in_keys=True)
    assert reqs[1] == KVRequest(1, 96, 0, value_dim=16, value_heads=3)
    assert reqs[2] == KVRequest(1, 16, 0)
    assert len(reqs) == 3          # the layers that read layer 1's keys keep nothing of their own
    cache = SequenceCache(reqs, max_tokens=256, max_positions=256, dtype=torch.float32, device="cpu", max_slots=2)
    kv = cache.view(1, writes=False)
    assert isinstance(kv, KVView) and tuple(kv.k.shape[1:]) == (1, 64, 96) and tuple(kv.v.shape[1:]) == (3, 64, 16)
    assert cache.bytes_per_position() == 4 * (68 + (96 + 48) + (16 + 16))
    latent = cache.view(0)
    assert latent.v.data_ptr() == latent.k.data_ptr() and tuple(latent.k.shape[1:]) == (1, 64, 68)


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
    (("layers", 2, "mixer", "kv_from"), 2), (("layers", 2, "mixer", "kv_from"), 1), (("layers", 2, "mixer", "kv_from"), 3),
    (("layers", 2, "mixer", "dim"), 32), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 7),
    (("layers", 0, "mixer", "rot", "dims"), 18), (("layers", 1, "mixer", "rot", "dims"), 6), (("layers", 1, "mixer", "rot_dim"), 7),
    (("layers", 1, "mixer", "mask", "size"), 0), (("layers", 1, "mixer", "kv_rank"), KeyError), (("layers", 0, "mixer", "scale"), -1.0),
    (("layers", 0, "mlp", "router", "top"), 6), (("layers", 1, "mlp", "kind"), "gated"), (("layers", 0, "type"), "mamba"),
    (("residual_mult",), KeyError), (("norm",), 1e-5), (("layers",), []), (("width",), 0),
])
def test_refused_configurations(path, value):
    with pytest.raises(ValueError):
        build(_with(dm.ALPHA, path, value))


def test_a_layer_cannot_read_the_keys_of_a_layer_that_reads_anothers():
    cfg = copy.deepcopy(dm.BETA)
    cfg["layers"][4]["mixer"]["kv_from"] = 3
    with pytest.raises(ValueError):
        build(cfg)


def test_command_line_inspects_and_writes_a_random_folder(tmp_path, capsys):
    from gopherllm_b200 import cli
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(dm.GAMMA))
    folder = tmp_path / "model"
    assert cli.main([str(folder), "--random-config", str(cfg_path), "--seed", "3"]) == 0
    cfg, tensors = dm.read_folder(str(folder))
    assert set(tensors) == set(dm.tensor_shapes(dm.GAMMA)) and tensors["l0.norm1"].shape == ()
    logits = pd.forward(cfg, tensors, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 91) and torch.isfinite(logits).all()
    assert cli.main([str(folder), "--inspect"]) == 0
    assert "darusun" in capsys.readouterr().out.lower()


# -- the plain implementation by hand ------------------------------------------------------------------------------
def test_plain_model_is_causal_and_its_windows_end():
    cfg = dm.ALPHA
    t = {k: v.double() for k, v in dm.draw(cfg, 3).items()}
    toks = [int(x) for x in np.random.default_rng(0).integers(0, cfg["vocab"], size=40)]
    a = pd.forward(cfg, t, toks)
    other = list(toks)
    other[30] = (other[30] + 1) % cfg["vocab"]
    b = pd.forward(cfg, t, other)
    assert float((a[:30] - b[:30]).abs().max()) == 0.0 and float((a[30:] - b[30:]).abs().max()) > 1e-6
    # a latent layer alone with a window of 3 forgets a token three positions on
    one = dm.only(dm.GAMMA, 1)
    t1 = {k: v.double() for k, v in dm.draw(one, 4).items()}
    toks = [int(x) for x in np.random.default_rng(1).integers(0, one["vocab"], size=12)]
    a = pd.forward(one, t1, toks)
    other = list(toks)
    other[4] = (other[4] + 1) % one["vocab"]
    b = pd.forward(one, t1, other)
    moved = (a - b).abs().max(-1).values
    assert (moved[4:7] > 1e-9).all() and float(moved[7:].max()) == 0.0 and float(moved[:4].max()) == 0.0


def test_plain_activation_router_and_rotations_by_hand():
    z = torch.tensor([-2.0, 0.0, 0.5, 3.0], dtype=torch.float64)
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-1.0, dtype=torch.float64)
    sp = lambda x: math.log1p(math.exp(x))
    want = [(0.5 + sp(-1.0)) * (math.exp(-2.0) - 1 + 2.0) - 1.0, 0.0, sp(0.3) * 0.25 + 0.25, sp(0.3) * 9 + 1.5]
    assert torch.allclose(pd.xielu(z, p, q), torch.tensor(want, dtype=torch.float64), atol=1e-12)
    # the router: bias added, the two largest chosen, a softmax over those two alone
    w = {"r.router": torch.eye(4, dtype=torch.float64), "r.router.b": torch.tensor([0.0, 0.0, 0.0, 2.5], dtype=torch.float64)}
    ids, weights = pd.route(torch.tensor([[1.0, 3.0, 2.0, 0.0]], dtype=torch.float64), w, "r.", 2)
    assert ids.tolist() == [[1, 3]]
    assert torch.allclose(weights, torch.tensor([[1 / (1 + math.exp(-0.5)), 1 / (1 + math.exp(0.5))]], dtype=torch.float64))
    # rotations: halves pair dim i with i + dims/2, neighbours dim 2i with 2i + 1; position 0 turns nothing
    x = torch.arange(12, dtype=torch.float64).view(2, 1, 6) + 1.0
    rot = {"dims": 4, "base": 100.0}
    h, n = pd.rotate_halves(x, rot), pd.rotate_neighbours(x, rot)
    assert torch.equal(h[0], x[0]) and torch.equal(n[0], x[0]) and torch.equal(h[..., 4:], x[..., 4:])
    a0, a1 = 1.0, 100.0 ** -0.5
    u = x[1, 0]
    assert torch.allclose(h[1, 0, :4], torch.tensor([u[0] * math.cos(a0) - u[2] * math.sin(a0), u[1] * math.cos(a1) - u[3] * math.sin(a1),
                                                    u[2] * math.cos(a0) + u[0] * math.sin(a0), u[3] * math.cos(a1) + u[1] * math.sin(a1)], dtype=torch.float64))
    assert torch.allclose(n[1, 0, :4], torch.tensor([u[0] * math.cos(a0) - u[1] * math.sin(a0), u[1] * math.cos(a0) + u[0] * math.sin(a0),
                                                    u[2] * math.cos(a1) - u[3] * math.sin(a1), u[3] * math.cos(a1) + u[2] * math.sin(a1)], dtype=torch.float64))


def test_plain_score_mixing_equals_wide_queries():
    """What the library relies on: mixing the heads' scores is a product of mixed queries with the key heads side by
    side."""
    g = torch.Generator().manual_seed(1)
    H, G, D, T = 6, 3, 5, 7
    q, k = torch.randn(T, H, D, generator=g, dtype=torch.float64), torch.randn(T, G, D, generator=g, dtype=torch.float64)
    table = torch.randn(H, H, generator=g, dtype=torch.float64)
    raw = torch.stack([q[:, h] @ k[:, h // (H // G)].T for h in range(H)])
    mixed = torch.einsum("hg,gij->hij", table, raw)
    wide = torch.zeros(T, H, G * D, dtype=torch.float64)
    for h in range(H):
        for c in range(G):
            for gq in range(c * (H // G), (c + 1) * (H // G)):
                wide[:, h, c * D:(c + 1) * D] += table[h, gq] * q[:, gq]
    again = torch.stack([wide[:, h] @ k.reshape(T, G * D).T for h in range(H)])
    assert torch.allclose(mixed, again, atol=1e-12)
