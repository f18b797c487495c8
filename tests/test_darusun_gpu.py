"""The Darusun design through the library's loader, cache, step function, scheduler and kernels, against
the plain implementation (tests/plain_darusun.py) on small models whose weights the tests make themselves."""
import copy
import json

import numpy as np
import pytest
import torch

import darusun_models as dm
import plain_darusun as pd

pytestmark = pytest.mark.gpu

# the largest |difference| of a position's logits is bounded by TOL * max(1, max|reference|), the mean over
# positions by MEAN_TOL
TOL = {"float32": 3e-4, "bfloat16": 1e-1}
MEAN_TOL = {"float32": 1e-4, "bfloat16": 3e-2}
_REF = {}


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _REF:
        cfg, t = dm.read_folder(folder)
        _REF[key] = pd.forward(cfg, t, list(tokens)).numpy()
    return _REF[key]


def load(folder, dtype, max_tokens=4096, **kw):
    import gopherllm_b200 as gl
    return gl.load(folder, dtype=dtype, max_tokens=max_tokens, **kw)


def feed(model, slot, tokens, cuts):
    """Feed ``tokens`` in pieces of the given sizes (the rest one by one); logits of every position."""
    out, at = [], 0
    cuts = list(cuts)
    while at < len(tokens):
        n = min(cuts.pop(0) if cuts else 1, len(tokens) - at)
        out.append(model.step([(slot, tokens[at:at + n])], [list(range(n))]).cpu().numpy())
        at += n
    return np.concatenate(out, 0)


def check(got, ref, dtype, what="", outliers=0):
    """``outliers``: so many positions are left out of the bound: positions where a sixteen-bit router logit falls on the
    other side of a close call and the token meets another expert than in the 64-bit run (with one expert a token that
    changes the whole feed-forward's output).  The 32-bit run of the same test allows none."""
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max(-1)
    bound = TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    if outliers:
        err = np.sort(err)[::-1][outliers:] if len(err) > outliers else err * 0
    worst = int(err.argmax())
    assert err.max() <= bound, f"{what} {dtype}: position {worst} differs by {err.max():.3e} (bound {bound:.3e})"
    mean_bound = MEAN_TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    assert err.mean() <= mean_bound, f"{what} {dtype}: positions differ by {err.mean():.3e} on average (bound {mean_bound:.3e})"


def loose(dtype, n):
    """Positions of n that a bfloat16 router may send to another expert than the 64-bit one."""
    return max(1, n // 40) if dtype == "bfloat16" else 0


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


FOLDERS = {}


def folder_for(name, cfg, seed, **kw):
    key = (name, seed, tuple(sorted(kw.items())))
    if key not in FOLDERS:
        FOLDERS[key] = dm.write_folder(cfg, dm.draw(cfg, seed, **kw))
    return FOLDERS[key]


def _double(tensors):
    return {k: v.double() for k, v in tensors.items()}


# layer sizes nearer a real model's: heads of 64 and 128, a latent of 256 + 64, a window of several pages, many experts
WIDE = dict(
    architecture="Darusun", vocab=500, width=256, norm={"eps": 1e-6}, residual_mult=0.8,
    layers=[
        {"type": "latent_attention",
         "mixer": {"heads": 8, "dim": 64, "rot_dim": 64, "vdim": 64, "q_rank": 192, "kv_rank": 256, "scale": 0.09,
                   "mask": {"size": 150}, "rot": {"dims": 64, "base": 10000.0}},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 32, "top": 4}, "shared": {"ff": 128}}},
        {"type": "attention",
         "mixer": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "rot": {"dims": 64, "base": 1e6}},
         "mlp": {"kind": "dense", "ff": 512}},
        {"type": "attention",
         "mixer": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "rot": {"dims": 64, "base": 1e6},
                   "kv_from": 1},
         "mlp": {"kind": "moe", "expert": {"ff": 128}, "router": {"experts": 8, "top": 2}}},
    ])

# more query heads than one block of the one-token kernel takes on a key head: sixteen (two runs of eight, value heads
# that span a run and value heads inside a run) and twelve (no whole runs: the kernel by pairs)
MANY = dict(
    architecture="Darusun", vocab=200, width=64, norm={"eps": 1e-6}, residual_mult=0.6,
    layers=[
        {"type": "latent_attention",
         "mixer": {"heads": 16, "dim": 8, "rot_dim": 8, "vdim": 8, "q_rank": 24, "kv_rank": 24, "scale": 0.3,
                   "mask": {"size": 100}, "rot": {"dims": 8, "base": 1000.0}}, "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 16, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.3, "rot": {"dims": 16, "base": 1000.0}},
         "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 16, "kv_heads": 8, "dim": 8, "vdim": 16, "scale": 0.3, "rot": {"dims": 4, "base": 1000.0}},
         "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 12, "kv_heads": 3, "dim": 8, "vdim": 8, "scale": 0.3, "rot": {"dims": 8, "base": 1000.0}},
         "mlp": None},
    ])

# sizes the tensor-core kernel of one-token steps takes (key and value sizes in sixteens, eight or more query heads on
# the key row): sixteen heads on a latent, runs of eight and of four heads that share a value head
ROWS = dict(
    architecture="Darusun", vocab=200, width=64, norm={"eps": 1e-6}, residual_mult=0.9,
    layers=[
        {"type": "latent_attention",
         "mixer": {"heads": 16, "dim": 8, "rot_dim": 16, "vdim": 8, "q_rank": 24, "kv_rank": 48, "scale": 0.3,
                   "mask": {"size": 100}, "rot": {"dims": 16, "base": 1000.0}}, "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 16, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "rot": {"dims": 16, "base": 1000.0}},
         "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 8, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.3, "rot": {"dims": 8, "base": 1000.0}},
         "mlp": None},
        {"type": "latent_attention",
         "mixer": {"heads": 32, "dim": 16, "rot_dim": 0, "vdim": 8, "q_rank": 24, "kv_rank": 32, "scale": 0.3},
         "mlp": None},
    ])

# key rows too long for a page of them in shared memory: four key heads of 160 side by side
LONG_ROWS = dict(
    architecture="Darusun", vocab=120, width=48, norm={"eps": 1e-6}, residual_mult=1.0,
    layers=[{"type": "attention",
             "mixer": {"heads": 4, "kv_heads": 4, "dim": 160, "vdim": 8, "scale": 0.1, "rot": {"dims": 6, "base": 100.0}},
             "mlp": None}])

ALONE = [("talking_heads_with_shared_expert", dm.only(dm.ALPHA, 0)), ("latent_dense", dm.only(dm.ALPHA, 1)),
         ("talking_heads_bare", dm.only(dm.ALPHA, 2, mlp=False)), ("latent_top1", dm.only(dm.ALPHA, 3)),
         ("latent_small_rotation_long_window", dm.only(dm.BETA, 0)), ("talking_full_rotation_top3", dm.only(dm.BETA, 1)),
         ("talking_six_on_one_no_rotation", dm.only(dm.BETA, 2)), ("talking_odd_all_experts", dm.only(dm.GAMMA, 0)),
         ("latent_one_head_window_three", dm.only(dm.GAMMA, 1)), ("latent_window_of_one", dm.only(dm.GAMMA, 2)),
         ("latent_sixteen_heads", dm.only(MANY, 0)), ("talking_sixteen_on_two", dm.only(MANY, 1)),
         ("talking_sixteen_on_eight", dm.only(MANY, 2)), ("talking_twelve_on_three", dm.only(MANY, 3)), ("many_heads", MANY),
         ("rows_latent_sixteen", dm.only(ROWS, 0)), ("rows_talking_runs_of_eight", dm.only(ROWS, 1)),
         ("rows_talking_runs_of_four", dm.only(ROWS, 2)), ("rows_latent_no_rotation_no_window", dm.only(ROWS, 3)), ("rows", ROWS), ("talking_long_key_rows", LONG_ROWS)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", ALONE, ids=[a[0] for a in ALONE])
def test_each_mechanism_alone(name, cfg, dtype):
    """One layer of one kind: a whole prompt across a page's edge, then single tokens."""
    folder = folder_for(name, cfg, 11)
    toks = tokens_for(cfg, 150 if name.startswith("rows") else 78, 1)
    m = load(folder, dtype)
    s = m.open_sequence()
    got = feed(m, s, toks, [70])
    m.engine.check_device()
    check(got, plain_logits(folder, toks), dtype, name, outliers=loose(dtype, 78))
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg_name", ["ALPHA", "BETA", "GAMMA"])
def test_whole_pieces_and_single_tokens(cfg_name, dtype):
    """The same tokens whole, in pieces of many sizes down to two, and mostly one by one."""
    cfg = getattr(dm, cfg_name)
    folder = folder_for(cfg_name, cfg, 5)
    toks = tokens_for(cfg, 150, 2)
    ref = plain_logits(folder, toks)
    m = load(folder, dtype)
    for cuts in ([150], [2, 2, 3, 57, 1, 64, 2, 19], [40]):
        s = m.open_sequence()
        got = feed(m, s, toks, cuts)
        m.close_sequence(s)
        check(got, ref, dtype, f"{cfg_name} cuts {cuts}", outliers=loose(dtype, 150))
    m.engine.check_device()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_nearer_a_real_layer(dtype):
    folder = folder_for("WIDE", WIDE, 21)
    toks = tokens_for(WIDE, 330, 4)
    ref = plain_logits(folder, toks)
    m = load(folder, dtype)
    for cuts in ([330], [130, 66, 100]):
        s = m.open_sequence()
        check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}", outliers=loose(dtype, 330))
        m.close_sequence(s)
    m.engine.check_device()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(dtype):
    """Sequences of one to four tokens: a window that is not full yet, a softmax over the sink and one key."""
    for cfg_name in ("ALPHA", "GAMMA"):
        cfg = getattr(dm, cfg_name)
        folder = folder_for(cfg_name, cfg, 5)
        m = load(folder, dtype)
        for n in (1, 2, 3, 4):
            toks = tokens_for(cfg, n, 20 + n)
            s = m.open_sequence()
            check(feed(m, s, toks, [n]), plain_logits(folder, toks), dtype, f"{cfg_name}: {n} tokens at once", outliers=loose(dtype, 1))
            m.close_sequence(s)
            s = m.open_sequence()
            check(feed(m, s, toks, []), plain_logits(folder, toks), dtype, f"{cfg_name}: {n} tokens one by one", outliers=loose(dtype, 1))
            m.close_sequence(s)
        m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(dtype):
    """Three prompts of different lengths as one batch, then decoded together while the shorter ones leave;
    every sequence must get what it gets alone."""
    cfg = dm.ALPHA
    folder = folder_for("ALPHA", cfg, 5)
    lens, prompt = [9, 140, 71], [5, 131, 66]
    seqs = [tokens_for(cfg, n, 30 + i) for i, n in enumerate(lens)]
    m = load(folder, dtype)
    slots = [m.open_sequence() for _ in seqs]
    got = [[] for _ in seqs]
    out = m.step([(slots[i], seqs[i][:prompt[i]]) for i in range(3)], [list(range(p)) for p in prompt]).cpu().numpy()
    at = 0
    for i, p in enumerate(prompt):
        got[i].append(out[at:at + p])
        at += p
    pos = list(prompt)
    while any(pos[i] < lens[i] for i in range(3)):
        live = [i for i in range(3) if pos[i] < lens[i]]
        out = m.step([(slots[i], [seqs[i][pos[i]]]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            pos[i] += 1
            if pos[i] == lens[i]:
                m.close_sequence(slots[i])
    m.engine.check_device()
    for i in range(3):
        check(np.concatenate(got[i], 0), plain_logits(folder, seqs[i]), dtype, f"sequence {i} in the batch",
              outliers=loose(dtype, lens[i]))
    if dtype == "float32":
        alone = load(folder, dtype)
        s = alone.open_sequence()
        one = feed(alone, s, seqs[2], [prompt[2]])
        assert np.abs(one - np.concatenate(got[2], 0)).max() <= 2e-5 * max(1.0, np.abs(one).max())
        alone.close()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype):
    """A sequence that takes the slot and the pages another one left must not see them; the window's groups give
    pages back while a sequence grows, and those are used again too."""
    cfg = dm.ALPHA
    folder = folder_for("ALPHA", cfg, 5)
    a, b, c = tokens_for(cfg, 130, 40), tokens_for(cfg, 90, 41), tokens_for(cfg, 70, 42)
    m = load(folder, dtype, max_tokens=512)
    sa = m.open_sequence()
    feed(m, sa, a, [100])
    sb = m.open_sequence()
    gb = [feed(m, sb, b[:50], [50])]
    m.close_sequence(sa)
    sc = m.open_sequence()                      # takes a's slot and pages while b is still live
    assert sc == sa
    gc = feed(m, sc, c, [33, 2])
    gb.append(feed(m, sb, b[50:], [7]))
    m.engine.check_device()
    check(gc, plain_logits(folder, c), dtype, "the sequence in the used slot", outliers=loose(dtype, 70))
    check(np.concatenate(gb, 0), plain_logits(folder, b), dtype, "the sequence that stayed", outliers=loose(dtype, 90))
    m.engine.cache.check()
    m.close()


def test_keys_at_the_windows_edges_decide():
    """Latent attention alone with a sharp softmax (scores of tens): a position's output is mostly the value of its
    best key, so a window one position too long or too short changes whole rows, and so does a missing sink or
    gate.  Prompts that end on, before and after the window's length and the pages' edges, pieces of two tokens, and
    single tokens while the window passes over decoded tokens."""
    cfg = dm.only(dm.ALPHA, 1, mlp=False)
    cfg["layers"][0]["mixer"]["scale"] = 1.0
    tensors = dm.draw(cfg, 17, sharp=3.0)
    folder = dm.write_folder(cfg, tensors)
    toks = tokens_for(cfg, 170, 3)
    ref = plain_logits(folder, toks)
    scale = max(1.0, float(np.abs(ref).max()))
    for off in (-1, 1):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["mask"]["size"] += off
        moved = np.abs(pd.forward(other, _double(tensors), toks).numpy() - ref).max(-1)
        assert (moved[25:] > 30 * TOL["float32"] * scale).sum() >= 5, "the test's model does not show its window's edge"
    no_sink = _double(tensors)
    no_sink["l0.mix.sink"] = no_sink["l0.mix.sink"] - 60.0
    assert np.abs(pd.forward(cfg, no_sink, toks).numpy() - ref).max() > 30 * TOL["float32"] * scale, "the sink does not show"
    no_gate = _double(tensors)
    no_gate["l0.mix.g"] = no_gate["l0.mix.g"] * 0.0
    assert np.abs(pd.forward(cfg, no_gate, toks).numpy() - ref).max() > 30 * TOL["float32"] * scale, "the gate does not show"
    for dtype in ("float32", "bfloat16"):
        m = load(folder, dtype)
        for cuts in ([170], [19], [20, 2, 2], [21], [63, 1, 1, 20, 2], [64, 19, 21, 20], [5]):
            s = m.open_sequence()
            check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}")
            m.close_sequence(s)
        m.engine.check_device()
        m.close()


def test_far_keys_and_page_edges():
    """Attention over all earlier positions with a sharp softmax and a table that mixes the heads strongly: the
    logits late in a sequence hang on single keys hundreds of positions back (the test changes early tokens and
    sees late logits move) and on every entry of the table; pieces end on, before and after the pages' edges."""
    cfg = dm.only(dm.ALPHA, 0, mlp=False)
    cfg["layers"][0]["mixer"]["scale"] = 2.5
    tensors = dm.draw(cfg, 23)
    folder = dm.write_folder(cfg, tensors)
    toks = tokens_for(cfg, 330, 50)
    ref = plain_logits(folder, toks)
    scale = max(1.0, float(np.abs(ref).max()))
    other = list(toks)
    for j in range(8):
        other[j] = (other[j] + 1 + j) % cfg["vocab"]
    moved = np.abs(plain_logits(folder, other)[300:] - ref[300:]).max(-1)
    assert (moved > 30 * TOL["float32"] * scale).sum() >= 3, "the test's model does not look far back"
    plain_table = _double(tensors)
    plain_table["l0.mix.talk"] = torch.eye(4, dtype=torch.float64)
    assert np.abs(pd.forward(cfg, plain_table, toks).numpy() - ref).max() > 100 * TOL["float32"] * scale, "the table does not show"
    for dtype in ("float32", "bfloat16"):
        m = load(folder, dtype)
        for cuts in ([330], [63, 1, 1, 63, 2], [129], [64, 64, 64], [65, 63], [320]):
            s = m.open_sequence()
            check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}")
            m.close_sequence(s)
        m.engine.check_device()
        m.close()


def test_router_and_shared_expert_by_hand():
    """A mixture alone behind a window of one: the router's bias decides between two experts whose logits are equal
    by construction, and the shared expert's share is the sigmoid of its own product."""
    cfg = dm.only(dm.GAMMA, 2)
    cfg["layers"][0]["mlp"] = {"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 6}}
    tensors = dm.draw(cfg, 29)
    tensors["l0.mlp.router"][1] = tensors["l0.mlp.router"][0]              # experts 0 and 1: the same logit but for the bias
    tensors["l0.mlp.router.b"] = torch.tensor([0.0, 0.5, -0.25, 0.25]).to(torch.bfloat16)
    folder = dm.write_folder(cfg, tensors)
    toks = tokens_for(cfg, 40, 6)
    ref = plain_logits(folder, toks)
    scale = max(1.0, float(np.abs(ref).max()))
    no_bias = _double(tensors)
    no_bias["l0.mlp.router.b"] = no_bias["l0.mlp.router.b"] * 0.0
    assert np.abs(pd.forward(cfg, no_bias, toks).numpy() - ref).max() > 30 * TOL["float32"] * scale, "the bias does not show"
    half = _double(tensors)
    half["l0.mlp.shared.sg"] = half["l0.mlp.shared.sg"] * 0.0
    assert np.abs(pd.forward(cfg, half, toks).numpy() - ref).max() > 30 * TOL["float32"] * scale, "the share does not show"
    m = load(folder, "float32")
    s = m.open_sequence()
    check(feed(m, s, toks, [33]), ref, "float32", "router with a bias")
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """A few tokens of prompt, then single tokens across two pages' edges and past the longer window (captured
    steps in bfloat16)."""
    cfg = dm.BETA
    folder = folder_for("BETA", cfg, 9)
    toks = tokens_for(cfg, 160, 60)
    m = load(folder, dtype)
    s = m.open_sequence()
    got = feed(m, s, toks, [3])
    m.engine.check_device()
    check(got, plain_logits(folder, toks), dtype, "long decoding", outliers=loose(dtype, 160))
    m.close()


def _greedy(folder, prompt, n):
    pcfg, t = dm.read_folder(folder)
    seq = list(prompt)
    for _ in range(n):
        logits = pd.forward(pcfg, t, seq)[-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) < 1e-3:        # a tie within rounding proves nothing either way
            break
        seq.append(int(logits.argmax()))
    return seq[len(prompt):]


def test_greedy_generation_through_the_scheduler():
    """Model.generate, greedy, for prompts of different lengths in one call: the tokens the plain
    implementation chooses; and the on-device loop chooses what Model.generate chooses."""
    from gopherllm_b200.sampling.sampler import DeviceSampler, SamplerConfig
    cfg = dm.GAMMA
    folder = folder_for("GAMMA", cfg, 3)
    prompts = [tokens_for(cfg, n, 70 + n) for n in (4, 37, 66)]
    m = load(folder, "float32")
    outs = m.generate(prompts, max_tokens=8, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())
    for p, o in zip(prompts, outs):
        want = _greedy(folder, p, 8)
        assert o.tokens[:len(want)] == want, (o.tokens, want)
    m.close()
    mb = load(folder_for("ALPHA", dm.ALPHA, 5), "bfloat16")
    prompt = tokens_for(dm.ALPHA, 21, 90)
    want = mb.generate([prompt], max_tokens=12, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())[0].tokens
    assert len(want) == 12
    s = mb.open_sequence()
    first = int(mb.step([(s, prompt)])[0].argmax())
    assert first == want[0]
    sampler = DeviceSampler(SamplerConfig.greedy(), [1], [prompt], dm.ALPHA["vocab"], mb.engine.device)
    chosen = mb.engine.decode_loop([s], [first], 11, sampler).cpu().numpy()[:, 0].tolist()
    assert [first] + chosen == want
    mb.engine.check_device()
    mb.close()


def test_command_line_generates():
    """python -m gopherllm_b200 on a Darusun folder: greedy tokens equal the plain implementation's, and the
    isolated kernel bench knows the parts' products."""
    import os
    import subprocess
    import sys
    cfg = dm.GAMMA
    folder = folder_for("GAMMA", cfg, 3)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = lambda *a: subprocess.run([sys.executable, "-m", "gopherllm_b200", folder, *a], cwd=root,
                                    capture_output=True, text=True, timeout=600)
    prompt = tokens_for(cfg, 9, 77)
    want = _greedy(folder, prompt, 5)
    p = run("--prompt", " ".join(map(str, prompt)), "--max-tokens", "5", "--temp", "0", "--repeat-penalty", "1",
            "--dtype", "float32", "--stop", "100000")
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()][:len(want)] == want
    p = run("--kernel-bench-json", "--kernel-bench-runs", "2")
    assert p.returncode == 0, p.stderr[-2000:]
    assert json.loads(p.stdout)["kernels"]


def test_replay_of_a_trace(tmp_path):
    """The trace runner's loop on a Darusun model: a batch of two requests, one ends, the other goes on."""
    from gopherllm_b200.engine.replay import run
    cfg = dm.ALPHA
    folder = folder_for("ALPHA", cfg, 5)
    a, b = tokens_for(cfg, 70, 80), tokens_for(cfg, 12, 81)
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 63, 65]},
                                                 {"id": "b", "tokens": b[:11], "want": []}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": a[66:67], "want": [0]},
                                                 {"id": "b", "tokens": b[11:], "want": [0]}], "end": ["b"]})]
    lines += [json.dumps({"step": 2 + i, "entries": [{"id": "a", "tokens": [a[67 + i]], "want": [0]}],
                          "end": ["a"] if i == 2 else []}) for i in range(3)]
    m = load(folder, "float32")
    said = []
    run(m, lines, str(tmp_path), said.append)
    assert said == [f"done {i}" for i in range(5)]
    ra, rb = plain_logits(folder, a), plain_logits(folder, b)
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(3, -1)
    check(got0, ra[[0, 63, 65]], "float32", "step 0")
    got1 = np.fromfile(tmp_path / "1.f32", dtype="<f4").reshape(2, -1)
    check(got1, np.stack([ra[66], rb[11]]), "float32", "step 1")
    got4 = np.fromfile(tmp_path / "4.f32", dtype="<f4").reshape(1, -1)
    check(got4, ra[69:70], "float32", "step 4")
    assert not m.engine.cache.live_slots()
    m.close()


def test_kernels_of_the_design_alone():
    """The per-head product with its rotated tail and its gate, the cache write with a table on the queries, and
    the router's softmax over the chosen logits, each against torch at sizes of their own."""
    from gopherllm_b200 import ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    # (sizes the tensor-core form of the product does not take, then sizes it does: two tiles of tokens, two of outputs)
    for T, H, N, K, tail in ((70, 3, 20, 12, 6), (70, 3, 72, 32, 8), (5, 2, 16, 80, 0)):
        x = torch.randn(T, H * (K + tail), generator=g)
        w = torch.randn(H, N, K, generator=g)
        ang = torch.randn(T, tail // 2, generator=g)
        gate = torch.randn(T, 5 + H, generator=g)
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
            xd, wd, gd = x.to(dev, dtype), w.to(dev, dtype), gate.to(dev, dtype)
            kw = dict(cos=torch.cos(ang).to(dev), sin=torch.sin(ang).to(dev)) if tail else {}
            got = ops.head_linear(xd, wd, K + tail, tail=tail, interleaved=True, gate=gd, gate_off=5, **kw).float().cpu().view(T, H, N + tail)
            xr, wr, gr = xd.float().cpu().view(T, H, K + tail), wd.float().cpu(), gd.float().cpu()
            want = torch.einsum("thk,hnk->thn", xr[..., :K], wr) * torch.sigmoid(gr[:, 5:5 + H])[..., None]
            assert (got[..., :N] - want).abs().max() <= tol * max(1.0, want.abs().max()), (T, H, N, K, dtype)
            if tail:
                a, b = xr[..., K::2], xr[..., K + 1::2]
                c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
                turned = torch.stack([a * c - b * s, b * c + a * s], -1).reshape(T, H, tail)        # (the copied columns are not gated)
                assert (got[..., N:] - turned).abs().max() <= tol * max(1.0, turned.abs().max())
    # the activation with two numbers: in the epilogue of every product kernel (few rows, many rows, 32-bit) and alone
    def xielu(z, up, down):
        return torch.where(z > 0, up * z * z + 0.5 * z, down * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)
    for rows in (5, 200):
        a, w = torch.randn(rows, 64, generator=g), torch.randn(48, 64, generator=g) * 0.2
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
            ad, wd = a.to(dev, dtype), w.to(dev, dtype)
            want = xielu(ad.float().cpu() @ wd.float().cpu().T, 0.7, 1.3)
            got = ops.linear(ad, wd, None, act=("xielu", 0.7, 1.3), out_dtype=torch.float32).cpu()
            assert (got - want).abs().max() <= tol * max(1.0, want.abs().max()), (rows, dtype)
            alone = ops.xielu((ad.float() @ wd.float().T).to(dtype), 0.7, 1.3).float().cpu()
            assert (alone - want).abs().max() <= tol * max(1.0, want.abs().max())
    logits = torch.randn(50, 7, generator=g)
    bias = torch.randn(7, generator=g)
    ids, weights = ops.moe_route(logits.to(dev), 3, bias=bias.to(dev), softmax_chosen=True)
    best = torch.topk(logits + bias, 3, dim=-1)
    assert (ids.cpu().long() == best.indices).all()
    assert (weights.cpu() - torch.softmax(best.values, -1)).abs().max() <= 1e-6
