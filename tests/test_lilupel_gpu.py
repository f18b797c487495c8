"""The Lilupel design through the library's loader, cache, step function, scheduler and kernels, against
the plain implementation (tests/plain_lilupel.py) on small models whose weights the tests make themselves."""
import copy
import json
import math

import numpy as np
import pytest
import torch

import lilupel_models as lm
import plain_lilupel as pl

pytestmark = pytest.mark.gpu

# the largest |difference| of a position's logits is bounded by TOL * max(1, max|reference|), the mean over
# positions by MEAN_TOL
TOL = {"float32": 3e-4, "bfloat16": 1e-1}
MEAN_TOL = {"float32": 1e-4, "bfloat16": 3e-2}
_REF = {}


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _REF:
        cfg, t = lm.read_folder(folder)
        _REF[key] = pl.forward(list(tokens), t, cfg).numpy()
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
    """``outliers``: so many positions may differ by up to twice the bound (a position where sixteen-bit
    rounding is amplified, which the 32-bit run of the same test shows to be rounding and nothing else)."""
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max(-1)
    bound = TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    if outliers:
        over = np.sort(err)[::-1][:outliers]
        assert (over <= 2 * bound).all(), f"{what} {dtype}: a position differs by {over[0]:.3e} (twice the bound: {2 * bound:.3e})"
        err = np.sort(err)[::-1][outliers:] if len(err) > outliers else err * 0
    worst = int(err.argmax())
    assert err.max() <= bound, f"{what} {dtype}: position {worst} differs by {err.max():.3e} (bound {bound:.3e})"
    mean_bound = MEAN_TOL[dtype] * max(1.0, float(np.abs(ref).max()))
    assert err.mean() <= mean_bound, f"{what} {dtype}: positions differ by {err.mean():.3e} on average (bound {mean_bound:.3e})"


def tokens_for(cfg, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], size=n)]


FOLDERS = {}


def folder_for(name, cfg, seed, **kw):
    key = (name, seed, tuple(sorted(kw.items())))
    if key not in FOLDERS:
        FOLDERS[key] = lm.write_folder(cfg, lm.draw(cfg, seed, **kw))
    return FOLDERS[key]


def one_side(cfg, index, left):
    """The pair of ``cfg``'s layer with one side's factor zero: the other mechanism alone behind the norm."""
    out = lm.only(cfg, index, mlp=False)
    out["layers"][0]["mixer"]["left_scale" if not left else "right_scale"] = 0.0
    return out


# layer sizes nearer a real model's: heads of 64 and 128, a state of 128, a window of several pages, many experts
WIDE = dict(
    architecture="Lilupel", vocab=500, width=256, norm={"eps": 1e-6},
    layers=[
        {"type": "mamba2", "mixer": {"heads": 8, "vdim": 64, "state": 128, "groups": 2, "conv": 4, "norm_groups": 4},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 32, "top": 4}}},
        {"type": "parallel",
         "mixer": {"left": {"heads": 8, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "mask": {"size": 150},
                            "rot": {"dims": 64, "base": 10000.0}},
                   "right": {"heads": 2, "dim": 128, "vdim": 128, "decay": [0.97, 0.999], "rot": {"dims": 128, "base": 1e6}},
                   "left_scale": 1.1, "right_scale": 0.8},
         "mlp": {"kind": "moe", "expert": {"ff": 128}, "router": {"experts": 8, "top": 2}}},
        {"type": "mamba2", "mixer": {"heads": 8, "vdim": 64, "state": 128, "groups": 2, "conv": 4, "norm_groups": 4},
         "mlp": {"kind": "moe", "expert": {"ff": 64}, "router": {"experts": 32, "top": 4}}, "weights_of": 0},
    ])

ALONE = [("state_space", lm.only(lm.ALPHA, 0)), ("pair", lm.only(lm.ALPHA, 1)),
         ("state_space_bare_one_group_two_taps", lm.only(lm.ALPHA, 2, mlp=False)),
         ("pair_bare_plain_retention", lm.only(lm.BETA, 0, mlp=False)), ("state_space_four_taps_top3", lm.only(lm.BETA, 1)),
         ("state_space_odd_one_tap", lm.only(lm.GAMMA, 0)), ("pair_six_on_one_window_three", lm.only(lm.GAMMA, 1)),
         ("pair_window_of_one", lm.only(lm.GAMMA, 2, mlp=False)),
         ("window_attention_alone", one_side(lm.ALPHA, 1, left=True)), ("retention_alone", one_side(lm.ALPHA, 1, left=False)),
         ("retention_alone_no_decay", one_side(lm.GAMMA, 1, left=False))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg", ALONE, ids=[a[0] for a in ALONE])
def test_each_mechanism_alone(name, cfg, dtype):
    """One layer of one kind: a whole prompt across a page's edge, then single tokens."""
    folder = folder_for(name, cfg, 11)
    toks = tokens_for(cfg, 78, 1)
    m = load(folder, dtype)
    s = m.open_sequence()
    got = feed(m, s, toks, [70])
    m.engine.check_device()
    check(got, plain_logits(folder, toks), dtype, name)
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cfg_name", ["ALPHA", "BETA", "GAMMA"])
def test_whole_pieces_and_single_tokens(cfg_name, dtype):
    """The same tokens whole, in pieces of many sizes down to two, and mostly one by one."""
    cfg = getattr(lm, cfg_name)
    folder = folder_for(cfg_name, cfg, 5)
    toks = tokens_for(cfg, 150, 2)
    ref = plain_logits(folder, toks)
    m = load(folder, dtype)
    for cuts in ([150], [2, 2, 3, 57, 1, 64, 2, 19], [40]):
        s = m.open_sequence()
        got = feed(m, s, toks, cuts)
        m.close_sequence(s)
        check(got, ref, dtype, f"{cfg_name} cuts {cuts}")
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
        check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}")
        m.close_sequence(s)
    m.engine.check_device()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(dtype):
    """Sequences of one to four tokens: the filter's zeros before the start, a window that is not full yet, a
    memory that starts empty, a softmax over the sink and one key."""
    for cfg_name in ("ALPHA", "GAMMA"):
        cfg = getattr(lm, cfg_name)
        folder = folder_for(cfg_name, cfg, 5)
        m = load(folder, dtype)
        for n in (1, 2, 3, 4):
            toks = tokens_for(cfg, n, 20 + n)
            s = m.open_sequence()
            check(feed(m, s, toks, [n]), plain_logits(folder, toks), dtype, f"{cfg_name}: {n} tokens at once")
            m.close_sequence(s)
            s = m.open_sequence()
            check(feed(m, s, toks, []), plain_logits(folder, toks), dtype, f"{cfg_name}: {n} tokens one by one")
            m.close_sequence(s)
        m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(dtype):
    """Three prompts of different lengths as one batch, then decoded together while the shorter ones leave;
    every sequence must get what it gets alone."""
    cfg = lm.ALPHA
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
              outliers=1 if dtype == "bfloat16" else 0)
    if dtype == "float32":
        alone = load(folder, dtype)
        s = alone.open_sequence()
        one = feed(alone, s, seqs[2], [prompt[2]])
        assert np.abs(one - np.concatenate(got[2], 0)).max() <= 2e-5 * max(1.0, np.abs(one).max())
        alone.close()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slots_and_pages_used_again(dtype):
    """A sequence that takes the slot, the state rows (both memories, the filter's inputs) and the pages another
    one left must not see them."""
    cfg = lm.ALPHA
    folder = folder_for("ALPHA", cfg, 5, long_memory=True)
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
    check(gc, plain_logits(folder, c), dtype, "the sequence in the used slot")
    check(np.concatenate(gb, 0), plain_logits(folder, b), dtype, "the sequence that stayed")
    m.engine.cache.check()
    m.close()


def _double(tensors):
    return {k: (v.double() if v.dtype != torch.int32 else v.long()) for k, v in tensors.items()}


def test_keys_at_the_windows_edges_decide():
    """Window attention alone with a sharp softmax (scores of tens): a position's output is mostly the value of
    its best key, so a window one position too long or too short changes whole rows.  Prompts that end on,
    before and after the window's length and the pages' edges, pieces of two tokens, and single tokens while the
    window passes over decoded tokens."""
    cfg = one_side(lm.ALPHA, 1, left=True)
    cfg["layers"][0]["mixer"]["left"]["scale"] = 1.5
    tensors = lm.draw(cfg, 17, sharp=6.0)
    folder = lm.write_folder(cfg, tensors)
    toks = tokens_for(cfg, 170, 3)
    ref = plain_logits(folder, toks)
    scale = max(1.0, float(np.abs(ref).max()))
    for off in (-1, 1):
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] += off
        moved = np.abs(pl.forward(toks, _double(tensors), other).numpy() - ref).max(-1)
        assert (moved[25:] > 30 * TOL["float32"] * scale).sum() >= 5, "the test's model does not show its window's edge"
    no_sink = _double(tensors)
    no_sink["l0.mix.left.sink"] = no_sink["l0.mix.left.sink"] - 60.0
    assert np.abs(pl.forward(toks, no_sink, cfg).numpy() - ref).max() > 30 * TOL["float32"] * scale, "the sink does not show"
    for dtype in ("float32", "bfloat16"):
        m = load(folder, dtype)
        for cuts in ([170], [19], [20, 2, 2], [21], [63, 1, 1, 20, 2], [64, 19, 21, 20], [5]):
            s = m.open_sequence()
            check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}")
            m.close_sequence(s)
        m.engine.check_device()
        m.close()


def test_far_tokens_and_page_edges():
    """Memories that decay slowly: the logits late in a sequence hang on single tokens hundreds of positions back,
    through the state-space layers' and the retention's states; pieces end on, before and after the pages' edges."""
    cfg = copy.deepcopy(lm.ALPHA)
    for i in (1, 3):
        cfg["layers"][i]["mixer"]["right"]["decay"] = [0.998, 1.0]
    folder = folder_for("ALPHA_far", cfg, 7, long_memory=True)
    toks = tokens_for(cfg, 260, 50)
    ref = plain_logits(folder, toks)
    other = list(toks)
    other[3] = (other[3] + 1) % cfg["vocab"]
    moved = np.abs(plain_logits(folder, other)[250:] - ref[250:]).max()
    assert moved > 20 * TOL["float32"] * max(1.0, np.abs(ref).max()), "the test's model forgets its early tokens"
    m = load(folder, "float32")
    for cuts in ([260], [63, 1, 1, 63, 2], [129], [64, 64, 64], [65, 63], [200]):
        s = m.open_sequence()
        check(feed(m, s, toks, cuts), ref, "float32", f"cuts {cuts}")
        m.close_sequence(s)
    m.close()
    m = load(folder, "bfloat16")
    s = m.open_sequence()
    got = feed(m, s, toks, [127])
    m.engine.check_device()
    check(got, ref, "bfloat16", "far tokens")
    m.close()


def test_one_far_token_in_a_retention():
    """A retention alone whose only head never forgets (decay 1): one early token's key is made, by hand, many
    times longer than the others', so every later read-out hangs on it, across hundreds of positions."""
    cfg = dict(architecture="Lilupel", vocab=120, width=48, norm={"eps": 1e-6}, layers=[
        {"type": "parallel", "mlp": None,
         "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.3, "mask": {"size": 4},
                            "rot": {"dims": 4, "base": 100.0}},
                   "right": {"heads": 1, "dim": 24, "vdim": 40, "decay": [1.0], "rot": {"dims": 24, "base": 10000.0}},
                   "left_scale": 0.0, "right_scale": 1.0}}])
    t = lm.draw(cfg, 19)
    toks = tokens_for(cfg, 400, 9)
    special = 119
    toks = [x if x != special else 0 for x in toks]
    toks[5] = special
    emb = t["embed"].float()
    emb[special] *= 12.0
    t["embed"] = emb.to(torch.bfloat16)
    folder = lm.write_folder(cfg, t)
    ref = plain_logits(folder, toks)
    other = list(toks)
    other[5] = 1
    assert np.abs(plain_logits(folder, other)[390:] - ref[390:]).max() > 0.05 * np.abs(ref).max()
    for dtype in ("float32", "bfloat16"):
        m = load(folder, dtype)
        for cuts in ([400], [300], [6, 2, 2, 190]):
            s = m.open_sequence()
            check(feed(m, s, toks, cuts), ref, dtype, f"cuts {cuts}")
            m.close_sequence(s)
        m.engine.check_device()
        m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """A few tokens of prompt, then single tokens across two pages' edges and twice the longer window (captured
    steps in bfloat16)."""
    cfg = lm.BETA
    folder = folder_for("BETA", cfg, 9, long_memory=True)
    toks = tokens_for(cfg, 160, 60)
    m = load(folder, dtype)
    s = m.open_sequence()
    got = feed(m, s, toks, [3])
    m.engine.check_device()
    check(got, plain_logits(folder, toks), dtype, "long decoding")
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_runs_walked_as_chunks(dtype, monkeypatch):
    """Long runs of both memories are cut into chunks that are walked side by side, with a carry between two
    walks.  With chunks of 16 tokens from 32 tokens on: a whole prompt (a ragged last chunk), pieces above and
    below the threshold that go on from a state, and a batch whose shorter sequence has fewer chunks."""
    from gopherllm_b200 import ops
    monkeypatch.setattr(ops, "DECAY_CHUNK_TOKENS", 16)
    monkeypatch.setattr(ops, "DECAY_CHUNK_TOKENS_SHORT", 16)
    monkeypatch.setattr(ops, "DECAY_CHUNKED_FROM", 32)
    for cfg_name, cfg in (("ALPHA", lm.ALPHA), ("BETA", lm.BETA), ("GAMMA", lm.GAMMA), ("WIDE", WIDE)):
        folder = folder_for(cfg_name, cfg, 5, long_memory=True)
        toks = tokens_for(cfg, 150, 2)
        ref = plain_logits(folder, toks)
        m = load(folder, dtype)
        for cuts in ([150], [33, 31, 64, 17]):
            s = m.open_sequence()
            check(feed(m, s, toks, cuts), ref, dtype, f"{cfg_name} cuts {cuts}")
            m.close_sequence(s)
        short = tokens_for(cfg, 37, 3)
        sa, sb = m.open_sequence(), m.open_sequence()
        out = m.step([(sa, short), (sb, toks[:100])], [list(range(37)), list(range(100))]).cpu().numpy()
        check(out[:37], plain_logits(folder, short), dtype, "the shorter of two")
        check(out[37:], ref[:100], dtype, "the longer of two")
        m.engine.check_device()
        m.close()


def _greedy(folder, prompt, n):
    pcfg, t = lm.read_folder(folder)
    seq = list(prompt)
    for _ in range(n):
        logits = pl.forward(seq, t, pcfg)[-1]
        top2 = torch.topk(logits, 2).values
        if float(top2[0] - top2[1]) < 1e-3:        # a tie within rounding proves nothing either way
            break
        seq.append(int(logits.argmax()))
    return seq[len(prompt):]


def test_greedy_generation_through_the_scheduler():
    """Model.generate, greedy, for prompts of different lengths in one call: the tokens the plain
    implementation chooses."""
    cfg = lm.GAMMA
    folder = folder_for("GAMMA", cfg, 3)
    prompts = [tokens_for(cfg, n, 70 + n) for n in (4, 37, 66)]
    m = load(folder, "float32")
    outs = m.generate(prompts, max_tokens=8, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())
    for p, o in zip(prompts, outs):
        want = _greedy(folder, p, 8)
        assert o.tokens[:len(want)] == want, (o.tokens, want)
    m.close()
    mb = load(folder, "bfloat16")
    outs_b = mb.generate(prompts, max_tokens=8, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())
    assert all(len(o.tokens) == 8 for o in outs_b)
    mb.engine.check_device()
    mb.close()


def test_generation_on_the_device_routes_by_the_chosen_token():
    """The on-device loop feeds tokens back without the host: the experts of the next step are those of the token
    just chosen.  Greedy, against Model.generate."""
    from gopherllm_b200.sampling.sampler import DeviceSampler, SamplerConfig
    cfg = lm.ALPHA
    folder = folder_for("ALPHA", cfg, 5)
    prompt = tokens_for(cfg, 21, 90)
    m = load(folder, "bfloat16")
    want = m.generate([prompt], max_tokens=12, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())[0].tokens
    s = m.open_sequence()
    logits = m.step([(s, prompt)])
    first = int(logits[0].argmax())
    assert first == want[0]
    sampler = DeviceSampler(SamplerConfig.greedy(), [1], [prompt], cfg["vocab"], m.engine.device)
    chosen = m.engine.decode_loop([s], [first], 11, sampler).cpu().numpy()[:, 0].tolist()
    assert [first] + chosen == want
    m.engine.check_device()
    m.close()


def test_command_line_generates_and_samples():
    """python -m gopherllm_b200 on a Lilupel folder: greedy tokens equal the plain implementation's, a sampled
    run with the sampler's options ends by length, and the isolated kernel bench knows the parts' products."""
    import os
    import subprocess
    import sys
    cfg = lm.GAMMA
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
    p = run("--prompt", " ".join(map(str, prompt)), "--max-tokens", "12", "--temp", "0.9", "--top-k", "20", "--top-p", "0.95",
            "--seed", "4", "--stop", "100000")
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(x) for x in p.stdout.split()]
    assert len(out) == 12 and all(0 <= x < cfg["vocab"] for x in out) and "finish=length" in p.stderr
    p = run("--kernel-bench-json", "--kernel-bench-runs", "2")
    assert p.returncode == 0, p.stderr[-2000:]
    assert json.loads(p.stdout)["kernels"]


def test_replay_of_a_trace(tmp_path):
    """The trace runner's loop on a Lilupel model: a batch of two requests, one ends, the other goes on."""
    from gopherllm_b200.engine.replay import run
    cfg = lm.ALPHA
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
