"""The Fezolorn decoder in the engine against the plain implementation: whole prompts, prefill against
token-by-token decoding, portions down to two tokens, unequal batches, slots, pages and state used
again, long decoding, greedy generation through the entry point, the replay program and the command
line; then each mechanism's kernels alone on inputs made so that a wrong window edge, a missed far
key, a sink left out, a lost state or a convolution that looks past a sequence's start shows."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from fezolorn_tiny import CONFIGS, FModel, make_weights, random_config, tokens_of, write_folder
from plain import fezolorn_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOTH = [(c, d) for c in ("P", "Q", "R") for d in ("float32", "bfloat16")]


def assert_close(got, ref, dtype, what=""):
    """32-bit: the head is the embedding table, whose rows these tests draw from N(0, 1), so logits are of the
    order of sqrt(width) (10 to 25) and 32-bit rounding through the layers is a few 1e-5 of that: the bound per
    logit is 2e-5 of the largest logit + 1e-4 |ref|.  bfloat16: an activation is rounded
    to 8 bits at a dozen places per layer, and a row whose softmax is sharp turns that into a few percent of
    its logits; the bound is 2 % of the logits' root mean square over all rows and 10 % of the largest logit
    for any one.  What a mechanism's fault does shows in the 32-bit run and in the kernels alone."""
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    err = got - ref
    if dtype == "float32":
        bad = np.abs(err) > 2e-5 * max(1.0, np.abs(ref).max()) + 1e-4 * np.abs(ref)
        assert not bad.any(), (f"{what}: max err {np.abs(err).max():.3e} of {np.abs(ref).max():.1f} "
                               f"(first bad row {np.argwhere(bad)[0]})")
        return
    rms = float(np.sqrt((err ** 2).mean()) / np.sqrt((ref ** 2).mean()))
    worst = float(np.abs(err).max() / np.abs(ref).max())
    assert rms <= 2e-2 and worst <= 1e-1, f"{what}: rms error {rms:.3e} of the logits' rms, worst logit {worst:.3e}"


def _feed(tm, slot, toks, cuts):
    """Feeds `toks` to one sequence in pieces of the sizes `cuts` (the rest one by one) and returns the
    logits of every position."""
    rows, at = [], 0
    for c in list(cuts) + [1] * len(toks):
        if at >= len(toks):
            break
        piece = toks[at:at + c]
        rows.append(tm.step_np([slot], [piece], "all"))
        at += len(piece)
    return np.concatenate(rows)


@pytest.mark.parametrize("name,dtype", BOTH)
def test_whole_prompt_and_decoding_and_portions(name, dtype):
    tm = FModel(name, dtype, seed=3)
    rng = np.random.default_rng(11)
    toks = tokens_of(rng, 150, tm.cfg["vocab"])
    ref = tm.reference(toks)
    for cuts, what in (([150], "whole"), ([40], "prefix, then one by one across windows and page borders"),
                       ([2, 3, 59, 2, 64, 1, 17, 2], "portions"), ([], "from the first token one by one"),
                       ([63, 2, 63, 2], "portions that end at and start on page borders"),
                       ([1, 1, 1, 2, 2], "portions shorter than the convolutions")):
        s = tm.engine.start_sequences(1)
        got = _feed(tm, s[0], toks, cuts)
        tm.engine.end_sequences(s)
        assert_close(got, ref, dtype, f"{name} {what}")
    tm.engine.check_kernels()
    tm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", [("R", "float32"), ("R", "bfloat16"), ("P", "float32")])
def test_a_long_prompt_takes_the_chunked_kernels(name, dtype):
    """600 tokens in one step (the recurrences' passes over chunks, the many-token projection kernels)
    against the same tokens in portions and one by one."""
    tm = FModel(name, dtype, seed=17, max_tokens=2048)
    toks = tokens_of(np.random.default_rng(23), 600, tm.cfg["vocab"])
    ref = tm.reference(toks)
    for cuts in ([600], [300, 280], [257, 256, 64]):
        s = tm.engine.start_sequences(1)
        got = _feed(tm, s[0], toks, cuts)
        tm.engine.end_sequences(s)
        assert_close(got, ref, dtype, f"{name} cut as {cuts}")


@pytest.mark.parametrize("name,dtype", BOTH)
def test_unequal_batches_equal_each_request_alone(name, dtype):
    tm = FModel(name, dtype, seed=5, max_tokens=1024)
    rng = np.random.default_rng(2)
    V = tm.cfg["vocab"]
    lens, pre = [1, 37, 141, 66], [1, 20, 100, 64]
    reqs = [tokens_of(rng, n, V) for n in lens]
    slots = tm.engine.start_sequences(4)
    out = tm.step_np(slots, [r[:p] for r, p in zip(reqs, pre)], "all")
    got, at = [], 0
    for p in pre:
        got.append([out[at:at + p]])
        at += p
    fed, live = list(pre), [i for i in range(4) if pre[i] < lens[i]]
    tm.engine.end_sequences([slots[i] for i in range(4) if pre[i] >= lens[i]])
    while live:
        out = tm.step_np([slots[i] for i in live], [[reqs[i][fed[i]]] for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
            fed[i] += 1
        done = [i for i in live if fed[i] >= lens[i]]
        tm.engine.end_sequences([slots[i] for i in done])      # shorter requests end earlier
        live = [i for i in live if i not in done]
    if dtype == "float32":
        for i, r in enumerate(reqs):
            assert_close(np.concatenate(got[i]), tm.reference(r), dtype, f"{name} request {i} of the batch")
    else:
        assert_close(np.concatenate([np.concatenate(g) for g in got]), np.concatenate([tm.reference(r) for r in reqs]),
                     dtype, f"{name} all requests of the batch")
    assert tm.engine.cache.slots.held_count == 0
    tm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("R", "bfloat16"), ("Q", "float32")])
def test_slots_pages_and_state_are_clean_when_used_again(name, dtype):
    """A cache that holds one request at a time: every request gets the slot, the pages, the recurrent
    states and the kept convolution inputs that the one before left behind."""
    tm = FModel(name, dtype, seed=8, max_tokens=192, max_batch=1)
    rng = np.random.default_rng(9)
    for n, cuts in ((170, [100]), (130, [130]), (150, [3, 90]), (5, [])):
        toks = tokens_of(rng, n, tm.cfg["vocab"])
        s = tm.engine.start_sequences(1)
        assert s == [0]
        got = _feed(tm, s[0], toks, cuts)
        tm.engine.end_sequences(s)
        assert_close(got, tm.reference(toks), dtype, f"{name} request of {n} tokens in a used slot")
        tm.engine.cache.check()
    toks = tokens_of(rng, 90, tm.cfg["vocab"])
    s = tm.engine.start_sequences(1)
    _feed(tm, s[0], tokens_of(rng, 70, tm.cfg["vocab"]), [70])
    tm.engine.reset(s[0])
    assert_close(_feed(tm, s[0], toks, [50]), tm.reference(toks), dtype, f"{name} after reset")
    tm.engine.end_sequences(s)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding(name):
    """400 tokens one by one: the recurrent states and the windows run far past every edge, and the decode
    steps are replayed from recorded graphs."""
    tm = FModel(name, "float32", seed=13)
    rng = np.random.default_rng(5)
    reqs = [tokens_of(rng, n, tm.cfg["vocab"]) for n in (400, 333)]
    slots = tm.engine.start_sequences(2)
    got = [[], []]
    for t in range(400):
        live = [i for i in (0, 1) if t < len(reqs[i])]
        out = tm.step_np([slots[i] for i in live], [[reqs[i][t]] for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(out[j])
    tm.engine.end_sequences(slots)
    assert len(tm.engine._graphs) > 0, "no decode step was replayed from a graph"
    for i in (0, 1):
        assert_close(np.stack(got[i]), tm.reference(reqs[i]), "float32", f"{name} sequence {i}")


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_entry_point(name):
    tm = FModel(name, "float32", seed=21, max_tokens=512)
    rng = np.random.default_rng(4)
    prompts = [tokens_of(rng, n, tm.cfg["vocab"]) for n in (1, 19, 70)]
    res = tm.model.generate(prompts, max_tokens=14, temperature=0.0, stop_ids=())
    for p, r in zip(prompts, res):
        seq, want = list(p), []
        for _ in range(14):
            want.append(int(np.argmax(tm.reference(seq)[-1])))
            seq.append(want[-1])
        assert r.tokens == want, f"prompt of {len(p)} tokens"
    assert tm.engine.steps_advanced_on_device > 0, "the decode steps were not fed from the device"
    assert tm.engine.cache.slots.held_count == 0


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_layers_one_by_one(name):
    """The stream after every layer (32-bit), so that a wrong layer is named."""
    tm = FModel(name, "float32", seed=6)
    toks = tokens_of(np.random.default_rng(1), 45, tm.cfg["vocab"])
    seen = []
    for b in tm.engine.model.blocks:
        def wrap(x, batch, *a, f=b.forward, **k):
            r = f(x, batch, *a, **k)
            seen.append(x.cpu().numpy().copy())
            return r
        b.forward = wrap
    s = tm.engine.start_sequences(1)
    tm.step_np(s, [toks], "last")
    ref = []
    plain.forward(tm.cfg, tm.weights, toks, streams_out=ref)
    assert len(seen) == len(ref)
    for i, (a, r) in enumerate(zip(seen, ref)):
        assert np.abs(a - r).max() <= 1e-4 * max(1.0, np.abs(r).max()), \
            f"layer {i} ({tm.cfg['layers'][i]['type']}): {np.abs(a - r).max():.3e}"


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_configurations_drawn_at_random(seed):
    cfg = random_config(seed)
    tm = FModel(cfg, "float32", seed=seed)
    rng = np.random.default_rng(seed)
    V = cfg["vocab"]
    toks = tokens_of(rng, 140, V)
    ref = tm.reference(toks)
    for cuts in ([140], [100], [2, 67, 3]):
        s = tm.engine.start_sequences(1)
        assert_close(_feed(tm, s[0], toks, cuts), ref, "float32", f"seed {seed} cut as {cuts}")
        tm.engine.end_sequences(s)
    reqs = [tokens_of(rng, n, V) for n in (9, 80, 33)]
    slots = tm.engine.start_sequences(3)
    out = tm.step_np(slots, reqs, "all")
    at = 0
    for r in reqs:
        assert_close(out[at:at + len(r)], tm.reference(r), "float32", f"seed {seed} batch")
        at += len(r)
    tm.engine.end_sequences(slots)
    tmb = FModel(cfg, "bfloat16", seed=seed)
    s = tmb.engine.start_sequences(1)
    assert_close(_feed(tmb, s[0], toks, [90]), tmb.reference(toks), "bfloat16", f"seed {seed} bfloat16")


def test_a_folder_may_hold_the_second_norm_of_a_layer_without_feed_forward():
    cfg = CONFIGS["P"]
    stored = make_weights(cfg, 4, torch.float32)
    stored["l2.norm2"] = torch.ones(cfg["width"])
    tm = FModel(cfg, "float32", weights=stored)
    toks = tokens_of(np.random.default_rng(0), 30, cfg["vocab"])
    s = tm.engine.start_sequences(1)
    assert_close(tm.step_np(s, [toks], "all"), tm.reference(toks), "float32", "unused norm present")


def test_replay_program_and_command_line(tmp_path):
    from test_trace_run_gpu import collect, run_trace
    cfg = CONFIGS["P"]
    stored = make_weights(cfg, 33, torch.float32)
    w = {k: v.double().numpy() for k, v in stored.items()}
    d = write_folder({**cfg, "vocab_size": cfg["vocab"]}, stored, str(tmp_path))   # the shared helper reads this key
    rng = np.random.default_rng(3)
    reqs = {"a": tokens_of(rng, 70, cfg["vocab"]), "b": tokens_of(rng, 33, cfg["vocab"])}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:60], "want": list(range(60))},
                                     {"id": "b", "tokens": reqs["b"][:30], "want": [0, 29]}], "end": []}]
    for t in range(10):
        ent = [{"id": "a", "tokens": [reqs["a"][60 + t]], "want": [0]}]
        if t < 3:
            ent.append({"id": "b", "tokens": [reqs["b"][30 + t]], "want": [0]})
        steps.append({"step": t + 1, "entries": ent, "end": ["b"] if t == 2 else (["a"] if t == 9 else [])})
    got = collect(steps, run_trace(d, "float32", 256, steps))
    for rid, toks in reqs.items():
        ref = plain.forward(cfg, w, toks)
        for pos, row in got[rid].items():
            assert_close(row[None], ref[pos][None], "float32", f"request {rid} position {pos}")
    assert sorted(got["a"]) == list(range(70)) and sorted(got["b"]) == [0, 29, 30, 31, 32]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "torchless"), "--temperature", "0",
                        "--max-tokens", "5", "--dtype", "float32", d, "3 17 200 ; 45"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    for prompt, line in zip(([3, 17, 200], [45]), r.stdout.strip().splitlines()):
        seq = list(prompt)
        for tok in line.split():
            assert int(tok) == int(np.argmax(plain.forward(cfg, w, seq)[-1]))
            seq.append(int(tok))


# ---------------------------------------------------------------------------------------------
# Kernels alone
# ---------------------------------------------------------------------------------------------
def _ops(dtype):
    from torchless_rs_b200.csrc import ops
    return ops.core_ops(dtype)


def _dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).cuda().contiguous()


def _i32(a):
    return torch.as_tensor(np.asarray(a, dtype=np.int32)).cuda()


def _pieces(n, cuts):
    """(start, count) of the steps that feed n tokens in pieces of `cuts`, the rest one by one."""
    out, at = [], 0
    for c in list(cuts) + [1] * n:
        if at >= n:
            break
        c = min(c, n - at)
        out.append((at, c))
        at += c
    return out


# ---- the gated delta rule ------------------------------------------------------------------------------
def _plain_delta_heads(z, taps_w, A_log, dt_bias, G, H, dim, vdim):
    """Head outputs o [n, H, vdim] of the plain recurrence from the projections z = [q | k | v | g | b | a]."""
    C = 2 * G * dim + H * vdim
    n = z.shape[0]
    conv = plain.silu(plain.short_convolution(z[:, :C], taps_w))
    q = conv[:, :G * dim].reshape(n, G, dim)
    k = conv[:, G * dim:2 * G * dim].reshape(n, G, dim)
    v = conv[:, 2 * G * dim:].reshape(n, H, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = plain.sigmoid(z[:, C + H * vdim:C + H * vdim + H])
    g = np.exp(-np.exp(A_log) * plain.softplus(z[:, C + H * vdim + H:] + dt_bias))
    o = np.zeros((n, H, vdim))
    for h in range(H):
        kv = h // (H // G)
        S = np.zeros((dim, vdim))
        for t in range(n):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            o[t, h] = S.T @ q[t, kv]
    return o


def _run_delta(z, taps_w, A_log, dt_bias, G, H, dim, vdim, seqs, slots, n_slots, state, kept):
    """One step of the package's three kernels on the rows of z that belong to `seqs` = [(start, count)]."""
    o = _ops(torch.float32)
    C = 2 * G * dim + H * vdim
    taps = taps_w.shape[1]
    T = z.shape[0]
    starts = np.concatenate([[0], np.cumsum([c for _, c in seqs])])
    token_seq = np.repeat(np.arange(len(seqs)), [c for _, c in seqs])
    zd = _dev(z)
    y = torch.zeros((T, C), device="cuda")
    gates = torch.zeros((T, 2 * H + G), device="cuda")
    out = torch.zeros((T, H * vdim), device="cuda")
    o.delta_prep(zd, _dev(taps_w), kept, y, gates, _dev(-np.exp(A_log)), _dev(dt_bias), C + H * vdim, C + H * vdim + H,
                 _i32(token_seq), _i32(starts), _i32(slots), G, H, dim, vdim, 1e-6, dim ** -0.5)
    if taps > 1:
        o.conv_state_update(zd, kept, _i32(starts), _i32(slots), C)
    o.delta_scan(y, gates, state, out, _i32(starts), _i32(slots), G, H, dim, vdim)
    return out.cpu().numpy().astype(np.float64).reshape(T, H, vdim)


@pytest.mark.parametrize("G,H,dim,vdim,taps", [(2, 4, 16, 8, 4), (2, 2, 33, 5, 1), (1, 3, 8, 36, 5), (1, 1, 64, 64, 2),
                                                (2, 8, 128, 20, 3), (1, 2, 200, 17, 4)])
def test_delta_rule_in_pieces_equals_the_plain_walk(G, H, dim, vdim, taps):
    """Two sequences of unequal lengths fed in pieces of every size (also shorter than the convolution)
    into slots that held another sequence's state before."""
    rng = np.random.default_rng(dim + taps)
    C = 2 * G * dim + H * vdim
    cols = C + H * vdim + 2 * H
    taps_w = rng.normal(0, 0.5, (C, taps))
    A_log, dt_bias = rng.normal(-1, 0.7, H), rng.normal(0, 1, H)
    n_slots = 4
    state = torch.full((n_slots, H, dim, vdim), 7.0, device="cuda")     # what an earlier sequence left
    kept = torch.full((n_slots, max(taps - 1, 1), C), -3.0, device="cuda")[:, :taps - 1]
    lens = {2: 150, 0: 61}
    zs = {s: rng.normal(0, 1.5, (n, cols)) for s, n in lens.items()}
    ref = {s: _plain_delta_heads(zs[s], taps_w, A_log, dt_bias, G, H, dim, vdim) for s in lens}
    for s in lens:                                                      # a slot is zeroed when it is taken
        state[s].zero_()
        kept[s].zero_()
    plans = {2: _pieces(150, [1, 2, 1, 70, 3, 64]), 0: _pieces(61, [40, 2])}
    got = {s: [] for s in lens}
    step = 0
    while any(step < len(p) for p in plans.values()):
        live = [s for s in plans if step < len(plans[s])]
        seqs = [plans[s][step] for s in live]
        z = np.concatenate([zs[s][a:a + c] for s, (a, c) in zip(live, seqs)])
        out = _run_delta(z, taps_w, A_log, dt_bias, G, H, dim, vdim, seqs, live, n_slots, state, kept)
        at = 0
        for s, (_, c) in zip(live, seqs):
            got[s].append(out[at:at + c])
            at += c
        step += 1
    for s in lens:
        g = np.concatenate(got[s])
        assert np.abs(g - ref[s]).max() <= 2e-4 * max(1.0, np.abs(ref[s]).max()), f"slot {s}: {np.abs(g - ref[s]).max():.3e}"
    assert float(state[1].min()) == 7.0 and float(state[3].max()) == 7.0, "another slot's state was touched"


def test_delta_rule_recalls_a_value_written_far_back():
    """With beta = 1 and no decay, a key written once is read back exactly hundreds of tokens later if the
    keys in between are orthogonal to it, and a second write under the same key replaces the value (the
    rule corrects, it does not add)."""
    G = H = 1
    dim, vdim, taps, n = 32, 16, 1, 400
    C = 2 * dim + vdim
    z = np.zeros((n, C + vdim + 2))
    rng = np.random.default_rng(0)
    for t in range(n):
        k = np.zeros(dim)
        k[1 + (t % (dim - 1))] = 30.0                   # unit vectors e_1 .. e_31 in turn
        z[t, dim:2 * dim] = k
        z[t, :dim] = k                                  # each token asks for its own key
        z[t, 2 * dim:C] = rng.uniform(20, 40, vdim)
    z[5, dim:2 * dim] = 0.0
    z[5, dim] = 30.0                                    # key e_0 is written at token 5 only ...
    z[5, 2 * dim:C] = 25.0
    z[390, :dim] = 0.0
    z[390, 0] = 30.0                                    # ... and asked for at token 390
    z[:, C + vdim] = 40.0                               # beta = sigmoid(40) = 1
    z[:, C + vdim + 1] = -60.0                          # softplus(-60) ~ 0: no decay
    taps_w = np.ones((C, 1))
    state = torch.zeros((1, 1, dim, vdim), device="cuda")
    kept = torch.zeros((1, 1, C), device="cuda")[:, :0]
    out = _run_delta(z, taps_w, np.zeros(1), np.zeros(1), G, H, dim, vdim, [(0, n)], [0], 1, state, kept)
    # token 390 reads key e_0 while writing its own key e_(1 + 390 % 31): o = S^T q picks row 0 of S
    assert np.allclose(out[390, 0] * np.sqrt(dim), plain.silu(25.0), rtol=1e-4)
    # token t's own read-out is its own value (beta = 1 replaces what the key held before)
    v_act = plain.silu(z[200, 2 * dim:C])
    assert np.allclose(out[200, 0] * np.sqrt(dim), v_act, rtol=1e-4)
    ref = _plain_delta_heads(z, taps_w, np.zeros(1), np.zeros(1), G, H, dim, vdim)
    assert np.abs(out - ref).max() <= 1e-4 * np.abs(ref).max()


def test_convolution_sees_zeros_before_a_sequence_starts_and_the_kept_inputs_after():
    G, H, dim, vdim, taps = 1, 1, 4, 4, 4
    C = 2 * dim + vdim
    o = _ops(torch.float32)
    rng = np.random.default_rng(1)
    z = rng.normal(0, 1, (9, C + vdim + 2))
    w = rng.normal(0, 1, (C, taps))
    ref = plain.silu(plain.short_convolution(z[:, :C], w))
    kept = torch.zeros((2, taps - 1, C), device="cuda")
    kept[0] = 99.0                                       # another slot's inputs must not leak in
    state = torch.zeros((2, H, dim, vdim), device="cuda")
    ys = []
    for a, c in ((0, 2), (2, 1), (3, 1), (4, 5)):
        y = torch.zeros((c, C), device="cuda")
        gates = torch.zeros((c, 2 * H + G), device="cuda")
        zd = _dev(z[a:a + c])
        o.delta_prep(zd, _dev(w), kept, y, gates, _dev([-1.0]), _dev([0.0]), C + vdim, C + vdim + 1, _i32([0] * c),
                     _i32([0, c]), _i32([1]), G, H, dim, vdim, 1e-6, 1.0)
        o.conv_state_update(zd, kept, _i32([0, c]), _i32([1]), C)
        ys.append(y.cpu().numpy())
    got = np.concatenate(ys)[:, 2 * dim:]                # the value channels are not normed
    assert np.abs(got - ref[:, 2 * dim:]).max() < 1e-5
    assert np.allclose(kept[1].cpu().numpy(), z[6:9, :C], atol=1e-6) and float(kept[0].min()) == 99.0


# ---- lightning attention ---------------------------------------------------------------------------------
def _plain_lightning(q, k, v, decay):
    n, H, dim = q.shape
    o = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        S = np.zeros((dim, v.shape[2]))
        for t in range(n):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    return o


@pytest.mark.parametrize("H,dim,vdim,decay", [(3, 16, 24, (0.5, 0.9, 0.999)), (1, 40, 12, (1.0,)), (4, 64, 32, (0.2, 0.8, 0.99, 0.97)),
                                              (2, 5, 9, (0.6, 0.95))])
def test_constant_decay_recurrence_whole_chunked_and_one_by_one(H, dim, vdim, decay):
    o = _ops(torch.float32)
    rng = np.random.default_rng(H + dim)
    n = 700
    z = np.abs(rng.normal(0, 1, (n, 2 * H * dim + H * vdim)))
    # a far key that stands out: written at token 3, asked for at token 690 by a query along the same direction
    hd = H * dim
    for h in range(H):
        z[3, hd + h * dim:hd + (h + 1) * dim] = 0.0
        z[3, hd + h * dim] = 50.0
        z[690, h * dim] = 50.0
    q, k, v = z[:, :hd].reshape(n, H, dim), z[:, hd:2 * hd].reshape(n, H, dim), z[:, 2 * hd:].reshape(n, H, vdim)
    ref = _plain_lightning(q, k, v, decay)
    decays = _dev(np.repeat(np.asarray(decay, dtype=np.float32), dim)[None])
    for cuts in ([700], [300, 399], [65, 1, 2, 512], [10] * 70):
        state = torch.zeros((2, H, dim, vdim), device="cuda")
        outs = []
        for a, c in _pieces(n, cuts):
            zd = _dev(z[a:a + c])
            out = torch.zeros((c, H * vdim), device="cuda")
            o.gla_scan(zd[:, :hd], zd[:, hd:2 * hd], zd[:, 2 * hd:], decays, None, 1.0, 1.0, state, out, _i32([0, c]),
                       _i32([1]), H, dim, vdim, given=True)
            outs.append(out.cpu().numpy())
        got = np.concatenate(outs).reshape(n, H, vdim)
        err = np.abs(got - ref).max(axis=(1, 2)) / np.maximum(1.0, np.abs(ref).max(axis=(1, 2)))
        assert err.max() <= 2e-4, f"cut as {cuts[:4]}: token {err.argmax()}: {err.max():.3e}"
        assert float(state[0].abs().max()) == 0.0


# ---- projections into the cache ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,rd,T", [(4, 2, 16, 8, 9), (3, 3, 24, 24, 5), (8, 2, 64, 32, 300), (2, 1, 20, 4, 270),
                                          (4, 1, 128, 64, 260), (1, 1, 32, 0, 7), (2, 2, 200, 100, 280)])
def test_projections_with_bias_whose_values_are_the_keys(dtype, H, G, dim, rd, T):
    """q and k get their bias, turn by position in neighbouring pairs and are divided by their root mean square;
    the value pages hold the biased keys as projected.  Few tokens and many (every kernel variant)."""
    from torchless_rs_b200.cache import PAGE
    o = _ops(dtype)
    rng = np.random.default_rng(dim + T)
    cols = (H + G) * dim
    z = rng.normal(0, 1, (T, cols)).astype(np.float32)
    bias = rng.normal(0, 1, cols).astype(np.float32)
    freq = plain.frequencies({"base": 300.0, "dims": rd, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}) \
        if rd else np.zeros(0)
    start = 50                                                   # positions 50 .. 50 + T - 1 of one sequence
    pos = np.arange(start, start + T)
    n_pages = (start + T + PAGE - 1) // PAGE
    table = np.full((3, n_pages + 1), -1, dtype=np.int32)
    order = list(rng.permutation(n_pages + 2)[:n_pages])
    table[1, :n_pages] = order
    kp = torch.zeros((n_pages + 2, G, PAGE, dim), dtype=dtype, device="cuda")
    vp = torch.zeros((n_pages + 2, G, dim, PAGE), dtype=dtype, device="cuda")
    qo = torch.zeros((T, H * dim), dtype=dtype, device="cuda")
    o.rotary_cache_write(_dev(z), _dev(freq.astype(np.float32)) if rd else None, rd, 1, True, 1e-6, qo, kp, vp, _i32(pos),
                         _i32([0] * T), _i32([1]), _i32(table), H, G, G, dim, dim, 1, bias=_dev(bias), values_are_keys=True)
    zb = z.astype(np.float64) + bias
    q = zb[:, :H * dim].reshape(T, H, dim)
    k = zb[:, H * dim:].reshape(T, G, dim)
    f = freq.astype(np.float32).astype(np.float64)
    qr = plain.rms_normalise(plain.rotate_pairs(q, pos.astype(np.float64), f), 1e-6)
    kr = plain.rms_normalise(plain.rotate_pairs(k, pos.astype(np.float64), f), 1e-6)
    tol = 5e-5 if dtype == torch.float32 else 1.2e-2
    assert np.abs(qo.float().cpu().numpy().reshape(T, H, dim) - qr).max() <= tol * max(1.0, np.abs(qr).max())
    kp, vp = kp.float().cpu().numpy(), vp.float().cpu().numpy()
    for t in range(T):
        page, at = order[pos[t] // PAGE], pos[t] % PAGE
        assert np.abs(kp[page, :, at] - kr[t]).max() <= tol * max(1.0, np.abs(kr).max()), f"key of token {t}"
        assert np.abs(vp[page, :, :, at] - k[t]).max() <= tol * max(1.0, np.abs(k).max()), f"value of token {t}"


# ---- attention with a sink over a window -------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,window", [(4, 2, 16, 20), (3, 3, 24, 1), (8, 2, 64, 130), (8, 1, 64, 65), (4, 4, 32, 64),
                                            (1, 1, 20, None), (2, 1, 128, 100)])
def test_windowed_attention_with_a_sink_sees_exactly_its_window(dtype, H, G, dim, window):
    """One key carries a score far above all others and a value that no other key has.  A query `window - 1`
    positions after it must return that value, a query `window` positions after it must not; without a window
    the key is seen from hundreds of positions on.  A sink far above the scores takes nearly all the weight, a
    sink far below none.  As a decode step, a few tokens, and a long run."""
    from torchless_rs_b200.cache import PAGE
    from torchless_rs_b200.parts.sink_attention import run_attention
    rng = np.random.default_rng(dim + (window or 0))
    n = 5 * PAGE + 9
    pages_of = [7, 2, 9, 4, 0, 5]
    slot = 3
    table = np.full((5, 8), -1, dtype=np.int32)
    table[slot, :len(pages_of)] = pages_of
    scale = 0.5
    for target in (PAGE - 1, PAGE, 3 * PAGE - 1, 200):
        k = rng.normal(0, 0.3, (n, G, dim))
        v = rng.normal(0, 0.3, (n, G, dim))
        k[target] = 0.0
        k[target, :, 0] = 9.0
        v[target, :, 0] = 50.0
        ks = torch.zeros((10, G, PAGE, dim), dtype=dtype)
        vs = torch.zeros((10, G, dim, PAGE), dtype=dtype)
        for p in range(n):
            ks[pages_of[p // PAGE], :, p % PAGE] = torch.as_tensor(k[p], dtype=dtype)
            vs[pages_of[p // PAGE], :, :, p % PAGE] = torch.as_tensor(v[p], dtype=dtype)
        kk = np.stack([ks[pages_of[p // PAGE], :, p % PAGE].float().numpy() for p in range(n)]).astype(np.float64)
        vv = np.stack([vs[pages_of[p // PAGE], :, :, p % PAGE].float().numpy() for p in range(n)]).astype(np.float64)
        ks, vs = ks.cuda(), vs.cuda()
        w = window or n
        edge = sorted({target, min(target + w - 1, n - 1), min(target + w, n - 1), n - 1})
        for qpos_list in ([[p] for p in edge] + [list(range(max(0, edge[1] - 2), min(n, edge[1] + 4)))] +
                          [list(range(n - 200, n))]):
            T = len(qpos_list)
            q = rng.normal(0, 0.3, (T, H, dim))
            q[:, :, 0] = 6.0
            q = torch.as_tensor(q, dtype=dtype).double().numpy()
            for sink in (rng.normal(0, 1, H), np.full(H, 40.0), np.full(H, -40.0)):
                out = torch.zeros((T, H * dim), dtype=dtype).cuda()
                run_attention(_ops(dtype), _dev(q.reshape(T, H * dim), dtype), ks, vs, None, _dev(sink), out, _i32(qpos_list),
                              _i32([0] * T), _i32([slot]), _i32(table), H, G, dim, dim, window, 0, scale, None)
                got = out.float().cpu().numpy().reshape(T, H, dim)
                for j, qpos in enumerate(qpos_list):
                    vis = plain.visible(n, window)[qpos]
                    for h in range(H):
                        g = h // (H // G)
                        s = (kk[:, g] @ q[j, h]) * scale
                        ref = plain.sink_softmax(s[None], vis[None], sink[h])[0] @ vv[:, g]
                        tol = 1e-4 if dtype == torch.float32 else 2e-2
                        assert np.abs(got[j, h] - ref).max() <= tol * max(1.0, np.abs(ref).max()), \
                            f"target {target} query {qpos} head {h} sink {sink[h]:.1f}: {got[j, h, 0]:.3f} vs {ref[0]:.3f}"


# ---- latent attention with a sink ----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,rank,rd", [(3, 44, 8), (4, 64, 16), (6, 128, 32), (2, 36, 6), (20, 32, 16)])
def test_latent_attention_counts_the_sink_once_however_the_keys_are_cut(dtype, H, rank, rd):
    """Scores against cached rows [c | r] with a far row that stands out; a decode step (whose keys the
    tensor-core kernel cuts into parts), a few tokens and a long run; sinks around, far above and far below
    the scores."""
    from torchless_rs_b200.cache import PAGE
    o = _ops(dtype)
    rng = np.random.default_rng(rank + H)
    n = 9 * PAGE + 5
    width = rank + rd
    rows = rng.normal(0, 0.4, (n, width))
    rows[70] = 0.0
    rows[70, 0] = 8.0                                           # the far row: a mark in the latent's first entry
    pages_of = list(rng.permutation(12)[:10])
    table = np.full((2, 12), -1, dtype=np.int32)
    table[1, :10] = pages_of
    store = torch.zeros((12, PAGE, width), dtype=dtype)
    for p in range(n):
        store[pages_of[p // PAGE], p % PAGE] = torch.as_tensor(rows[p], dtype=dtype)
    cached = np.stack([store[pages_of[p // PAGE], p % PAGE].float().numpy() for p in range(n)]).astype(np.float64)
    store = store.cuda()
    inv_freq = (100.0 ** (-np.arange(rd // 2) / (rd // 2))).astype(np.float32)
    scale = 0.3
    for qpos_list in ([n - 1], [70], list(range(300, 305)), list(range(n - 260, n))):
        T = len(qpos_list)
        q = rng.normal(0, 0.5, (T, H, width)).astype(np.float32)
        q[:, :, 0] = 7.0
        for sink in (rng.normal(0, 1, H), np.full(H, 60.0), np.full(H, -60.0)):
            out = torch.zeros((T, H, rank), device="cuda")
            qd = _dev(q.reshape(T, H * width))
            o.latent_attn(qd, width, qd, width, rank, store, out, _i32(qpos_list), _i32([0] * T), _i32([1]), _i32(table),
                          _dev(inv_freq), H, rank, rd, rd, None, scale, max_keys=1024, sink=_dev(sink))
            got = out.cpu().numpy()
            for j, qpos in enumerate(qpos_list):
                a = qpos * inv_freq.astype(np.float64)
                qq = q[j].astype(np.float64).copy()
                u, w = qq[:, rank:rank + rd // 2].copy(), qq[:, rank + rd // 2:].copy()
                qq[:, rank:rank + rd // 2] = u * np.cos(a) - w * np.sin(a)       # the kernels' pairs (i, i + rd/2)
                qq[:, rank + rd // 2:] = w * np.cos(a) + u * np.sin(a)
                for h in range(H):
                    s = (cached[:qpos + 1] @ qq[h]) * scale
                    p = plain.sink_softmax(s[None], np.ones((1, qpos + 1), bool), sink[h])[0]
                    ref = p @ cached[:qpos + 1, :rank]
                    tol = 1e-4 if dtype == torch.float32 else 2.5e-2
                    assert np.abs(got[j, h] - ref).max() <= tol * max(1.0, np.abs(ref).max()), \
                        f"query {qpos} head {h} sink {sink[h]:.1f}: {got[j, h, 0]:.3f} vs {ref[0]:.3f}"


# ---- the small kernels ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    o = _ops(dtype)
    rng = np.random.default_rng(0)
    # silu over a range of columns of strided rows
    for T, n, ld in ((5, 12, 20), (300, 30, 37)):
        x = rng.normal(0, 2, (T, ld)).astype(np.float32)
        xd = _dev(x)
        o.silu_rows(xd[:, :n])
        ref = x.copy().astype(np.float64)
        ref[:, :n] = plain.silu(ref[:, :n])
        assert np.abs(xd.cpu().numpy() - ref).max() < 1e-5
    # a weighted sum of terms with and without a bias, stored and accumulated
    T, n = 7, 33
    ys = [rng.normal(0, 1, (T, n)).astype(np.float32) for _ in range(3)]
    b1 = rng.normal(0, 1, n).astype(np.float32)
    base = rng.normal(0, 1, (T, n)).astype(np.float32)
    ref = 0.7 * (ys[0] + b1) - 1.3 * ys[1] + 2.0 * ys[2]
    for acc in (False, True):
        out = _dev(base)
        o.weighted_sum([_dev(y) for y in ys], [_dev(b1), None, None], [0.7, -1.3, 2.0], out, accumulate=acc)
        assert np.abs(out.cpu().numpy() - (ref + (base if acc else 0))).max() < 1e-5
    # a norm over the concatenated heads with a sigmoid gate, and per head with a silu gate
    for heads, vdim, sig in ((1, 72, True), (3, 24, False), (1, 1000, True)):
        x = rng.normal(0, 2, (6, heads * vdim)).astype(np.float32)
        g = rng.normal(0, 2, (6, heads * vdim)).astype(np.float32)
        w = rng.normal(1, 0.2, vdim).astype(np.float32)
        out = torch.zeros((6, heads * vdim), dtype=dtype, device="cuda")
        o.headnorm_silu_gate(_dev(x), _dev(w), 1e-5, _dev(g), out, heads, vdim, sigmoid=sig)
        xn = plain.rms_normalise(x.astype(np.float64).reshape(6, heads, vdim), 1e-5) * w
        ref = xn.reshape(6, -1) * (plain.sigmoid(g) if sig else plain.silu(g.astype(np.float64)))
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    # one small product per head into the activation type, without a gate
    for M in (3, 70):
        H, N, K = 3, 20, 24
        a = rng.normal(0, 1, (M, H * K)).astype(np.float32)
        w = torch.as_tensor(rng.normal(0, 1, (H, N, K)), dtype=dtype)
        c = torch.zeros((M, H * N), dtype=dtype, device="cuda")
        o.headwise_gemm(_dev(a), K, w.cuda(), c, N, act_out=True)
        ad = a if dtype == torch.float32 or M <= 16 else torch.as_tensor(a).bfloat16().float().numpy()
        ref = np.einsum("mhk,hnk->mhn", ad.reshape(M, H, K).astype(np.float64), w.double().numpy()).reshape(M, H * N)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert np.abs(c.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
