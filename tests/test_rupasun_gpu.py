"""The Rupasun decoder in the engine against the plain implementation: whole prompts, prefill
against token-by-token decoding, portions down to two tokens, unequal batches, slots and pages used
again, long decoding, greedy generation through the entry point, the replay program and the command
line; then each mechanism's kernels alone on inputs made so that a wrong window edge, a missed far
key, a confused map, a wrong rotation or a wrong expert shows."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers_gpu import assert_close as _assert_close_32
from plain import rupasun_plain as plain
from rupasun_tiny import CONFIGS, TModel, make_weights, random_config, sure_tokens, tokens_of, write_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOTH = [(c, d) for c in ("P", "Q", "R") for d in ("float32", "bfloat16")] + [("S", "bfloat16")]


def assert_close(got, ref, dtype, what=""):
    """32-bit: the package's stated bound (5e-5 + 1e-4 |ref| per logit).  bfloat16: activations are rounded
    to 8 bits at some ten places per layer, and a sharp softmax or a router's close call turns that into
    a few percent of a row's logits: 2 % of the logits' root mean square over all rows and 10 % of the
    largest logit for any one.  What a mechanism's fault does shows in the 32-bit run and in the kernels'
    own tests below."""
    if dtype == "float32":
        return _assert_close_32(got, ref, dtype, what)
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    err = got - ref
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
    tm = TModel(name, dtype, seed=3)
    rng = np.random.default_rng(11)
    toks = sure_tokens(tm, rng, 150)
    ref = tm.reference(toks)
    for cuts, what in (([150], "whole"), ([40], "prefix, then one by one across windows and page borders"),
                       ([2, 3, 59, 2, 64, 1, 17, 2], "portions"), ([], "from the first token one by one"),
                       ([63, 2, 63, 2], "portions that end at and start on page borders")):
        s = tm.engine.start_sequences(1)
        got = _feed(tm, s[0], toks, cuts)
        tm.engine.end_sequences(s)
        assert_close(got, ref, dtype, f"{name} {what}")
    tm.engine.check_kernels()
    tm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", BOTH)
def test_unequal_batches_equal_each_request_alone(name, dtype):
    tm = TModel(name, dtype, seed=5, max_tokens=1024)
    rng = np.random.default_rng(2)
    V = tm.cfg["vocab"]
    lens, pre = [1, 37, 141, 66], [1, 20, 100, 64]
    reqs = [sure_tokens(tm, rng, n) for n in lens]
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


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("R", "bfloat16"), ("Q", "float32"), ("S", "bfloat16")])
def test_slots_and_pages_are_clean_when_used_again(name, dtype):
    """A cache that holds one request at a time: every request gets the slot and the pages that the one
    before left behind, keys of the longer request still in them."""
    tm = TModel(name, dtype, seed=8, max_tokens=192, max_batch=1)
    rng = np.random.default_rng(9)
    for n, cuts in ((170, [100]), (130, [130]), (150, [3, 90]), (5, [])):
        toks = sure_tokens(tm, rng, n)
        s = tm.engine.start_sequences(1)
        assert s == [0]
        got = _feed(tm, s[0], toks, cuts)
        tm.engine.end_sequences(s)
        assert_close(got, tm.reference(toks), dtype, f"{name} request of {n} tokens in a used slot")
        tm.engine.cache.check()
    toks = sure_tokens(tm, rng, 90)
    s = tm.engine.start_sequences(1)
    _feed(tm, s[0], tokens_of(rng, 70, tm.cfg["vocab"]), [70])
    tm.engine.reset(s[0])
    assert_close(_feed(tm, s[0], toks, [50]), tm.reference(toks), dtype, f"{name} after reset")
    tm.engine.end_sequences(s)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding(name):
    """400 tokens one by one: the windows run far past every edge, the maps without a window see every key
    from the first on, and the decode steps are replayed from recorded graphs."""
    tm = TModel(name, "float32", seed=13)
    rng = np.random.default_rng(5)
    reqs = [sure_tokens(tm, rng, n) for n in (400, 333)]
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [3, 8, 13, 14])
def test_configurations_drawn_at_random(seed, dtype):
    """Other sizes, head counts, layer orders, windows and constants than the named configurations have: a whole
    prompt, a prefix and then token by token, and three unequal requests in one batch that are then decoded
    together, against the plain implementation."""
    tm = TModel(random_config(seed), dtype, seed=100 + seed, max_tokens=2048)
    rng = np.random.default_rng(seed)
    reqs = [sure_tokens(tm, rng, n) for n in (230, 150, 40)]
    refs = [tm.reference(q) for q in reqs]
    s = tm.engine.start_sequences(1)
    assert_close(tm.step_np(s, [reqs[0]], "all"), refs[0], dtype, f"seed {seed} whole")
    tm.engine.end_sequences(s)
    s = tm.engine.start_sequences(1)
    got = [tm.step_np(s, [reqs[0][:180]], "all")] + [tm.step_np(s, [[t]], "all") for t in reqs[0][180:]]
    assert_close(np.concatenate(got), refs[0], dtype, f"seed {seed} prefix, then one by one")
    tm.engine.end_sequences(s)
    s = tm.engine.start_sequences(3)
    cut = [len(q) - 20 for q in reqs]
    first = tm.step_np(s, [q[:c] for q, c in zip(reqs, cut)], "all")
    rows = [[first[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
    for k in range(20):
        out = tm.step_np(s, [[q[c + k]] for q, c in zip(reqs, cut)], "last")
        for i in range(3):
            rows[i].append(out[i:i + 1])
    tm.engine.end_sequences(s)
    for i in range(3):
        assert_close(np.concatenate(rows[i]), refs[i], dtype, f"seed {seed} request {i} of a batch")
    tm.engine.check_kernels()
    tm.engine.cache.check()


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_entry_point(name):
    tm = TModel(name, "float32", seed=21, max_tokens=512)
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
    tm = TModel(name, "float32", seed=6)
    toks = tokens_of(np.random.default_rng(1), 45, tm.cfg["vocab"])
    seen = []
    for b in tm.engine.model.blocks:
        def wrap(x, batch, carry=None, next_norm=None, f=b.forward, **kw):
            r = f(x, batch, carry, next_norm, **kw)
            seen.append(x.cpu().numpy().copy())
            return r
        b.forward = wrap
    s = tm.engine.start_sequences(1)
    tm.step_np(s, [toks], "last")
    _, ref = plain.forward(tm.cfg, tm.weights, toks, return_layers=True)
    assert len(seen) == len(ref)
    for i, (a, r) in enumerate(zip(seen, ref)):
        assert np.abs(a - r).max() <= 1e-4 * max(1.0, np.abs(r).max()), f"layer {i}: {np.abs(a - r).max():.3e}"


def test_a_folder_may_hold_the_unused_norms_of_a_layer_without_feed_forward():
    cfg = CONFIGS["P"]
    stored = make_weights(cfg, 4, torch.float32)
    none = [i for i, l in enumerate(cfg["layers"]) if l["mlp"] is None]
    assert none
    for i in none:
        stored.update({f"l{i}.norm2": torch.zeros(cfg["width"]), f"l{i}.norm2b": torch.ones(cfg["width"])})
    tm = TModel(cfg, "float32", weights=stored)
    toks = tokens_of(np.random.default_rng(0), 30, cfg["vocab"])
    s = tm.engine.start_sequences(1)
    assert_close(tm.step_np(s, [toks], "all"), tm.reference(toks), "float32", "unused tensors present")


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
# Mechanisms alone
# ---------------------------------------------------------------------------------------------
def _ops(dtype):
    from torchless_rs_b200.csrc import ops
    return ops.core_ops(dtype)


def _dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=dtype).cuda().contiguous()


def _i32(a):
    return torch.as_tensor(np.asarray(a, dtype=np.int32)).cuda()


def _inv_freq(rot, base):
    return _dev(base ** (-2.0 * np.arange(rot // 2) / rot)) if rot else None


class _Pages:
    """Pages of one sequence, out of order, in a table that also holds other slots."""

    def __init__(self, dtype, n, G, width, vdim, n_slots=5, slot=3):
        from torchless_rs_b200.cache import PAGE
        self.PAGE = PAGE
        count = (n + PAGE - 1) // PAGE
        order = list(np.random.default_rng(n).permutation(count + 4))[:count]
        self.table = np.full((n_slots, count + 2), -1, dtype=np.int32)
        self.table[slot, :count] = order
        self.slot = slot
        self.k = torch.zeros((count + 4, G, PAGE, width), dtype=dtype).cuda()
        self.v = torch.zeros((count + 4, G, vdim, PAGE), dtype=dtype).cuda()


def _write(o, pages, z, pos, rot, base, style, unit_norm, eps, H, G, dim, vdim, slots, dtype):
    """The step's projections through the package's kernel into `pages`; returns q [T, H * slots * width]."""
    T = len(pos)
    q = torch.zeros((T, H * slots * slots * dim), dtype=dtype).cuda()
    o.rotary_cache_write(_dev(z), _inv_freq(rot, base), rot, style, unit_norm, eps, q, pages.k, pages.v, _i32(pos),
                         _i32([0] * T), _i32([pages.slot]), _i32(pages.table), H * slots, G * slots, G, dim, vdim, slots)
    return q


def _join(zq, zk, zv):
    n = zq.shape[0]
    return np.concatenate([zq.reshape(n, -1), zk.reshape(n, -1), zv.reshape(n, -1)], axis=1).astype(np.float32)


def _split(z, H, G, dim, vdim, slots):
    n = z.shape[0]
    a, b = H * slots * dim, (H + G) * slots * dim
    return (z[:, :a].reshape(n, H * slots, dim), z[:, a:b].reshape(n, G * slots, dim),
            z[:, b:b + G * vdim].reshape(n, G, vdim))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,vdim,rot,slots,style,unit", [
    (3, 1, 20, 7, 8, 1, 1, True), (2, 2, 16, 24, 16, 2, 0, False), (4, 2, 64, 32, 32, 1, 0, True),
    (1, 1, 24, 10, 0, 2, 0, False), (4, 4, 48, 112, 48, 2, 1, False), (2, 1, 128, 64, 128, 1, 1, True),
    (2, 1, 64, 16, 24, 1, 1, True), (2, 2, 32, 8, 12, 2, 0, False), (3, 1, 128, 40, 64, 1, 0, True), (5, 5, 16, 16, 8, 2, 1, True)])
def test_projections_are_rotated_normed_and_written_to_their_pages(dtype, H, G, dim, vdim, rot, slots, style, unit):
    """Both pairings, rotation of a part and of nothing, with and without the unit norm, one and two maps
    per head: q, and k and v where the pages hold them; positions up to some thousands (32-bit angles),
    a step that crosses a page border, steps of few and of many tokens; pages of other sequences stay
    untouched."""
    o = _ops(dtype)
    rng = np.random.default_rng(dim + rot)
    base, eps = 5000.0, 1e-5
    cols = (H + G) * slots * dim + G * vdim
    for first, T in ((0, 70), (60, 70), (3000, 70), (37, 300), (1000, 257)):      # few tokens; many (another kernel)
        pos = np.arange(first, first + T)
        pages = _Pages(dtype, first + T, G, slots * dim, vdim)
        z = rng.normal(0, 1.0, (T, cols + 3)).astype(np.float32)        # further columns follow and are not read
        q = _write(o, pages, z, pos, rot, base, style, unit, eps, H, G, dim, vdim, slots, dtype).float().cpu().numpy()
        zq, zk, zv = _split(z.astype(np.float64), H, G, dim, vdim, slots)
        p64 = pos.astype(np.float64)
        qr = plain.rotate(zq, p64, rot, base, style == 1)
        kr = plain.rotate(zk, p64, rot, base, style == 1)
        if unit:
            qr, kr = plain.rms_normalise(qr, eps), plain.rms_normalise(kr, eps)
        # angles are 32-bit: at position p the rounding of p * f moves sine and cosine by about p * 6e-8
        tol = (2e-5 + first * 2e-7) if dtype == torch.float32 else 1e-2
        scale = max(np.abs(qr).max(), np.abs(kr).max())
        q = q.reshape(T, H * slots, slots, dim)
        for j in range(H * slots):
            assert np.abs(q[:, j, j % slots] - qr[:, j]).max() <= tol * scale
            for other in range(slots):
                if other != j % slots:
                    assert (q[:, j, other] == 0).all(), "a query is not zero in the other map's half"
        kg, vg = pages.k.float().cpu().numpy(), pages.v.float().cpu().numpy()
        used = set()
        for t, p in enumerate(pos):
            page = pages.table[pages.slot, p // pages.PAGE]
            used.add(int(page))
            assert np.abs(kg[page, :, p % pages.PAGE].reshape(G * slots, dim) - kr[t]).max() <= tol * scale
            assert np.abs(vg[page, :, :, p % pages.PAGE] - zv[t]).max() <= tol * np.abs(zv).max()
        rest = [i for i in range(kg.shape[0]) if i not in used]
        assert float(np.abs(kg[rest]).sum()) == 0.0 and float(np.abs(vg[rest]).sum()) == 0.0


def _attend(dtype, q, pos, pages, H, G, width, vdim, window, scale, cap):
    from torchless_rs_b200.parts.sink_attention import run_attention
    T = len(pos)
    out = torch.zeros((T, H * vdim), dtype=dtype).cuda()
    run_attention(_ops(dtype), q, pages.k, pages.v, None, None, out, _i32(pos), _i32([0] * T), _i32([pages.slot]),
                  _i32(pages.table), H, G, width, vdim, window, 0, scale, cap)
    return out


def _forms(qpos):
    """The positions of a step that ends with `qpos`: one (a decode step), a few, a long run (a prompt)."""
    return {"decode": qpos, "few": max(0, qpos - 5), "prompt": max(0, qpos - 309)}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,vdim,rot,window,cap", [
    (3, 1, 16, 24, 16, 70, 30.0), (2, 2, 40, 12, 20, 64, None), (4, 2, 64, 64, 64, 130, 25.0), (8, 2, 32, 64, 32, 1, 50.0),
    (2, 1, 128, 128, 64, 65, 40.0), (4, 4, 64, 32, 0, 20, None), (2, 1, 64, 80, 64, None, 30.0)])
def test_window_attention_sees_exactly_its_window(dtype, H, G, dim, vdim, rot, window, cap):
    """Rotation (neighbouring pairs), unit norm, cache, attention with cap and window, and the gate, as the
    mixer chains them.  One key points where every query points, far more than the others, and carries a
    value that no other key has: a query `window - 1` positions after it returns that value, a query
    `window` positions after it does not.  The key also lies on page borders and hundreds of keys back
    among look-alikes (no window: seen from everywhere).  The marked entry's pair turns by less than a
    thousandth of a turn over the whole sequence, so the mark survives the rotation."""
    o = _ops(dtype)
    rng = np.random.default_rng(dim + (window or 0))
    base, eps = 1e7, 1e-6
    n = 5 * 64 + 9
    mark = (rot - 2) if rot else 0                # the slowest pair's first entry (style 1), or an unrotated one
    # after the unit norm the marked key is sqrt(dim) in the marked entry and a query q_mark / rms(q) there:
    # a score of 16 for the marked key, while the other keys (zero in that entry) score around +-1.6
    scale = 16.0 / (3.0 / np.sqrt((9.0 + (dim - 1) * 0.09) / dim) * np.sqrt(dim))
    pos_all = np.arange(n)
    for target in (63, 64, 3 * 64 - 1, 200, 0):
        zq = rng.normal(0, 0.3, (n, H, dim))
        zk = rng.normal(0, 0.3, (n, G, dim))
        zv = rng.normal(0, 0.3, (n, G, vdim))
        zk[:, :, mark] = 0.0
        zk[target] = 0.0
        zk[target, :, mark] = 4.0
        zv[target, :, 0] = 50.0
        zq[:, :, mark] = 3.0                                 # every query looks for the mark
        z = _join(zq, zk, zv)
        gate = rng.normal(0, 1.0, (n, H * vdim)).astype(np.float32)
        pages = _Pages(dtype, n, G, dim, vdim)
        q = _write(o, pages, z, pos_all, rot, base, 1, True, eps, H, G, dim, vdim, 1, dtype)
        z64 = z.astype(np.float64)
        zq, zk, zv = _split(z64, H, G, dim, vdim, 1)
        p64 = pos_all.astype(np.float64)
        qr = plain.rms_normalise(plain.rotate(zq, p64, rot, base, True), eps)
        kr = plain.rms_normalise(plain.rotate(zk, p64, rot, base, True), eps)
        vis = plain.visible(p64, window)
        for qpos in sorted({target, target + (window or 1) - 1, target + (window or 1), n - 1}):
            if qpos >= n:
                continue
            ref = np.zeros((H, vdim))
            for h in range(H):
                g = h // (H // G)
                s = (kr[:, g] @ qr[qpos, h]) * scale
                if cap:
                    s = cap * np.tanh(s / cap)
                ref[h] = plain.softmax_rows(s[None], vis[qpos][None])[0] @ zv[:, g]
            ref = ref.reshape(-1) * plain.sigmoid(gate[qpos].astype(np.float64))
            sees = bool(vis[qpos, target])
            strong = np.abs(ref.reshape(H, vdim)[:, 0]) > 5.0 * plain.sigmoid(gate[qpos].reshape(H, vdim)[:, 0])
            assert strong.all() == sees and (sees or not strong.any()), "the test's own mark does not stand out"
            for form, first in _forms(qpos).items():
                rows = np.arange(first, qpos + 1)
                out = _attend(dtype, q[first:qpos + 1].contiguous(), rows, pages, H, G, dim, vdim, window, scale, cap)
                o.sigmoid_gate(out, _dev(gate[first:qpos + 1]))
                got = out.float().cpu().numpy()[-1]
                tol = 3e-5 if dtype == torch.float32 else 2.5e-2
                assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max()), \
                    f"target {target} query {qpos} ({form}): {np.abs(got - ref).max():.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,vdim,rot,lam,diff", [
    (3, 1, 16, 24, 8, 0.45, 0.3), (2, 2, 8, 8, 0, 1.3, 0.8), (4, 2, 32, 64, 32, 0.7, 0.5), (4, 1, 48, 112, 48, 0.2, 0.1),
    (2, 1, 64, 32, 16, 0.9, 0.6)])
def test_differential_attention_keeps_its_maps_apart_and_sees_far_keys(dtype, H, G, dim, vdim, rot, lam, diff):
    """Rotation (halves), cache with both maps' keys side by side, attention, and the difference with its
    per-head norm, as the mixer chains them.  One key stands out in ONE map only (first the one, then the
    other) and carries a value of its own: the head's output then points along that value with the sign
    of the map (plus for the first, minus for the second), from the key's own position to hundreds of
    keys later, across page borders."""
    o = _ops(dtype)
    rng = np.random.default_rng(dim + rot)
    base, eps, scale = 1e7, 1e-6, 0.3              # the marked key scores 16, the others around +-0.6
    n = 5 * 64 + 9
    mark = (rot // 2 - 1) if rot else 0           # the slowest pair's first entry (style 0), or an unrotated one
    pos_all = np.arange(n)
    p64 = pos_all.astype(np.float64)
    vis = plain.visible(p64, None)
    for target, which in ((0, 0), (63, 1), (64, 0), (200, 1)):
        zq = rng.normal(0, 0.3, (n, 2 * H, dim))
        zk = rng.normal(0, 0.3, (n, 2 * G, dim))
        zv = rng.normal(0, 0.3, (n, G, vdim))
        zk[target, which::2] = 0.0
        zk[target, which::2, mark] = 9.0
        zv[target, :, 0] = 50.0
        zq[:, :, mark] = 6.0
        z = _join(zq, zk, zv)
        pages = _Pages(dtype, n, G, 2 * dim, vdim)
        q = _write(o, pages, z, pos_all, rot, base, 0, False, eps, H, G, dim, vdim, 2, dtype)
        zq, zk, zv = _split(z.astype(np.float64), H, G, dim, vdim, 2)
        qr = plain.rotate(zq, p64, rot, base, False).reshape(n, H, 2, dim)
        kr = plain.rotate(zk, p64, rot, base, False).reshape(n, G, 2, dim)
        for qpos in sorted({target, target + 1, min(n - 1, target + 130), n - 1}):
            ref = np.zeros((H, vdim))
            for h in range(H):
                g = h // (H // G)
                a = [plain.softmax_rows(((kr[:, g, m] @ qr[qpos, h, m]) * scale)[None], vis[qpos][None])[0] @ zv[:, g]
                     for m in (0, 1)]
                ref[h] = plain.rms_normalise(a[0] - lam * a[1], eps) * (1.0 - diff)
            # the marked value dominates the head: entry 0 is close to +-(1 - diff) sqrt(vdim)
            sign = 1.0 if which == 0 else -1.0
            if qpos > 0:          # at the first position both maps see one key only: o = (1 - lambda) v
                assert (sign * ref[:, 0] > 0.8 * (1.0 - diff) * np.sqrt(vdim)).all(), "the test's own mark does not stand out"
            for form, first in _forms(qpos).items():
                rows = np.arange(first, qpos + 1)
                maps = _attend(dtype, q[first:qpos + 1].contiguous(), rows, pages, 2 * H, G, 2 * dim, vdim, None, scale, None)
                out = torch.zeros((len(rows), H * vdim), dtype=dtype).cuda()
                o.diff_heads(maps, lam, eps, 1.0 - diff, out, H, vdim)
                got = out.float().cpu().numpy()[-1].reshape(H, vdim)
                tol = 3e-5 if dtype == torch.float32 else 2.5e-2
                assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max()), \
                    f"target {target} map {which} query {qpos} ({form}): {np.abs(got - ref).max():.3e}"


@pytest.mark.parametrize("E,groups,keep,top", [(6, 3, 2, 2), (4, 4, 2, 2), (6, 3, 2, 4), (4, 2, 2, 3), (3, 1, 1, 1), (15, 5, 4, 2),
                                               (64, 8, 3, 6), (40, 40, 7, 7), (9, 3, 1, 3)])
def test_router_chooses_among_the_best_groups(E, groups, keep, top):
    """Groups of one, two and more members, all groups kept, one group kept, a choice of one and of all that
    can be chosen; tokens whose choice hangs on a gap that 32-bit rounding can move are left out.  Some
    rows are made so that the largest score of all lies in a group that is not kept."""
    o = _ops(torch.float32)
    rng = np.random.default_rng(E + top)
    T, scale = 300, 2.5
    z = rng.normal(0, 1.5, (T, E + 2)).astype(np.float32)                # further columns follow and are not read
    size = E // groups
    if size > 2 and keep < groups:
        z[:40, :E] = rng.normal(-1.0, 0.3, (40, E))
        z[:40, 0] = 4.0                                                  # group 0: one large score, the rest small
        z[:40, size:E] += 2.5                                            # the other groups: two good scores each
    idx = torch.zeros((T, top), dtype=torch.int32).cuda()
    wt = torch.zeros((T, top), dtype=torch.float32).cuda()
    o.moe_route_grouped(_dev(z)[:, :E], groups, keep, top, scale, idx, wt)
    idx, wt = idx.cpu().numpy(), wt.cpu().numpy()
    s = plain.sigmoid(z[:, :E].astype(np.float64))
    checked = struck = 0
    for t in range(T):
        chosen, allowed = plain.route(s[t], top, groups, keep)
        per = np.sort(s[t].reshape(groups, size), axis=1)[:, ::-1][:, :2].sum(axis=1)
        gs = np.sort(per)[::-1]
        rest = np.sort(np.where(allowed, s[t], -1.0))[::-1]
        close = (keep < groups and gs[keep - 1] - gs[keep] < 1e-5) or (top < allowed.sum() and rest[top - 1] - rest[top] < 1e-5)
        if close:
            continue
        checked += 1
        struck += int(not allowed[np.argmax(s[t])])
        assert list(idx[t]) == list(chosen), f"token {t}: {idx[t]} for {chosen}"
        ref = s[t, chosen] / (s[t, chosen].sum() + 1e-20) * scale
        assert np.abs(wt[t] - ref).max() <= 1e-5
    assert checked > T // 2
    if size > 2 and keep < groups:
        assert struck >= 30, "no row has its largest score outside the kept groups"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,f,E,groups,keep,top,shared,T", [(96, 24, 6, 3, 2, 2, (40, 1.5), 70), (80, 40, 4, 4, 2, 2, None, 9),
                                                            (64, 16, 3, 1, 1, 1, None, 150), (128, 64, 40, 8, 3, 6, (32, 0.4), 300),
                                                            (64, 32, 8, 2, 2, 8, (64, 5.0), 1)])
def test_experts_are_chosen_weighted_and_summed(dtype, W, f, E, groups, keep, top, shared, T):
    """The feed-forward part alone against the plain one on the same (already rounded) input; tokens whose
    choice hangs on a gap below what the rounding of the router's product can move are left out."""
    from torchless_rs_b200.config.spec import PartSpec
    from torchless_rs_b200.parts import Runtime, lookup
    rt = Runtime("cuda:0", torch.float32 if dtype == "float32" else torch.bfloat16)
    store = rt.act_dtype
    rng = np.random.default_rng(W + E)
    limit, scale = 0.7, 1.7
    spec = PartSpec("moe_grouped_sigmoid", {"hidden_size": W, "ff": f, "experts": E, "top": top, "limit": limit,
                                            "groups": groups, "keep": keep, "route_scale": scale,
                                            "shared_ff": shared[0] if shared else None,
                                            "shared_limit": shared[1] if shared else None})
    cls = lookup("feed_forward", "moe_grouped_sigmoid")
    w = {}
    for n, ts in cls.expected_tensors(spec, "m").items():
        std = (2.0 if n.endswith("router") else 1.0) / np.sqrt(ts.shape[-1])
        w[n] = torch.as_tensor(rng.normal(0, std, ts.shape), dtype=torch.float32).to(store)
    part = cls(spec, "m", rt)
    part.load(w)
    h = torch.as_tensor(rng.normal(0, 1.0, (T, W)), dtype=torch.float32).to(store)
    w64 = {k[2:]: v.double().numpy() for k, v in w.items()}
    h64 = h.double().numpy()
    p = {"kind": "moe", "router": {"experts": E, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}},
         "expert": {"ff": f, "limit": limit}}
    if shared:
        p["shared"] = {"ff": shared[0], "limit": shared[1]}
    ref = plain.expert_ff(h64, w64, p)
    s = plain.sigmoid(h64 @ w64["router"].T)
    gap_needed = 1e-5 if dtype == "float32" else 2e-2
    sure = np.ones(T, bool)
    for t in range(T):
        _, allowed = plain.route(s[t], top, groups, keep)
        gs = np.sort(np.sort(s[t].reshape(groups, E // groups), axis=1)[:, ::-1][:, :2].sum(axis=1))[::-1]
        rest = np.sort(np.where(allowed, s[t], -1.0))[::-1]
        if (keep < groups and gs[keep - 1] - gs[keep] < 2 * gap_needed) or \
                (top < allowed.sum() and rest[top - 1] - rest[top] < gap_needed):
            sure[t] = False
    assert sure.sum() > T // 8
    out = torch.full((T, W), 3.0).cuda()
    part.forward(h.cuda(), out, None, overwrite=True)
    got = out.cpu().numpy()
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert np.abs(got - ref)[sure].max() <= tol * np.abs(ref).max(), f"{np.abs(got - ref)[sure].max():.3e}"
    part.forward(h.cuda(), out, None)                  # adds into what is there
    assert np.abs(out.cpu().numpy() - 2 * ref)[sure].max() <= 2 * tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,f,T", [(96, 160, 70), (80, 36, 1), (256, 1024, 300)])
def test_dense_feed_forward_squares_its_relu(dtype, W, f, T):
    from torchless_rs_b200.config.spec import PartSpec
    from torchless_rs_b200.parts import Runtime, lookup
    rt = Runtime("cuda:0", torch.float32 if dtype == "float32" else torch.bfloat16)
    rng = np.random.default_rng(W)
    spec = PartSpec("relu_squared", {"hidden_size": W, "intermediate_size": f})
    cls = lookup("feed_forward", "relu_squared")
    w = {n: torch.as_tensor(rng.normal(0, ts.shape[-1] ** -0.5, ts.shape), dtype=torch.float32).to(rt.act_dtype)
         for n, ts in cls.expected_tensors(spec, "m").items()}
    part = cls(spec, "m", rt)
    part.load(w)
    h = torch.as_tensor(rng.normal(0, 1.0, (T, W)), dtype=torch.float32).to(rt.act_dtype)
    ref = plain.dense_ff(h.double().numpy(), {k[2:]: v.double().numpy() for k, v in w.items()})
    out = torch.full((T, W), 3.0).cuda()
    part.forward(h.cuda(), out, None, overwrite=True)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert np.abs(out.cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    part.forward(h.cuda(), out, None)
    assert np.abs(out.cpu().numpy() - 2 * ref).max() <= 2 * tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [40, 96, 1000, 1030, 4100, 9000])
def test_sublayer_output_is_normed_added_and_normed_again(dtype, H):
    """Rows of very different size (the norms divide them out), widths inside and past what a block keeps in
    registers; alone and together with the next norm the stream is the same."""
    o = _ops(dtype)
    rng = np.random.default_rng(H)
    T = 21
    y = (rng.normal(0, 1.0, (T, H + 3)) * rng.choice([1e-3, 1.0, 300.0], (T, 1))).astype(np.float32)
    x = rng.normal(0, 2.0, (T, H)).astype(np.float32)
    for wdt in (torch.float32, torch.bfloat16):
        w1 = torch.as_tensor(rng.normal(1, 0.3, H), dtype=torch.float32).to(wdt)
        w2 = torch.as_tensor(rng.normal(1, 0.3, H), dtype=torch.float32).to(wdt)
        new = x.astype(np.float64) + plain.norm(y[:, :H].astype(np.float64), w1.double().numpy(), 1e-5)
        x1, x2 = _dev(x), _dev(x)
        o.norm_add_norm(_dev(y)[:, :H], w1.cuda(), 1e-5, x1)
        xn = torch.zeros((T, H), dtype=dtype).cuda()
        o.norm_add_norm(_dev(y)[:, :H], w1.cuda(), 1e-5, x2, w2.cuda(), 3e-6, xn)
        assert np.abs(x1.cpu().numpy() - new).max() <= 1e-5 * np.abs(new).max() and torch.equal(x1, x2)
        ref = plain.norm(new, w2.double().numpy(), 3e-6)
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert np.abs(xn.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations_of_the_feed_forwards(dtype):
    o = _ops(dtype)
    rng = np.random.default_rng(0)
    T, n = 37, 50
    z = rng.normal(0, 2.0, (T, 2 * n + 5)).astype(np.float32)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    out = torch.zeros((T, n), dtype=dtype).cuda()
    o.relu_squared(_dev(z)[:, 3:3 + n], out)
    ref = np.maximum(z[:, 3:3 + n].astype(np.float64), 0.0) ** 2
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    for limit in (0.5, 1.0, 7.0):
        o.clamped_glu(_dev(z)[:, 5:], limit, 1.702, out)
        g = np.minimum(z[:, 5:5 + n].astype(np.float64), limit)
        u = np.clip(z[:, 5 + n:].astype(np.float64), -limit, limit)
        ref = g * plain.sigmoid(1.702 * g) * (u + 1.0)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= max(tol, 2e-6) * np.abs(ref).max()
    for m, skip in ((n, 4), (n, 3), (52, 8), (256, 4)):        # rows that are and are not taken four entries at a time
        x = torch.as_tensor(rng.normal(0, 1.0, (T, m)), dtype=dtype)
        gate = rng.normal(0, 3.0, (T, m + skip)).astype(np.float32)
        xd = x.cuda()
        o.sigmoid_gate(xd, _dev(gate)[:, skip:])
        ref = x.double().numpy() * plain.sigmoid(gate[:, skip:].astype(np.float64))
        assert np.abs(xd.float().cpu().numpy() - ref).max() <= max(tol, 2e-6) * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,vdim", [(3, 7), (2, 24), (5, 128), (1, 132), (2, 512), (1, 260)])
def test_difference_of_maps_is_normed_per_head(dtype, H, vdim):
    """o = a1 - lambda a2, o / rms(o) * mult per head, for value sizes that are and are not taken four at a time;
    one head's maps nearly cancel (the norm then lifts what is left)."""
    o = _ops(dtype)
    rng = np.random.default_rng(H * vdim)
    T, lam, eps, mult = 19, 0.6, 1e-5, 0.7
    a = rng.normal(0, 1.0, (T, H, 2, vdim))
    a[3, 0, 0] = lam * a[3, 0, 1] + 1e-2 * rng.normal(0, 1.0, vdim)
    ad = torch.as_tensor(a, dtype=torch.float32).to(dtype)
    a64 = ad.double().numpy()
    d = a64[:, :, 0] - lam * a64[:, :, 1]
    ref = plain.rms_normalise(d, eps) * mult
    out = torch.zeros((T, H * vdim), dtype=dtype).cuda()
    o.diff_heads(ad.reshape(T, -1).cuda(), lam, eps, mult, out, H, vdim)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert np.abs(out.float().cpu().numpy().reshape(T, H, vdim) - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (8, 1408, 2048), (40, 384, 4096), (100, 512, 1024), (130, 640, 512),
                                   (200, 4096, 2048), (300, 1024, 256), (700, 1408, 1024), (2048, 2816, 1024)])
def test_products_apply_the_activations_in_their_epilogues(M, N, K):
    """The tensor-core product with the squared relu and with the clamped gate in its epilogue, on every
    one of its kernels (few tokens with and without a K split, single SMs, pairs), against 64-bit sums
    of the same bfloat16 inputs; limits that cut many of the values, and one that cuts none."""
    from torchless_rs_b200.csrc import ops
    from torchless_rs_b200.csrc.gemm_bf16 import GemmBf16
    gm = GemmBf16.get()
    rng = np.random.default_rng(M + N)
    a = torch.as_tensor(rng.normal(0, 1.0, (M, K)), dtype=torch.float32).bfloat16()
    w = torch.as_tensor(rng.normal(0, K ** -0.5, (2 * N, K)), dtype=torch.float32).bfloat16()
    z = a.double().numpy() @ w.double().numpy().T
    out = torch.zeros((M, N), dtype=torch.bfloat16).cuda()
    assert gm.run(a.cuda(), w[:N].cuda(), out, ops.MODE_STORE_ACT, act=(ops.ACT_RELU_SQUARED,))
    ref = np.maximum(z[:, :N], 0.0) ** 2
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 1e-2 * np.abs(ref).max()
    assert gm.run(a.cuda(), w[:N].cuda(), out, ops.MODE_STORE_ACT)            # and the plain mode is what it was
    assert np.abs(out.float().cpu().numpy() - z[:, :N]).max() <= 1e-2 * np.abs(z).max()
    for limit in (0.4, 1.0, 50.0):
        assert gm.run(a.cuda(), w.cuda(), out, ops.MODE_SWIGLU, act=(ops.ACT_CLAMPED_GLU, limit, 1.702))
        g, u = np.minimum(z[:, :N], limit), np.clip(z[:, N:], -limit, limit)
        ref = g * plain.sigmoid(1.702 * g) * (u + 1.0)
        assert np.abs(out.float().cpu().numpy() - ref).max() <= 1e-2 * np.abs(ref).max(), limit
    assert gm.run(a.cuda(), w.cuda(), out, ops.MODE_SWIGLU)
    ref = z[:, :N] * plain.sigmoid(z[:, :N]) * z[:, N:]
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 1e-2 * np.abs(ref).max()
    assert gm.take_error() == 0


class _Step:
    """What the attention kernels read of a step: one sequence's tokens first..last."""

    def __init__(self, pages, first, last):
        self.n_seqs, self.is_decode, self.max_new = 1, False, last - first + 1
        self.seq_start, self.seq_len, self.seq_slot = _i32([0, last - first + 1]), _i32([last + 1]), _i32([pages.slot])


class _View:
    def __init__(self, pages):
        self.k_pages, self.v_pages, self.page_table = pages.k, pages.v, _i32(pages.table)


@pytest.mark.parametrize("H,G,dim,rot,window,cap", [(4, 2, 64, 32, 70, 8.0), (2, 1, 128, 64, 130, 30.0), (4, 4, 64, 64, None, 9.0),
                                                   (2, 2, 128, 128, 64, None), (8, 1, 64, 0, 1, 20.0)])
def test_tensor_memory_attention_takes_caps_and_windows(H, G, dim, rot, window, cap):
    """Prompt steps of at least 128 tokens on the kernels of the plain attention (keys as wide as values, 64
    or 128), with and without a cap: every row of a whole prompt and of a portion that continues a held
    sequence against the plain softmax.  One key scores 16 where the others score around 1.6 and has a value
    of its own, on and beside page borders: the rows up to `window - 1` after it return that value, the next
    one does not, and the cap (below 16) decides how much of it."""
    from torchless_rs_b200.csrc.attention_bf16 import AttentionBf16
    dtype, vdim = torch.bfloat16, dim
    o = _ops(dtype)
    fast = AttentionBf16.get(dim)
    rng = np.random.default_rng(dim + (window or 0))
    base, eps = 1e7, 1e-6
    n = 5 * 64 + 9
    mark = (rot - 2) if rot else 0
    scale = 16.0 / (3.0 / np.sqrt((9.0 + (dim - 1) * 0.09) / dim) * np.sqrt(dim))
    pos_all = np.arange(n)
    for target in (63, 64, 3 * 64 - 1, 130):
        zq = rng.normal(0, 0.3, (n, H, dim))
        zk = rng.normal(0, 0.3, (n, G, dim))
        zv = rng.normal(0, 0.3, (n, G, vdim))
        zk[:, :, mark] = 0.0
        zk[target] = 0.0
        zk[target, :, mark] = 4.0
        zv[target, :, 0] = 50.0
        zq[:, :, mark] = 3.0
        z = _join(zq, zk, zv)
        pages = _Pages(dtype, n, G, dim, vdim)
        q = _write(o, pages, z, pos_all, rot, base, 1, True, eps, H, G, dim, vdim, 1, dtype)
        zq, zk, zv = _split(z.astype(np.float64), H, G, dim, vdim, 1)
        p64 = pos_all.astype(np.float64)
        qr = plain.rms_normalise(plain.rotate(zq, p64, rot, base, True), eps)
        kr = plain.rms_normalise(plain.rotate(zk, p64, rot, base, True), eps)
        vis = plain.visible(p64, window)
        ref = np.zeros((n, H, vdim))
        for h in range(H):
            g = h // (H // G)
            s = (qr[:, h] @ kr[:, g].T) * scale
            if cap:
                s = cap * np.tanh(s / cap)
            ref[:, h] = plain.softmax_rows(s, vis) @ zv[:, g]
        last_seen = n - 1 if window is None else min(n - 1, target + window - 1)
        assert (np.abs(ref[last_seen, :, 0]) > 5.0).all(), "the test's own mark does not stand out"
        if last_seen + 1 < n:
            assert (np.abs(ref[last_seen + 1, :, 0]) < 2.0).all(), "the mark is seen outside the window"
        for first, last in ((0, n - 1), (n - 200, n - 1), (target + 1, target + 128), (0, 127)):
            if last >= n:
                continue
            out = torch.zeros((last - first + 1, H * vdim), dtype=dtype).cuda()
            step, view = _Step(pages, first, last), _View(pages)
            qs = q[first:last + 1].contiguous()
            if cap:
                assert fast.run_capped(qs, view, out, step, H, G, window, scale, cap), "the kernel did not take the step"
            else:
                fast.prefill(qs, view.k_pages, view.v_pages, out, step.seq_start, step.seq_len, step.seq_slot,
                             view.page_table, 1, step.max_new, H, G, window, scale, variant="tc")
            got = out.float().cpu().numpy().reshape(-1, H, vdim)
            err = np.abs(got - ref[first:last + 1])
            assert err.max() <= 2.5e-2 * max(1.0, np.abs(ref).max()), \
                f"target {target} rows {first}..{last}: {err.max():.3e} at row {first + int(err.max(axis=(1, 2)).argmax())}"
        assert fast.take_error() == 0
