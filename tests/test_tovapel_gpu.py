"""The Tovapel decoder in the engine against the plain implementation: whole prompts, prefill
against token-by-token decoding, portions down to two tokens, unequal batches, slots, pages and
state used again, long decoding, greedy generation through the entry point, the replay program and
the command line; then each mechanism's kernels alone on inputs made so that a wrong window edge, a
missed far or kept key, a sink left out, a lost state or a wrong expert shows."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers_gpu import assert_close as _assert_close_32
from plain import tovapel_plain as plain
from tovapel_tiny import CONFIGS, DECAY_RANKS, TModel, make_weights, tokens_of, write_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOTH = [(c, d) for c in ("P", "Q", "R") for d in ("float32", "bfloat16")]


def assert_close(got, ref, dtype, what=""):
    """32-bit: the package's stated bound (5e-5 + 1e-4 |ref| per logit).  bfloat16: this design rounds an
    activation to 8 bits at some twenty places per layer (two branches, two norms on each, gates, experts), and a
    row whose softmax or router is sharp turns that into a few percent of its logits; measured on these
    configurations the error over all rows is 0.7 to 1 % of the logits' root mean square and the worst row's
    largest error 1.5 to 4.5 % of the largest logit.  The bound is 2 % over all rows and 10 % for any one
    logit: what a mechanism's fault does to the 32-bit run (bound 1e-4) and to the kernels alone (bound
    2e-2 on inputs that stand out) is tested there."""
    if dtype == "float32":
        return _assert_close_32(got, ref, dtype, what)
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    err = got - ref
    rms = float(np.sqrt((err ** 2).mean()) / np.sqrt((ref ** 2).mean()))
    worst = float(np.abs(err).max() / np.abs(ref).max())
    assert rms <= 2e-2 and worst <= 1e-1, f"{what}: rms error {rms:.3e} of the logits' rms, worst logit {worst:.3e}"


def _feed(tm, slot, toks, cuts):
    """Feeds `toks` to one sequence in pieces of the sizes `cuts` (the rest one by one) and
    returns the logits of every position."""
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
    toks = tokens_of(rng, 150, tm.cfg["vocab"])
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
        # the bfloat16 bound is one over all rows (a request of one token is one row: at a sequence's first
        # token the recurrence's output is sign(q . k) v / rms(v), which rounding can move a lot)
        assert_close(np.concatenate([np.concatenate(g) for g in got]), np.concatenate([tm.reference(r) for r in reqs]),
                     dtype, f"{name} all requests of the batch")
    assert tm.engine.cache.slots.held_count == 0
    tm.engine.cache.check()


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("R", "bfloat16"), ("Q", "float32")])
def test_slots_pages_and_state_are_clean_when_used_again(name, dtype):
    """A cache that holds one request at a time: every request gets the slot, the pages (also those of
    the kept first keys) and the recurrent state that the one before left behind."""
    tm = TModel(name, dtype, seed=8, max_tokens=192, max_batch=1)
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
    """400 tokens one by one: the recurrent state and the windows run far past every edge while the kept
    first keys stay, and the decode steps are replayed from recorded graphs."""
    tm = TModel(name, "float32", seed=13)
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


@pytest.mark.parametrize("name", ["P", "Q"])
def test_layers_one_by_one(name):
    """The sum of the streams after every layer (32-bit), so that a wrong layer is named."""
    tm = TModel(name, "float32", seed=6)
    toks = tokens_of(np.random.default_rng(1), 45, tm.cfg["vocab"])
    seen = []
    for b in tm.engine.model.blocks:
        def wrap(xs, batch, carry=None, next_norm=None, next_block=None, f=b.forward):
            r = f(xs, batch, carry, next_norm, next_block=next_block)
            seen.append(xs.sum(dim=1).cpu().numpy().copy())
            return r
        b.forward = wrap
    s = tm.engine.start_sequences(1)
    tm.step_np(s, [toks], "last")
    _, ref = plain.forward(tm.cfg, tm.weights, toks, return_layers=True)
    for i, (a, r) in enumerate(zip(seen, ref)):
        # 32-bit sums of some hundred terms, two norms per branch: a few 1e-5 of the largest entry
        assert np.abs(a - r).max() <= 1e-4 * max(1.0, np.abs(r).max()), f"layer {i}: {np.abs(a - r).max():.3e}"


def test_a_folder_may_hold_the_unused_tensors_of_a_layer_without_feed_forward():
    cfg = CONFIGS["P"]
    stored = make_weights(cfg, 4, torch.float32, DECAY_RANKS["P"])
    W, S = cfg["width"], cfg["streams"]
    stored.update({"l2.norm2": torch.zeros(W), "l2.hc2.in": torch.ones(S), "l2.hc2.out": torch.ones(S),
                   "l2.hc2.mix": torch.eye(S)})
    tm = TModel(cfg, "float32", weights=stored)
    toks = tokens_of(np.random.default_rng(0), 30, cfg["vocab"])
    s = tm.engine.start_sequences(1)
    assert_close(tm.step_np(s, [toks], "all"), tm.reference(toks), "float32", "unused tensors present")


def test_a_single_stream_may_come_without_its_connections():
    """One stream whose folder stores no connections is the plain pre-norm block: the same logits as with
    stored connections that are all one."""
    cfg = CONFIGS["Q"]
    stored = make_weights(cfg, 9, torch.float32, DECAY_RANKS["Q"])
    ones = {k: torch.ones_like(v) for k, v in stored.items() if ".hc" in k}
    toks = tokens_of(np.random.default_rng(0), 40, cfg["vocab"])
    with_ones = TModel(cfg, "float32", weights={**stored, **ones})
    s = with_ones.engine.start_sequences(1)
    ref = with_ones.step_np(s, [toks], "all")
    assert_close(ref, with_ones.reference(toks), "float32", "connections of ones")
    bare = {k: v for k, v in stored.items() if ".hc" not in k}
    import shutil
    import torchless_rs_b200 as tl
    d = write_folder(cfg, bare)
    try:
        model = tl.load(d, dtype="float32", max_tokens=256)
    finally:
        shutil.rmtree(d, ignore_errors=True)
    s = model.engine.start_sequences(1)
    got = model.engine.step(s, [toks], "all").float().cpu().numpy()
    assert np.array_equal(got, ref)


def test_replay_program_and_command_line(tmp_path):
    from test_trace_run_gpu import collect, run_trace
    cfg = CONFIGS["P"]
    stored = make_weights(cfg, 33, torch.float32, DECAY_RANKS["P"])
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


def _attend(dtype, q, pos, seq, slots, table, k_store, v_store, gate, sink, H, G, dim, vdim, window, keep, scale, cap):
    """The package's attention on made pages: the kernel the mixer would take for this step."""
    from torchless_rs_b200.parts.sink_attention import run_attention
    T = len(pos)
    out = torch.zeros((T, H * vdim), dtype=dtype).cuda()
    run_attention(_ops(dtype), _dev(q, dtype), k_store, v_store, _dev(gate) if gate is not None else None,
                  _dev(sink) if sink is not None else None, out, _i32(pos), _i32(seq), _i32(slots), _i32(table),
                  H, G, dim, vdim, window, keep, scale, cap)
    return out.float().cpu().numpy().reshape(T, H, vdim)


def _plain_attend(q, kk, vv, visible, sink, gate, scale, cap):
    """One query [H, dim] over keys kk [n, G, dim], values vv [n, G, vdim] with a visibility row [n]."""
    H, G = q.shape[0], kk.shape[1]
    out = np.zeros((H, vv.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (kk[:, g] @ q[h]) * scale
        if cap:
            s = cap * np.tanh(s / cap)
        p = plain.sink_softmax(s[None], visible[None], sink[h] if sink is not None else -np.inf)[0]
        out[h] = (p @ vv[:, g]) * (plain.sigmoid(gate[h]) if gate is not None else 1.0)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dim,vdim,window,keep", [(3, 1, 16, 24, 70, 3), (2, 2, 40, 12, 64, 0), (4, 2, 64, 64, 130, 5),
                                                      (8, 2, 32, 64, 64, 70), (2, 1, 128, 128, 100, 1), (4, 4, 64, 32, 20, 66)])
def test_attention_sees_exactly_its_window_and_the_kept_first_keys(dtype, H, G, dim, vdim, window, keep):
    """One key carries a score far above all others and a value that no other key has.  A query
    `window - 1` positions after it must return that value, a query `window` positions after it must
    not, unless the key is one of the kept first ones: the last kept key is seen from everywhere, the
    key after it is not.  The key also lies on page borders and hundreds of keys back among
    look-alikes.  Called with one position (a decode step), a few, and a long run (a prompt)."""
    from torchless_rs_b200.cache import PAGE
    rng = np.random.default_rng(dim + window)
    n = 5 * PAGE + 9
    pages_of = [7, 2, 9, 4, 0, 5]                      # the sequence's pages, out of order
    slot = 3
    table = np.full((5, 8), -1, dtype=np.int32)
    table[slot, :len(pages_of)] = pages_of
    scale, cap = 0.5, 40.0
    targets = [t for t in (PAGE - 1, PAGE, 3 * PAGE - 1, 200, keep - 1, keep) if 0 <= t < n]
    for target in targets:
        k = rng.normal(0, 0.3, (n, G, dim))
        v = rng.normal(0, 0.3, (n, G, vdim))
        k[target] = 0.0
        k[target, :, 0] = 9.0                           # a mark in coordinate 0 only
        v[target, :, 0] = 50.0
        ks = torch.zeros((10, G, PAGE, dim), dtype=dtype)
        vs = torch.zeros((10, G, vdim, PAGE), dtype=dtype)
        for p in range(n):
            ks[pages_of[p // PAGE], :, p % PAGE] = torch.as_tensor(k[p], dtype=dtype)
            vs[pages_of[p // PAGE], :, :, p % PAGE] = torch.as_tensor(v[p], dtype=dtype)
        kk = np.stack([ks[pages_of[p // PAGE], :, p % PAGE].float().numpy() for p in range(n)]).astype(np.float64)
        vv = np.stack([vs[pages_of[p // PAGE], :, :, p % PAGE].float().numpy() for p in range(n)]).astype(np.float64)
        ks, vs = ks.cuda(), vs.cuda()
        for qpos in sorted({target, target + window - 1, target + window, n - 1}):
            if qpos >= n:
                continue
            q = rng.normal(0, 0.3, (H, dim))
            q[:, 0] = 6.0                               # times the mark: a score of 27 above the rest
            q = torch.as_tensor(q, dtype=dtype).double().numpy()
            sink = rng.normal(0, 1.0, H)
            gate = rng.normal(0, 1.0, H)
            j = np.arange(n)
            vis = (j <= qpos) & ((qpos - j < window) | (j < keep))
            ref = _plain_attend(q, kk, vv, vis, sink, gate, scale, cap)
            sees = bool(vis[target])
            assert sees == (target <= qpos and (qpos - target < window or target < keep))
            strong = np.abs(ref[:, 0]) > 5.0 * plain.sigmoid(gate)
            assert strong.all() == sees and (sees or not strong.any())
            for form in ("decode", "few", "prompt"):
                first = {"decode": qpos, "few": max(0, qpos - 5), "prompt": max(0, qpos - 309)}[form]
                pos = list(range(first, qpos + 1))
                T = len(pos)
                q_t = np.zeros((T, H * dim)); q_t[-1] = q.reshape(-1)
                g_t = np.zeros((T, H)); g_t[-1] = gate
                got = _attend(dtype, q_t, pos, [0] * T, [slot], table, ks, vs, g_t, sink, H, G, dim, vdim, window,
                              keep, scale, cap)[-1]
                tol = 2e-5 if dtype == torch.float32 else 2e-2
                assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max()), \
                    f"target {target} query {qpos} ({form}): {np.abs(got - ref).max():.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,keep,cap", [(None, 0, None), (130, 4, 25.0), (64, 0, 8.0)])
def test_attention_of_a_long_packed_step(dtype, window, keep, cap):
    """A step of 1300 tokens of two sequences that each continue a sequence which already holds keys, the
    border between them inside a tile of the tensor-core kernel; rows against numpy on the values that the
    pages hold.  With and without window, kept keys and cap; the sink and the gate always."""
    from torchless_rs_b200.cache import PAGE
    H, G, dim, vdim = 4, 2, 64, 32
    rng = np.random.default_rng(7)
    past, new = [70, 5], [701, 599]
    n_pages = sum((p + n + PAGE - 1) // PAGE for p, n in zip(past, new))
    order = rng.permutation(n_pages + 3)
    table = np.full((4, 16), -1, dtype=np.int32)
    slots, at = [2, 0], 0
    for s, p, n in zip(slots, past, new):
        c = (p + n + PAGE - 1) // PAGE
        table[s, :c] = order[at:at + c]
        at += c
    ks = torch.as_tensor(rng.normal(0, 0.5, (n_pages + 3, G, PAGE, dim)), dtype=dtype)
    vs = torch.as_tensor(rng.normal(0, 0.5, (n_pages + 3, G, vdim, PAGE)), dtype=dtype)
    kk, vv = ks.double().numpy(), vs.double().numpy()
    T = sum(new)
    q = torch.as_tensor(rng.normal(0, 0.6, (T, H * dim)), dtype=dtype).double().numpy()
    gate, sink = rng.normal(0, 1.0, (T, H)), rng.normal(0, 1.0, H)
    pos = np.concatenate([np.arange(p, p + n) for p, n in zip(past, new)])
    seq = np.concatenate([np.full(n, i) for i, n in enumerate(new)])
    got = _attend(dtype, q, pos, seq, slots, table, ks.cuda(), vs.cuda(), gate, sink, H, G, dim, vdim, window, keep,
                  0.25, cap)
    worst = 0.0
    for t in list(range(0, T, 37)) + [699, 700, 701, 702, 703, T - 1]:
        s, p = slots[seq[t]], int(pos[t])
        j = np.arange(p + 1)
        vis = ((p - j < window) | (j < keep)) if window else np.ones(p + 1, bool)
        keys = np.stack([kk[table[s, i // PAGE], :, i % PAGE] for i in j])
        vals = np.stack([vv[table[s, i // PAGE], :, :, i % PAGE] for i in j])
        ref = _plain_attend(q[t].reshape(H, dim), keys, vals, vis, sink, gate[t], 0.25, cap)
        worst = max(worst, np.abs(got[t] - ref).max() / np.abs(ref).max())
    assert worst <= (2e-5 if dtype == torch.float32 else 2e-2), f"{worst:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_projections_are_biased_normed_and_written_to_their_pages(dtype):
    from torchless_rs_b200.cache import PAGE
    o = _ops(dtype)
    rng = np.random.default_rng(3)
    H, G, dim, vdim, T = 3, 1, 20, 7, 70
    cols = (H + G) * dim + G * vdim
    z = rng.normal(0, 1.0, (T, cols + H)).astype(np.float32)        # the gate's columns follow and stay untouched
    bias, qw, kw = rng.normal(0, 0.5, cols), rng.normal(1, 0.2, dim), rng.normal(1, 0.2, dim)
    pos = np.arange(60, 60 + T)                                     # crosses a page border
    table = np.array([[5, 1, 3]], dtype=np.int32)
    kp = torch.zeros((6, G, PAGE, dim), dtype=dtype).cuda()
    vp = torch.zeros((6, G, vdim, PAGE), dtype=dtype).cuda()
    q = torch.zeros((T, H * dim), dtype=dtype).cuda()
    o.qk_norm_cache_write(_dev(z), _dev(bias), _dev(qw), _dev(kw), 1e-5, q, kp, vp, _i32(pos), _i32([0] * T), _i32([0]),
                          _i32(table), H, G, dim, vdim)
    zb = z[:, :cols].astype(np.float64) + bias.astype(np.float32)
    qr = (plain.rms_normalise(zb[:, :H * dim].reshape(T, H, dim), 1e-5) * qw.astype(np.float32)).reshape(T, -1)
    kr = plain.rms_normalise(zb[:, H * dim:(H + G) * dim].reshape(T, G, dim), 1e-5) * kw.astype(np.float32)
    vr = zb[:, (H + G) * dim:].reshape(T, G, vdim)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert np.abs(q.float().cpu().numpy() - qr).max() <= tol * np.abs(qr).max()
    kg, vg = kp.float().cpu().numpy(), vp.float().cpu().numpy()
    for t, p in enumerate(pos):
        page = table[0, p // PAGE]
        assert np.abs(kg[page, :, p % PAGE] - kr[t]).max() <= tol * np.abs(kr).max()
        assert np.abs(vg[page, :, :, p % PAGE] - vr[t]).max() <= tol * np.abs(vr).max()
    assert float(kp[[0, 2, 4]].abs().sum()) == 0.0 and float(vp[[0, 2, 4]].abs().sum()) == 0.0


@pytest.mark.parametrize("heads,dim,vdim,tau", [(2, 16, 8, 8.0), (1, 40, 20, 1.0), (3, 70, 33, 16.0), (2, 128, 64, 4.0),
                                                (1, 256, 12, 2.0)])
def test_linear_attention_carries_its_state(heads, dim, vdim, tau):
    """The recurrence over a batch of two sequences, whole and in pieces down to one token, from the state
    that the piece before left in the sequence's slot; a zeroed slot starts a new sequence; other slots
    stay untouched.  Decays close to one, so that the first tokens still count at the end."""
    o = _ops(torch.float32)
    rng = np.random.default_rng(dim)
    lens = [300, 47]
    T, hd, hv = sum(lens), heads * dim, heads * vdim
    z = rng.normal(0, 1.0, (T, 2 * hd + 2 * hv)).astype(np.float32)
    za = rng.normal(2.0, 1.5, (T, hd)).astype(np.float32)
    bias = rng.normal(1.0, 1.0, hd).astype(np.float32)
    q_scale = dim ** -0.5
    refs, at = [], 0
    for n in lens:
        S = np.zeros((heads, dim, vdim))
        out = np.zeros((n, heads, vdim))
        for t in range(n):
            row = z[at + t].astype(np.float64)
            a = plain.sigmoid(za[at + t].astype(np.float64) + bias) ** (1.0 / tau)
            S = a.reshape(heads, dim, 1) * S + row[hd:2 * hd].reshape(heads, dim, 1) * \
                row[2 * hd:2 * hd + hv].reshape(heads, 1, vdim)
            out[t] = np.einsum("hdv,hd->hv", S, row[:hd].reshape(heads, dim) * q_scale)
        refs.append((out.reshape(n, hv), S))
        at += n
    ref = np.concatenate([r[0] for r in refs])
    slots = [4, 1]
    for cuts in ([300], [1] * 5 + [2, 100, 7, 64], [256, 44]):
        state = torch.full((6, heads, dim, vdim), 7.0).cuda()
        state[slots] = 0.0
        got = np.zeros((T, hv), dtype=np.float32)
        fed = [0, 0]
        for c in cuts + [10 ** 6]:
            take = [min(c, lens[i] - fed[i]) for i in (0, 1)]
            rows = [i for i in (0, 1) if take[i] > 0]
            if not rows:
                break
            idx = np.concatenate([np.arange(sum(lens[:i]) + fed[i], sum(lens[:i]) + fed[i] + take[i]) for i in rows])
            zz = _dev(z[idx])
            hd2 = 2 * hd
            out = torch.zeros((len(idx), hv)).cuda()
            start = np.concatenate([[0], np.cumsum([take[i] for i in rows])])
            o.gla_scan(zz[:, :hd], zz[:, hd:hd2], zz[:, hd2:hd2 + hv], _dev(za[idx]), _dev(bias), tau, q_scale, state,
                       out, _i32(start), _i32([slots[i] for i in rows]), heads, dim, vdim)
            got[idx] = out.cpu().numpy()
            for i in rows:
                fed[i] += take[i]
        scale = np.abs(ref).max()
        assert np.abs(got - ref).max() <= 3e-5 * scale, f"cuts {cuts}: {np.abs(got - ref).max() / scale:.3e}"
        st = state.cpu().numpy()
        for i in (0, 1):
            assert np.abs(st[slots[i]] - refs[i][1]).max() <= 3e-5 * np.abs(refs[i][1]).max()
        assert (st[[0, 2, 3, 5]] == 7.0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,vdim", [(2, 8), (3, 33), (1, 128)])
def test_head_norm_with_gate(dtype, H, vdim):
    o = _ops(dtype)
    rng = np.random.default_rng(vdim)
    T = 19
    x = rng.normal(0, 2.0, (T, H * vdim)).astype(np.float32)
    g = rng.normal(0, 2.0, (T, H * vdim + 5)).astype(np.float32)
    w = rng.normal(1, 0.3, vdim).astype(np.float32)
    out = torch.zeros((T, H * vdim), dtype=dtype).cuda()
    o.headnorm_silu_gate(_dev(x), _dev(w), 1e-5, _dev(g)[:, 5:], out, H, vdim)
    ref = (plain.rms_normalise(x.astype(np.float64).reshape(T, H, vdim), 1e-5) * w).reshape(T, -1) * \
        plain.silu(g[:, 5:].astype(np.float64))
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,H", [(1, 40), (3, 96), (4, 320), (8, 72), (2, 4100), (7, 64)])
def test_streams_are_read_written_and_summed(dtype, S, H):
    o = _ops(dtype)
    rng = np.random.default_rng(S * H)
    T = 33
    x0 = rng.normal(0, 1.0, (T, H)).astype(np.float32)
    xs = torch.zeros((T, S, H)).cuda()
    o.stream_spread(_dev(x0), xs)
    assert (xs.cpu().numpy() == x0[:, None, :]).all()
    X = rng.normal(0, 1.0, (T, S, H)).astype(np.float32)
    a, a2, b = (rng.normal(0.5, 0.5, S).astype(np.float32) for _ in range(3))
    M = rng.normal(0.3, 0.5, (S, S)).astype(np.float32)
    w, w2 = (rng.normal(1.0, 0.2, H).astype(np.float32) for _ in range(2))
    y = rng.normal(0, 1.0, (T, H)).astype(np.float32)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    out = torch.zeros((T, H), dtype=dtype).cuda()
    o.hc_read_norm(_dev(X), _dev(a), _dev(w), 1e-5, out)
    X64 = X.astype(np.float64)
    ref = plain.rms_normalise(np.einsum("s,tsd->td", a.astype(np.float64), X64), 1e-5) * w
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()
    # writing, alone and together with the next read, gives the same streams
    new = np.einsum("sj,tsd->tjd", M.astype(np.float64), X64) + b.astype(np.float64)[None, :, None] * y[:, None, :]
    x1, x2 = _dev(X), _dev(X)
    o.hc_write(x1, _dev(M), _dev(b), _dev(y))
    out2 = torch.zeros((T, H), dtype=dtype).cuda()
    o.hc_write(x2, _dev(M), _dev(b), _dev(y), next_read=(_dev(a2), _dev(w2), 1e-5, out2))
    assert np.abs(x1.cpu().numpy() - new).max() <= 1e-5 * np.abs(new).max() and torch.equal(x1, x2)
    ref2 = plain.rms_normalise(np.einsum("s,tsd->td", a2.astype(np.float64), new), 1e-5) * w2
    assert np.abs(out2.float().cpu().numpy() - ref2).max() <= tol * np.abs(ref2).max()
    rows = [5, 0, 32]
    sm = torch.zeros((3, H)).cuda()
    o.stream_sum(x1, sm, _i32(rows))
    assert np.abs(sm.cpu().numpy() - new[rows].sum(1)).max() <= 1e-5 * np.abs(new).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_branches_are_normed_and_averaged(dtype):
    o = _ops(dtype)
    rng = np.random.default_rng(0)
    T, H = 21, 100
    ys = [rng.normal(0, s, (T, H)).astype(np.float32) for s in (0.1, 30.0, 1.0)]
    ws = [rng.normal(1, 0.3, H).astype(np.float32) for _ in ys]
    for n in (1, 2, 3):
        ref = sum(plain.rms_normalise(y.astype(np.float64), 1e-6) * w for y, w in zip(ys[:n], ws[:n])) / n
        out = torch.full((T, H), 2.0).cuda()
        o.branch_norm_mean([_dev(y) for y in ys[:n]], [_dev(w) for w in ws[:n]], 1e-6, out, accumulate=False)
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
        o.branch_norm_mean([_dev(y) for y in ys[:n]], [_dev(w) for w in ws[:n]], 1e-6, out, accumulate=True)
        assert np.abs(out.cpu().numpy() - 2 * ref).max() <= 2e-5 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,f,E,I,top,T", [(96, 24, 5, 2, 3, 70), (80, 40, 3, 0, 1, 9), (64, 16, 3, 1, 4, 150),
                                           (128, 64, 40, 3, 6, 300), (64, 32, 2, 30, 2, 64)])
def test_experts_are_chosen_weighted_and_summed(dtype, W, f, E, I, top, T):
    """The feed-forward part alone against the plain one on the same (already rounded) input.  Tokens
    whose choice hangs on a gap below what the rounding of the router's product can move are left out
    of the comparison (tokens do not influence one another here)."""
    from torchless_rs_b200.config.spec import PartSpec
    from torchless_rs_b200.parts import Runtime, lookup
    rt = Runtime("cuda:0", torch.float32 if dtype == "float32" else torch.bfloat16)
    store = rt.act_dtype
    rng = np.random.default_rng(W + E)
    spec = PartSpec("moe_clamped", {"hidden_size": W, "ff": f, "experts": E, "identity": I, "top": top, "limit": 0.7})
    names = lookup("feed_forward", "moe_clamped").expected_tensors(spec, "m")
    w = {}
    for n, ts in names.items():
        std = 0.1 if n.endswith("correction") else (2.0 if n.endswith("router") else 1.0) / np.sqrt(ts.shape[-1])
        w[n] = torch.as_tensor(rng.normal(0, std, ts.shape), dtype=torch.float32).to(store)
    part = lookup("feed_forward", "moe_clamped")(spec, "m", rt)
    part.load(w)
    h = torch.as_tensor(rng.normal(0, 1.0, (T, W)), dtype=torch.float32).to(store)
    w64 = {k[2:]: v.double().numpy() for k, v in w.items()}
    h64 = h.double().numpy()
    p = {"router": {"experts": E, "identity": I, "top": top}, "expert": {"ff": f, "limit": 0.7}}
    ref = plain.moe_ff(h64, w64, p)
    z = h64 @ w64["router"].T
    s = np.exp(z - z.max(-1, keepdims=True)); s /= s.sum(-1, keepdims=True)
    c = np.sort(s + w64["correction"], axis=-1)[:, ::-1]
    gap = c[:, top - 1] - c[:, top] if top < E + I else np.full(T, 1.0)
    sure = gap > (1e-5 if dtype == "float32" else 2e-2)
    assert sure.sum() > T // 8
    out = torch.full((T, W), 3.0).cuda()
    part.forward(h.cuda(), out, None, overwrite=True)
    got = out.cpu().numpy()
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert np.abs(got - ref)[sure].max() <= tol * np.abs(ref).max(), f"{np.abs(got - ref)[sure].max():.3e}"
    part.forward(h.cuda(), out, None)                  # adds into what is there
    assert np.abs(out.cpu().numpy() - 2 * ref)[sure].max() <= 2 * tol * np.abs(ref).max()
