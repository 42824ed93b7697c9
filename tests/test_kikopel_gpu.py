"""The Kikopel decoder in the engine against the plain implementation: whole prompts, prefill
against token-by-token decoding, portions down to two tokens, unequal batches, slots and pages
used again, long decoding, greedy generation through the entry point, the replay program and the
command line; then each kernel alone on inputs made so that a wrong window edge, a missed far
key or a lost state shows."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers_gpu import assert_close
from kikopel_tiny import CONFIGS, KModel, make_weights, tokens_of, write_folder
from plain import kikopel_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOTH = [(c, d) for c in ("P", "Q", "R") for d in ("float32", "bfloat16")]


def _feed(km, slot, toks, cuts):
    """Feeds `toks` to one sequence in pieces of the sizes `cuts` (the rest one by one) and
    returns the logits of every position."""
    rows, at = [], 0
    for c in list(cuts) + [1] * len(toks):
        if at >= len(toks):
            break
        piece = toks[at:at + c]
        rows.append(km.step_np([slot], [piece], "all"))
        at += len(piece)
    return np.concatenate(rows)


@pytest.mark.parametrize("name,dtype", BOTH)
def test_whole_prompt_and_decoding_and_portions(name, dtype):
    km = KModel(name, dtype, seed=3)
    rng = np.random.default_rng(11)
    toks = tokens_of(rng, 150, km.cfg["vocab"])
    ref = km.reference(toks)
    for cuts, what in (([150], "whole"), ([40], "prefix, then one by one across windows and page borders"),
                       ([2, 3, 59, 2, 64, 1, 17, 2], "portions"), ([], "from the first token one by one"),
                       ([63, 2, 63, 2], "portions that end at and start on page borders")):
        s = km.engine.start_sequences(1)
        got = _feed(km, s[0], toks, cuts)
        km.engine.end_sequences(s)
        assert_close(got, ref, dtype, f"{name} {what}")
    km.engine.check_kernels()
    km.engine.cache.check()


@pytest.mark.parametrize("name,dtype", BOTH)
def test_unequal_batches_equal_each_request_alone(name, dtype):
    km = KModel(name, dtype, seed=5, max_tokens=1024)
    rng = np.random.default_rng(2)
    V = km.cfg["vocab"]
    lens, pre = [1, 37, 141, 66], [1, 20, 100, 64]
    reqs = [tokens_of(rng, n, V) for n in lens]
    slots = km.engine.start_sequences(4)
    out = km.step_np(slots, [r[:p] for r, p in zip(reqs, pre)], "all")
    got, at = [], 0
    for p in pre:
        got.append([out[at:at + p]])
        at += p
    fed, live = list(pre), [i for i in range(4) if pre[i] < lens[i]]
    km.engine.end_sequences([slots[i] for i in range(4) if pre[i] >= lens[i]])
    while live:
        out = km.step_np([slots[i] for i in live], [[reqs[i][fed[i]]] for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
            fed[i] += 1
        done = [i for i in live if fed[i] >= lens[i]]
        km.engine.end_sequences([slots[i] for i in done])      # shorter requests end earlier
        live = [i for i in live if i not in done]
    for i, r in enumerate(reqs):
        assert_close(np.concatenate(got[i]), km.reference(r), dtype, f"{name} request {i} of the batch")
    assert km.engine.cache.slots.held_count == 0
    km.engine.cache.check()


@pytest.mark.parametrize("name,dtype", [("P", "float32"), ("R", "bfloat16"), ("Q", "float32")])
def test_slots_pages_and_state_are_clean_when_used_again(name, dtype):
    """A cache that holds one request at a time: every request gets the slot, the pages, the
    recurrent state and the remembered token that the one before left behind."""
    km = KModel(name, dtype, seed=8, max_tokens=192, max_batch=1)
    rng = np.random.default_rng(9)
    for n, cuts in ((170, [100]), (130, [130]), (150, [3, 90]), (5, [])):
        toks = tokens_of(rng, n, km.cfg["vocab"])
        s = km.engine.start_sequences(1)
        assert s == [0]
        got = _feed(km, s[0], toks, cuts)
        km.engine.end_sequences(s)
        assert_close(got, km.reference(toks), dtype, f"{name} request of {n} tokens in a used slot")
        km.engine.cache.check()
    # reset: the same slot starts again without being given back
    toks = tokens_of(rng, 90, km.cfg["vocab"])
    s = km.engine.start_sequences(1)
    _feed(km, s[0], tokens_of(rng, 70, km.cfg["vocab"]), [70])
    km.engine.reset(s[0])
    assert_close(_feed(km, s[0], toks, [50]), km.reference(toks), dtype, f"{name} after reset")
    km.engine.end_sequences(s)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding(name):
    """400 tokens one by one: the recurrent state and the windows run far past every edge, and the
    decode steps are replayed from recorded graphs."""
    km = KModel(name, "float32", seed=13)
    rng = np.random.default_rng(5)
    reqs = [tokens_of(rng, n, km.cfg["vocab"]) for n in (400, 333)]
    slots = km.engine.start_sequences(2)
    got = [[], []]
    for t in range(400):
        live = [i for i in (0, 1) if t < len(reqs[i])]
        out = km.step_np([slots[i] for i in live], [[reqs[i][t]] for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(out[j])
    km.engine.end_sequences(slots)
    for i in (0, 1):
        assert_close(np.stack(got[i]), km.reference(reqs[i]), "float32", f"{name} sequence {i}")


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_through_the_entry_point(name):
    km = KModel(name, "float32", seed=21, max_tokens=512)
    rng = np.random.default_rng(4)
    prompts = [tokens_of(rng, n, km.cfg["vocab"]) for n in (1, 19, 70)]
    res = km.model.generate(prompts, max_tokens=14, temperature=0.0, stop_ids=())
    for p, r in zip(prompts, res):
        seq, want = list(p), []
        for _ in range(14):
            want.append(int(np.argmax(km.reference(seq)[-1])))
            seq.append(want[-1])
        assert r.tokens == want, f"prompt of {len(p)} tokens"
    assert km.engine.steps_advanced_on_device > 0, "the decode steps were not fed from the device"
    assert km.engine.cache.slots.held_count == 0


def test_layers_one_by_one():
    """The stream after every layer (32-bit), so that a wrong layer is named."""
    km = KModel("P", "float32", seed=6)
    toks = tokens_of(np.random.default_rng(1), 45, km.cfg["vocab"])
    seen = []
    for b in km.engine.model.blocks:
        def wrap(x, batch, carry=None, next_norm=None, f=b.forward):
            r = f(x, batch, carry, next_norm)
            seen.append(x.detach().cpu().numpy().copy())
            return r
        b.forward = wrap
    s = km.engine.start_sequences(1)
    km.step_np(s, [toks], "last")
    _, ref = plain.forward(km.cfg, km.weights, toks, every_layer=True)
    for i, (a, r) in enumerate(zip(seen, ref)):
        assert np.abs(a - r).max() <= 2e-5 * max(1.0, np.abs(r).max()), f"layer {i}: {np.abs(a - r).max():.3e}"


def test_replay_program_and_command_line(tmp_path):
    from test_trace_run_gpu import collect, run_trace
    cfg = CONFIGS["P"]
    stored = make_weights(cfg, 33, torch.float32)
    w = {k: v.double().numpy() for k, v in stored.items()}
    d = write_folder(cfg, stored, str(tmp_path))
    rng = np.random.default_rng(3)
    reqs = {"a": tokens_of(rng, 70, cfg["vocab"]), "b": tokens_of(rng, 33, cfg["vocab"])}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:60], "want": list(range(60))},
                                     {"id": "b", "tokens": reqs["b"][:30], "want": [0, 29]}], "end": []}]
    for t in range(10):
        ent = [{"id": "a", "tokens": [reqs["a"][60 + t]], "want": [0]}]
        if t < 3:
            ent.append({"id": "b", "tokens": [reqs["b"][30 + t]], "want": [0]})
        steps.append({"step": t + 1, "entries": ent, "end": ["b"] if t == 2 else (["a"] if t == 9 else [])})
    # config.json of this design has `vocab`, which the shared helper reads under another name
    cj = json.load(open(os.path.join(d, "config.json")))
    json.dump({**cj, "vocab_size": cj["vocab"]}, open(os.path.join(d, "config.json"), "w"))
    got = collect(steps, run_trace(d, "float32", 256, steps))
    for rid, toks in reqs.items():
        ref = plain.forward_logits(cfg, w, toks)
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
            assert int(tok) == int(np.argmax(plain.forward_logits(cfg, w, seq)[-1]))
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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot,dims,heads,window", [(24, 8, 8, 3, 70), (40, 12, 4, 1, 64), (16, 0, 0, 2, 130),
                                                        (32, 16, 16, 3, 70), (96, 32, 8, 16, 64), (144, 16, 16, 20, 130),
                                                        (512, 64, 64, 5, 100)])
def test_latent_attention_sees_exactly_its_window(dtype, rank, rot, dims, heads, window):
    """One key carries a score far above all others and a value that no other key has.  A query
    `window - 1` positions after it must return that value, a query `window` positions after it
    must not; the key also lies on a page border, hundreds of keys back among look-alikes.  The
    same kernel is called with all positions at once (a prompt) and with one (a decode step)."""
    from torchless_rs_b200.cache import PAGE
    o = _ops(dtype)
    rng = np.random.default_rng(rank)
    n = 5 * PAGE + 9
    width = rank + rot
    keys = rng.normal(0, 0.3, (n, width))
    pages_of = [7, 2, 9, 4, 0, 5]                      # the sequence's pages, out of order
    slot = 3
    table = np.full((5, 8), -1, dtype=np.int32)
    table[slot, :len(pages_of)] = pages_of
    inv_freq = np.array([10000.0 ** (-2.0 * i / dims) for i in range(dims // 2)]) if dims else None
    for target in (PAGE - 1, PAGE, 3 * PAGE - 1, 200):
        k = keys.copy()
        k[target, :rank] = 0.0
        k[target, 0] = 9.0                                 # its c: a mark in coordinate 0 only
        store = torch.zeros((10, PAGE, width), dtype=dtype)
        rotated = k.copy()
        if rot:
            rotated[:, rank:] = plain.rotate(k[:, rank:], np.arange(n), 10000.0, dims) if dims else k[:, rank:]
        for p in range(n):
            store[pages_of[p // PAGE], p % PAGE] = torch.as_tensor(rotated[p], dtype=dtype)
        kept = store.float().numpy()
        store = store.cuda()
        for qpos in (target, target + window - 1, target + window, n - 1):
            if qpos >= n:
                continue
            qa = rng.normal(0, 0.3, (heads, rank))
            qa[:, 0] = 6.0                                 # times the mark: a score of 54 * scale above the rest
            qr = rng.normal(0, 0.3, (heads, rot))
            lo = max(0, qpos - window + 1)
            # the plain result from the values as the cache holds them
            kk = np.stack([kept[pages_of[p // PAGE], p % PAGE] for p in range(lo, qpos + 1)]).astype(np.float64)
            qrot = plain.rotate(qr[None], [qpos], 10000.0, dims)[0] if dims else qr
            s = (qa @ kk[:, :rank].T + qrot @ kk[:, rank:].T) * 0.5
            w = np.exp(s - s.max(-1, keepdims=True))
            ref = (w / w.sum(-1, keepdims=True)) @ kk[:, :rank]
            sees = lo <= target <= qpos
            assert (ref[:, 0] > 8.0).all() == sees and (sees or (np.abs(ref[:, 0]) < 2.0).all())
            for form in ("decode", "prompt", "long prompt"):
                if form == "long prompt" and qpos < 310:
                    continue          # (more than 296 tokens: the tensor-core kernel then does not cut the keys)
                pos = [qpos] if form == "decode" else list(range(max(0, qpos - (5 if form == "prompt" else 309)), qpos + 1))
                T = len(pos)
                qa_t = np.zeros((T, heads, rank)); qa_t[-1] = qa
                q_t = np.zeros((T, heads * (3 + rot))); q_t[-1] = np.concatenate(
                    [np.concatenate([np.zeros(3), qr[h]]) for h in range(heads)])
                out = torch.zeros((T, heads, rank), dtype=torch.float32).cuda()
                o.latent_attn(_dev(qa_t.reshape(T, heads * rank)), rank, _dev(q_t), 3 + rot, 3, store, out, _i32(pos), _i32([0] * T), _i32([slot]),
                              _i32(table), _dev(inv_freq) if dims else None, heads, rank, rot, dims, window, 0.5)
                got = out[-1].cpu().numpy()
                tol = 2e-5 if dtype == torch.float32 else 2e-2
                assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max()), \
                    f"target {target} query {qpos} ({form}): {np.abs(got - ref).max():.3e}"


@pytest.mark.parametrize("window", [None, 130])
@pytest.mark.parametrize("heads,rank,rot", [(16, 64, 32), (5, 512, 64), (20, 128, 16)])
def test_latent_attention_of_a_long_packed_step(window, heads, rank, rot):
    """A step of 1300 tokens of two sequences whose border falls inside a block of the tensor-core
    kernel (the tokens of a block share their key chunks), each continuing a sequence that already
    holds keys; every row against numpy on the values that the pages hold."""
    from torchless_rs_b200.cache import PAGE
    o = _ops(torch.bfloat16)
    rng = np.random.default_rng(rank + heads)
    width = rank + rot
    past, new = [70, 5], [701, 599]
    n_pages = sum((p + n + PAGE - 1) // PAGE for p, n in zip(past, new))
    order = rng.permutation(n_pages + 3)
    table = np.full((4, 16), -1, dtype=np.int32)
    slots, at = [2, 0], 0
    for s, p, n in zip(slots, past, new):
        k = (p + n + PAGE - 1) // PAGE
        table[s, :k] = order[at:at + k]
        at += k
    store = torch.as_tensor(rng.normal(0, 0.5, (n_pages + 3, PAGE, width)), dtype=torch.bfloat16)
    kept = store.float().numpy().astype(np.float64)
    T = sum(new)
    q = rng.normal(0, 0.6, (T, heads * width))
    inv_freq = np.array([10000.0 ** (-2.0 * i / rot) for i in range(rot // 2)])
    pos = np.concatenate([np.arange(p, p + n) for p, n in zip(past, new)])
    seq = np.concatenate([np.full(n, i) for i, n in enumerate(new)])
    out = torch.zeros((T, heads, rank), dtype=torch.float32).cuda()
    qd = _dev(q)
    o.latent_attn(qd, width, qd, width, rank, store.cuda(), out, _i32(pos), _i32(seq), _i32(slots), _i32(table),
                  _dev(inv_freq), heads, rank, rot, rot, window, 0.25)
    got = out.cpu().numpy()
    q32 = q.astype(np.float32).astype(np.float64).reshape(T, heads, width)
    worst = 0.0
    for t in list(range(0, T, 37)) + [699, 700, 701, 702, 703, T - 1]:
        s, p = slots[seq[t]], int(pos[t])
        lo = max(0, p - window + 1) if window else 0
        kk = np.stack([kept[table[s, i // PAGE], i % PAGE] for i in range(lo, p + 1)])
        qq = np.concatenate([q32[t, :, :rank], plain.rotate(q32[t:t + 1, :, rank:], [p], 10000.0, rot)[0]], axis=-1)
        sc = (qq @ kk.T) * 0.25
        w = np.exp(sc - sc.max(-1, keepdims=True))
        ref = (w / w.sum(-1, keepdims=True)) @ kk[:, :rank]
        worst = max(worst, np.abs(got[t] - ref).max() / np.abs(ref).max())
    assert worst <= 2e-2, f"{worst:.3e}"


@pytest.mark.parametrize("heads,dim,vdim", [(2, 16, 8), (1, 40, 20), (3, 70, 33), (2, 128, 64), (1, 300, 12)])
def test_gated_scan_carries_its_state(heads, dim, vdim):
    """The recurrence over a batch of two sequences, whole and in pieces down to one token, from
    the state that the piece before left in the sequence's slot; a slot's state that is zeroed
    starts a new sequence.  Decays close to one, so that the first tokens still count at the end."""
    o = _ops(torch.float32)
    rng = np.random.default_rng(dim)
    lens = [300, 47]      # 300: long enough for the path that shares the state's rows out over several warps
    T, hd = sum(lens), heads * dim
    z = rng.normal(0, 1.0, (T, 2 * hd + heads * vdim))
    bias, low = rng.normal(2.0, 1.0, hd), rng.uniform(0.5, 0.99, hd)
    refs, at = [], 0
    for n in lens:
        zz = z[at:at + n]
        q = (zz[:, :hd] / (1 + np.exp(-zz[:, :hd]))).reshape(n, heads, dim)
        f = (low + (1 - low) / (1 + np.exp(-(zz[:, hd:2 * hd] + bias)))).reshape(n, heads, dim)
        v = zz[:, 2 * hd:].reshape(n, heads, vdim)
        S, out = np.zeros((heads, dim, vdim)), np.zeros((n, heads, vdim))
        for t in range(n):
            S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
            out[t] = np.einsum("hdv,hd->hv", S, q[t])
        refs.append((out.reshape(n, heads * vdim), S))
        at += n
    slots = [4, 1]
    for cuts in ([300], [1] * 10 + [2, 3, 64, 71, 150], [299, 1]):
        state = torch.full((6, heads, dim, vdim), 7.0).cuda()
        state[slots] = 0.0
        got = [np.zeros((n, heads * vdim)) for n in lens]
        fed = [0, 0]
        for c in cuts:
            take = [min(c, lens[i] - fed[i]) for i in (0, 1)]
            rows = [i for i in (0, 1) if take[i] > 0]
            zs = np.concatenate([z[sum(lens[:i]) + fed[i]: sum(lens[:i]) + fed[i] + take[i]] for i in rows])
            starts = np.cumsum([0] + [take[i] for i in rows])
            out = torch.zeros((len(zs), heads * vdim)).cuda()
            o.gated_scan(_dev(zs), _dev(bias), _dev(low), state, out, _i32(starts), _i32([slots[i] for i in rows]),
                         heads, dim, vdim)
            out = out.cpu().numpy()
            for j, i in enumerate(rows):
                got[i][fed[i]:fed[i] + take[i]] = out[starts[j]:starts[j + 1]]
                fed[i] += take[i]
        for i in (0, 1):
            assert fed[i] == lens[i]
            assert np.abs(got[i] - refs[i][0]).max() <= 2e-5 * np.abs(refs[i][0]).max(), f"cuts {cuts[:3]} sequence {i}"
            assert np.abs(state[slots[i]].cpu().numpy() - refs[i][1]).max() <= 2e-5
        assert (state[[0, 2, 3, 5]] == 7.0).all(), "another slot's state was touched"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_hash_embedding_and_its_remembered_token(dtype):
    o = _ops(dtype)
    rng = np.random.default_rng(0)
    H, V, buckets, mp, mc = 24, 1000, 53, 3000017, 77
    table = torch.as_tensor(rng.normal(0, 1, (buckets + 1, H)), dtype=dtype).cuda()
    tab = table.float().cpu().numpy()
    seqs = [tokens_of(rng, 9, V), tokens_of(rng, 4, V), tokens_of(rng, 1, V)]
    slots = [5, 0, 2]
    last = torch.full((7, 1), -5, dtype=torch.int32).cuda()

    def run(pieces, past, src=None):
        toks = [t for p in pieces for t in p]
        T = len(toks)
        x = torch.zeros((T, H)).cuda()
        starts = np.cumsum([0] + [len(p) for p in pieces])
        pos = [past[i] + j for i, p in enumerate(pieces) for j in range(len(p))]
        seq = [i for i, p in enumerate(pieces) for _ in p]
        if src is None:
            o.pair_embed_add(_i32(toks), None, None, _i32(pos), _i32(seq), _i32(slots), _i32(starts), last, table, x,
                             V, buckets, mp, mc)
        else:     # tokens taken from a device buffer, as a decode step fed by the sampler takes them
            o.pair_embed_add(_i32([0] * T), _i32(list(range(T))), _i32(toks), _i32(pos), _i32(seq), _i32(slots),
                             _i32(starts), last, table, x, V, buckets, mp, mc)
        return x.cpu().numpy()

    def rows(s, a, b):
        return np.stack([tab[buckets if p == 0 else (s[p - 1] * mp + s[p] * mc) % buckets] for p in range(a, b)])
    x = run([seqs[0][:5], seqs[1][:3], seqs[2]], [0, 0, 0])
    assert np.array_equal(x, np.concatenate([rows(seqs[0], 0, 5), rows(seqs[1], 0, 3), rows(seqs[2], 0, 1)]))
    assert last[slots, 0].tolist() == [seqs[0][4], seqs[1][2], seqs[2][0]] and int(last[1, 0]) == -5
    slots = slots[:2]
    x = run([seqs[0][5:8], seqs[1][3:]], [5, 3])
    assert np.array_equal(x, np.concatenate([rows(seqs[0], 5, 8), rows(seqs[1], 3, 4)]))
    slots = slots[:1]
    x = run([seqs[0][8:]], [8], src=True)
    assert np.array_equal(x, rows(seqs[0], 8, 9)) and int(last[5, 0]) == seqs[0][8]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(3, 96), (70, 1030), (2, 5000)])
def test_branch_norm_add_and_poly_norm(dtype, rows, width):
    o = _ops(dtype)
    rng = np.random.default_rng(width)
    y, x0 = rng.normal(0, 3.0, (rows, width)), rng.normal(0, 1.0, (rows, width))
    gain, m, eps = 1.3, 0.7, 1e-3
    x = _dev(x0)
    xb = torch.zeros((rows, width), dtype=dtype).cuda() if dtype != torch.float32 else None
    ybuf = torch.zeros((rows, width + 8)).cuda()
    ybuf[:, :width] = _dev(y)
    o.branch_norm_add(ybuf[:, :width], _dev([gain]), m, eps, x, xb)
    y32, x32 = y.astype(np.float32).astype(np.float64), x0.astype(np.float32).astype(np.float64)
    ref = x32 + m * gain * plain.rms_normalise(y32, eps)
    assert np.abs(x.cpu().numpy() - ref).max() <= 1e-5
    if xb is not None:
        assert torch.equal(xb, x.to(dtype))
    coeff = np.array([0.6, -0.3, 0.2, 0.05])
    out = torch.zeros((rows, width), dtype=dtype).cuda()
    o.poly_norm(ybuf[:, :width], _dev(coeff), eps, out)
    ref = plain.poly_norm(y32, coeff, eps)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert np.abs(out.float().cpu().numpy() - ref).max() <= tol * np.abs(ref).max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,heads,N,K", [(1, 3, 20, 24), (16, 2, 7, 40), (17, 1, 70, 33), (200, 4, 48, 96),
                                         (130, 3, 80, 64), (64, 2, 128, 512), (300, 17, 10, 24)])
def test_headwise_products(dtype, M, heads, N, K):
    o = _ops(dtype)
    rng = np.random.default_rng(M)
    a_head, c_head = K + (8 if K % 8 == 0 else 5), N + 3     # aligned strides let the tensor-core kernel run
    a = rng.normal(0, 1, (M, heads * a_head))
    w = torch.as_tensor(rng.normal(0, 1, (heads, N, K)), dtype=dtype).cuda()
    w64 = w.double().cpu().numpy()
    a64 = a.astype(np.float32).astype(np.float64)
    ref = np.stack([a64[:, h * a_head:h * a_head + K] @ w64[h].T for h in range(heads)], axis=1)   # [M, heads, N]
    c = torch.zeros((M, heads * c_head)).cuda()
    o.headwise_gemm(_dev(a), a_head, w, c, c_head)
    got = c.cpu().numpy().reshape(M, heads, c_head)
    assert np.abs(got[:, :, :N] - ref).max() <= 1e-4 and (got[:, :, N:] == 0).all()
    gate = rng.normal(0, 2, (M, heads * N))
    g64 = gate.astype(np.float32).astype(np.float64)
    cg = torch.zeros((M, heads * N), dtype=dtype).cuda()
    o.headwise_gemm(_dev(a), a_head, w, cg, N, gate=_dev(gate))
    refg = ref.reshape(M, heads * N) / (1 + np.exp(-g64))
    tol = 1e-4 if dtype == torch.float32 else 2e-2 * np.abs(refg).max()
    assert np.abs(cg.float().cpu().numpy() - refg).max() <= tol
