"""The Tovapel configuration, its tensor list, what its parts ask of the cache (pages whose first
positions a window keeps, values of another size than keys, a mixer that asks for two things), and
the plain implementation's mechanisms against closed forms (no device needed)."""
import copy

import numpy as np
import pytest
import torch

import torchless_rs_b200 as tl
from plain import tovapel_plain as plain
from torchless_rs_b200.cache import Cache, PAGE, PagedKVRequest, StateRequest
from torchless_rs_b200.config import ConfigError
from torchless_rs_b200.engine.model import expected_tensors
from tovapel_tiny import CONFIGS, DECAY_RANKS, tensor_shapes


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_keys_are_read_and_written_back(name):
    raw = CONFIGS[name]
    cfg = tl.config_from_dict(raw)
    assert type(cfg).__name__ == "TovapelConfig"
    assert tl.config_from_dict(cfg.to_dict()) == cfg
    assert (cfg.width, cfg.vocab, cfg.streams, cfg.eps) == (raw["width"], raw["vocab"], raw["streams"], raw["norm"]["eps"])
    assert cfg.logit_softcap == raw.get("logit_softcap")
    for layer, entry in zip(cfg.layers, raw["layers"]):
        a, b = entry["mixer"]["left"], entry["mixer"]["right"]
        l, r = layer.mixer.left, layer.mixer.right
        assert (l.heads, l.kv_heads, l.dim, l.vdim, l.scale) == (a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["scale"])
        assert l.window == (a.get("mask") or {}).get("size") and l.softcap == a.get("softcap")
        assert l.keep_first == ((a.get("mask") or {}).get("keep_first", 0) if l.window else 0)
        assert (r.heads, r.dim, r.vdim, r.tau, r.rank) == (b["heads"], b["dim"], b["vdim"], b["tau"], None)
        mlp = entry["mlp"]
        if mlp is None:
            assert layer.mlp is None
        elif mlp["kind"] == "dense":
            assert layer.mlp.ff == mlp["ff"]
        else:
            assert (layer.mlp.ff, layer.mlp.limit) == (mlp["expert"]["ff"], mlp["expert"]["limit"])
            assert (layer.mlp.experts, layer.mlp.identity, layer.mlp.top) == \
                (mlp["router"]["experts"], mlp["router"]["identity"], mlp["router"]["top"])


def test_errors_name_the_key():
    base = CONFIGS["P"]
    for change, word in ((lambda c: c["layers"][0].__setitem__("type", "serial"), "type"),
                         (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
                         (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
                         (lambda c: c["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 2), "kv_heads"),
                         (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
                         (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
                         (lambda c: c["layers"][0]["mixer"]["right"].__setitem__("tau", 0), "tau"),
                         (lambda c: c.__setitem__("streams", 9), "streams"),
                         (lambda c: c.pop("width"), "width")):
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError) as e:
            tl.config_from_dict(c)
        assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_model_asks_for_the_designs_tensors(name):
    exp = expected_tensors(tl.config_from_dict(CONFIGS[name]).model_spec())
    want = tensor_shapes(CONFIGS[name], DECAY_RANKS[name])
    # (optional: what a layer without feed-forward does not use, and a single stream's connections)
    got = {n: tuple(s.shape) for n, s in exp.items() if not s.optional or n in want}
    assert sorted(got) == sorted(want)
    assert all(s.optional == (CONFIGS[name]["streams"] == 1) for n, s in exp.items() if ".hc" in n and n in want)
    for n, shape in got.items():
        # the decay map's inner size is the stored tensors' business: the model leaves it open
        assert all(a == -1 or a == b for a, b in zip(shape, want[n])) and len(shape) == len(want[n]), n
        assert (-1 in shape) == n.endswith((".a1", ".a2")), n
    # a layer without a feed-forward accepts the norm and connections it does not use
    if name == "P":
        assert {n for n, s in exp.items() if s.optional} == {"l2.norm2", "l2.hc2.in", "l2.hc2.out", "l2.hc2.mix"}


def test_the_decay_rank_may_be_stated():
    raw = copy.deepcopy(CONFIGS["Q"])
    raw["layers"][0]["mixer"]["right"]["rank"] = 6
    cfg = tl.config_from_dict(raw)
    assert cfg.layers[0].mixer.right.rank == 6 and cfg.to_dict()["layers"][0]["mixer"]["right"]["rank"] == 6
    exp = expected_tensors(cfg.model_spec())
    assert exp["l0.mix.right.a1"].shape == (6, 80) and exp["l1.mix.right.a1"].shape == (-1, 80)


def test_parts_and_what_they_ask_of_the_cache():
    spec = tl.config_from_dict(CONFIGS["P"]).model_spec()
    assert spec.streams == 3 and spec.logit_softcap == 8.0 and spec.final_norm.kind == "rmsnorm_one_plus"
    kinds = [(l.block.kind, l.mixer.kind, l.feed_forward.kind) for l in spec.layers]
    assert kinds == [("hyper_connections", "parallel", "swiglu"), ("hyper_connections", "parallel", "moe_clamped"),
                     ("hyper_connections_mixer_only", "parallel", "none")]
    names = [[(n, ps.kind) for n, ps in l.mixer.params["branches"]] for l in spec.layers]
    assert names[0] == [("left", "sink_window_attention"), ("right", "gated_linear_attention")]


def test_a_mixer_that_asks_for_two_things_gets_two_views():
    a = (PagedKVRequest(1, 16, 20, v_head_dim=24, keep_first=3), StateRequest((2, 16, 8)))
    b = (PagedKVRequest(2, 32, 70, v_head_dim=10, keep_first=1), StateRequest((1, 40, 20)))
    c = Cache([a, b, a, None], max_tokens=4 * PAGE, max_slots=2, dtype=torch.float32, device="cpu")
    assert len(c.paged) == 2 and len(c.states) == 2
    kv, st = c.view(0)
    assert tuple(kv.k_pages.shape) == (4, 1, PAGE, 16) and tuple(kv.v_pages.shape) == (4, 1, 24, PAGE)
    assert kv.window == 20 and kv.keep_first == 3 and tuple(st.shape) == (2, 2, 16, 8)
    assert c.view(2)[0].group is kv.group and c.view(2)[0].k_pages.data_ptr() != kv.k_pages.data_ptr()
    assert c.view(3) is None
    # keys and values of one layer do not overlap, and neither do two layers
    kv.k_pages.fill_(1.0)
    kv.v_pages.fill_(2.0)
    assert float(c.view(2)[0].k_pages.sum()) == 0.0 and float(c.view(2)[0].v_pages.sum()) == 0.0
    assert float(kv.k_pages.sum()) == kv.k_pages.numel() and float(kv.v_pages.sum()) == 2 * kv.v_pages.numel()
    s = c.acquire(1)
    st[s[0]].fill_(3.0)
    c.release(s)
    assert c.acquire(1) == s and float(st[s[0]].abs().sum()) == 0.0


@pytest.mark.parametrize("window,keep", [(20, 3), (70, 1), (64, 70), (5, 130), (130, 0)])
def test_a_window_never_gives_back_the_pages_of_the_kept_first_keys(window, keep):
    c = Cache([PagedKVRequest(1, 8, window, keep_first=keep)], max_tokens=8 * PAGE, max_slots=2,
              dtype=torch.float32, device="cpu")
    g = c.paged[0]
    s = c.acquire(1)[0]
    length = 0
    for step in [150] + [1] * 200 + [37, 1, 1]:
        length += step
        if length > 8 * PAGE:
            break
        c.prepare([s], [length])
        c.commit([s], [length])
        c.check()
        # every key that the next position sees is held; every other whole page has gone back
        seen = {j for j in range(length) if j < keep or length - j < window}        # by position `length`
        held = {col for col in range(g.n_cols[s]) if g.table_host[s, col] >= 0}
        need = {j // PAGE for j in seen}
        assert need <= held, (length, sorted(need - held))
        last = (length - 1) // PAGE
        assert held - need <= {last}, (length, sorted(held - need))
    c.release([s])
    assert g.pool.held_count == 0
    c.check()
    # the slot and its pages are used again from the start
    s2 = c.acquire(1)[0]
    c.prepare([s2], [3 * PAGE + 1])
    assert all(g.table_host[s2, :4] >= 0)
    c.commit([s2], [3 * PAGE + 1])
    c.reset(s2)
    assert g.pool.held_count == 0 and c.length(s2) == 0


# ---- the plain mechanisms against closed forms -----------------------------------------------------------
def test_plain_visibility():
    m = plain.visible(12, 4, 2)
    for i in range(12):
        for j in range(12):
            assert m[i, j] == (j <= i and (i - j < 4 or j < 2))
    assert plain.visible(5, None, 0).sum() == 15 and (plain.visible(6, 1, 0) == np.eye(6, dtype=bool)).all()


def test_plain_sink_softmax():
    s = np.array([[0.3, -1.0, 2.0]])
    p = plain.sink_softmax(s, np.array([[True, True, False]]), sink=0.7)
    e = np.exp([0.3, -1.0, 0.7])
    assert np.allclose(p, [[e[0] / e.sum(), e[1] / e.sum(), 0.0]]) and p.sum() < 1.0
    # a sink far below the scores changes nothing; one far above takes all the weight
    assert np.allclose(plain.sink_softmax(s, np.ones((1, 3), bool), -60.0).sum(), 1.0)
    assert plain.sink_softmax(s, np.ones((1, 3), bool), 60.0).sum() < 1e-20


def test_plain_linear_attention_is_its_unrolled_sum():
    rng = np.random.default_rng(0)
    n, W, H, d, v = 9, 12, 2, 3, 4
    w = {"q": rng.normal(size=(H * d, W)), "k": rng.normal(size=(H * d, W)), "v": rng.normal(size=(H * v, W)),
         "g": rng.normal(size=(H * v, W)), "o": np.eye(H * v), "norm": np.ones(v), "a1": rng.normal(size=(2, W)),
         "a2": rng.normal(size=(H * d, 2)), "a2.b": rng.normal(size=H * d)}
    h = rng.normal(size=(n, W))
    p = {"heads": H, "dim": d, "vdim": v, "tau": 2.0}
    out, S = plain.gated_linear_attention(h, w, p, 0.0)
    a = plain.decay(h, w, 2.0).reshape(n, H, d)
    assert np.allclose(a, np.sqrt(plain.sigmoid((h @ w["a1"].T) @ w["a2"].T + w["a2.b"])).reshape(n, H, d))
    q = (h @ w["q"].T).reshape(n, H, d) / np.sqrt(d)
    k = (h @ w["k"].T).reshape(n, H, d)
    vv = (h @ w["v"].T).reshape(n, H, v)
    o = np.zeros((n, H, v))
    for t in range(n):
        for j in range(t + 1):
            o[t] += np.einsum("hd,hv->hv", q[t] * k[j] * np.prod(a[j + 1:t + 1], axis=0), vv[j])
    ref = plain.rms_normalise(o, 0.0).reshape(n, H * v) * plain.silu(h @ w["g"].T)
    assert np.allclose(out, ref)
    # carried state: two pieces give what the whole gives
    o1, S1 = plain.gated_linear_attention(h[:4], w, p, 0.0)
    o2, S2 = plain.gated_linear_attention(h[4:], w, p, 0.0, state=S1)
    assert np.allclose(np.concatenate([o1, o2]), out) and np.allclose(S2, S)


def test_plain_router_and_experts():
    rng = np.random.default_rng(1)
    W, E, I, f = 6, 3, 2, 4
    w = {"router": rng.normal(size=(E + I, W)), "correction": np.array([0.0, 5.0, 0.0, 0.0, -5.0])}
    for e in range(E):
        w.update({f"e{e}.gate": rng.normal(size=(f, W)), f"e{e}.up": rng.normal(size=(f, W)),
                  f"e{e}.down": rng.normal(size=(W, f))})
    h = rng.normal(size=(7, W))
    idx, wt = plain.route(h, w, 2)
    z = h @ w["router"].T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    assert (idx[:, 0] == 1).all() and (idx != 4).all()          # the correction decides the choice ...
    assert np.allclose(wt[:, 0], s[:, 1]) and (wt.sum(-1) < 1.0).all()   # ... but not the weights, which are not renormalised
    p = {"router": {"experts": E, "identity": I, "top": 2}, "expert": {"ff": f, "limit": 0.5}}
    out = plain.moe_ff(h, w, p)
    for t in range(7):
        ref = np.zeros(W)
        for e, a in zip(idx[t], wt[t]):
            if e >= E:
                ref += a * h[t]
            else:
                g = np.minimum(w[f"e{e}.gate"] @ h[t], 0.5)
                u = np.clip(w[f"e{e}.up"] @ h[t], -0.5, 0.5)
                ref += a * (w[f"e{e}.down"] @ (g / (1 + np.exp(-1.702 * g)) * (u + 1)))
        assert np.allclose(out[t], ref)


def test_plain_hyper_connections_reduce_to_the_residual_sum():
    rng = np.random.default_rng(2)
    X = rng.normal(size=(1, 5, 8))
    w = {"hc1.in": np.ones(1), "hc1.mix": np.ones((1, 1)), "hc1.out": np.ones(1)}
    got = plain.hyper_step(X, w, "hc1", np.zeros(8), 1e-6, lambda h: 2.0 * h)
    assert np.allclose(got[0], X[0] + 2.0 * plain.rms_normalise(X[0], 1e-6))
    # several streams: the mix is indexed [from, to]
    X = rng.normal(size=(2, 3, 4))
    w = {"hc1.in": np.array([1.0, 0.0]), "hc1.mix": np.array([[0.0, 1.0], [0.0, 0.0]]), "hc1.out": np.array([0.0, 0.0])}
    got = plain.hyper_step(X, w, "hc1", np.zeros(4), 1e-6, lambda h: h)
    assert np.allclose(got[1], X[0]) and np.allclose(got[0], 0.0)
