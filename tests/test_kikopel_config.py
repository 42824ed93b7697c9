"""The Kikopel configuration, its tensor list, what its parts ask of the cache, and the plain
implementation's mechanisms against closed forms (no device needed)."""
import numpy as np
import pytest
import torch

import torchless_rs_b200 as tl
from kikopel_tiny import CONFIGS, make_weights, tensor_shapes
from plain import kikopel_plain as plain
from torchless_rs_b200.cache import PagedLatentRequest, StateRequest
from torchless_rs_b200.config import ConfigError
from torchless_rs_b200.engine.model import expected_tensors


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_keys_are_read_and_written_back(name):
    cfg = tl.config_from_dict(CONFIGS[name])
    assert type(cfg).__name__ == "KikopelConfig"
    assert tl.config_from_dict(cfg.to_dict()) == cfg
    raw = CONFIGS[name]
    assert cfg.width == raw["width"] and cfg.vocab == raw["vocab"] and cfg.eps == raw["norm"]["eps"]
    assert cfg.residual_mult == raw["residual_mult"] and cfg.embedding_scale == raw["embedding"]["scale"]
    for layer, entry in zip(cfg.layers, raw["layers"]):
        assert layer.mixer.type == entry["type"]
        assert layer.ff == (entry["mlp"]["ff"] if entry["mlp"] else None)
        if entry["type"] == "latent_attention":
            m = entry["mixer"]
            assert layer.mixer.window == (m.get("mask") or {}).get("size")
            assert (layer.mixer.rot_base, layer.mixer.rot_dims) == (m["rot"]["base"], m["rot"]["dims"])
            assert layer.mixer.scale == m["scale"]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_model_asks_for_the_designs_tensors(name):
    exp = expected_tensors(tl.config_from_dict(CONFIGS[name]).model_spec())
    want = tensor_shapes(CONFIGS[name])
    assert {n: tuple(s.shape) for n, s in exp.items() if not s.optional} == want


def test_what_the_parts_ask_of_the_cache():
    spec = tl.config_from_dict(CONFIGS["P"]).model_spec()
    assert spec.embedding_addend.kind == "pair_hash" and spec.embedding_scale == 2.0
    kinds = [(l.block.kind, l.mixer.kind, l.feed_forward.kind) for l in spec.layers]
    assert kinds == [("branchnorm", "latent_attention", "polynorm"), ("branchnorm", "hgrn2", "polynorm"),
                     ("branchnorm", "latent_attention", "polynorm"), ("branchnorm_mixer_only", "hgrn2", "none")]
    assert spec.layers[2].position.params == {"head_dim": 8, "theta": 500000.0}
    assert tl.config_from_dict(CONFIGS["Q"]).model_spec().embedding_addend is None


def test_latent_pages_and_state_in_the_cache():
    from torchless_rs_b200.cache import Cache, PAGE
    reqs = [PagedLatentRequest(40, 20), StateRequest((3, 16, 8)), PagedLatentRequest(40, 20),
            PagedLatentRequest(64, None), StateRequest((1,), torch.int32)]
    c = Cache(reqs, max_tokens=4 * PAGE, max_slots=2, dtype=torch.float32, device="cpu")
    assert len(c.paged) == 2 and len(c.states) == 2
    v = c.view(0)
    assert tuple(v.pages.shape) == (4, PAGE, 40) and v.window == 20 and c.view(2).group is v.group
    assert tuple(c.view(3).pages.shape) == (4, PAGE, 64) and c.view(4).dtype == torch.int32
    s = c.acquire(1)
    c.view(1)[s[0]].fill_(3.0)
    c.prepare(s, [PAGE + 30])
    c.commit(s, [PAGE + 30])
    # the window of 20 has left the first page behind, the group without a window holds both
    assert c.paged[0].pool.held_count == 1 and c.paged[1].pool.held_count == 2
    c.release(s)
    assert c.acquire(1) == s and float(c.view(1)[s[0]].abs().max()) == 0.0
    c.check()


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=9), "rot.dims"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_errors_name_the_key(change, needle):
    import copy
    cfg = copy.deepcopy(CONFIGS["P"])
    change(cfg)
    with pytest.raises(ConfigError, match=needle):
        tl.config_from_dict(cfg)


def test_random_weights_of_the_design(tmp_path):
    cfg = tl.config_from_dict(CONFIGS["Q"])
    d = tl.write_random_model(cfg, str(tmp_path), 4, torch.float32)
    from torchless_rs_b200.weights.loader import load_checked
    w, src = load_checked(d, expected_tensors(cfg.model_spec()), torch.float32)
    assert tuple(w["l0.norm1"].shape) == () and 0.5 < float(w["final.norm"]) < 1.5
    assert {n: tuple(t.shape) for n, t in w.items()} == tensor_shapes(CONFIGS["Q"])
    logits = plain.forward_logits(CONFIGS["Q"], {k: v.double().numpy() for k, v in w.items()}, [3, 9, 9, 1])
    src.close()
    assert logits.shape == (4, CONFIGS["Q"]["vocab"]) and np.isfinite(logits).all()


# ---- the plain mechanisms against closed forms -------------------------------------------------
def test_plain_recurrence_is_an_exponential_average_for_a_constant_gate():
    H, dim, vdim, n = 1, 3, 2, 30
    w = {"q": np.zeros((dim, 4)), "f": np.zeros((dim, 4)), "f.b": np.zeros(dim), "lower": np.full(dim, 0.5),
         "v": np.zeros((vdim, 4)), "norm": np.ones(vdim), "o": np.eye(4)[:, :vdim]}
    w["v"][:, 0] = [1.0, -2.0]
    w["q"][:, 1] = 50.0                      # silu(50) = 50
    h = np.zeros((n, 4)); h[:, 0] = 1.0; h[:, 1] = 1.0
    out, S = plain.hgrn2(h, w, {"heads": H, "dim": dim, "vdim": vdim}, 0.0)
    f = 0.5 + 0.5 * 0.5                      # sigmoid(0) = 1/2
    assert np.allclose(S, (1 - f ** n) * np.array([1.0, -2.0])[None, None, :])
    assert np.allclose(out[-1][:2], np.array([1.0, -2.0]) / np.sqrt(2.5))    # normalised over vdim
    # a state that is handed on gives the same as one pass
    a, Sa = plain.hgrn2(h[:11], w, {"heads": H, "dim": dim, "vdim": vdim}, 0.0)
    b, Sb = plain.hgrn2(h[11:], w, {"heads": H, "dim": dim, "vdim": vdim}, 0.0, state=Sa)
    assert np.allclose(np.concatenate([a, b]), out) and np.allclose(Sb, S)


def test_plain_window_rotation_embedding_and_activation():
    m = plain.window_mask(6, 3)
    assert m[4].tolist() == [False, False, True, True, True, False] and plain.window_mask(4, None)[3].all()
    x = np.array([[1.0, 0.0, 0.0, 1.0, 5.0]])
    y = plain.rotate(x, [1], 10000.0, 4)     # pairs (0, 2) and (1, 3); entry 4 passes
    a0, a1 = 1.0, 10000.0 ** -0.5
    assert np.allclose(y[0], [np.cos(a0), -np.sin(a1), np.sin(a0), np.cos(a1), 5.0])
    e = plain.embed(np.eye(3), np.arange(12.0).reshape(4, 3), [2, 0, 1], 2.0, 3, 5, 7)
    assert np.allclose(e, 2.0 * np.eye(3)[[2, 0, 1]] + np.arange(12.0).reshape(4, 3)[[3, (2 * 5 + 0) % 3, (0 * 5 + 7) % 3]])
    z = np.array([[1.0, -1.0, 1.0, -1.0]])
    assert np.allclose(plain.poly_norm(z, [2.0, 3.0, 5.0, 0.5], 0.0), 2 * z + 3 + 5 * z + 0.5)


def test_plain_attention_of_one_head_is_ordinary_attention():
    rng = np.random.default_rng(0)
    n, W, dim, rank, vdim = 7, 6, 4, 5, 3
    p = {"heads": 1, "dim": dim, "rot_dim": 0, "vdim": vdim, "q_rank": 6, "kv_rank": rank, "scale": 0.5,
         "rot": {"base": 1.0, "dims": 0}, "mask": {"size": 3}}
    w = {k: rng.normal(size=s) for k, s in (("dq", (6, W)), ("uq", (dim, 6)), ("dkv", (rank, W)), ("uk", (dim, rank)),
                                            ("uv", (vdim, rank)), ("g", (vdim, W)), ("o", (W, vdim)))}
    w["dq.norm"], w["dkv.norm"] = np.ones(6), np.ones(rank)
    h = rng.normal(size=(n, W))
    got = plain.latent_attention(h, w, p, 1e-6)
    q = plain.rms_normalise(h @ w["dq"].T, 1e-6) @ w["uq"].T
    c = plain.rms_normalise(h @ w["dkv"].T, 1e-6)
    k, v = c @ w["uk"].T, c @ w["uv"].T
    out = np.zeros((n, vdim))
    for i in range(n):
        js = list(range(max(0, i - 2), i + 1))
        s = np.array([q[i] @ k[j] for j in js]) * 0.5
        a = np.exp(s - s.max()); a /= a.sum()
        out[i] = sum(a[t] * v[j] for t, j in enumerate(js))
    assert np.allclose(got, (out / (1 + np.exp(-(h @ w["g"].T)))) @ w["o"].T)


def test_a_folder_may_store_the_second_gain_of_a_layer_without_feed_forward(tmp_path):
    from safetensors.torch import save_file
    from torchless_rs_b200.weights.loader import load_checked
    import os
    cfg = CONFIGS["Q"]                                   # its layer 1 has no feed-forward
    w = make_weights(cfg, 2, torch.float32)
    assert "l1.norm2" not in w
    w["l1.norm2"] = torch.tensor(1.25)
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(tmp_path, "model.safetensors"))
    exp = expected_tensors(tl.config_from_dict(cfg).model_spec())
    got, src = load_checked(str(tmp_path), exp, torch.float32)
    src.close()
    assert exp["l1.norm2"].optional and "l1.norm2" in got
    w["l1.norm3"] = torch.tensor(1.0)                    # any other name is still refused
    save_file({k: v.contiguous() for k, v in w.items()}, os.path.join(tmp_path, "model.safetensors"))
    with pytest.raises(tl.WeightsMismatchError, match="norm3"):
        load_checked(str(tmp_path), exp, torch.float32)
