"""Plain, slow restatement of the Kikopel decoder, for tests only: numpy, whole sequences,
no cache, one function per mechanism.  It shares no code with the package under test.

The design in short.  Tokens are embedded (a table row times a multiplier) and a row of a
second table, chosen by a hash of (previous token, token), is added.  Every layer is
    x <- x + m * G1(mixer(x)),   x <- x + m * G2(ff(x))
where G is an RMS norm with a single gain and the sublayers read x itself.  A mixer is
either attention through low-rank latents with a sliding window and an output gate, or a
gated linear recurrence (HGRN2) whose forget gate also sets what is written.  The
feed-forward is up-projection, a polynomial activation of normalised powers, and a
down-projection.  Arrays are float64 by default, so this is also the oracle for error
budgets."""
from __future__ import annotations

import numpy as np


def rms_normalise(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def embed(table: np.ndarray, pair_table: np.ndarray, tokens, scale: float, buckets: int,
          mul_prev: int, mul_cur: int) -> np.ndarray:
    """Row of `table` times `scale`, plus the row of `pair_table` that the pair (previous
    token, token) hashes to; a sequence's first token takes the table's last row."""
    toks = [int(t) for t in tokens]
    out = table[toks] * scale
    for i, t in enumerate(toks):
        row = buckets if i == 0 else (toks[i - 1] * mul_prev + t * mul_cur) % buckets
        out[i] = out[i] + pair_table[row]
    return out


def rotate(x: np.ndarray, positions, base: float, dims: int) -> np.ndarray:
    """Rotary position on the first `dims` entries of the last axis: entry i pairs with entry
    i + dims/2, angle = position * base^(-2i/dims); the other entries pass.  x: [n, ..., d]."""
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return np.concatenate([u * c - v * s, v * c + u * s, x[..., dims:]], axis=-1)


def window_mask(n: int, size) -> np.ndarray:
    """[n, n] booleans: query i sees key j iff 0 <= i - j < size (no size: every j <= i)."""
    d = np.arange(n)[:, None] - np.arange(n)[None, :]
    return (d >= 0) & ((d < size) if size else True)


def latent_attention(h: np.ndarray, w: dict, p: dict, eps: float) -> np.ndarray:
    """h: [n, width]; w: the mixer's tensors by short name; p: its sizes and constants."""
    n = h.shape[0]
    H, dim, rot, vdim, rank = p["heads"], p["dim"], p["rot_dim"], p["vdim"], p["kv_rank"]
    pos = np.arange(n)
    base, dims = p["rot"]["base"], p["rot"]["dims"]
    cq = rms_normalise(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).reshape(n, H, dim + rot)
    q_flat, q_turn = q[..., :dim], rotate(q[..., dim:], pos, base, dims)
    down = h @ w["dkv"].T
    c = rms_normalise(down[:, :rank], eps) * w["dkv.norm"]
    k_turn = rotate(down[:, rank:], pos, base, dims)                 # one per token, for all heads
    k_flat = (c @ w["uk"].T).reshape(n, H, dim)
    v = (c @ w["uv"].T).reshape(n, H, vdim)
    scores = (np.einsum("ihd,jhd->hij", q_flat, k_flat) + np.einsum("ihd,jd->hij", q_turn, k_turn)) * p["scale"]
    size = (p.get("mask") or {}).get("size")
    scores = np.where(window_mask(n, size)[None], scores, -np.inf)
    scores = scores - scores.max(axis=-1, keepdims=True)
    e = np.exp(scores)
    prob = e / e.sum(axis=-1, keepdims=True)
    out = np.einsum("hij,jhd->ihd", prob, v).reshape(n, H * vdim)
    gate = 1.0 / (1.0 + np.exp(-(h @ w["g"].T)))
    return (out * gate) @ w["o"].T


def hgrn2(h: np.ndarray, w: dict, p: dict, eps: float, state=None):
    """Returns (output [n, width], state [heads, dim, vdim] after the last token)."""
    n = h.shape[0]
    H, dim, vdim = p["heads"], p["dim"], p["vdim"]
    z = h @ w["q"].T
    q = (z / (1.0 + np.exp(-z))).reshape(n, H, dim)
    v = (h @ w["v"].T).reshape(n, H, vdim)
    low = w["lower"].reshape(H, dim)
    f = low + (1.0 - low) / (1.0 + np.exp(-((h @ w["f"].T + w["f.b"]).reshape(n, H, dim))))
    S = np.zeros((H, dim, vdim)) if state is None else state.copy()
    o = np.zeros((n, H, vdim))
    for t in range(n):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_normalise(o, eps) * w["norm"]
    return o.reshape(n, H * vdim) @ w["o"].T, S


def poly_norm(z: np.ndarray, coeff, eps: float) -> np.ndarray:
    """a N(z) + b N(z^2) + c N(z^3) + e with N = division by the root mean square."""
    a, b, c, e = (float(x) for x in coeff)
    return a * rms_normalise(z, eps) + b * rms_normalise(z * z, eps) + c * rms_normalise(z * z * z, eps) + e


def feed_forward(h: np.ndarray, w: dict, eps: float) -> np.ndarray:
    return poly_norm(h @ w["up"].T, w["act"], eps) @ w["down"].T


def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens, dtype=np.float64, every_layer: bool = False):
    """Logits [n, vocab] of one sequence from its first token; with `every_layer` also the
    stream after each layer, [layers, n, width]."""
    w = {k: np.asarray(v, dtype=dtype) for k, v in weights.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    e = cfg["embedding"]
    big = e.get("bigram")
    if big:
        x = embed(w["embed"], w["bigram"], tokens, e["scale"], big["buckets"], big["mul_prev"], big["mul_cur"])
    else:
        x = w["embed"][[int(t) for t in tokens]] * e["scale"]
    seen = []
    for i, layer in enumerate(cfg["layers"]):
        mw = _sub(w, f"l{i}.mix.")
        if layer["type"] == "latent_attention":
            y = latent_attention(x, mw, layer["mixer"], eps)
        elif layer["type"] == "hgrn2":
            y, _ = hgrn2(x, mw, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * rms_normalise(y, eps) * w[f"l{i}.norm1"]
        if layer.get("mlp"):
            y = feed_forward(x, _sub(w, f"l{i}.mlp."), eps)
            x = x + m * rms_normalise(y, eps) * w[f"l{i}.norm2"]
        seen.append(x.copy())
    logits = (rms_normalise(x, eps) * w["final.norm"]) @ w["head"].T
    return (logits, np.stack(seen)) if every_layer else logits


def forward_logits(cfg: dict, weights: dict, tokens, dtype=np.float64) -> np.ndarray:
    return forward(cfg, weights, tokens, dtype)
