"""Plain, slow restatement of the Tovapel decoder, for tests only: numpy, whole sequences, no
cache, one function per mechanism.  It shares no code with the package under test.

The design in short.  The embedded token is copied into `streams` residual streams
(hyper-connections).  A sublayer reads a weighted sum of the streams through a norm, and its output
goes back into every stream while the streams are mixed among themselves:
    u = sum_s a[s] X_s;   y = sublayer(N(u));   X'_t = sum_s M[s, t] X_s + b[t] y
N is an RMS norm whose stored weight lies around zero (it multiplies by 1 + w).  A layer has a mixer
and, optionally, a feed-forward.  The mixer runs two branches on the same input and averages their
outputs after an RMS norm of each over the model width:
  * softmax attention with grouped key/value heads, biased projections, a per-head RMS norm of
    queries and keys, no positional rotation, tanh-capped scores, a sliding window that also keeps
    the sequence's first keys, a learned "sink" logit per head that only enters the denominator,
    and a sigmoid gate per head;
  * gated linear attention: a matrix state per head that decays per key channel,
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, followed by a per-head RMS norm
    and a silu gate.
The feed-forward is SwiGLU, or a mixture of experts whose router may also pick experts that hand
the input through.  Arrays are float64 by default, so this is also the oracle for error budgets."""
from __future__ import annotations

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_normalise(x: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """The layer norm of the design: the stored weight lies around zero."""
    return rms_normalise(x, eps) * (1.0 + w)


def visible(n: int, size, keep_first: int) -> np.ndarray:
    """[n, n] booleans: query i sees key j iff j <= i and (i - j < size or j < keep_first);
    without a size every j <= i."""
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    near = (i - j < size) if size else np.ones((n, n), bool)
    return (j <= i) & (near | (j < keep_first))


def sink_softmax(scores: np.ndarray, mask: np.ndarray, sink: float) -> np.ndarray:
    """Softmax over the visible keys of each row whose denominator also holds exp(sink)."""
    s = np.where(mask, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


def window_attention(h: np.ndarray, w: dict, p: dict, eps: float) -> np.ndarray:
    """h: [n, width]; w: the branch's tensors by short name; p: its sizes and constants."""
    n = h.shape[0]
    H, G, dim, vdim = p["heads"], p["kv_heads"], p["dim"], p["vdim"]
    q = (h @ w["q"].T + w["q.b"]).reshape(n, H, dim)
    k = (h @ w["k"].T + w["k.b"]).reshape(n, G, dim)
    v = (h @ w["v"].T + w["v.b"]).reshape(n, G, vdim)
    q = rms_normalise(q, eps) * w["q.norm"]
    k = rms_normalise(k, eps) * w["k.norm"]
    mask_p = p.get("mask") or {}
    mask = visible(n, mask_p.get("size"), int(mask_p.get("keep_first", 0)))
    cap = p.get("softcap")
    gate = sigmoid(h @ w["g"].T)                                   # [n, H]
    out = np.zeros((n, H, vdim))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * p["scale"]
        if cap:
            s = cap * np.tanh(s / cap)
        prob = sink_softmax(s, mask, float(w["sink"][head]))
        out[:, head] = (prob @ v[:, g]) * gate[:, head:head + 1]
    return out.reshape(n, H * vdim) @ w["o"].T


def decay(h: np.ndarray, w: dict, tau: float) -> np.ndarray:
    """alpha = sigmoid(W_a2 (W_a1 h) + b)^(1/tau), one per key channel."""
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    return sigmoid(z) ** (1.0 / tau)


def gated_linear_attention(h: np.ndarray, w: dict, p: dict, eps: float, state=None):
    """Returns (output [n, width], state [heads, dim, vdim] after the last token)."""
    n = h.shape[0]
    H, dim, vdim = p["heads"], p["dim"], p["vdim"]
    q = (h @ w["q"].T).reshape(n, H, dim) * dim ** -0.5
    k = (h @ w["k"].T).reshape(n, H, dim)
    v = (h @ w["v"].T).reshape(n, H, vdim)
    alpha = decay(h, w, p["tau"]).reshape(n, H, dim)
    S = np.zeros((H, dim, vdim)) if state is None else state.copy()
    o = np.zeros((n, H, vdim))
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_normalise(o, eps) * w["norm"]
    return (o.reshape(n, H * vdim) * silu(h @ w["g"].T)) @ w["o"].T, S


def parallel_mixer(h: np.ndarray, w: dict, p: dict, eps: float) -> np.ndarray:
    """Half the sum of the two branches, each RMS-normed over the width with its own weight.
    `w` holds the tensors under `left.` / `right.`."""
    sub = lambda side: {k[len(side) + 1:]: v for k, v in w.items() if k.startswith(side + ".")}
    left = window_attention(h, sub("left"), p["left"], eps)
    right, _ = gated_linear_attention(h, sub("right"), p["right"], eps)
    return 0.5 * (rms_normalise(left, eps) * w["left.out"] + rms_normalise(right, eps) * w["right.out"])


def dense_ff(h: np.ndarray, w: dict) -> np.ndarray:
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def expert(h: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray, limit: float) -> np.ndarray:
    """A clamped, gated expert: g is bounded above, u on both sides, and u enters as u + 1."""
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h: np.ndarray, w: dict, top: int):
    """Returns (chosen experts [n, top], their weights [n, top]).  The softmax runs over every
    router output; the correction only influences the choice; weights are not renormalised."""
    z = h @ w["router"].T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(axis=-1, keepdims=True)
    choice = s + w["correction"]
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1)


def moe_ff(h: np.ndarray, w: dict, p: dict) -> np.ndarray:
    """`experts` real experts e0.., followed by `identity` router outputs whose expert hands its
    input through."""
    E, top = p["router"]["experts"], p["router"]["top"]
    limit = p["expert"]["limit"]
    idx, wt = route(h, w, top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t], wt[t]):
            if e >= E:
                out[t] += a * h[t]
            else:
                out[t] += a * expert(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    return out


def hyper_step(X: np.ndarray, w: dict, which: str, norm_w: np.ndarray, eps: float, sublayer) -> np.ndarray:
    """One sublayer over the streams X [streams, n, width]; `which` is hc1 or hc2."""
    u = np.einsum("s,snd->nd", w[f"{which}.in"], X)
    y = sublayer(norm_one_plus(u, norm_w, eps))
    return np.einsum("st,snd->tnd", w[f"{which}.mix"], X) + w[f"{which}.out"][:, None, None] * y[None]


def layer(X: np.ndarray, w: dict, cfg: dict, eps: float) -> np.ndarray:
    """w: the layer's tensors without the `l<i>.` prefix.  X: [streams, n, width]."""
    sub = lambda pre: {k[len(pre) + 1:]: v for k, v in w.items() if k.startswith(pre + ".")}
    X = hyper_step(X, w, "hc1", w["norm1"], eps, lambda h: parallel_mixer(h, sub("mix"), cfg["mixer"], eps))
    mlp = cfg.get("mlp")
    if mlp is not None:
        ff = (lambda h: dense_ff(h, sub("mlp"))) if mlp["kind"] == "dense" else (lambda h: moe_ff(h, sub("mlp"), mlp))
        X = hyper_step(X, w, "hc2", w["norm2"], eps, ff)
    return X


def forward(cfg: dict, w: dict, tokens, return_layers: bool = False):
    """Logits [n, vocab] for one whole sequence; with `return_layers` also the sum of the streams
    after every layer [layers, n, width]."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][[int(t) for t in tokens]]
    X = np.repeat(x[None], int(cfg["streams"]), axis=0)
    after = []
    for i, lc in enumerate(cfg["layers"]):
        pre = f"l{i}."
        X = layer(X, {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}, lc, eps)
        after.append(X.sum(axis=0))
    x = norm_one_plus(X.sum(axis=0), w["final.norm"], eps)
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(after)) if return_layers else logits
