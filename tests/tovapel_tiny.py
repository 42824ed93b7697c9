"""Small Tovapel configurations with weights made here (numpy, not the package's generator), a
model folder written with the `safetensors` package, and a loader through the package's entry
point.  Matrices are N(0, 1/in) so that activations are of order one and attention scores spread
over a few units: a key that is wrongly seen or missed, a sink that is left out or a lost state
changes the result by far more than rounding.

The configurations differ from one another, layer by layer, in every size: streams (also one),
heads and key/value heads (also equal, also one), key and value sizes that differ and are no
multiples of 4, windows smaller than a page, across pages and absent, kept first keys (none, one,
several), caps present and absent, recurrences whose state is not square, decay ranks, layers without
a feed-forward, experts with and without pass-through outputs, a choice of one and of all."""
from __future__ import annotations

import json
import os
import shutil
import tempfile

import numpy as np
import torch

from plain import tovapel_plain as plain


def left(heads, kv_heads, dim, vdim, window, keep_first=0, scale=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else 1.0 / float(np.sqrt(dim))}
    if softcap:
        m["softcap"] = softcap
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    return m


def right(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, identity, top, limit=1.0):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top}}


def layer(l, r, mlp):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp}


def config(width, vocab, streams, layers, eps=1e-5, logit_softcap=None):
    c = {"architecture": "Tovapel", "width": width, "vocab": vocab, "streams": streams, "norm": {"eps": eps},
         "layers": layers}
    if logit_softcap:
        c["logit_softcap"] = logit_softcap
    return c


# the inner size of each layer's decay map is no key of config.json: the stored tensors give it
DECAY_RANKS = {"P": (4, 7, 2), "Q": (3, 5), "R": (16, 8, 8)}

CONFIGS = {
    # a window inside a page with kept keys; a window across pages with one kept key and experts; no window,
    # no cap, no feed-forward
    "P": config(96, 211, 3, [
        layer(left(3, 1, 16, 24, window=20, keep_first=3, softcap=6.0), right(2, 16, 8, tau=8.0), dense(160)),
        layer(left(2, 2, 32, 10, window=70, keep_first=1, scale=0.15, softcap=20.0), right(1, 40, 20, tau=3.0),
              moe(24, experts=5, identity=2, top=3, limit=0.8)),
        layer(left(4, 2, 8, 8, window=None), right(3, 8, 12, tau=1.0), None),
    ], eps=1e-6, logit_softcap=8.0),
    # one stream; a window of one key; a choice of one expert among real ones only; a choice of all outputs
    "Q": config(80, 130, 1, [
        layer(left(1, 1, 24, 12, window=1, keep_first=0), right(2, 24, 36, tau=16.0), moe(40, 3, 0, 1, limit=2.5)),
        layer(left(4, 1, 8, 6, window=5, keep_first=9, softcap=3.0), right(1, 33, 5, tau=2.0),
              moe(16, 3, 1, 4, limit=0.5)),
    ], eps=3e-5),
    # sizes that the tensor-core kernels take (multiples of 16 and more), windows across pages
    "R": config(192, 520, 2, [
        layer(left(4, 2, 64, 64, window=130, keep_first=5, softcap=30.0), right(4, 32, 64, tau=16.0), dense(448)),
        layer(left(8, 2, 32, 64, window=64, keep_first=70, softcap=50.0), right(2, 64, 32, tau=8.0),
              moe(64, experts=8, identity=1, top=2)),
        layer(left(2, 2, 128, 128, window=None, softcap=10.0), right(3, 64, 64, tau=4.0), dense(256)),
    ], logit_softcap=30.0),
}


def tensor_shapes(cfg: dict, ranks) -> dict:
    """Tensor names and shapes, as the design lays them out."""
    W, S, out = cfg["width"], cfg["streams"], {}
    out["embed"] = (cfg["vocab"], W)
    for i, l in enumerate(cfg["layers"]):
        a, b, p = l["mixer"]["left"], l["mixer"]["right"], f"l{i}."
        H, G, d, v = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        out.update({p + "norm1": (W,), p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S),
                    p + "mix.left.q": (H * d, W), p + "mix.left.q.b": (H * d,), p + "mix.left.k": (G * d, W),
                    p + "mix.left.k.b": (G * d,), p + "mix.left.v": (G * v, W), p + "mix.left.v.b": (G * v,),
                    p + "mix.left.q.norm": (d,), p + "mix.left.k.norm": (d,), p + "mix.left.sink": (H,),
                    p + "mix.left.g": (H, W), p + "mix.left.o": (W, H * v), p + "mix.left.out": (W,)})
        H, d, v, r = b["heads"], b["dim"], b["vdim"], ranks[i]
        out.update({p + "mix.right.q": (H * d, W), p + "mix.right.k": (H * d, W), p + "mix.right.v": (H * v, W),
                    p + "mix.right.g": (H * v, W), p + "mix.right.o": (W, H * v), p + "mix.right.norm": (v,),
                    p + "mix.right.a1": (r, W), p + "mix.right.a2": (H * d, r), p + "mix.right.a2.b": (H * d,),
                    p + "mix.right.out": (W,)})
        mlp = l.get("mlp")
        if mlp:
            out.update({p + "norm2": (W,), p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
            if mlp["kind"] == "dense":
                out.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
            else:
                E, I, f = mlp["router"]["experts"], mlp["router"]["identity"], mlp["expert"]["ff"]
                out.update({p + "mlp.router": (E + I, W), p + "mlp.correction": (E + I,)})
                for e in range(E):
                    out.update({p + f"mlp.e{e}.gate": (f, W), p + f"mlp.e{e}.up": (f, W), p + f"mlp.e{e}.down": (W, f)})
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def make_weights(cfg: dict, seed: int, store: torch.dtype, ranks=(4,) * 16, static_choice: bool = False) -> dict:
    """name -> torch tensor in `store`.  `static_choice`: the router's corrections lie so far apart that
    they alone decide which experts are chosen (for runs in bfloat16, whose rounding of the router's
    input could otherwise flip a close choice against the float64 oracle); the weights still vary."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if leaf.endswith(".mix") and "hc" in leaf:
            v = 0.7 * np.eye(shape[0]) + rng.normal(0, 0.1, shape)
        elif leaf.endswith(".in") and "hc" in leaf:
            # all of one sign: the streams start equal, and a read whose weights cancel would turn the
            # rounding of the streams into the signal
            v = rng.uniform(0.5, 1.5, shape) / shape[0]
        elif leaf.endswith(".out") and "hc" in leaf:
            v = rng.uniform(0.5, 1.5, shape) * rng.choice([-1.0, 1.0], shape)
        elif leaf in ("norm1", "norm2", "final.norm"):
            v = rng.normal(0.0, 0.2, shape)                # stored around zero
        elif leaf.endswith(".sink"):
            v = rng.normal(0.5, 1.0, shape)
        elif leaf.endswith(".a2.b"):
            v = rng.normal(2.0, 1.0, shape)
        elif leaf.endswith(".a2"):
            v = rng.normal(0, 1.0, shape)
        elif leaf.endswith(".correction"):
            v = rng.permutation(shape[0]) * 1.5 if static_choice else rng.normal(0, 0.1, shape)
        elif leaf.endswith(".router"):
            v = rng.normal(0, 2.0 / np.sqrt(shape[1]), shape)
        elif leaf.endswith(".b"):
            v = rng.normal(0, 0.5, shape)
        elif len(shape) == 1:
            v = 1.0 + rng.normal(0, 0.2, shape)
        elif name == "embed":
            v = rng.normal(0, 1.0, shape)
        else:
            v = rng.normal(0, 1.0 / np.sqrt(shape[1]), shape)
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(store)
    return out


def write_folder(cfg: dict, weights: dict, where: str | None = None) -> str:
    from safetensors.torch import save_file
    d = where or tempfile.mkdtemp(prefix="tl_tovapel_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


class TModel:
    """A configuration loaded through the package's entry point, with the plain implementation (in
    float64, on the stored values) beside it."""

    def __init__(self, cfg, dtype: str, seed: int = 0, max_tokens: int = 1024, max_batch=None, weights=None):
        import torchless_rs_b200 as tl
        name = cfg if isinstance(cfg, str) else None
        self.cfg = CONFIGS[cfg] if isinstance(cfg, str) else cfg
        self.dtype = dtype
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        self.stored = weights if weights is not None else make_weights(
            self.cfg, seed, store, DECAY_RANKS.get(name, (4,) * 16), static_choice=dtype != "float32")
        self.weights = {k: v.to(torch.float64).numpy() for k, v in self.stored.items()}
        d = write_folder(self.cfg, self.stored)
        try:
            self.model = tl.load(d, dtype=dtype, max_tokens=max_tokens, max_batch=max_batch)
        finally:
            shutil.rmtree(d, ignore_errors=True)
        self.engine = self.model.engine
        self._ref = {}

    def reference(self, tokens) -> np.ndarray:
        key = tuple(tokens)
        if key not in self._ref:
            self._ref[key] = plain.forward(self.cfg, self.weights, list(tokens))
        return self._ref[key]

    def step_np(self, slots, tokens, want) -> np.ndarray:
        return self.engine.step(slots, tokens, want).float().cpu().numpy().copy()


def tokens_of(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]
