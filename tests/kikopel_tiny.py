"""Small Kikopel configurations with weights made here (numpy, not the package's generator), a
model folder written with the `safetensors` package, and a loader through the package's entry
point.  Matrices are N(0, 1/in) so that activations are of order one and attention scores spread
over a few units: a key that is wrongly seen or missed changes the result by far more than rounding.

The configurations differ from one another, layer by layer, in every size: heads (also one),
plain and rotated query sizes, rotated entries fewer than the rotated part, value sizes that are
no multiples of 4, latent ranks smaller and larger than the head size, windows smaller than a
page, larger than a page and absent, recurrences whose state is not square and whose sizes are no
multiples of 32, layers without a feed-forward, a model without the second embedding table."""
from __future__ import annotations

import json
import os
import shutil
import tempfile

import numpy as np
import torch

from plain import kikopel_plain as plain


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, base=10000.0, dims=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims},
         "scale": scale if scale is not None else 1.0 / float(np.sqrt(dim + rot_dim))}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def recur(heads, dim, vdim):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}}


def with_ff(layer, ff):
    return {**layer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(width, vocab, layers, eps=1e-5, mult=0.6, scale=1.0, bigram=(37, 5, 3)):
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    return {"architecture": "Kikopel", "width": width, "vocab": vocab, "embedding": emb, "norm": {"eps": eps},
            "residual_mult": mult, "layers": layers}


CONFIGS = {
    # attention, recurrence, attention of other sizes with a partial rotation, recurrence without feed-forward
    "P": config(96, 211, [
        with_ff(latent(3, 16, 8, 24, 40, 32, window=20), 160),
        with_ff(recur(3, 16, 8), 72),
        with_ff(latent(2, 32, 16, 10, 24, 48, window=70, base=500000.0, dims=8, scale=0.2), 100),
        with_ff(recur(1, 40, 20), None),
    ], eps=1e-6, mult=0.5, scale=2.0, bigram=(37, 5, 3)),
    # recurrence first, attention without a window and with one head, no second table, multiplier one
    "Q": config(80, 130, [
        with_ff(recur(2, 24, 36), 96),
        with_ff(latent(1, 24, 4, 12, 16, 8, window=None, dims=4), None),
        with_ff(latent(4, 8, 24, 6, 56, 20, window=1), 64),
    ], eps=3e-5, mult=1.0, scale=1.0, bigram=None),
    # sizes that the tensor-core products take (multiples of 8 and more), a window across pages
    "R": config(256, 520, [
        with_ff(latent(4, 32, 32, 48, 64, 96, window=130, base=250000.0), 448),
        with_ff(recur(4, 64, 32), 256),
        with_ff(latent(4, 32, 32, 48, 64, 96, window=64), 448),
    ], eps=1e-5, mult=0.8, scale=4.0, bigram=(1021, 131, 17)),
}


def tensor_shapes(cfg: dict) -> dict:
    """Tensor names and shapes, as the design lays them out."""
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    big = cfg["embedding"].get("bigram")
    if big:
        out["bigram"] = (big["buckets"] + 1, W)
    for i, l in enumerate(cfg["layers"]):
        m, p = l["mixer"], f"l{i}."
        out[p + "norm1"] = ()
        if l["type"] == "latent_attention":
            H, d, r, v, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + r), qr),
                        p + "mix.dkv": (kr + r, W), p + "mix.dkv.norm": (kr,), p + "mix.uk": (H * d, kr),
                        p + "mix.uv": (H * v, kr), p + "mix.g": (H * v, W), p + "mix.o": (W, H * v)})
        else:
            H, d, v = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.f": (H * d, W), p + "mix.f.b": (H * d,),
                        p + "mix.lower": (H * d,), p + "mix.v": (H * v, W), p + "mix.norm": (v,),
                        p + "mix.o": (W, H * v)})
        if l.get("mlp"):
            ff = l["mlp"]["ff"]
            out.update({p + "norm2": (), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff), p + "mlp.act": (4,)})
    out["final.norm"] = ()
    out["head"] = (cfg["vocab"], W)
    return out


def make_weights(cfg: dict, seed: int, store: torch.dtype) -> dict:
    """name -> torch tensor in `store`."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".lower"):
            v = rng.uniform(0.05, 0.9, shape)
        elif name.endswith(".f.b"):
            v = rng.normal(0.5, 1.0, shape)
        elif name.endswith(".act"):
            v = np.array([0.6, 0.3, -0.2, 0.1]) + rng.normal(0, 0.05, 4)
        elif len(shape) <= 1:
            v = 1.0 + rng.normal(0, 0.2, shape)
        elif name in ("embed", "bigram"):
            v = rng.normal(0, 1.0, shape)
        else:
            v = rng.normal(0, 1.0 / np.sqrt(shape[1]), shape)
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(store)
    return out


def write_folder(cfg: dict, weights: dict, where: str | None = None) -> str:
    from safetensors.torch import save_file
    d = where or tempfile.mkdtemp(prefix="tl_kikopel_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


class KModel:
    """A configuration loaded through the package's entry point, with the plain implementation (in
    float64, on the stored values) beside it."""

    def __init__(self, cfg, dtype: str, seed: int = 0, max_tokens: int = 1024, max_batch=None, weights=None):
        import torchless_rs_b200 as tl
        self.cfg = CONFIGS[cfg] if isinstance(cfg, str) else cfg
        self.dtype = dtype
        store = torch.float32 if dtype == "float32" else torch.bfloat16
        self.stored = weights if weights is not None else make_weights(self.cfg, seed, store)
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
            self._ref[key] = plain.forward_logits(self.cfg, self.weights, list(tokens))
        return self._ref[key]

    def step_np(self, slots, tokens, want) -> np.ndarray:
        return self.engine.step(slots, tokens, want).float().cpu().numpy().copy()


def tokens_of(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]
