"""HGRN2: a gated linear recurrence with a matrix state per head, in which the forget gate also
decides what is written.

With h the mixer's input, per token and head (q, f of `dim` channels; v of `vdim`):
    q = silu(W_q h),   v = W_v h,   f = low + (1 - low) * sigmoid(W_f h + b)
    S <- diag(f) S + (1 - f) v^T,   o = S^T q
each head's o is RMS-normed over its `vdim` entries with one weight vector shared by the heads,
the heads are concatenated and projected by W_o.  S starts at zero, is 32-bit and is carried
from token to token in the cache's per-sequence state (`StateRequest`), so a prompt may come in
any number of pieces.  The three projections are one stacked product whose 32-bit outputs the
scan kernel reads; it applies the activations itself."""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.requests import StateRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_mixer
from .runtime import Runtime


@register_mixer("hgrn2")
class GatedLinearRecurrence:
    """Parameters: `hidden_size`, `heads`, `dim`, `vdim`, `eps` (of the output norm).
    Tensors under the prefix: q, f, f.b, lower, v, norm, o."""
    graph_safe = True
    can_overwrite = True
    state_attributes = ("state",)

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p["vdim"])
        self.eps = float(p["eps"])
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)
        self.state = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, dim, vdim = int(p["hidden_size"]), int(p["heads"]), int(p["dim"]), int(p["vdim"])
        return {
            f"{prefix}.q": TensorSpec((H * dim, hidden)),
            f"{prefix}.f": TensorSpec((H * dim, hidden)),
            f"{prefix}.f.b": TensorSpec((H * dim,), init=(1.0, 1.0)),
            f"{prefix}.lower": TensorSpec((H * dim,), init=(0.15, 0.5)),
            f"{prefix}.v": TensorSpec((H * vdim, hidden)),
            f"{prefix}.norm": TensorSpec((vdim,)),
            f"{prefix}.o": TensorSpec((hidden, H * vdim)),
        }

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        self.w_in = rt.stack([weights[f"{p}.q"], weights[f"{p}.f"], weights[f"{p}.v"]])
        self.w_o = rt.matrix(weights[f"{p}.o"])
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        self.bias = f32(weights[f"{p}.f.b"])
        self.low = f32(weights[f"{p}.lower"])
        self.norm_w = f32(weights[f"{p}.norm"])

    def cache_request(self):
        return StateRequest((self.heads, self.dim, self.vdim), torch.float32)

    def bind_cache(self, view) -> None:
        self.state = view        # [slots, heads, dim, vdim]

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        H, dim, vdim = self.heads, self.dim, self.vdim
        z = ws.get("scan_in", (T, 2 * H * dim + H * vdim), torch.float32)
        self.matmul(xn, self.w_in, z, ops.MODE_STORE_F32)
        out = ws.get("scan_out", (T, H * vdim), torch.float32)
        rt.ops.gated_scan(z, self.bias, self.low, self.state, out, batch.seq_start, batch.seq_slot, H, dim, vdim,
                          workspace=ws)
        normed = ws.get("scan_normed", (T * H, vdim), rt.act_dtype)
        rt.ops.rmsnorm(out.view(T * H, vdim), self.norm_w, self.eps, normed)
        self.matmul(normed.view(T, H * vdim), self.w_o, residual,
                    ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)
