"""Softmax attention with grouped key/value heads, a sliding window that keeps the sequence's first
keys, capped scores, a sink in the softmax's denominator and a gate per head.

With h the mixer's input, per token i and query head (using key/value head floor(head / (H / G))):
    q = N_q(W_q h + b_q),  k = N_k(W_k h + b_k),  v = W_v h + b_v      N: RMS norm over the head's
                                                                        entries, one weight for all heads
    score(i, j) = cap * tanh(scale * (q_i . k_j) / cap)
    j is visible iff j <= i and (i - j < window or j < keep_first)
    p(i, j) = exp(score(i, j)) / (sum over visible j' of exp(score(i, j')) + exp(sink_head))
    out_i = sigmoid(w_g,head . h) * sum_j p(i, j) v_j,   then W_o over the concatenated heads
Positions do not enter the scores.  q, k, v and the gate come from one stacked product; one kernel
adds the biases, norms q and k and writes k and v into the cache pages; attention reads pages only,
for prompts and decode steps alike."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.requests import PagedKVRequest
from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorSpec
from .linear import Matmul
from .registry import register_mixer
from .runtime import Runtime


def run_attention(core_ops, q, k_pages, v_pages, gate, sink, out, token_pos, token_seq, seq_slot, page_table,
                  nh, nkv, dim, vdim, window, keep_first, scale, softcap, batch=None, workspace=None) -> None:
    """Attention of one step over the pages, by the kernel that takes these sizes: in bfloat16 the
    tensor-core kernels where they do (key and value sizes that are multiples of 16), else the CUDA-core
    kernel, which takes every size and is the whole of the 32-bit path.  Which kernel runs changes the
    order of the sums only."""
    if q.dtype == torch.bfloat16:
        from ..csrc import sink_attention_bf16
        if sink_attention_bf16.run(q, k_pages, v_pages, gate, sink, out, token_pos, token_seq, seq_slot, page_table,
                                   nh, nkv, dim, vdim, window, keep_first, scale, softcap, batch, workspace):
            return
    core_ops.sink_attn(q, k_pages, v_pages, gate, sink, out, token_pos, token_seq, seq_slot, page_table, nh, nkv,
                       dim, vdim, window, keep_first, scale, softcap)


@register_mixer("sink_window_attention")
class SinkWindowAttention:
    """Parameters: `hidden_size`, `heads`, `kv_heads`, `dim`, `vdim`, `window` (None: all keys),
    `keep_first`, `scale`, `softcap` (None: no cap), `eps` (of the query and key norms).
    Tensors under the prefix: q, q.b, k, k.b, v, v.b, q.norm, k.norm, sink, g, o."""
    graph_safe = True
    can_overwrite = True

    def __init__(self, spec: PartSpec, prefix: str, rt: Runtime, position=None):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.window = int(p["window"]) if p.get("window") else None
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.scale = float(p["scale"])
        self.softcap = float(p["softcap"]) if p.get("softcap") else None
        self.eps = float(p["eps"])
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads cannot share {self.nkv} key/value heads")
        if position is not None:
            raise ValueError("this attention takes no positional rotation")
        self.prefix = prefix
        self.rt = rt
        self.matmul = Matmul(rt)
        self.cache = None

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        p = spec.params
        hidden, H, G, dim, vdim = (int(p[k]) for k in ("hidden_size", "heads", "kv_heads", "dim", "vdim"))
        std = hidden ** -0.5
        return {
            f"{prefix}.q": TensorSpec((H * dim, hidden), init=(std, 0.0)),
            f"{prefix}.q.b": TensorSpec((H * dim,), init=(0.1, 0.0)),
            f"{prefix}.k": TensorSpec((G * dim, hidden), init=(std, 0.0)),
            f"{prefix}.k.b": TensorSpec((G * dim,), init=(0.1, 0.0)),
            f"{prefix}.v": TensorSpec((G * vdim, hidden), init=(std, 0.0)),
            f"{prefix}.v.b": TensorSpec((G * vdim,), init=(0.1, 0.0)),
            f"{prefix}.q.norm": TensorSpec((dim,)),
            f"{prefix}.k.norm": TensorSpec((dim,)),
            f"{prefix}.sink": TensorSpec((H,), init=(1.0, 0.0)),
            f"{prefix}.g": TensorSpec((H, hidden), init=(std, 0.0)),
            f"{prefix}.o": TensorSpec((hidden, H * vdim), init=((H * vdim) ** -0.5, 0.0)),
        }

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        p, rt = self.prefix, self.rt
        self.w_in = rt.stack([weights[f"{p}.q"], weights[f"{p}.k"], weights[f"{p}.v"], weights[f"{p}.g"]])
        self.w_o = rt.matrix(weights[f"{p}.o"])
        f32 = lambda t: t.to(device=rt.device, dtype=torch.float32).contiguous()
        self.bias = torch.cat([f32(weights[f"{p}.q.b"]), f32(weights[f"{p}.k.b"]), f32(weights[f"{p}.v.b"])])
        self.q_norm = f32(weights[f"{p}.q.norm"])
        self.k_norm = f32(weights[f"{p}.k.norm"])
        self.sink = f32(weights[f"{p}.sink"])

    def cache_request(self):
        return PagedKVRequest(self.nkv, self.dim, self.window, v_head_dim=self.vdim, keep_first=self.keep_first)

    def bind_cache(self, view) -> None:
        self.cache = view

    def forward(self, xn: torch.Tensor, residual: torch.Tensor, batch, emit=None, overwrite: bool = False) -> None:
        rt, ws = self.rt, self.rt.workspace
        T = residual.shape[0]
        c = self.cache
        H, G, dim, vdim = self.nh, self.nkv, self.dim, self.vdim
        g_off = (H + G) * dim + G * vdim
        z = ws.get("swa_in", (T, g_off + H), torch.float32)
        self.matmul(xn, self.w_in, z, ops.MODE_STORE_F32)
        q = ws.get("swa_q", (T, H * dim), rt.act_dtype)
        rt.ops.qk_norm_cache_write(z, self.bias, self.q_norm, self.k_norm, self.eps, q, c.k_pages, c.v_pages,
                                   batch.token_pos, batch.token_seq, batch.seq_slot, c.page_table, H, G, dim, vdim)
        out = ws.get("swa_out", (T, H * vdim), rt.act_dtype)
        gate = z[:, g_off:]
        run_attention(rt.ops, q, c.k_pages, c.v_pages, gate, self.sink, out, batch.token_pos, batch.token_seq,
                      batch.seq_slot, c.page_table, H, G, dim, vdim, self.window, self.keep_first, self.scale,
                      self.softcap, batch, ws)
        self.matmul(out, self.w_o, residual, ops.MODE_STORE_F32 if overwrite else ops.MODE_ACCUM_F32)
