"""Hyper-connections: a layer over several residual streams instead of one.

The model keeps `streams` copies X_1 .. X_S of the stream (all equal to the embedded token at the
start; their sum is the model's output stream).  A sublayer q of a layer has three small learned
tensors: a read vector a_q [S], a mixing matrix M_q [S, S] indexed [from, to], and a write vector
b_q [S]:
    u = sum_s a_q[s] X_s;   y = sublayer(norm_q(u));   X'_t = sum_s M_q[s, t] X_s + b_q[t] y
(all streams at once from the old ones).  With S = 1, a = b = M = 1 this is the pre-norm block.

The streams lie token-major in one 32-bit tensor [tokens, S, hidden].  Reading and the norm are one
kernel; writing a sublayer's output and the next sublayer's read and norm are one kernel too, also
across layers (the block hands the next block its first input already normed)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorSpec
from .registry import register_block
from .runtime import Runtime


class StreamsRead:
    """What a hyper-connection block hands to the next one: the input of that block's first sublayer,
    read from the streams and normed by the kernel that last wrote them.  (`valid` is False so that a
    block that expects the prepared input of a plain norm ignores it.)"""
    valid = False

    def __init__(self, xn: torch.Tensor, norm):
        self.xn, self.norm = xn, norm


@register_block("hyper_connections")
class HyperConnectionBlock:
    """Parameters: `streams`, `names` = the tensor names of the two sublayers' connections under the
    layer's prefix (default hc1, hc2): `<prefix>.<name>.in` [S], `.mix` [S, S], `.out` [S].  Any
    registered mixer and feed-forward fit (one that says `can_overwrite` stores its output, any other
    adds into a zeroed buffer); norms must offer a 32-bit factor per coordinate as `weight`.

    `multi_stream = True` tells the model to hand `forward` the streams [tokens, S, hidden]."""
    norm_roles = ("mixer_norm", "feed_forward_norm")
    takes_carry = True
    multi_stream = True
    sublayers = ("mixer", "feed_forward")

    def __init__(self, spec, rt: Runtime, mixer, feed_forward, norms):
        self.rt = rt
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)
        self.streams = int(spec.params["streams"])
        self.prefix = str(spec.params["prefix"])
        self.names = tuple(spec.params.get("names") or ("hc1", "hc2"))[:len(self.sublayers)]
        self.read, self.mix, self.write = [], [], []

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> Dict[str, TensorSpec]:
        S = int(spec.params["streams"])
        names = tuple(spec.params.get("names") or ("hc1", "hc2"))[:len(cls.sublayers)]
        out = {}
        # with one stream and no stored connections the block is the plain pre-norm block (all ones)
        opt = S == 1
        for n in names:
            out[f"{prefix}.{n}.in"] = TensorSpec((S,), init=(0.2, 1.0 / S), optional=opt)
            out[f"{prefix}.{n}.out"] = TensorSpec((S,), init=(0.2, 1.0), optional=opt)
            out[f"{prefix}.{n}.mix"] = TensorSpec((S, S), init=(0.2, 1.0 / S), optional=opt)
        return out

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        S = self.streams

        def f32(name, shape):
            t = weights.get(name)
            if t is None:      # only a single stream may come without its connections
                return torch.ones(shape, dtype=torch.float32, device=self.rt.device)
            return t.to(device=self.rt.device, dtype=torch.float32).contiguous()
        for n in self.names:
            self.read.append(f32(f"{self.prefix}.{n}.in", (S,)))
            self.mix.append(f32(f"{self.prefix}.{n}.mix", (S, S)))
            self.write.append(f32(f"{self.prefix}.{n}.out", (S,)))
        self._norm_list = [self.norms[r] for r in self.norm_roles]
        for norm in self._norm_list:
            if norm.weight.dtype != torch.float32:
                norm.weight = norm.weight.to(torch.float32)

    @property
    def first_norm(self):
        return self.norms[self.norm_roles[0]]

    def first_read(self):
        """(read vector, norm factor, eps) of this block's first sublayer, for the kernel that writes the
        streams before it."""
        n = self.first_norm
        return self.read[0], n.weight, n.eps

    def _run(self, part, xn, y, batch):
        if getattr(part, "can_overwrite", False):
            part.forward(xn, y, batch, overwrite=True)
        else:
            y.zero_()
            part.forward(xn, y, batch)

    def forward(self, xs: torch.Tensor, batch, carry=None, next_norm=None, next_block=None):
        rt, ws = self.rt, self.rt.workspace
        T, S, H = xs.shape
        parts = [getattr(self, name) for name in self.sublayers]
        xn = None
        if isinstance(carry, StreamsRead) and carry.norm is self.first_norm and carry.xn.shape == (T, H):
            xn = carry.xn
        if xn is None:
            xn = ws.get("hc_normed_0", (T, H), rt.act_dtype)
            rt.ops.hc_read_norm(xs, self.read[0], self._norm_list[0].weight, self._norm_list[0].eps, xn)
        y = ws.get("hc_branch_out", (T, H), torch.float32)
        handed = None
        for q, part in enumerate(parts):
            self._run(part, xn, y, batch)
            nxt = None
            if q + 1 < len(parts):
                n = self._norm_list[q + 1]
                nxt = (self.read[q + 1], n.weight, n.eps)
            elif next_block is not None and getattr(next_block, "multi_stream", False) and \
                    getattr(next_block, "streams", None) == S:
                nxt = next_block.first_read()
            if nxt is None:
                rt.ops.hc_write(xs, self.mix[q], self.write[q], y)
                continue
            # the normed input alternates between two buffers: the one being written is not the one
            # the sublayer that just ran has read (kernels of a stream run in order, but the buffer a
            # block hands on must outlive this call)
            out = ws.get(f"hc_normed_{(q + 1) % 2 if q + 1 < len(parts) else 0}", (T, H), rt.act_dtype)
            rt.ops.hc_write(xs, self.mix[q], self.write[q], y, next_read=(*nxt, out))
            if q + 1 < len(parts):
                xn = out
            else:
                handed = StreamsRead(out, next_block.first_norm)
        return handed


@register_block("hyper_connections_mixer_only")
class HyperConnectionMixerBlock(HyperConnectionBlock):
    """The same block for a layer without a feed-forward."""
    norm_roles = ("mixer_norm",)
    sublayers = ("mixer",)
