"""Tensor-core attention of the bfloat16 path for the attention with a sink, capped scores and a window
that keeps the first keys (kernels in sink_attention_mma.cu), one library per pair of key and value
sizes, built when a model first needs it.  `run` returns False for sizes it does not take; the caller
then uses the CUDA-core kernel."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong
from typing import Dict, Tuple

import torch

from . import build
from .ops import _check, _ptr, _sm_count, _stream

MAX_SIZE = 128          # key and value sizes: multiples of 16 up to this
MAX_GROUP = 16          # query heads per key/value head in the kernel for steps of few tokens
FEW_TOKENS = 8          # a step whose sequences bring at most this many tokens each takes that kernel
COMMON_SIZES = ((64, 64), (128, 128))     # built by the build check; others are built at first use

_libs: Dict[Tuple[int, int], object] = {}


def library_name(dim: int, vdim: int) -> str:
    return f"sink_attn_bf16_d{dim}_v{vdim}"


def register(dim: int, vdim: int) -> str:
    name = library_name(dim, vdim)
    if name not in build.LIBRARIES:
        build.register_library(name, ("sink_attention_mma.cu",), ("-DTL_DTYPE=1", f"-DSA_DIM={dim}", f"-DSA_VDIM={vdim}"))
    return name


for _d, _v in COMMON_SIZES:
    register(_d, _v)


def takes(dim: int, vdim: int) -> bool:
    return dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= MAX_SIZE and 16 <= vdim <= MAX_SIZE


def _lib(dim: int, vdim: int):
    key = (dim, vdim)
    if key not in _libs:
        lib = build.load_library(register(dim, vdim))
        lib.tl_sink_attn_mma.restype = c_int
        lib.tl_sink_attn_split.restype = c_int
        lib.tl_sink_attn_split_floats.restype = c_longlong
        _libs[key] = lib
    return _libs[key]


def split_count(n_tokens: int, nkv: int, span: int, sms: int) -> int:
    """How many blocks share the pages of one (token, key/value head): enough to put some four blocks on
    every SM, never more than there are pages.  The kernel shares out whatever pages a token has by this
    count, so a count chosen for another length is slower, not wrong."""
    pages = max(1, (span + build.PAGE_TOKENS - 1) // build.PAGE_TOKENS)
    return max(1, min(pages, (4 * sms) // max(1, n_tokens * nkv)))


def run(q, k_pages, v_pages, gate, sink, out, token_pos, token_seq, seq_slot, page_table, nh, nkv, dim, vdim,
        window, keep_first, scale, softcap, batch=None, workspace=None) -> bool:
    if not takes(dim, vdim) or q.dtype != torch.bfloat16:
        return False
    T, n_seqs = q.shape[0], seq_slot.numel()
    lib = _lib(dim, vdim)
    ldg = gate.stride(0) if gate is not None else 0
    few = (batch.max_new <= FEW_TOKENS) if batch is not None and hasattr(batch, "max_new") else T <= 4 * n_seqs
    if few and nh // nkv <= MAX_GROUP:
        max_len = getattr(batch, "len_bucket", None) or getattr(batch, "max_len", None) or 4096
        span = min(max_len, window + keep_first + build.PAGE_TOKENS) if window else max_len
        splits = split_count(T, nkv, span, _sm_count(q.device))
        n = int(lib.tl_sink_attn_split_floats(c_int(T), c_int(nh), c_int(nkv), c_int(splits)))
        part = (workspace.get("sink_attn_parts", (n,), torch.float32) if workspace is not None
                else torch.empty(n, dtype=torch.float32, device=q.device))
        _check(lib.tl_sink_attn_split(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(gate), c_int(ldg), _ptr(sink), _ptr(out), _ptr(part),
            _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)),
            c_int(T), c_int(nh), c_int(nkv), c_int(window or 0), c_int(keep_first or 0), c_float(scale),
            c_float(softcap or 0.0), c_int(splits), _stream()), "sink_attn_split")
        _check(0, "sink_attn_merge")
        return True
    seq_start = getattr(batch, "seq_start", None)
    if seq_start is None:
        # the rows' offsets from the rows' sequences, on the device
        counts = torch.bincount(token_seq.to(torch.int64), minlength=n_seqs)
        seq_start = torch.zeros(n_seqs + 1, dtype=torch.int32, device=q.device)
        seq_start[1:] = torch.cumsum(counts, 0).to(torch.int32)
    _check(lib.tl_sink_attn_mma(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(gate), c_int(ldg), _ptr(sink), _ptr(out), _ptr(token_pos),
        _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), c_int(page_table.stride(0)), c_int(T), c_int(n_seqs),
        c_int(nh), c_int(nkv), c_int(window or 0), c_int(keep_first or 0), c_float(scale), c_float(softcap or 0.0),
        _stream()), "sink_attn_mma")
    return True
