"""Tensor-core attention of the bfloat16 path for the attention with a sink, capped scores and a window
that keeps the first keys (kernels in sink_attention_mma.cu).  `run` returns False for sizes it does not
take; the caller then uses the CUDA-core kernel."""
from __future__ import annotations


def run(q, k_pages, v_pages, gate, sink, out, token_pos, token_seq, seq_slot, page_table, nh, nkv, dim, vdim,
        window, keep_first, scale, softcap, batch=None, workspace=None) -> bool:
    return False
