"""Tree topology tables and the initial parents, computed by the CUDA library.

Mirrors hierarchical_attention/ops/topology.py of the reference project (same names, arguments
and results): `build_tree_topology` (:6-150) and `generate_span_input_Y` (:153-169).
"""
from __future__ import annotations

import math
from ctypes import c_void_p
from typing import Dict, Optional

import torch

from .. import _lib


def build_tree_topology(seq_len: int, is_causal: bool = True, device="cuda", dtype=torch.int32) -> Dict[str, torch.Tensor]:
    """Tables {"forward_idx" [N,L], "forward_mask" [N,L] bool, "backward_gather" [2N-1,3]}.

    Bit-identical to the reference builder.  The tables are produced on a CUDA device by
    `hsa_topology_build`; asking for a CPU result copies them back.
    """
    assert seq_len >= 1 and (seq_len & (seq_len - 1)) == 0, "seq_len must be power of 2"
    lib = _lib.load()
    dev = torch.device(device)
    run_dev = dev if dev.type == "cuda" else torch.device("cuda")
    if not torch.cuda.is_available():
        raise _lib.HsaError("build_tree_topology needs a CUDA device (there is no CPU path)")
    if run_dev.index is None:
        run_dev = torch.device("cuda", torch.cuda.current_device())
    L = int(math.log2(seq_len))
    with _lib.on_device(run_dev):
        idx = torch.empty((seq_len, L), dtype=torch.int32, device=run_dev)
        mask = torch.empty((seq_len, L), dtype=torch.uint8, device=run_dev)
        gather = torch.empty((2 * seq_len - 1, 3), dtype=torch.int32, device=run_dev)
        rc = lib.hsa_topology_build(seq_len, int(bool(is_causal)), c_void_p(idx.data_ptr()),
                                    c_void_p(mask.data_ptr()), c_void_p(gather.data_ptr()),
                                    _lib.stream_ptr(run_dev))
        _lib.check(rc, "hsa_topology_build")
    out = {"forward_idx": idx.to(dtype), "forward_mask": mask.to(torch.bool), "backward_gather": gather.to(dtype)}
    if dev.type != "cuda":
        out = {k: v.to(dev) for k, v in out.items()}
    return out


class _SpanInputY(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        lib = _lib.load()
        dev = _lib.require_cuda(x)
        x = _lib.as_rows(x)
        B, N, D = x.shape
        M = int(lib.hsa_span_input_y_rows(N))
        y = torch.empty((B, M, D), dtype=x.dtype, device=dev)
        with _lib.on_device(dev):
            rc = lib.hsa_span_input_y_fwd(_lib.rows_view(x), _lib.rows_view(y), B, N, D, _lib.dtype_code(x),
                                          _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_span_input_y_fwd")
        ctx.shape = (B, N, D)
        return y

    @staticmethod
    def backward(ctx, gy):
        lib = _lib.load()
        B, N, D = ctx.shape
        gy = _lib.as_rows(gy)
        dev = gy.device
        gx = torch.empty((B, N, D), dtype=gy.dtype, device=dev)
        with _lib.on_device(dev):
            rc = lib.hsa_span_input_y_bwd(_lib.rows_view(gy), _lib.rows_view(gx), B, N, D, _lib.dtype_code(gy),
                                          _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_span_input_y_bwd")
        return gx


def generate_span_input_Y(x: torch.Tensor) -> Optional[torch.Tensor]:
    """Initializes Y by averaging adjacent pairs of X, level by level: [B,N,D] -> [B,N-1,D]."""
    if x.size(1) < 2:
        return None
    return _SpanInputY.apply(x)
