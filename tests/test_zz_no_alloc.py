"""The workspace-free backward entry point (hsa_span_attn_bwd_static), called through the C ABI.

Some hosts cannot allocate device memory around the call (plugin execute hooks that only get
pre-bound buffers, servers with fully partitioned GPU memory), so this variant keeps its scratch in
a fixed array inside the library.  It must give what hsa_span_attn_bwd gives, call after call: the
array keeps the previous call's contents.  This file sorts last on purpose, so a run that stops
at the first failure has already been through every other test.
"""
from ctypes import c_void_p

import pytest
import torch

from sparseattention_b200 import _lib
from sparseattention_b200.ops import functional as F


def _static_bwd(Q, K, V, Out, LSE, dOut, R, causal):
    lib = _lib.load()
    B, N, H, D = Q.shape
    dQ = torch.empty_like(Q)
    dK = torch.empty_like(K)
    dV = torch.empty_like(V)
    rc = lib.hsa_span_attn_bwd_static(
        *(_lib.rows_view(t) for t in (Q, K, V, Out)), c_void_p(LSE.data_ptr()),
        *(_lib.rows_view(t) for t in (dOut, dQ, dK, dV)),
        B, N, H, D, R, int(causal), _lib.dtype_code(Q), _lib.stream_ptr(Q.device))
    return rc, dQ, dK, dV


@pytest.mark.gpu
def test_static_backward_matches_workspace_backward_twice():
    torch.cuda.set_device(0)
    gen = torch.Generator().manual_seed(21)
    for call, (B, N, H, D, R, causal, dtype) in enumerate([(2, 256, 4, 64, 8, True, torch.float32),
                                                           (1, 128, 3, 32, 5, False, torch.bfloat16)]):
        Q = torch.randn(B, N, H, D, generator=gen).to(dtype).cuda()
        K = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype).cuda()
        V = torch.randn(B, 2 * N - 1, H, D, generator=gen).to(dtype).cuda()
        dOut = torch.randn(B, N, H, D, generator=gen).to(dtype).cuda()
        Out, LSE = F.span_attention_forward(Q, K, V, R, causal, need_lse=True, algo=_lib.ALGO_PORTABLE)
        want = F.span_attention_backward(Q, K, V, Out, LSE, dOut, R, causal, algo=_lib.ALGO_PORTABLE)
        rc, dQ, dK, dV = _static_bwd(Q, K, V, Out, LSE, dOut, R, causal)
        _lib.check(rc, "hsa_span_attn_bwd_static")
        torch.cuda.synchronize()
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for got, ref in zip((dQ, dK, dV), want):
            err = float((got.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-30))
            assert err < tol, (call, err)


def test_static_backward_rejects_oversize():
    lib = _lib.load()
    B, N, H, D = 1, 1 << 20, 2, 8          # B*N*H = 2^21 > the built-in 2^20 entries
    v = _lib.HsaView(0x1000, 0, 0)
    rc = lib.hsa_span_attn_bwd_static(v, v, v, v, c_void_p(0x1000), v, v, v, v, B, N, H, D, 1, 1, 0, None)
    assert rc == -4
    assert b"exceeds the built-in scratch" in lib.hsa_last_error()
