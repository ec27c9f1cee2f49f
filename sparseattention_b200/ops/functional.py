"""Functional ops of the hierarchical attention path, backed by the CUDA library.

Mirrors hierarchical_attention/ops/functional.py of the reference project:
`build_parent_nodes` (:271) and `hierarchical_attention` (:274), with the same argument
meaning, output dtype (= input dtype) and autograd contract (tables and window_size get no
gradient).  Differences a caller can observe:
  * the backward is deterministic (no floating-point atomics);
  * instead of the softmax weights the forward saves one log-sum-exp per (batch, leaf, head);
  * batch-strided views (as produced by torch.split along dim 1) are consumed without a copy.
"""
from __future__ import annotations

import math
import weakref
from ctypes import c_void_p
from typing import Dict, Optional, Tuple

import torch

from .. import _lib

# ---------------------------------------------------------------------------------------------
# build_parent_nodes
# ---------------------------------------------------------------------------------------------


class BuildParentNodesFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q_p, K_p, V_p, K_c, V_c):
        lib = _lib.load()
        dev = _lib.require_cuda(Q_p, K_p, V_p, K_c, V_c)
        Q_p, K_p, V_p, K_c, V_c = (_lib.as_rows(t) for t in (Q_p, K_p, V_p, K_c, V_c))
        B, P, H, D = Q_p.shape
        assert K_c.shape[1] == 2 * P, "Child count mismatch"
        assert K_p.shape == Q_p.shape == V_p.shape and V_c.shape == K_c.shape == (B, 2 * P, H, D)
        dt = _lib.dtype_code(Q_p)
        assert all(t.dtype == Q_p.dtype for t in (K_p, V_p, K_c, V_c)), "dtype mismatch"
        Out = torch.empty((B, P, H, D), dtype=Q_p.dtype, device=dev)
        with _lib.on_device(dev):
            rc = lib.hsa_parent_nodes_fwd(*(_lib.rows_view(t) for t in (Q_p, K_p, V_p, K_c, V_c, Out)),
                                          None, B, P, H, D, dt, _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_parent_nodes_fwd")
        ctx.save_for_backward(Q_p, K_p, V_p, K_c, V_c)
        return Out

    @staticmethod
    def backward(ctx, grad_output):
        lib = _lib.load()
        Q_p, K_p, V_p, K_c, V_c = ctx.saved_tensors
        dev = Q_p.device
        B, P, H, D = Q_p.shape
        grad_output = _lib.as_rows(grad_output)
        dQ, dKp, dVp = (torch.empty((B, P, H, D), dtype=Q_p.dtype, device=dev) for _ in range(3))
        dKc, dVc = (torch.empty((B, 2 * P, H, D), dtype=Q_p.dtype, device=dev) for _ in range(2))
        with _lib.on_device(dev):
            rc = lib.hsa_parent_nodes_bwd(
                *(_lib.rows_view(t) for t in (grad_output, Q_p, K_p, V_p, K_c, V_c, dQ, dKp, dVp, dKc, dVc)),
                B, P, H, D, _lib.dtype_code(Q_p), _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_parent_nodes_bwd")
        return dQ, dKp, dVp, dKc, dVc


def build_parent_nodes(Q_p, K_p, V_p, K_c, V_c):
    """Three-way attention of every parent over (itself, left child, right child).

    Q_p, K_p, V_p: [B, P, H, D]; K_c, V_c: [B, 2P, H, D]; returns [B, P, H, D].
    """
    return BuildParentNodesFunc.apply(Q_p, K_p, V_p, K_c, V_c)


# ---------------------------------------------------------------------------------------------
# hierarchical_attention (span attention)
# ---------------------------------------------------------------------------------------------

# The kernels derive the tree in closed form.  Tables passed by the caller are accepted for API
# compatibility and verified (once per tensor) to be the canonical ones; anything else is refused
# rather than silently ignored.
_verified_tables: Dict[int, Tuple[int, int, int]] = {}      # id(tensor) -> stamp; the entry dies with the tensor


def _verify_tables(idx_table, mask_table, N: int) -> None:
    L = int(math.log2(N)) if N > 1 else 0
    assert idx_table.shape[0] == N and idx_table.shape[1] == L, \
        f"idx_table shape {tuple(idx_table.shape)} does not match N={N}, levels={L}"
    if mask_table is not None:
        assert tuple(mask_table.shape) == (N, L), "mask_table shape mismatch"
    for t, kind in ((idx_table, 0), (mask_table, 1)):
        if t is None or t.numel() == 0:
            continue
        # a verdict is remembered per tensor OBJECT (and dropped with it), for its current version counter
        stamp = (t._version, kind, N)
        if _verified_tables.get(id(t)) == stamp:
            continue
        n = torch.arange(N, device=t.device).unsqueeze(1)
        l = torch.arange(L, device=t.device).unsqueeze(0)
        if kind == 0:
            base = torch.where(l == 0, torch.zeros_like(l), 2 * N - (torch.full_like(l, N) >> (l - 1).clamp_min(0)))
            want = base + ((n >> l) ^ 1)
            ok = bool((t.to(torch.int64) == want).all())
        else:
            want = ((n >> l) & 1) == 0
            ok = bool((t.to(torch.bool) == want).all())
        if not ok:
            raise _lib.HsaError(
                "hierarchical_attention: the tables passed are not the canonical binary-tree topology "
                "(build_tree_topology); custom topologies are not supported")
        if id(t) not in _verified_tables:
            weakref.finalize(t, _verified_tables.pop, id(t), None)
        _verified_tables[id(t)] = stamp


def span_attention_forward(Q, K, V, window_size: int, is_causal: bool, need_lse: bool = True,
                           algo: int = _lib.ALGO_AUTO):
    """Raw forward on [B,N,H,D] / [B,2N-1,H,D] tensors: returns (Out, LSE or None). No autograd."""
    lib = _lib.load()
    dev = _lib.require_cuda(Q, K, V)
    Q, K, V = (_lib.as_rows(t) for t in (Q, K, V))
    B, N, H, D = Q.shape
    assert K.shape == (B, 2 * N - 1, H, D) and V.shape == K.shape, "K/V must be [B, 2N-1, H, D]"
    assert K.dtype == Q.dtype and V.dtype == Q.dtype, "dtype mismatch"
    Out = torch.empty((B, N, H, D), dtype=Q.dtype, device=dev)
    LSE = torch.empty((B, N, H), dtype=torch.float32, device=dev) if need_lse else None
    with _lib.on_device(dev):
        rc = lib.hsa_span_attn_fwd(*(_lib.rows_view(t) for t in (Q, K, V, Out)),
                                   c_void_p(LSE.data_ptr()) if need_lse else None,
                                   B, N, H, D, int(window_size), int(is_causal), _lib.dtype_code(Q), algo,
                                   _lib.stream_ptr(dev))
    _lib.check(rc, "hsa_span_attn_fwd")
    _lib.debug_check_waits("hsa_span_attn_fwd")
    return Out, LSE


def span_attention_backward(Q, K, V, Out, LSE, dOut, window_size: int, is_causal: bool,
                            algo: int = _lib.ALGO_AUTO):
    """Raw backward: returns (dQ, dK, dV); dK/dV cover all 2N-1 rows."""
    lib = _lib.load()
    dev = Q.device
    B, N, H, D = Q.shape
    dOut = _lib.as_rows(dOut)
    dQ = torch.empty((B, N, H, D), dtype=Q.dtype, device=dev)
    dK = torch.empty((B, 2 * N - 1, H, D), dtype=Q.dtype, device=dev)
    dV = torch.empty_like(dK)
    dt = _lib.dtype_code(Q)
    nbytes = int(lib.hsa_span_attn_bwd_workspace_bytes(B, N, H, D, int(window_size), int(is_causal), dt, algo))
    ws = torch.empty((max(nbytes, 256) + 255) // 256 * 256, dtype=torch.uint8, device=dev)
    with _lib.on_device(dev):
        rc = lib.hsa_span_attn_bwd(
            *(_lib.rows_view(t) for t in (Q, K, V, Out)), c_void_p(LSE.data_ptr()),
            *(_lib.rows_view(t) for t in (dOut, dQ, dK, dV)), c_void_p(ws.data_ptr()), ws.numel(),
            B, N, H, D, int(window_size), int(is_causal), dt, algo, _lib.stream_ptr(dev))
    _lib.check(rc, "hsa_span_attn_bwd")
    _lib.debug_check_waits("hsa_span_attn_bwd")
    return dQ, dK, dV


def span_attention_logits(Q, K, window_size: int, is_causal: bool, weights: bool = False):
    """Per-leaf candidate logits of span attention, float32 [B, N, H, 2*window_size + 1 + log2 N]: window slots
    (key leaf n - window_size + c) first, then one slot per tree level.  weights=False: q.k / sqrt(D), -inf where
    a slot is masked or outside the sequence; weights=True: the softmax weights (0 where masked), i.e. the
    `Weights` tensor the reference's forward saves (ops/functional.py:131-132).  No autograd."""
    lib = _lib.load()
    dev = _lib.require_cuda(Q, K)
    Q, K = _lib.as_rows(Q), _lib.as_rows(K)
    B, N, H, D = Q.shape
    assert K.shape == (B, 2 * N - 1, H, D) and K.dtype == Q.dtype, "K must be [B, 2N-1, H, D] of Q's dtype"
    L = int(math.log2(N)) if N > 1 else 0
    out = torch.empty((B, N, H, 2 * int(window_size) + 1 + L), dtype=torch.float32, device=dev)
    with _lib.on_device(dev):
        rc = lib.hsa_span_attn_logits(_lib.rows_view(Q), _lib.rows_view(K), c_void_p(out.data_ptr()), B, N, H, D,
                                      int(window_size), int(is_causal), int(weights), _lib.dtype_code(Q),
                                      _lib.stream_ptr(dev))
    _lib.check(rc, "hsa_span_attn_logits")
    return out


def build_hierarchical_logits(ALL_Q, ALL_K, H: int, D: int, seq_len: int):
    """The logits op of the reference's first prototype (Hierarchical_Attention_Triton.py:456), same signature:
    ALL_Q, ALL_K [B, total_nodes, H*D] -> (RES_SELF [B, seq_len, H], RES_CROSS [B, total_nodes-1, H]), float32;
    RES_SELF[b,t] = q_t.k_t / sqrt(D), RES_CROSS[b,r] = q_{r^1}.k_r / sqrt(D) (a node's key against its sibling's
    query).  No autograd (the prototype is forward only)."""
    lib = _lib.load()
    dev = _lib.require_cuda(ALL_Q, ALL_K)
    B, total, DH = ALL_Q.shape
    assert DH == H * D and ALL_K.shape == ALL_Q.shape and ALL_K.dtype == ALL_Q.dtype
    q = ALL_Q.contiguous().view(B, total, H, D)
    k = ALL_K.contiguous().view(B, total, H, D)
    res_self = torch.empty((B, seq_len, H), dtype=torch.float32, device=dev)
    res_cross = torch.empty((B, total - 1, H), dtype=torch.float32, device=dev)
    with _lib.on_device(dev):
        rc = lib.hsa_sibling_logits(_lib.rows_view(q), _lib.rows_view(k), c_void_p(res_self.data_ptr()),
                                    c_void_p(res_cross.data_ptr()), B, total, int(seq_len), H, D, _lib.dtype_code(q),
                                    _lib.stream_ptr(dev))
    _lib.check(rc, "hsa_sibling_logits")
    return res_self, res_cross


def span_attention_decode(q, K, V, n: int, window_size: int):
    """Span attention of the single new leaf `n` of every sequence: q [B, H, D] (or [B, 1, H, D]) against the
    key/value caches K, V [B, 2N-1, H, D]; only rows of leaves <= n and of completed left siblings are read.
    Returns [B, H, D].  No autograd."""
    lib = _lib.load()
    dev = _lib.require_cuda(q, K, V)
    B, rows, H, D = K.shape
    N = (rows + 1) // 2
    q4 = q.reshape(B, 1, H, D).contiguous()
    K, V = _lib.as_rows(K), _lib.as_rows(V)
    out = torch.empty_like(q4)
    with _lib.on_device(dev):
        rc = lib.hsa_span_attn_decode(_lib.rows_view(q4), _lib.rows_view(K), _lib.rows_view(V), _lib.rows_view(out),
                                      B, N, H, D, int(window_size), int(n), _lib.dtype_code(q4), _lib.stream_ptr(dev))
    _lib.check(rc, "hsa_span_attn_decode")
    return out.view(B, H, D)


class HierarchicalAttentionFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, idx_table, gather_table, mask_table=None, window_size=16):
        B, N, H, D = Q.shape
        _verify_tables(idx_table, mask_table, N)
        is_causal = mask_table is not None
        need_lse = any(ctx.needs_input_grad[:3])
        Q, K, V = (_lib.as_rows(t) for t in (Q, K, V))
        Out, LSE = span_attention_forward(Q, K, V, window_size, is_causal, need_lse=need_lse)
        if need_lse:
            ctx.save_for_backward(Q, K, V, Out, LSE)
        ctx.window_size, ctx.is_causal = int(window_size), is_causal
        return Out

    @staticmethod
    def backward(ctx, grad_output):
        Q, K, V, Out, LSE = ctx.saved_tensors
        dQ, dK, dV = span_attention_backward(Q, K, V, Out, LSE, grad_output, ctx.window_size, ctx.is_causal)
        return dQ, dK, dV, None, None, None, None


def hierarchical_attention(Q, K, V, idx_table, gather_table, mask_table=None, window_size=16):
    """Span attention: each leaf attends to its radius-`window_size` window and to one sibling
    node per tree level.  Q: [B,N,H,D]; K,V: [B,2N-1,H,D] (leaves then parents); returns [B,N,H,D].
    `mask_table` not None selects the causal variant.
    """
    return HierarchicalAttentionFunc.apply(Q, K, V, idx_table, gather_table, mask_table, window_size)


# ---------------------------------------------------------------------------------------------
# Host-resident inputs (inference): copy in, compute and copy out overlapped over batch chunks
# ---------------------------------------------------------------------------------------------
_host_streams: Dict[int, Tuple[torch.cuda.Stream, torch.cuda.Stream]] = {}
_host_buffers: Dict[tuple, list] = {}


def host_entry_h2d_bytes(B: int, N: int, H: int, D: int, esize: int, is_causal: bool) -> int:
    """Bytes `hierarchical_attention_from_host` copies to the device per call: Q and, of K and V, the rows a
    query can attend to (causal: the N leaves and the N/2 even parent rows; otherwise all 2N-1 rows)."""
    row = H * D * esize
    kv_rows = (N + N // 2) if (is_causal and N > 1) else (2 * N - 1)
    return B * row * (N + 2 * kv_rows)


def hierarchical_attention_from_host(Q, K, V, window_size=16, is_causal=True, out=None, device=None, chunks=8):
    """Span attention on HOST tensors (pinned memory recommended): Q [B,N,H,D], K,V [B,2N-1,H,D].

    The batch is cut into `chunks` pieces; piece i+1 is copied to the device while piece i is computed and
    piece i-1 is copied back, so the call costs about max(copy-in, copy-out, compute) instead of their
    sum.  In the causal case only the key/value rows that can be attended to are copied: the leaves and the
    left-child parents (the even rows from N on); the other rows of the device buffers stay zero, which is
    what the kernels need of rows they load but mask.  Device buffers are kept per shape and reused.
    Returns a host tensor [B,N,H,D] (`out` if given; pinned otherwise).  No autograd.
    """
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, N, H, D = Q.shape
    assert not Q.is_cuda and not K.is_cuda and not V.is_cuda, "inputs of this entry point live on the host"
    assert K.shape == (B, 2 * N - 1, H, D) and V.shape == K.shape
    assert Q.is_contiguous() and K.is_contiguous() and V.is_contiguous(), "host inputs must be contiguous"
    if out is None:
        out = torch.empty((B, N, H, D), dtype=Q.dtype).pin_memory()
    if dev.index not in _host_streams:
        _host_streams[dev.index] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    work, back = _host_streams[dev.index]
    nchunk = max(1, min(int(chunks), B))
    bounds = [(B * i) // nchunk for i in range(nchunk + 1)]
    pieces = [(lo, hi) for lo, hi in zip(bounds[:-1], bounds[1:]) if hi > lo]
    compact = bool(is_causal) and N > 1
    # device buffers of every piece, zero-filled once (the rows never copied must read as finite numbers)
    key = (dev.index, B, N, H, D, Q.dtype, nchunk, compact)
    if key not in _host_buffers:
        if len(_host_buffers) >= 4:
            _host_buffers.clear()
        _host_buffers[key] = [(torch.empty((hi - lo, N, H, D), dtype=Q.dtype, device=dev),
                               torch.zeros((hi - lo, 2 * N - 1, H, D), dtype=Q.dtype, device=dev),
                               torch.zeros((hi - lo, 2 * N - 1, H, D), dtype=Q.dtype, device=dev)) for lo, hi in pieces]
    buffers = _host_buffers[key]
    row = H * D * Q.element_size()
    cur = torch.cuda.current_stream(dev)
    work.wait_stream(cur)
    back.wait_stream(cur)
    keep = []
    for (lo, hi), (q, k, v) in zip(pieces, buffers):
        with torch.cuda.stream(work), torch.cuda.device(dev):
            st = _lib.stream_ptr(dev)
            q.copy_(Q[lo:hi], non_blocking=True)
            if not compact:
                k.copy_(K[lo:hi], non_blocking=True)
                v.copy_(V[lo:hi], non_blocking=True)
            else:
                for host, devt in ((K, k), (V, v)):
                    for j in range(hi - lo):
                        devt[j, :N].copy_(host[lo + j, :N], non_blocking=True)               # the leaves: one block
                        _lib.check(lib.hsa_copy_rows_async(                                  # parents N, N+2, ...
                            c_void_p(devt[j, N].data_ptr()), 2 * row, c_void_p(host[lo + j, N].data_ptr()), 2 * row,
                            row, N // 2, 0, st), "hsa_copy_rows_async")
            o, _ = span_attention_forward(q, k, v, window_size, is_causal, need_lse=False)
            done = torch.cuda.Event()
            done.record(work)
        with torch.cuda.stream(back):
            back.wait_event(done)
            out[lo:hi].copy_(o, non_blocking=True)
        keep.append(o)
    cur.wait_stream(back)
    for t in keep:                            # the caching allocator must not hand these out before `cur` passes
        t.record_stream(cur)
    return out
