"""One decoder layer of the hierarchical LM as a single autograd node with a hand-written backward.

Same function as DecoderLayer.forward run eagerly under bf16 autocast
(hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:379-427 around
hierarchical_attention/modules/attention.py:79-220): refresh the parents bottom-up, span attention on the
leaves, feed-forward, with float32 residual streams x [B, N, d] and y [B, N-1, d] and bfloat16 products.
What changes is how it is put on the GPU:

  * every product runs on the library's tcgen05 kernel (`ops.gemm.gemm`), with what used to be separate
    element-wise kernels folded into its epilogue: bias, relu, dropout (value columns only, where the reference
    drops values; regenerated from a counter-based hash in the backward instead of stored), the residual add, and a
    bfloat16 copy of a float32 result;
  * nothing is concatenated, split, stacked or made contiguous: level outputs are written straight into their rows of
    one [B, N-1, d] buffer and read back from there as batch-strided operands, the key/value projection of
    cat[x, y] is two products into the two row ranges of one buffer, projections of one input share one product on
    row-stacked weights, and gradients of stacked projections land in one buffer that the next product reads whole;
  * the weight gradient of the per-level child projections is ONE product over all levels (children rows of level
    l are the output rows of level l-1, so the stacked gradients and the stacked inputs line up);
  * LayerNorm reads float32 and writes bfloat16 directly; its backward adds the residual-path gradient on the way.

The eager module path stays the reference for numerics (and serves float32 and any shape this path does not take);
tests compare the two.
"""
from __future__ import annotations

from ctypes import c_void_p
from typing import List, Optional, Tuple

import torch

from . import _lib
from .ops.gemm import DropoutSpec, column_sums, gemm, masked_cast_with_sums

BF16 = torch.bfloat16

# dropout sites (independent masks) of one layer
S_LEAF_A, S_LEAF_B, S_CHILD, S_YDELTA, S_VALUES, S_ATTN, S_FFN_HIDDEN, S_FFN_OUT = range(1, 9)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else c_void_p(t.data_ptr())


def _ln_fwd(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, raw_copy: bool = False):
    """float32 [.., d] -> (bfloat16 [.., d], mean [rows], rstd [rows]); raw_copy: also the input itself as bfloat16."""
    lib = _lib.load()
    d = x.size(-1)
    rows = x.numel() // d
    y = torch.empty(x.shape, dtype=BF16, device=x.device)
    xb = torch.empty(x.shape, dtype=BF16, device=x.device) if raw_copy else None
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = lib.hsa_layer_norm_fwd_mixed(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(xb), _ptr(mean),
                                      _ptr(rstd), rows, d, float(eps), _lib.stream_ptr(x.device))
    _lib.check(rc, "hsa_layer_norm_fwd_mixed")
    return (y, xb, mean, rstd) if raw_copy else (y, mean, rstd)


def _ln_bwd(x, dy, gamma, mean, rstd, add):
    """dx = add + d(norm)/dx . dy (float32), dgamma, dbeta (float32)."""
    lib = _lib.load()
    d = x.size(-1)
    rows = x.numel() // d
    dx = torch.empty_like(x)
    dgamma = torch.empty(d, dtype=torch.float32, device=x.device)
    dbeta = torch.empty(d, dtype=torch.float32, device=x.device)
    partial = torch.empty(int(lib.hsa_layer_norm_bwd_ctas(rows)) * 2 * d, dtype=torch.float32, device=x.device)
    rc = lib.hsa_layer_norm_bwd_mixed(_ptr(x), _ptr(dy), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(add), _ptr(dx),
                                      _ptr(dgamma), _ptr(dbeta), _ptr(partial), rows, d, _lib.stream_ptr(x.device))
    _lib.check(rc, "hsa_layer_norm_bwd_mixed")
    return dx, dgamma, dbeta


def _heads(t: torch.Tensor, H: int) -> torch.Tensor:
    """[B, rows, d] (any row stride) -> [B, rows, H, d/H] view."""
    B, rows, d = t.shape
    return t.unflatten(2, (H, d // H))


def _parent_fwd(q, k, v, kc, vc, out, H):
    lib = _lib.load()
    B, P, d = q.shape
    views = [_lib.rows_view(_heads(t, H)) for t in (q, k, v, kc, vc, out)]
    rc = lib.hsa_parent_nodes_fwd(*views, None, B, P, H, d // H, _lib.HSA_BF16, _lib.stream_ptr(q.device))
    _lib.check(rc, "hsa_parent_nodes_fwd")


def _parent_bwd(dout, q, k, v, kc, vc, dq, dk, dv, dkc, dvc, H):
    lib = _lib.load()
    B, P, d = q.shape
    views = [_lib.rows_view(_heads(t, H)) for t in (dout, q, k, v, kc, vc, dq, dk, dv, dkc, dvc)]
    rc = lib.hsa_parent_nodes_bwd(*views, B, P, H, d // H, _lib.HSA_BF16, _lib.stream_ptr(q.device))
    _lib.check(rc, "hsa_parent_nodes_bwd")


def _span_fwd(q, k, v, out, lse, N, H, R, causal):
    lib = _lib.load()
    B, _, d = q.shape
    rc = lib.hsa_span_attn_fwd(*(_lib.rows_view(_heads(t, H)) for t in (q, k, v, out)), _ptr(lse), B, N, H, d // H, R,
                               int(causal), _lib.HSA_BF16, _lib.ALGO_AUTO, _lib.stream_ptr(q.device))
    _lib.check(rc, "hsa_span_attn_fwd")


def _span_bwd(q, k, v, out, lse, dout, dq, dk, dv, N, H, R, causal):
    lib = _lib.load()
    B, _, d = q.shape
    Dh = d // H
    nbytes = int(lib.hsa_span_attn_bwd_workspace_bytes(B, N, H, Dh, R, int(causal), _lib.HSA_BF16, _lib.ALGO_AUTO))
    ws = torch.empty(max(nbytes, 256) + 256, dtype=torch.uint8, device=q.device)
    wp = (ws.data_ptr() + 255) // 256 * 256
    rc = lib.hsa_span_attn_bwd(*(_lib.rows_view(_heads(t, H)) for t in (q, k, v, out)), _ptr(lse),
                               *(_lib.rows_view(_heads(t, H)) for t in (dout, dq, dk, dv)), c_void_p(wp), nbytes,
                               B, N, H, Dh, R, int(causal), _lib.HSA_BF16, _lib.ALGO_AUTO, _lib.stream_ptr(q.device))
    _lib.check(rc, "hsa_span_attn_bwd")


# Levels from this one up run as one cooperative launch per tree and direction (csrc/parent_tree.cu); the levels below
# it are large enough for a launch per level to stream at HBM speed.  None switches the tree kernel off.
TREE_START_LEVEL: Optional[int] = 2


def _tree_start(L: int, d: int) -> Optional[int]:
    if TREE_START_LEVEL is None or d % 256 != 0:
        return None
    start = max(1, int(TREE_START_LEVEL))
    return start if start < L else None


def _tree_state(dev) -> torch.Tensor:
    return torch.empty(int(_lib.load().hsa_parent_tree_state_bytes()) // 4, dtype=torch.int32, device=dev)


def _tree_drop(spec):
    if spec is None:
        return None, 0, 0, 1.0
    return c_void_p(spec.key.data_ptr()), spec.site0, spec.threshold, spec.scale


def _parent_tree_fwd(QKVp, Rb, KVc, Wkv, N, H, start, spec):
    lib = _lib.load()
    B, M, d3 = QKVp.shape
    d = d3 // 3
    state = _tree_state(QKVp.device)
    key, site, thr, scale = _tree_drop(spec)
    rc = lib.hsa_parent_tree_fwd(_lib.rows_view(QKVp[..., :d]), _lib.rows_view(QKVp[..., d:2 * d]), _lib.rows_view(QKVp[..., 2 * d:]),
                                 _lib.rows_view(Rb), _lib.rows_view(KVc), _ptr(Wkv), B, N, H, d // H, start, key, site, thr, scale,
                                 _ptr(state), _lib.stream_ptr(QKVp.device))
    _lib.check(rc, "hsa_parent_tree_fwd")
    return state


def _parent_tree_bwd(QKVp, KVc, dRf, dRb, dQKVp, dKVc, Wkv, N, H, start, spec):
    lib = _lib.load()
    B, M, d3 = QKVp.shape
    d = d3 // 3
    state = _tree_state(QKVp.device)
    key, site, thr, scale = _tree_drop(spec)
    rc = lib.hsa_parent_tree_bwd(_lib.rows_view(QKVp[..., :d]), _lib.rows_view(QKVp[..., d:2 * d]), _lib.rows_view(QKVp[..., 2 * d:]),
                                 _lib.rows_view(KVc), _lib.rows_view(dRf), _lib.rows_view(dRb), _lib.rows_view(dQKVp[..., :d]),
                                 _lib.rows_view(dQKVp[..., d:2 * d]), _lib.rows_view(dQKVp[..., 2 * d:]), _lib.rows_view(dKVc),
                                 _ptr(Wkv), B, N, H, d // H, start, key, site, thr, scale, _ptr(state),
                                 _lib.stream_ptr(QKVp.device))
    _lib.check(rc, "hsa_parent_tree_bwd")
    return state


def parent_tree_status(state: torch.Tensor) -> int:
    """0 when every level of the tree launch that used `state` completed; non-zero when a thread block gave up at the
    grid barrier (1) or inside a level (2).  Synchronises."""
    import ctypes
    st = ctypes.c_uint(0)
    _lib.check(_lib.load().hsa_parent_tree_status(_ptr(state), ctypes.byref(st)), "hsa_parent_tree_status")
    return int(st.value)


def level_layout(N: int) -> Tuple[List[int], List[int]]:
    sizes, offsets, off = [], [], 0
    n = N
    while n > 1:
        n //= 2
        sizes.append(n)
        offsets.append(off)
        off += n
    return sizes, offsets


def _rowsum(t: torch.Tensor) -> torch.Tensor:
    return column_sums(t)


class FusedDecoderLayerFunction(torch.autograd.Function):
    """(x, y) -> (x_out, y_next) of one decoder layer; parameters in the order of `fused_layer_parameters`."""

    @staticmethod
    def forward(ctx, x, y, cfg, rng_key, *params):
        (gy, by, Wq_y, Wk_y, Wv_y, Wo_y, bo_y, g1, b1n, Wq_x, Wk_x, Wv_x, Wo_x, bo_x, g2, b2n, W1, bf1, W2, bf2) = params
        H, R, causal, p, eps = cfg["heads"], cfg["window"], cfg["causal"], cfg["p"], cfg["eps"]
        dev = x.device
        B, N, d = x.shape
        M = N - 1
        dff = W1.size(0)
        sizes, offs = level_layout(N)
        drop = (lambda s0, s1=0: DropoutSpec(rng_key, p, s0, s1)) if p > 0.0 else (lambda s0, s1=0: None)
        new = lambda *shape, dtype=BF16: torch.empty(shape, dtype=dtype, device=dev)      # noqa: E731
        with _lib.on_device(dev):
            # row-stacked bfloat16 weights: one product per shared input
            w16 = cfg.get("w16")
            if w16 is not None:                     # kept by the model, refreshed once per step for all layers
                Wqkv_y, Wqkv_x, Wo_yb, Wo_xb, W1b, W2b = w16
            else:
                Wqkv_y = torch.cat([Wq_y, Wk_y, Wv_y], dim=0).to(BF16)
                Wqkv_x = torch.cat([Wq_x, Wk_x, Wv_x], dim=0).to(BF16)
                Wo_yb, Wo_xb, W1b, W2b = Wo_y.to(BF16), Wo_x.to(BF16), W1.to(BF16), W2.to(BF16)
            Wkv_y = Wqkv_y[d:]
            Wkv_x = Wqkv_x[d:]

            # ---------------- bottom-up: refresh the parents
            yn, mean_y, rstd_y = _ln_fwd(y, gy, by, eps)
            QKVp = gemm(yn, Wqkv_y)                                             # [B, M, 3d]
            # the leaves' norm is taken here already: the same pass over x leaves its bfloat16 copy for the child projection
            xn, xb, mean1, rstd1 = _ln_fwd(x, g1, b1n, eps, raw_copy=True)
            KVc0 = gemm(xb, Wkv_y, dropout=drop(S_LEAF_A, S_LEAF_B), drop_cols=(d, 2 * d))       # leaf values dropped twice
            Rb = new(B, M, d)                                                   # refreshed parents, level after level
            KVc = new(B, M, 2 * d)                                              # child projections of levels >= 1 (row = child's row in Rb)
            tree_start = _tree_start(len(sizes), d)
            for lvl, (P, off) in enumerate(zip(sizes, offs)):
                if tree_start is not None and lvl >= tree_start:
                    # every level from here up in one cooperative launch
                    _parent_tree_fwd(QKVp, Rb, KVc, Wkv_y, N, H, tree_start, drop(S_CHILD))
                    break
                if lvl == 0:
                    kc, vc = KVc0[..., :d], KVc0[..., d:]
                else:
                    po, pp = offs[lvl - 1], sizes[lvl - 1]
                    gemm(Rb[:, po:po + pp], Wkv_y, out=KVc[:, po:po + pp], dropout=drop(S_CHILD), drop_cols=(d, 2 * d),
                         drop_rows_total=M, drop_row_offset=po)
                    kc, vc = KVc[:, po:po + pp, :d], KVc[:, po:po + pp, d:]
                sl = QKVp[:, off:off + P]
                _parent_fwd(sl[..., :d], sl[..., d:2 * d], sl[..., 2 * d:], kc, vc, Rb[:, off:off + P], H)
            y_next = new(B, M, d, dtype=torch.float32)
            ynb = new(B, M, d)
            gemm(Rb, Wo_yb, bias=bo_y, out=y_next, dropout=drop(S_YDELTA), residual=y, copy_bf16=ynb)

            # ---------------- top-down: span attention on the leaves
            Q = gemm(xn, Wqkv_x[:d])
            KV = new(B, 2 * N - 1, 2 * d)
            gemm(xn, Wkv_x, out=KV[:, :N], dropout=drop(S_VALUES), drop_cols=(d, 2 * d), drop_rows_total=2 * N - 1)
            gemm(ynb, Wkv_x, out=KV[:, N:], dropout=drop(S_VALUES), drop_cols=(d, 2 * d), drop_rows_total=2 * N - 1,
                 drop_row_offset=N)
            attn = new(B, N, d)
            lse = new(B, N, H, dtype=torch.float32)
            _span_fwd(Q, KV[..., :d], KV[..., d:], attn, lse, N, H, R, causal)
            x1 = new(B, N, d, dtype=torch.float32)
            gemm(attn, Wo_xb, bias=bo_x, out=x1, dropout=drop(S_ATTN), residual=x)

            # ---------------- feed-forward
            x1n, mean2, rstd2 = _ln_fwd(x1, g2, b2n, eps)
            h = gemm(x1n, W1b, bias=bf1, relu=True, dropout=drop(S_FFN_HIDDEN))
            x2 = new(B, N, d, dtype=torch.float32)
            gemm(h, W2b, bias=bf2, out=x2, dropout=drop(S_FFN_OUT), residual=x1)

        ctx.cfg = cfg
        ctx.rng_key = rng_key
        ctx.save_for_backward(x, y, mean_y, rstd_y, yn, QKVp, xb, KVc0, Rb, KVc, ynb, mean1, rstd1, xn, Q, KV, attn, lse,
                              x1, mean2, rstd2, x1n, h, Wqkv_y, Wqkv_x, Wo_yb, Wo_xb, W1b, W2b, gy, g1, g2)
        return x2, y_next

    @staticmethod
    def backward(ctx, dx2, dy_next):
        (x, y, mean_y, rstd_y, yn, QKVp, xb, KVc0, Rb, KVc, ynb, mean1, rstd1, xn, Q, KV, attn, lse,
         x1, mean2, rstd2, x1n, h, Wqkv_y, Wqkv_x, Wo_yb, Wo_xb, W1b, W2b, gy, g1, g2) = ctx.saved_tensors
        cfg, rng_key = ctx.cfg, ctx.rng_key
        H, R, causal, p = cfg["heads"], cfg["window"], cfg["causal"], cfg["p"]
        dev = x.device
        B, N, d = x.shape
        M = N - 1
        sizes, offs = level_layout(N)
        Wkv_y, Wkv_x = Wqkv_y[d:], Wqkv_x[d:]
        f32 = torch.float32
        new = lambda *shape, dtype=BF16: torch.empty(shape, dtype=dtype, device=dev)      # noqa: E731
        spec = (lambda s0, s1=0: DropoutSpec(rng_key, p, s0, s1)) if p > 0.0 else (lambda s0, s1=0: None)

        def masked_bf16(src, site):
            """bfloat16 of (dropout mask of `site`) * src, src float32 [B, rows, cols], and its column sums."""
            return masked_cast_with_sums(src, spec(site))

        dx2 = dx2.contiguous() if dx2.dtype == f32 else dx2.float().contiguous()
        dy_next = dy_next.contiguous() if dy_next.dtype == f32 else dy_next.float().contiguous()
        with _lib.on_device(dev):
            # ---------------- feed-forward
            dz2, dbf2 = masked_bf16(dx2, S_FFN_OUT)
            dW2 = gemm(dz2, h, a_t=True, b_t=True, out_dtype=f32)
            keep = 1.0 / (1.0 - p) if p > 0.0 else 1.0
            dz1 = gemm(dz2, W2b, b_t=True, gate=h, gate_scale=keep)              # through dropout and relu in one step
            dbf1 = _rowsum(dz1)
            dW1 = gemm(dz1, x1n, a_t=True, b_t=True, out_dtype=f32)
            dx1n = gemm(dz1, W1b, b_t=True)
            dx1, dg2, db2n = _ln_bwd(x1, dx1n, g2, mean2, rstd2, dx2)

            # ---------------- top-down
            dzo, dbo_x = masked_bf16(dx1, S_ATTN)
            dWo_x = gemm(dzo, attn, a_t=True, b_t=True, out_dtype=f32)
            dattn = gemm(dzo, Wo_xb, b_t=True)
            G = new(B, 2 * N - 1, 3 * d)                                         # [dQ | dK | dV] (dQ: first N rows only)
            _span_bwd(Q, KV[..., :d], KV[..., d:], attn, lse, dattn, G[:, :N, :d], G[..., d:2 * d], G[..., 2 * d:], N, H, R, causal)
            if p > 0.0:
                spec(S_VALUES).apply(G, G, 2 * d, d, 2 * d, 2 * N - 1, 0, -d)    # dV sits in columns 2d..3d of G, V in d..2d of KV
            # weight gradients of [Wq_x; Wk_x; Wv_x] in one buffer: leaves give all three, parents K and V only
            dWqkv_x = gemm(G[:, :N], xn, a_t=True, b_t=True, out_dtype=f32)
            gemm(G[:, N:, d:], ynb, a_t=True, b_t=True, out=dWqkv_x[d:], accumulate=True)
            dxn = gemm(G[:, :N], Wqkv_x, b_t=True)
            dx_a, dg1, db1n = _ln_bwd(x, dxn, g1, mean1, rstd1, dx1)
            dyn_total = new(B, M, d, dtype=f32)                                  # gradient of y_next: next layer + key/value path
            gemm(G[:, N:, d:], Wkv_x, b_t=True, out=dyn_total, residual=dy_next)

            # ---------------- bottom-up
            dzy, dbo_y = masked_bf16(dyn_total, S_YDELTA)
            dWo_y = gemm(dzy, Rb, a_t=True, b_t=True, out_dtype=f32)
            dRf = new(B, M, d, dtype=f32)
            dRb = new(B, M, d)
            gemm(dzy, Wo_yb, b_t=True, out=dRf, copy_bf16=dRb)
            dQKVp = new(B, M, 3 * d)
            dKVc = new(B, M, 2 * d)
            dKVc0 = new(B, N, 2 * d)
            tree_start = _tree_start(len(sizes), d)
            top = len(sizes) - 1
            if tree_start is not None:
                _parent_tree_bwd(QKVp, KVc, dRf, dRb, dQKVp, dKVc, Wkv_y, N, H, tree_start, spec(S_CHILD))
                top = tree_start - 1
            for lvl in range(top, -1, -1):
                P, off = sizes[lvl], offs[lvl]
                sl, dsl = QKVp[:, off:off + P], dQKVp[:, off:off + P]
                if lvl == 0:
                    kc, vc, dkv = KVc0[..., :d], KVc0[..., d:], dKVc0
                else:
                    po, pp = offs[lvl - 1], sizes[lvl - 1]
                    kc, vc, dkv = KVc[:, po:po + pp, :d], KVc[:, po:po + pp, d:], dKVc[:, po:po + pp]
                _parent_bwd(dRb[:, off:off + P], sl[..., :d], sl[..., d:2 * d], sl[..., 2 * d:], kc, vc,
                            dsl[..., :d], dsl[..., d:2 * d], dsl[..., 2 * d:], dkv[..., :d], dkv[..., d:], H)
                if lvl == 0:
                    if p > 0.0:
                        spec(S_LEAF_A, S_LEAF_B).apply(dKVc0, dKVc0, d, d, 2 * d, N)
                else:
                    if p > 0.0:
                        spec(S_CHILD).apply(dkv, dkv, d, d, 2 * d, M, po)
                    # the children are the outputs of the level below: their gradient gets this level's share
                    gemm(dkv, Wkv_y, b_t=True, out=dRf[:, po:po + pp], accumulate=True, copy_bf16=dRb[:, po:po + pp])
            # [Wq_y; Wk_y; Wv_y] in one buffer: the parents' own projections give all three, the child projections (leaves
            # from x, every higher level from the refreshed rows below it, one product each) add to the K and V parts
            dWqkv_y = gemm(dQKVp, yn, a_t=True, b_t=True, out_dtype=f32)
            gemm(dKVc0, xb, a_t=True, b_t=True, out=dWqkv_y[d:], accumulate=True)
            if M > 1:
                gemm(dKVc[:, :M - 1], Rb[:, :M - 1], a_t=True, b_t=True, out=dWqkv_y[d:], accumulate=True)
            dx = new(B, N, d, dtype=f32)
            gemm(dKVc0, Wkv_y, b_t=True, out=dx, residual=dx_a)
            dyn = gemm(dQKVp, Wqkv_y, b_t=True)
            dy, dgy, dby = _ln_bwd(y, dyn, gy, mean_y, rstd_y, dyn_total)

        grads = (dgy, dby, dWqkv_y[:d], dWqkv_y[d:2 * d], dWqkv_y[2 * d:], dWo_y, dbo_y, dg1, db1n,
                 dWqkv_x[:d], dWqkv_x[d:2 * d], dWqkv_x[2 * d:], dWo_x, dbo_x, dg2, db2n, dW1, dbf1, dW2, dbf2)
        return (dx, dy, None, None) + grads


class Bf16Weights:
    """bfloat16 copies of the weight matrices of a stack of decoder layers, row-stacked the way the fused layer multiplies
    them ([Wq; Wk; Wv] per stream), in one flat buffer that a single multi-tensor copy refreshes: a training step then
    converts its weights with one launch instead of nine small ones per layer."""

    def __init__(self, layers):
        self.sources, shapes = [], []
        for layer in layers:
            a, ff = layer.self_attn, layer.feed_forward
            groups = ([a.Wq_y.weight, a.Wk_y.weight, a.Wv_y.weight], [a.Wq_x.weight, a.Wk_x.weight, a.Wv_x.weight],
                      [a.out_proj_y.weight], [a.out_proj_x.weight], [ff.fc1.weight], [ff.fc2.weight])
            self.sources.append(groups)
            shapes.append([(sum(w.size(0) for w in g), g[0].size(1)) for g in groups])
        dev = self.sources[0][0][0].device
        self.flat = torch.empty(sum(r * c for sh in shapes for r, c in sh), dtype=BF16, device=dev)
        self.per_layer, self._dst, self._src, off = [], [], [], 0
        for groups, sh in zip(self.sources, shapes):
            mats = []
            for g, (r, c) in zip(groups, sh):
                m = self.flat[off: off + r * c].view(r, c)
                off += r * c
                mats.append(m)
                row = 0
                for w in g:
                    self._dst.append(m[row: row + w.size(0)])
                    self._src.append(w)
                    row += w.size(0)
            self.per_layer.append(tuple(mats))

    def matches(self, layers) -> bool:
        if len(layers) != len(self.sources):
            return False
        flat_src = [w for groups in self.sources for g in groups for w in g]
        now = [w for layer in layers for w in (layer.self_attn.Wq_y.weight, layer.self_attn.Wk_y.weight, layer.self_attn.Wv_y.weight,
                                              layer.self_attn.Wq_x.weight, layer.self_attn.Wk_x.weight, layer.self_attn.Wv_x.weight,
                                              layer.self_attn.out_proj_y.weight, layer.self_attn.out_proj_x.weight,
                                              layer.feed_forward.fc1.weight, layer.feed_forward.fc2.weight)]
        return all(a is b for a, b in zip(flat_src, now)) and now[0].device == self.flat.device

    def refresh(self) -> None:
        with torch.no_grad():
            torch._foreach_copy_(self._dst, self._src)


def fused_layer_parameters(layer) -> tuple:
    """The parameters of a DecoderLayer in the order FusedDecoderLayerFunction takes them."""
    a, ff = layer.self_attn, layer.feed_forward
    return (layer.norm_y.weight, layer.norm_y.bias, a.Wq_y.weight, a.Wk_y.weight, a.Wv_y.weight, a.out_proj_y.weight,
            a.out_proj_y.bias, layer.norm1.weight, layer.norm1.bias, a.Wq_x.weight, a.Wk_x.weight, a.Wv_x.weight,
            a.out_proj_x.weight, a.out_proj_x.bias, layer.norm2.weight, layer.norm2.bias, ff.fc1.weight, ff.fc1.bias,
            ff.fc2.weight, ff.fc2.bias)


_rng_state = {}


def next_rng_key(device: torch.device) -> torch.Tensor:
    """A fresh 1-element int64 key for the dropout masks of one layer call: a device counter that only kernels touch
    (so a CUDA graph replay draws new masks), seeded from torch's CUDA seed on first use."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _rng_state:
        _rng_state[idx] = torch.tensor([torch.cuda.initial_seed() & 0x7fffffffffff], dtype=torch.int64, device=device)
    state = _rng_state[idx]
    key = state.clone()
    state.add_(0x9E3779B97F4A7C15 & 0x7fffffffffffffff)
    return key


def fused_layer_supported(layer, x: torch.Tensor, y: torch.Tensor, mask) -> bool:
    lib = _lib.load()
    a = layer.self_attn
    d = x.size(-1)
    return (x.is_cuda and x.dtype == torch.float32 and y is not None and y.dtype == torch.float32 and x.dim() == 3 and
            torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16 and
            bool(lib.hsa_layer_norm_supported(d)) and d % 64 == 0 and (d // a.num_heads) in (64, 128) and
            x.size(1) >= 128 and (x.size(1) & (x.size(1) - 1)) == 0 and y.size(1) == x.size(1) - 1 and
            type(layer.norm1).__name__ == "LayerNorm" and a.out_proj_x.bias is not None)


def fused_decoder_layer(layer, x: torch.Tensor, y: torch.Tensor, mask) -> Tuple[torch.Tensor, torch.Tensor]:
    """DecoderLayer.forward through the fused node (call only when fused_layer_supported(...))."""
    a = layer.self_attn
    p = float(layer.dropout.p) if layer.training else 0.0
    cfg = {"heads": a.num_heads, "window": int(a.window_size), "causal": mask is not None, "p": p, "eps": float(layer.norm1.eps),
           "w16": getattr(layer, "_w16", None)}
    key = next_rng_key(x.device) if p > 0.0 else torch.zeros(1, dtype=torch.int64, device=x.device)
    return FusedDecoderLayerFunction.apply(x.contiguous(), y.contiguous(), cfg, key, *fused_layer_parameters(layer))
