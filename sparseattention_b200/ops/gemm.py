"""Dense bf16 products on the tcgen05 tensor cores (`hsa_gemm`), and the Linear layer built on them.

The reference calls nn.Linear (a library GEMM) for every projection of the layer
(hierarchical_attention/modules/attention.py:101-103,116-117,141-142,162,182-187,220) and for the feed-forward
pair and LM head of the model around it (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:331-340,480).
`linear` is the drop-in for F.linear on CUDA bf16 tensors: Y = X W^T + b forward, dX = dY W and dW = dY^T X backward,
all three on the same kernel (operands are read transposed through their shared-memory descriptors, never copied);
batch-strided views (level slices of a [B, N-1, d] tensor) are taken as they are.
"""
from __future__ import annotations

from ctypes import c_void_p
from typing import Optional

import torch

from .. import _lib


def _view3(t: torch.Tensor) -> torch.Tensor:
    """[rows, cols] -> [1, rows, cols]; a 3-D tensor must have a contiguous last dimension."""
    if t.dim() == 2:
        t = t.unsqueeze(0)
    assert t.dim() == 3, "operands are [rows, cols] or [batches, rows, cols]"
    if t.stride(2) != 1 or t.stride(1) % 8 or (t.size(0) > 1 and t.stride(0) % 8) or t.data_ptr() % 16:
        t = t.contiguous()
    return t


class DropoutSpec:
    """A dropout that runs inside a product's epilogue and is regenerated in the backward: `key` is a 1-element int64
    CUDA tensor (seed + step counter), `site0` / `site1` name independent masks (site1 = 0: one mask), `p` the drop
    probability.  Element ids are positions in the logical [batches, rows_total, N] tensor."""

    def __init__(self, key: torch.Tensor, p: float, site0: int, site1: int = 0):
        assert key.dtype == torch.int64 and key.numel() == 1 and key.is_cuda
        assert 0.0 < p < 1.0 and site0 > 0
        self.key, self.p, self.site0, self.site1 = key, float(p), int(site0), int(site1)
        self.threshold = min(int(round(p * 4294967296.0)), 4294967295)
        keep = 1.0 / (1.0 - p)
        self.scale = keep * keep if site1 else keep

    def apply(self, src: torch.Tensor, out: torch.Tensor, col_begin: int, ncols: int, N: int, rows_total: int,
              row_offset: int = 0, col_shift: int = 0) -> torch.Tensor:
        """out[..., col_begin:col_begin+ncols] = mask * scale * src[...] (bfloat16 out; src float32 or bfloat16; src and
        out are [batches, rows, >= col_begin+ncols] with contiguous rows; in place when src is out).  The masks are those
        of columns col_begin+col_shift.. of the logical [batches, rows_total, N] tensor, rows row_offset.. ."""
        lib = _lib.load()
        dev = src.device
        with _lib.on_device(dev):
            rc = lib.hsa_dropout_apply(_lib.rows_view(src), _lib.dtype_code(src), _lib.rows_view(out), src.size(0), src.size(1),
                                       int(col_begin), int(ncols), int(N), int(rows_total), int(row_offset), int(col_shift),
                                       c_void_p(self.key.data_ptr()), self.site0, self.site1, self.threshold, self.scale,
                                       _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_dropout_apply")
        return out


def gemm(A: torch.Tensor, B: torch.Tensor, *, a_t: bool = False, b_t: bool = False, bias: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None, accumulate: bool = False,
         splits: Optional[int] = None, relu: bool = False, dropout: Optional[DropoutSpec] = None,
         drop_cols: Optional[tuple] = None, drop_rows_total: Optional[int] = None, drop_row_offset: int = 0,
         gate: Optional[torch.Tensor] = None, gate_scale: float = 1.0, residual: Optional[torch.Tensor] = None,
         copy_bf16: Optional[torch.Tensor] = None, ce_partial: Optional[torch.Tensor] = None,
         ce_targets: Optional[torch.Tensor] = None, ce_classes: int = 0, ce_skip_store: bool = False) -> torch.Tensor:
    """C = A @ op(B) (+ bias), bfloat16 operands, float32 accumulation.  No autograd.

    a_t=False: A [batches, rows, K] (or [rows, K]); B is one matrix: [N, K] (b_t=False, C = A B^T) or [K, N] (b_t=True,
               C = A B).  C: [batches, rows, N].
    a_t=True : A [batches, K, rows], B [batches, K, N] (b_t must be True): C [rows, N] = sum over batch entries of
               A[b]^T B[b].
    `out` may be a (strided) view with a contiguous last dimension; out_dtype bfloat16 (default) or float32;
    accumulate adds to `out` (float32 only); splits=None lets the library choose a split-K factor.
    Fused tail (see hsa_gemm_epilogue): relu; `dropout` on columns drop_cols=(begin, end) (default: all), element ids
    relative to a logical tensor of drop_rows_total rows per batch entry of which this product writes rows
    drop_row_offset..; `gate` (bfloat16, shaped like the output): v = gate > 0 ? v * gate_scale : 0; `residual`
    (float32, shaped like the output) added last; `copy_bf16`: a bfloat16 copy of a float32 output;
    `ce_partial` / `ce_targets` / `ce_classes`: cross-entropy statistics of the output taken as logits (see
    ops.loss.linear_cross_entropy), with ce_skip_store the logits themselves are not written.
    """
    lib = _lib.load()
    dev = _lib.require_cuda(A, B)
    assert A.dtype == torch.bfloat16 and B.dtype == torch.bfloat16, "hsa_gemm takes bfloat16 operands"
    squeeze = A.dim() == 2 and not a_t
    A3 = _view3(A)
    if a_t:
        assert b_t, "a transposed A needs B stored [K, N]"
        B3 = _view3(B)
        batches, K, rows = A3.shape
        assert B3.shape[:2] == (batches, K), "A and B must share [batches, K]"
        N = B3.size(2)
        out_shape = (rows, N)
    else:
        B3 = _view3(B)
        assert B3.size(0) == 1, "B is one matrix shared by all batch entries"
        batches, rows, K = A3.shape
        N = B3.size(2) if b_t else B3.size(1)
        assert (B3.size(1) if b_t else B3.size(2)) == K, "inner dimensions disagree"
        out_shape = (rows, N) if squeeze else (batches, rows, N)
    odt = out_dtype or (out.dtype if out is not None else torch.bfloat16)
    assert odt in (torch.bfloat16, torch.float32)
    if out is None and ce_skip_store:
        out = torch.empty(out_shape[:-1] + (8,), dtype=odt, device=dev)           # never written: only its pointer is passed
        out_shape = tuple(out.shape)
    if out is None:
        assert not accumulate, "accumulate needs an `out` tensor"
        out = torch.empty(out_shape, dtype=odt, device=dev)
    else:
        assert tuple(out.shape) == out_shape and out.dtype == odt and out.stride(-1) == 1
    out3 = out.unsqueeze(0) if out.dim() == 2 else out
    bias32 = None
    if bias is not None:
        bias32 = bias.detach()
        if bias32.dtype != torch.float32 or not bias32.is_contiguous():
            bias32 = bias32.float().contiguous()
        assert bias32.numel() == N
    ob = 1 if a_t else batches
    epi = None
    if relu or dropout is not None or gate is not None or residual is not None or copy_bf16 is not None or ce_partial is not None:
        assert not a_t, "a fused tail needs the plain A layout"
        epi = _lib.GemmEpilogue()
        epi.relu = int(relu)
        if dropout is not None:
            c0, c1 = drop_cols if drop_cols is not None else (0, N)
            epi.rng_state = dropout.key.data_ptr()
            epi.drop_site0, epi.drop_site1 = dropout.site0, dropout.site1
            epi.drop_threshold, epi.drop_scale = dropout.threshold, dropout.scale
            epi.drop_col_begin, epi.drop_col_end = int(c0), int(c1)
            epi.drop_rows_total = int(drop_rows_total if drop_rows_total is not None else rows)
            epi.drop_row_offset = int(drop_row_offset)
        keep = []
        for name, t, want in (("gate", gate, torch.bfloat16), ("residual", residual, torch.float32),
                              ("copy_bf16", copy_bf16, torch.bfloat16)):
            if t is None:
                continue
            t3 = t.unsqueeze(0) if t.dim() == 2 else t
            assert t3.dtype == want and tuple(t3.shape) == tuple(out3.shape) and t3.stride(-1) == 1, name
            if name == "gate":
                epi.gate, epi.gate_bs, epi.gate_rs, epi.gate_scale = t3.data_ptr(), t3.stride(0), t3.stride(1), float(gate_scale)
            elif name == "residual":
                epi.residual, epi.res_bs, epi.res_rs = t3.data_ptr(), t3.stride(0), t3.stride(1)
            else:
                epi.copy_bf16, epi.copy_bs, epi.copy_rs = t3.data_ptr(), t3.stride(0), t3.stride(1)
            keep.append(t3)
        if ce_partial is not None:
            assert ce_targets is not None and ce_targets.dtype == torch.int64 and ce_targets.numel() == batches * rows
            assert ce_partial.dtype == torch.float32 and ce_partial.is_contiguous() and ce_targets.is_contiguous()
            epi.ce_partial, epi.ce_targets = ce_partial.data_ptr(), ce_targets.data_ptr()
            epi.ce_classes, epi.ce_skip_store = int(ce_classes), int(ce_skip_store)
        splits = 1
    if splits is None:
        splits = int(lib.hsa_gemm_choose_splits(ob, rows, N, K * (batches if a_t else 1)))
    need = int(lib.hsa_gemm_workspace_bytes(ob, rows, N, K, int(a_t), int(b_t), splits)) if splits > 1 else 0
    ws = torch.empty(need + 256, dtype=torch.uint8, device=dev) if need else None
    ws_ptr = ((ws.data_ptr() + 255) // 256 * 256) if need else 0
    import ctypes
    with _lib.on_device(dev):
        rc = lib.hsa_gemm_ex(_lib.rows_view(A3), _lib.rows_view(B3), _lib.rows_view(out3),
                             c_void_p(bias32.data_ptr()) if bias32 is not None else None,
                             batches, rows, N, K, int(a_t), int(b_t), _lib.dtype_code(out), int(accumulate), int(splits),
                             c_void_p(ws_ptr) if need else None, need,
                             ctypes.cast(ctypes.pointer(epi), c_void_p) if epi is not None else None, _lib.stream_ptr(dev))
    _lib.check(rc, "hsa_gemm")
    return out


def column_sums(x: torch.Tensor) -> torch.Tensor:
    """Float32 sums over all leading dimensions of a bfloat16 tensor [..., cols] (contiguous rows): a bias gradient."""
    lib = _lib.load()
    cols = x.size(-1)
    x2 = x.reshape(-1, cols)
    if x2.stride(1) != 1 or x2.stride(0) % 8 or cols % 8 or x2.dtype != torch.bfloat16 or x2.data_ptr() % 16:
        return x2.sum(dim=0, dtype=torch.float32)
    rows = x2.size(0)
    out = torch.empty(cols, dtype=torch.float32, device=x.device)
    partial = torch.empty(int(lib.hsa_column_sums_partial_bytes(rows, cols)) // 4, dtype=torch.float32, device=x.device)
    with _lib.on_device(x.device):
        rc = lib.hsa_column_sums(c_void_p(x2.data_ptr()), x2.stride(0), rows, cols, c_void_p(out.data_ptr()),
                                 c_void_p(partial.data_ptr()), _lib.stream_ptr(x.device))
    _lib.check(rc, "hsa_column_sums")
    return out


def masked_cast_with_sums(src: torch.Tensor, dropout: Optional[DropoutSpec]) -> tuple:
    """(bfloat16(mask * src), float32 column sums of it) for a contiguous float32 tensor [..., cols] in one pass: a
    gradient on its way back through a dropout that ran in a product's epilogue (the mask is that of the logical tensor
    `src` itself), and the bias gradient of the projection under it.  dropout=None: a plain cast with its column sums."""
    lib = _lib.load()
    cols = src.size(-1)
    assert src.dtype == torch.float32 and src.is_contiguous() and cols % 8 == 0 and src.data_ptr() % 16 == 0
    rows = src.numel() // cols
    out = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    sums = torch.empty(cols, dtype=torch.float32, device=src.device)
    partial = torch.empty(int(lib.hsa_column_sums_partial_bytes(rows, cols)) // 4, dtype=torch.float32, device=src.device)
    if dropout is None:
        key, s0, s1, thr, scale = None, 0, 0, 0, 1.0
    else:
        key, s0, s1, thr, scale = c_void_p(dropout.key.data_ptr()), dropout.site0, dropout.site1, dropout.threshold, dropout.scale
    with _lib.on_device(src.device):
        rc = lib.hsa_dropout_cast_colsum(c_void_p(src.data_ptr()), cols, c_void_p(out.data_ptr()), cols, rows, cols, key, s0, s1, thr,
                                         scale, c_void_p(sums.data_ptr()), c_void_p(partial.data_ptr()), _lib.stream_ptr(src.device))
    _lib.check(rc, "hsa_dropout_cast_colsum")
    return out, sums


def gemm_aborts() -> int:
    """Thread blocks of hsa_gemm that gave up a bounded wait (0 in a healthy run); synchronises."""
    import ctypes
    count = ctypes.c_uint(0)
    _lib.check(_lib.load().hsa_gemm_aborts(ctypes.byref(count)), "hsa_gemm_aborts")
    return int(count.value)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        wb = weight if weight.dtype == torch.bfloat16 else weight.to(torch.bfloat16)
        lead = xb.shape[:-1]
        x3 = xb if xb.dim() == 3 else xb.reshape(1, -1, xb.size(-1))
        y = gemm(x3, wb, bias=bias)
        ctx.save_for_backward(x3, wb)
        ctx.meta = (lead, x.dtype, weight.dtype, None if bias is None else bias.dtype, x.dim())
        return y.view(*lead, wb.size(0))

    @staticmethod
    def backward(ctx, gy):
        x3, wb = ctx.saved_tensors
        lead, xdt, wdt, bdt, _ = ctx.meta
        g3 = gy.to(torch.bfloat16) if gy.dtype != torch.bfloat16 else gy
        g3 = g3 if g3.dim() == 3 else g3.reshape(1, -1, g3.size(-1))
        if g3.shape[0] != x3.shape[0]:
            g3 = g3.reshape(x3.shape[0], x3.shape[1], -1)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(g3, wb, b_t=True).view(*lead, wb.size(1)).to(xdt)
        if ctx.needs_input_grad[1]:
            dw = gemm(g3, x3, a_t=True, b_t=True, out_dtype=torch.float32 if wdt == torch.float32 else torch.bfloat16)
            dw = dw.to(wdt)
        if bdt is not None and ctx.needs_input_grad[2]:
            db = g3.reshape(-1, g3.size(-1)).sum(dim=0, dtype=torch.float32).to(bdt)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """F.linear on the library's tcgen05 kernel: bfloat16 operands (others are cast, as autocast would), float32
    accumulation, output bfloat16; gradients for x (bfloat16 product, returned in x's dtype), weight (float32 when the
    weight is float32) and bias."""
    return _Linear.apply(x, weight, bias)
