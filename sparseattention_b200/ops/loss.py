"""Label-smoothed cross entropy on (column-padded) logits, backed by the CUDA library.

Stands in for `nn.CrossEntropyLoss(ignore_index=..., label_smoothing=...)` as the reference's training
loop uses it (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:514, 562-572), with one
addition: the logits may carry padding columns beyond `num_classes` (the LM pads its vocabulary matrix
so the LM-head GEMM stays on aligned tensor-core tiles); they are excluded from the softmax and get
zero gradient.  The logits are read once forward and once backward, in their own dtype.

Two deviations from nn.CrossEntropyLoss: a target that is neither `ignore_index` nor inside [0, num_classes)
gives a NaN loss (PyTorch raises a device-side assertion); a batch in which every row is ignored gives 0
(PyTorch gives NaN), because the row count is clamped to 1 without a host synchronisation.
"""
from __future__ import annotations

from ctypes import c_void_p

import torch

from .. import _lib


class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, num_classes, label_smoothing, ignore_index):
        lib = _lib.load()
        dev = _lib.require_cuda(logits, targets)
        assert logits.dim() == 2 and targets.dim() == 1 and targets.numel() == logits.size(0)
        assert targets.dtype == torch.int64, "targets must be int64"
        if logits.stride(1) != 1:
            logits = logits.contiguous()
        targets = targets.contiguous()
        M, Vp = logits.shape
        V = int(num_classes)
        assert 1 <= V <= Vp
        loss_rows = torch.empty(M, dtype=torch.float32, device=dev)
        lse = torch.empty(M, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            rc = lib.hsa_cross_entropy_fwd(c_void_p(logits.data_ptr()), logits.stride(0), c_void_p(targets.data_ptr()),
                                           c_void_p(loss_rows.data_ptr()), c_void_p(lse.data_ptr()), M, V,
                                           float(label_smoothing), int(ignore_index), _lib.dtype_code(logits),
                                           _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_cross_entropy_fwd")
        count = (targets != ignore_index).sum().clamp_min(1).to(torch.float32)
        ctx.save_for_backward(logits, targets, lse, count)
        ctx.meta = (V, float(label_smoothing), int(ignore_index))
        return loss_rows.sum() / count

    @staticmethod
    def backward(ctx, grad_out):
        lib = _lib.load()
        logits, targets, lse, count = ctx.saved_tensors
        V, eps, ignore = ctx.meta
        dev = logits.device
        M, Vp = logits.shape
        scale = (grad_out.to(torch.float32) / count).reshape(1).contiguous()
        dlogits = torch.empty_like(logits)
        with _lib.on_device(dev):
            rc = lib.hsa_cross_entropy_bwd(c_void_p(logits.data_ptr()), logits.stride(0), c_void_p(targets.data_ptr()),
                                           c_void_p(lse.data_ptr()), c_void_p(scale.data_ptr()),
                                           c_void_p(dlogits.data_ptr()), dlogits.stride(0), M, V, Vp, eps, ignore,
                                           _lib.dtype_code(logits), _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_cross_entropy_bwd")
        return dlogits, None, None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, num_classes: int | None = None,
                  label_smoothing: float = 0.0, ignore_index: int = -100) -> torch.Tensor:
    """Mean label-smoothed cross entropy.  logits [M, Vp] (columns >= num_classes are padding),
    targets [M] int64.  Same value and gradient as F.cross_entropy(logits[:, :num_classes].float(), ...)."""
    if num_classes is None:
        num_classes = logits.size(-1)
    return _CrossEntropy.apply(logits, targets, num_classes, label_smoothing, ignore_index)


class _LinearCrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, targets, num_classes, label_smoothing, ignore_index):
        from .gemm import gemm
        lib = _lib.load()
        dev = _lib.require_cuda(x, weight, targets)
        assert x.dim() == 2 and weight.dim() == 2 and weight.size(1) == x.size(1) and targets.numel() == x.size(0)
        assert targets.dtype == torch.int64
        M, Vp, V = x.size(0), weight.size(0), int(num_classes)
        xb = x.detach() if x.dtype == torch.bfloat16 else x.detach().to(torch.bfloat16)
        wb = weight.detach() if weight.dtype == torch.bfloat16 else weight.detach().to(torch.bfloat16)
        targets = targets.contiguous()
        need_grad = any(ctx.needs_input_grad[:3])
        partial = torch.empty(int(lib.hsa_linear_ce_partial_bytes(M, Vp)) // 4, dtype=torch.float32, device=dev)
        logits = torch.empty((M, Vp), dtype=torch.bfloat16, device=dev) if need_grad else None
        gemm(xb, wb, bias=bias, out=logits, ce_partial=partial, ce_targets=targets, ce_classes=V, ce_skip_store=not need_grad)
        loss_rows = torch.empty(M, dtype=torch.float32, device=dev)
        lse = torch.empty(M, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            rc = lib.hsa_linear_ce_combine(c_void_p(partial.data_ptr()), M, Vp, c_void_p(targets.data_ptr()),
                                           c_void_p(loss_rows.data_ptr()), c_void_p(lse.data_ptr()), V, float(label_smoothing),
                                           int(ignore_index), _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_linear_ce_combine")
        count = (targets != ignore_index).sum().clamp_min(1).to(torch.float32)
        if need_grad:
            ctx.save_for_backward(xb, wb, logits, targets, lse, count)
        ctx.meta = (V, float(label_smoothing), int(ignore_index), x.dtype, weight.dtype, None if bias is None else bias.dtype)
        return loss_rows.sum() / count

    @staticmethod
    def backward(ctx, grad_out):
        from .gemm import gemm
        lib = _lib.load()
        xb, wb, logits, targets, lse, count = ctx.saved_tensors
        V, eps, ignore, xdt, wdt, bdt = ctx.meta
        dev = logits.device
        M, Vp = logits.shape
        scale = (grad_out.to(torch.float32) / count).reshape(1).contiguous()
        col_sums = torch.empty(Vp, dtype=torch.float32, device=dev)
        partial = torch.empty(int(lib.hsa_column_sums_partial_bytes(M, Vp)) // 4, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):          # the gradient overwrites the logits in place; its column sums are the bias gradient
            rc = lib.hsa_cross_entropy_bwd_inplace(c_void_p(logits.data_ptr()), logits.stride(0), c_void_p(targets.data_ptr()),
                                                   c_void_p(lse.data_ptr()), c_void_p(scale.data_ptr()), M, V, Vp, eps, ignore,
                                                   c_void_p(col_sums.data_ptr()), c_void_p(partial.data_ptr()), _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_cross_entropy_bwd_inplace")
        dlogits = logits
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dlogits, wb, b_t=True, out_dtype=torch.float32 if xdt == torch.float32 else torch.bfloat16).to(xdt)
        if ctx.needs_input_grad[1]:
            dw = gemm(dlogits.unsqueeze(0), xb.unsqueeze(0), a_t=True, b_t=True,
                      out_dtype=torch.float32 if wdt == torch.float32 else torch.bfloat16).to(wdt)
        if bdt is not None and ctx.needs_input_grad[2]:
            db = col_sums.to(bdt)
        return dx, dw, db, None, None, None, None


def linear_cross_entropy(x: torch.Tensor, weight: torch.Tensor, bias, targets: torch.Tensor, num_classes: int | None = None,
                         label_smoothing: float = 0.0, ignore_index: int = -100) -> torch.Tensor:
    """Mean label-smoothed cross entropy of logits = x @ weight^T + bias without a second pass over the logits: the
    product runs on the library's tcgen05 kernel, whose epilogue keeps the per-row softmax statistics (the reference
    computes fc_out(x) and then nn.CrossEntropyLoss over the stored logits: Hierarchical_Transformer_Pretrain.py:480,514).
    x [M, d], weight [Vp, d] (rows >= num_classes are padding), targets [M] int64.  When no gradient is asked for the
    logits are never written; otherwise they are stored once in bfloat16 and overwritten by their gradient in the backward.
    Operands are used in bfloat16 (as under autocast)."""
    if num_classes is None:
        num_classes = weight.size(0)
    return _LinearCrossEntropy.apply(x, weight, bias, targets, num_classes, label_smoothing, ignore_index)
