"""LayerNorm backed by the CUDA library (used by the LM around the attention layer).

Same parameters and results as `nn.LayerNorm(d)` (weight, bias, eps); one read of the input forward, one read
of input and upstream gradient backward, weight/bias gradients summed in a fixed order.  Widths the kernel
does not take (see `hsa_layer_norm_supported`) go through `torch.nn.functional.layer_norm`.
"""
from __future__ import annotations

from ctypes import c_void_p

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _lib


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        lib = _lib.load()
        dev = _lib.require_cuda(x, weight, bias)
        xc = x.contiguous()
        d = xc.size(-1)
        rows = xc.numel() // d
        w32 = weight.detach().to(torch.float32).contiguous()
        b32 = bias.detach().to(torch.float32).contiguous()
        y = torch.empty_like(xc)
        mean = torch.empty(rows, dtype=torch.float32, device=dev)
        rstd = torch.empty(rows, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            rc = lib.hsa_layer_norm_fwd(c_void_p(xc.data_ptr()), c_void_p(w32.data_ptr()), c_void_p(b32.data_ptr()),
                                        c_void_p(y.data_ptr()), c_void_p(mean.data_ptr()), c_void_p(rstd.data_ptr()),
                                        rows, d, float(eps), _lib.dtype_code(xc), _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_layer_norm_fwd")
        ctx.save_for_backward(xc, w32, mean, rstd)
        ctx.param_dtypes = (weight.dtype, bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load()
        xc, w32, mean, rstd = ctx.saved_tensors
        dev = xc.device
        d = xc.size(-1)
        rows = xc.numel() // d
        dy = dy.contiguous()
        if dy.dtype != xc.dtype:
            dy = dy.to(xc.dtype)
        dx = torch.empty_like(xc)
        dgamma = torch.empty(d, dtype=torch.float32, device=dev)
        dbeta = torch.empty(d, dtype=torch.float32, device=dev)
        ctas = int(lib.hsa_layer_norm_bwd_ctas(rows))
        partial = torch.empty(ctas * 2 * d, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            rc = lib.hsa_layer_norm_bwd(c_void_p(xc.data_ptr()), c_void_p(dy.data_ptr()), c_void_p(w32.data_ptr()),
                                        c_void_p(mean.data_ptr()), c_void_p(rstd.data_ptr()), c_void_p(dx.data_ptr()),
                                        c_void_p(dgamma.data_ptr()), c_void_p(dbeta.data_ptr()),
                                        c_void_p(partial.data_ptr()), rows, d, _lib.dtype_code(xc), _lib.stream_ptr(dev))
        _lib.check(rc, "hsa_layer_norm_bwd")
        wd, bd = ctx.param_dtypes
        return dx, dgamma.to(wd), dbeta.to(bd), None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    d = x.size(-1)
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16, torch.float16) and _lib.load().hsa_layer_norm_supported(d):
        return _LayerNorm.apply(x, weight, bias, eps)
    return F.layer_norm(x, (d,), weight, bias, eps)


class LayerNorm(nn.LayerNorm):
    """Drop-in for nn.LayerNorm(d) (same parameters, same state_dict) running the library kernels."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if len(self.normalized_shape) != 1 or self.weight is None or self.bias is None:
            return super().forward(x)
        return layer_norm(x, self.weight, self.bias, self.eps)
