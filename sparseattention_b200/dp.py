"""Data-parallel gradient averaging for one process per GPU (torch.distributed, NCCL over NVLink).

The reference has no multi-process training (it only wraps the model in nn.DataParallel,
hierarchical_attention_project/Hierarchical_Transformer_Triton_WikiText103.py:619-624); this is the
batch-sharded equivalent.  All gradients live in a few flat buckets (parameters' .grad are views into
them), filled by autograd in reverse layer order; a bucket is all-reduced asynchronously the moment
its last gradient has been accumulated, so the transfers overlap the rest of the backward.
"""
from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist


class BucketedGradAverager:
    def __init__(self, params, bucket_bytes: int = 32 << 20, process_group=None, communicate: bool = True):
        """`communicate=False` keeps the bucket layout and the bookkeeping but leaves the collectives out
        (each rank then trains on its own shard alone): what a benchmark compares a step against to see how
        much of the all-reduce time is left exposed."""
        self.group = process_group
        self.world = dist.get_world_size(process_group) if (dist.is_initialized() and communicate) else 1
        self.params = [p for p in params if p.requires_grad]
        backend = dist.get_backend(process_group) if dist.is_initialized() else "none"
        self._avg_op = backend == "nccl"            # gloo has no AVG: sum, then scale
        # buckets in reverse registration order = roughly the order gradients become ready
        self.buckets: List[dict] = []
        cur, cur_bytes = [], 0
        for p in reversed(self.params):
            nbytes = p.numel() * p.element_size()
            if cur and (cur_bytes + nbytes > bucket_bytes or p.dtype != cur[0].dtype):
                self._close(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
        if cur:
            self._close(cur)
        self._handles = []
        for bi, b in enumerate(self.buckets):
            for p in b["params"]:
                p.register_post_accumulate_grad_hook(self._make_hook(bi))

    def _close(self, plist):
        flat = torch.zeros(sum(p.numel() for p in plist), dtype=plist[0].dtype, device=plist[0].device)
        off = 0
        for p in plist:
            p.grad = flat[off: off + p.numel()].view_as(p)
            off += p.numel()
        self.buckets.append({"params": list(plist), "flat": flat, "pending": len(plist), "views": [p.grad for p in plist]})

    def _make_hook(self, bi: int):
        def hook(param):
            b = self.buckets[bi]
            b["pending"] -= 1
            if b["pending"] == 0 and self.world > 1:
                op = dist.ReduceOp.AVG if self._avg_op else dist.ReduceOp.SUM
                self._handles.append((dist.all_reduce(b["flat"], op=op, group=self.group, async_op=True), bi))
        return hook

    def zero_grad(self):
        """Clear the flat buckets and re-point .grad at them (an optimizer may have replaced them)."""
        for b in self.buckets:
            b["flat"].zero_()
            b["pending"] = len(b["params"])
            for p, v in zip(b["params"], b["views"]):
                p.grad = v

    def finish(self):
        """Wait for the outstanding all-reduces of this backward; gradients are then averaged."""
        for h, bi in self._handles:
            h.wait()
            if not self._avg_op and self.world > 1:
                self.buckets[bi]["flat"].div_(self.world)
        self._handles.clear()
        for b in self.buckets:
            if b["pending"] != 0 and self.world > 1:
                raise RuntimeError("a parameter received no gradient this step; its bucket was never reduced")

    def bytes_per_step(self) -> int:
        return sum(b["flat"].numel() * b["flat"].element_size() for b in self.buckets)
