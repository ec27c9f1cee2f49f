"""Data-parallel gradient averaging for one process per GPU (torch.distributed, NCCL over NVLink).

The reference has no multi-process training (it only wraps the model in nn.DataParallel,
hierarchical_attention_project/Hierarchical_Transformer_Triton_WikiText103.py:619-624); this is the
batch-sharded equivalent.  Gradients are gathered into a few flat buckets in reverse layer order (one
multi-tensor copy per bucket when its last gradient has arrived); a bucket is all-reduced asynchronously at
that moment, so the transfers overlap the rest of the backward, and afterwards the parameters' .grad are
views into the averaged buckets.
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
        # the flat buckets are used whenever the job has more than one rank (also with communicate=False, so that only
        # the collective itself is left out of that comparison); a single process keeps autograd's own gradient tensors
        self.bucketed = dist.is_initialized() and dist.get_world_size(process_group) > 1
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
        views, off = [], 0
        for p in plist:
            views.append(flat[off: off + p.numel()].view_as(p))
            off += p.numel()
        self.buckets.append({"params": list(plist), "flat": flat, "pending": len(plist), "views": views})

    def _make_hook(self, bi: int):
        def hook(param):
            b = self.buckets[bi]
            b["pending"] -= 1
            if b["pending"] == 0 and self.bucketed:
                # the bucket's gradients are complete: one multi-tensor copy into the flat buffer, then its all-reduce.
                # A bucket of one parameter (the tied embedding / head matrix, whose gradient arrives last) is reduced
                # where autograd left it: no copy stands between the end of the backward and the collective.
                single = len(b["params"]) == 1 and b["params"][0].grad.is_contiguous()
                b["reduced"] = b["params"][0].grad if single else b["flat"]
                if not single:
                    torch._foreach_copy_(b["views"], [p.grad for p in b["params"]])
                if self.world > 1:
                    op = dist.ReduceOp.AVG if self._avg_op else dist.ReduceOp.SUM
                    self._handles.append((dist.all_reduce(b["reduced"], op=op, group=self.group, async_op=True), bi))
        return hook

    def zero_grad(self):
        """Drop last step's gradients.  Autograd then hands each parameter its gradient as a fresh tensor (no zero fill,
        no `grad += new` kernel per parameter); the flat buckets are filled by one copy per bucket when it is complete."""
        for b in self.buckets:
            b["pending"] = len(b["params"])
        for p in self.params:
            p.grad = None

    def finish(self):
        """Wait for the outstanding all-reduces of this backward; `.grad` of every parameter then is the averaged
        gradient (a view into its bucket when the job has more than one rank)."""
        for h, bi in self._handles:
            h.wait()
            if not self._avg_op and self.world > 1:
                self.buckets[bi]["reduced"].div_(self.world)
        self._handles.clear()
        for b in self.buckets:
            if b["pending"] != 0 and self.world > 1:
                raise RuntimeError("a parameter received no gradient this step; its bucket was never reduced")
            if self.bucketed and b["pending"] == 0 and b.get("reduced") is b["flat"]:
                for p, v in zip(b["params"], b["views"]):
                    p.grad = v

    def bytes_per_step(self) -> int:
        return sum(b["flat"].numel() * b["flat"].element_size() for b in self.buckets)
