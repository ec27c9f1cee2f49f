"""Training-loop helpers for models built on the hierarchical attention layer.

`GraphedStep` captures one whole training step (forward, loss, backward, gradient all-reduce, clipping,
optimizer update) into a CUDA graph and replays it: a step of the hierarchical LM launches a few thousand
small kernels (one group per tree level, layer and direction), and on B200 issuing them from Python costs more
host time than the GPU needs to run them.  The reference trains eagerly
(hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:540-590); this is the launch-overhead
remedy its author asks for in hierarchical_attention/ops/triton/build_parents.py:207-216, applied to the
whole step instead of one kernel.

    step = GraphedStep(body, device)        # body() works on static tensors only (copy new inputs into them)
    for batch in loader:
        static_tokens.copy_(batch, non_blocking=True)
        step()

Rules for `body`: no host synchronisation (no .item(), no python branching on tensor values), every tensor it
reads or writes keeps its address between calls, optimizers are built with capturable=True, and NCCL
collectives inside it are fine (they are captured with the rest).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


class GraphedStep:
    def __init__(self, body: Callable[[], None], device: torch.device, warmup: int = 3, enabled: bool = True):
        self.body = body
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.error: Optional[str] = None
        if not enabled:
            return
        try:
            # warm up on a side stream (allocator pools, lazy initialisation, autotuned library calls)
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                for _ in range(max(1, warmup)):
                    body()
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                body()
            self.graph = graph
        except Exception as exc:                                  # capture refused: run eagerly
            self.graph = None
            self.error = f"{type(exc).__name__}: {exc}"[:300]
            torch.cuda.synchronize(device)

    @property
    def captured(self) -> bool:
        return self.graph is not None

    def drop_graph(self) -> None:
        """Fall back to eager launches (all ranks of a job have to take the same path)."""
        self.graph = None

    def __call__(self) -> None:
        if self.graph is not None:
            self.graph.replay()
        else:
            self.body()
