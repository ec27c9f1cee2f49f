"""The attention module of the hierarchical attention path.

Public surface of hierarchical_attention/modules/attention.py of the reference project — constructor,
parameter names (state_dict compatible), `forward`, `cross_update_Y`, `update_X_from_Y`, the cache
attributes — with the device work in the CUDA library (`..ops`) and the projections arranged for it:

  * projections that read the same input run as ONE GEMM against the row-stacked weights
    ([Wq_y; Wk_y; Wv_y] on the parents, [Wk_y; Wv_y] on every level's children, [Wk_x; Wv_x] on
    leaves+parents); Q/K/V are then strided views of that result, which the kernels consume as they
    are (row stride = 2d or 3d, no copies, half to a third of the GEMM launches);
  * level slices of the parent projections stay batch-strided views (no `.contiguous()` per level).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.functional import build_parent_nodes, hierarchical_attention
from ..ops.topology import build_tree_topology, generate_span_input_Y  # noqa: F401  (re-exported like the reference)


def _stacked_projection(inp: torch.Tensor, layers: Sequence[nn.Linear], heads: int) -> Tuple[torch.Tensor, ...]:
    """Apply several bias-free Linear layers of equal shape to `inp` [B, rows, d] with one GEMM.

    Returns one [B, rows, heads, d/heads] view per layer; the views share storage (row stride len(layers)*d).
    """
    weight = torch.cat([layer.weight for layer in layers], dim=0)
    out = F.linear(inp, weight)
    B, rows, _ = out.shape
    d = layers[0].weight.size(0)
    # unbind (not indexing): its backward writes the stacked gradient once instead of zero-filling per view
    return out.view(B, rows, len(layers), heads, d // heads).unbind(dim=2)


class HierarchicalAttention(nn.Module):
    """Binary-tree hierarchical sparse attention (reference: attention.py:10-270).

    forward(query, key, value, y=None, mask=None, return_attention=False)
        hierarchical mode when `y` is given and the three lengths agree: leaves attend to a
        radius-`window_size` window plus one sibling node per level of the parents `y`;
        `mask is not None` selects the causal variant (its content is not read).
    cross_update_Y(x, y_in)  bottom-up refresh of the parents from x.
    update_X_from_Y(x, y, mask=None)  the top-down pass used by forward.
    """

    def __init__(self, dim: int, num_heads: int, dropout: float = 0.1, window_size: int = 16):
        super().__init__()
        self.dim = dim
        self.num_heads = num_heads
        self.head_dim = dim // num_heads
        self.window_size = window_size
        # parameter names and creation order follow the reference (attention.py:20-29)
        for name in ("Wq_y", "Wk_y", "Wv_y"):
            setattr(self, name, nn.Linear(dim, dim, bias=False))
        self.out_proj_y = nn.Linear(dim, dim)
        for name in ("Wq_x", "Wk_x", "Wv_x"):
            setattr(self, name, nn.Linear(dim, dim, bias=False))
        self.out_proj_x = nn.Linear(dim, dim)
        self.dropout = nn.Dropout(dropout)

        self.cached_tables = None
        self.cached_seq_len = -1
        self.cached_is_causal = None
        self.sizes: Optional[List[int]] = None
        self.offsets: Optional[List[int]] = None

    # ------------------------------------------------------------------ cached host-side state
    def _get_lookup_table(self, L: int, is_causal: bool, device: torch.device):
        hit = (self.cached_tables is not None and self.cached_seq_len == L and self.cached_is_causal == is_causal
               and self.cached_tables["forward_idx"].device == device)
        if not hit:
            self.cached_tables = build_tree_topology(L, is_causal=is_causal, device=device)
            self.cached_seq_len, self.cached_is_causal = L, is_causal
        return self.cached_tables

    @staticmethod
    def _build_level_info(N: int):
        sizes = [N >> l for l in range(1, N.bit_length()) if (N >> l) >= 1]
        offsets = [0]
        for s in sizes[:-1]:
            offsets.append(offsets[-1] + s)
        return sizes, offsets

    # ------------------------------------------------------------------ bottom-up: leaves -> parents
    def cross_update_Y(self, x: torch.Tensor, y_in: torch.Tensor) -> torch.Tensor:
        B, N, D = x.shape
        H = self.num_heads
        assert y_in is not None, "y_in cannot be None"
        assert y_in.size(1) == N - 1, f"y_in size {y_in.size(1)} mismatch! Expected N-1 ({N-1}) for N={N} leaves."
        # The reference computes the level sizes once and keeps them for good (attention.py:92-93); here they
        # follow N, so one module serves several sequence lengths.
        if self.sizes is None or self.sizes[0] != N // 2:
            self.sizes, self.offsets = self._build_level_info(N)

        # all parents at once: one GEMM, then per-level (batch-strided) slices
        q_all, k_all, v_all = _stacked_projection(y_in, (self.Wq_y, self.Wk_y, self.Wv_y), H)
        q_lv = torch.split(q_all, self.sizes, dim=1)
        k_lv = torch.split(k_all, self.sizes, dim=1)
        v_lv = torch.split(v_all, self.sizes, dim=1)

        children = x
        refreshed = []
        for level, count in enumerate(self.sizes):
            k_c, v_c = _stacked_projection(children, (self.Wk_y, self.Wv_y), H)
            v_c = self.dropout(v_c)
            if level == 0:
                v_c = self.dropout(v_c)          # the reference drops the leaf values twice (attention.py:117,135)
            heads = build_parent_nodes(q_lv[level], k_lv[level], v_lv[level], k_c, v_c)
            children = heads.reshape(B, count, D)   # this level's parents are the next level's children
            refreshed.append(children)
        return self.out_proj_y(torch.cat(refreshed, dim=1))

    # ------------------------------------------------------------------ top-down: parents -> leaves
    def update_X_from_Y(self, x: torch.Tensor, y: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, N, D = x.shape
        H, Dh = self.num_heads, self.head_dim
        assert y is not None, "y (parents) cannot be None during top-down update"

        q = self.Wq_x(x).view(B, N, H, Dh)
        k, v = _stacked_projection(torch.cat([x, y], dim=1), (self.Wk_x, self.Wv_x), H)   # rows: leaves, then parents
        v = self.dropout(v)

        is_causal = mask is not None
        tables = self._get_lookup_table(N, is_causal, device=x.device)
        out = hierarchical_attention(q, k, v, tables["forward_idx"], tables["backward_gather"],
                                     tables["forward_mask"] if is_causal else None, self.window_size)
        return self.out_proj_x(out.reshape(B, N, D))

    # ------------------------------------------------------------------ dense attention when no parents are given
    def _standard_attention(self, Q, K, V, mask):
        scores = (Q @ K.transpose(-1, -2)) * (1.0 / math.sqrt(Q.size(-1)))
        if mask is not None:
            scores = scores.masked_fill(mask == 0, float("-inf"))
        attn = self.dropout(scores.softmax(dim=-1))
        return attn @ V, attn

    def forward(self, query, key, value, y=None, mask=None, return_attention=False):
        B, L_Q, D = query.shape
        if y is not None and L_Q == key.size(1) == value.size(1):
            output = self.update_X_from_Y(query, y, mask)
            return (output, None) if return_attention else output
        # the reference's fallback branch (attention.py:257-270): plain multi-head attention on the X projections
        H, Dh = self.num_heads, self.head_dim
        split = lambda t, proj: proj(t).view(B, t.size(1), H, Dh).transpose(1, 2)        # noqa: E731
        ctx, weights = self._standard_attention(split(query, self.Wq_x), split(key, self.Wk_x),
                                                split(value, self.Wv_x), mask)
        output = self.out_proj_x(ctx.transpose(1, 2).reshape(B, L_Q, D))
        return (output, weights) if return_attention else output
