"""The attention module of the hierarchical attention path.

Mirrors hierarchical_attention/modules/attention.py of the reference project: same constructor,
parameter names (state_dict compatible), public methods and results.  Projections are nn.Linear
(cuBLAS); the tree work runs in the CUDA library through `..ops`.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn

from ..ops.functional import build_parent_nodes, hierarchical_attention
from ..ops.topology import build_tree_topology, generate_span_input_Y  # noqa: F401  (re-exported like the reference)


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

        # bottom-up (Y) projections
        self.Wq_y = nn.Linear(dim, dim, bias=False)
        self.Wk_y = nn.Linear(dim, dim, bias=False)
        self.Wv_y = nn.Linear(dim, dim, bias=False)
        self.out_proj_y = nn.Linear(dim, dim)
        # top-down (X) projections
        self.Wq_x = nn.Linear(dim, dim, bias=False)
        self.Wk_x = nn.Linear(dim, dim, bias=False)
        self.Wv_x = nn.Linear(dim, dim, bias=False)
        self.out_proj_x = nn.Linear(dim, dim)

        self.dropout = nn.Dropout(dropout)

        self.cached_tables = None
        self.cached_seq_len = -1
        self.cached_is_causal = None
        self.sizes: Optional[List[int]] = None
        self.offsets: Optional[List[int]] = None

    # -- helpers ---------------------------------------------------------------------------
    def _get_lookup_table(self, L: int, is_causal: bool, device: torch.device):
        if (self.cached_tables is not None and self.cached_seq_len == L
                and self.cached_is_causal == is_causal
                and self.cached_tables["forward_idx"].device == device):
            return self.cached_tables
        tables = build_tree_topology(L, is_causal=is_causal, device=device)
        self.cached_tables, self.cached_seq_len, self.cached_is_causal = tables, L, is_causal
        return tables

    def _build_level_info(self, N: int):
        sizes, curr = [], N
        while curr > 1:
            sizes.append(curr // 2)
            curr //= 2
        offsets = [0]
        for s in sizes[:-1]:
            offsets.append(offsets[-1] + s)
        return sizes, offsets

    # -- bottom-up -------------------------------------------------------------------------
    def cross_update_Y(self, x: torch.Tensor, y_in: torch.Tensor) -> torch.Tensor:
        B, N, D = x.shape
        H, Dh = self.num_heads, self.head_dim
        assert y_in is not None, "y_in cannot be None"
        assert y_in.size(1) == N - 1, f"y_in size {y_in.size(1)} mismatch! Expected N-1 ({N-1}) for N={N} leaves."
        # The reference caches the level sizes on first use and never refreshes them
        # (attention.py:92-93); here they follow N, so one module serves several lengths.
        if self.sizes is None or self.sizes[0] != N // 2:
            self.sizes, self.offsets = self._build_level_info(N)

        Q_p_all = self.Wq_y(y_in).view(B, -1, H, Dh)
        K_p_all = self.Wk_y(y_in).view(B, -1, H, Dh)
        V_p_all = self.Wv_y(y_in).view(B, -1, H, Dh)
        Q_p_levels = torch.split(Q_p_all, self.sizes, dim=1)
        K_p_levels = torch.split(K_p_all, self.sizes, dim=1)
        V_p_levels = torch.split(V_p_all, self.sizes, dim=1)

        new_Y_levels = []
        prev_sources = x
        K_leaves = self.Wk_y(prev_sources).view(B, -1, H, Dh)
        V_leaves = self.dropout(self.Wv_y(prev_sources).view(B, -1, H, Dh))

        for level, parent_count in enumerate(self.sizes):
            if level == 0:
                K_c = K_leaves
                V_c = self.dropout(V_leaves)   # applied twice at level 0, as attention.py:117,135 does
            else:
                K_c = self.Wk_y(prev_sources).view(B, -1, H, Dh)
                V_c = self.dropout(self.Wv_y(prev_sources).view(B, -1, H, Dh))
            updated_heads = build_parent_nodes(Q_p_levels[level], K_p_levels[level], V_p_levels[level], K_c, V_c)
            prev_sources = updated_heads.reshape(B, parent_count, D)
            new_Y_levels.append(prev_sources)

        return self.out_proj_y(torch.cat(new_Y_levels, dim=1))

    # -- top-down --------------------------------------------------------------------------
    def update_X_from_Y(self, x: torch.Tensor, y: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, N, D = x.shape
        H, Dh = self.num_heads, self.head_dim
        assert y is not None, "y (parents) cannot be None during top-down update"

        XY = torch.cat([x, y], dim=1)
        Q = self.Wq_x(x).view(B, N, H, Dh)
        K_full = self.Wk_x(XY).view(B, -1, H, Dh)
        V_full = self.dropout(self.Wv_x(XY).view(B, -1, H, Dh))

        is_causal = mask is not None
        tables = self._get_lookup_table(N, is_causal, device=x.device)
        out = hierarchical_attention(Q, K_full, V_full, tables["forward_idx"], tables["backward_gather"],
                                     tables["forward_mask"] if is_causal else None, self.window_size)
        return self.out_proj_x(out.view(B, N, D))

    def _standard_attention(self, Q, K, V, mask):
        scores = torch.matmul(Q, K.transpose(-1, -2)) / math.sqrt(Q.size(-1))
        if mask is not None:
            scores = scores.masked_fill(mask == 0, float("-inf"))
        attn = self.dropout(torch.softmax(scores, dim=-1))
        return torch.matmul(attn, V), attn

    def forward(self, query, key, value, y=None, mask=None, return_attention=False):
        x = query
        B, L_Q, D = x.size()
        H, Dh = self.num_heads, self.head_dim
        L_K, L_V = key.size(1), value.size(1)
        if L_Q == L_K == L_V and y is not None:
            output = self.update_X_from_Y(x, y, mask)
            return (output, None) if return_attention else output
        # dense attention when no parents are given (the reference's fallback branch, attention.py:257-270)
        Q = self.Wq_x(query).view(B, L_Q, H, Dh).transpose(1, 2)
        K = self.Wk_x(key).view(B, L_K, H, Dh).transpose(1, 2)
        V = self.Wv_x(value).view(B, L_V, H, Dh).transpose(1, 2)
        output_leaf, attn_weights = self._standard_attention(Q, K, V, mask)
        output = self.out_proj_x(output_leaf.transpose(1, 2).reshape(B, L_Q, D))
        return (output, attn_weights) if return_attention else output
