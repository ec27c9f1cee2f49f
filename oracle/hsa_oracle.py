"""CPU oracle for the hierarchical sparse attention path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain numpy / eager PyTorch on the CPU, the algorithm of
the reference project's `hierarchical_attention` package and of its eager twin
`HierarchicalSparseAttentionRef`.  It is the checker the parity tests, the smoke
check and the CPU-baseline leg of the benchmark compare the CUDA library with.
Nothing in the shipped package imports it, and it is never the thing measured
as the product.

Parity status: PINNED.  Every function below is checked (tests/test_oracle_golden.py)
against vectors generated in a container where the reference itself is importable,
by `tests/golden/make_golden.py`, from

  * the reference's own `build_tree_topology` and `generate_span_input_Y`,
  * the reference's eager layer `HierarchicalSparseAttentionRef`
    (forward, cross_update_Y and their autograd gradients), and
  * the reference's Triton package ops run under the Triton CPU interpreter
    (`build_parent_nodes`, `hierarchical_attention`, forward and backward).

Reference citations use paths inside the reference project.
"""
from __future__ import annotations

import functools
import hashlib
import math
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F


# ---------------------------------------------------------------------------
# Topology (integer work, numpy, bit-exact)
# ---------------------------------------------------------------------------

def build_tree_topology(seq_len: int, is_causal: bool = True) -> Dict[str, np.ndarray]:
    """Tables of hierarchical_attention/ops/topology.py:6-150, by explicit climbing.

    forward_idx[n, l]  : key row of the sibling subtree a leaf sees at level l
                         (topology.py:37-59; eager twin
                         hierarchical_attention_project/Hierarchical_Attention_Triton_Test.py:73-102)
    forward_mask[n, l] : True when that sibling lies to the right (future) and the
                         mode is causal (topology.py:49-57)
    backward_gather[r] : (start, end, level) = leaf range under r's sibling, for the
                         nodes that receive gradient (topology.py:103-122)
    """
    assert seq_len >= 1 and (seq_len & (seq_len - 1)) == 0, "seq_len must be power of 2"
    N = seq_len
    total = 2 * N - 1
    levels = int(math.log2(N))
    max_valid = total - 2

    fwd_idx = np.full((N, levels), -1, dtype=np.int32)
    fwd_mask = np.zeros((N, levels), dtype=np.bool_)
    for n in range(N):
        cur = n
        for lvl in range(levels):
            if lvl == 0:
                nxt, pair = cur ^ 1, cur
            else:
                pair = cur // 2 + N
                nxt = pair ^ 1
            if nxt <= max_valid:
                fwd_idx[n, lvl] = nxt
                if is_causal:
                    fwd_mask[n, lvl] = pair < nxt
            cur = nxt

    # subtree ranges and levels, bottom-up (topology.py:64-100)
    lo = np.zeros(total, dtype=np.int64)
    hi = np.zeros(total, dtype=np.int64)
    lev = np.zeros(total, dtype=np.int64)
    lo[:N] = np.arange(N)
    hi[:N] = np.arange(N) + 1
    start, count = 0, N
    for lvl in range(levels):
        nstart, ncount = start + count, count // 2
        for i in range(ncount):
            p = nstart + i
            lo[p] = lo[start + 2 * i]
            hi[p] = hi[start + 2 * i + 1]
            lev[p] = lvl + 1
        start, count = nstart, ncount

    gather = np.full((total, 3), -1, dtype=np.int32)
    for r in range(total):
        sib = min(r ^ 1, total - 1)          # topology.py:104-105
        take = (sib > r) if is_causal else (sib != r)
        take = take and (sib != r)           # root has no sibling (topology.py:115)
        if take:
            gather[r] = (lo[sib], hi[sib], lev[r])
    return {"forward_idx": fwd_idx, "forward_mask": fwd_mask, "backward_gather": gather}


def topology_digest(tables: Dict[str, np.ndarray]) -> str:
    """First 32 hex digits of sha256(idx int32 | mask 1 byte/elem | gather int32)."""
    h = hashlib.sha256()
    h.update(np.ascontiguousarray(tables["forward_idx"], dtype=np.int32).tobytes())
    h.update(np.ascontiguousarray(tables["forward_mask"], dtype=np.bool_).tobytes())
    h.update(np.ascontiguousarray(tables["backward_gather"], dtype=np.int32).tobytes())
    return h.hexdigest()[:32]


# ---------------------------------------------------------------------------
# generate_span_input_Y  (topology.py:153-169)
# ---------------------------------------------------------------------------

def generate_span_input_Y(x: torch.Tensor) -> Optional[torch.Tensor]:
    """Initial parents: pairwise mean pyramid of x, levels concatenated."""
    B, N, D = x.shape
    levels: List[torch.Tensor] = []
    cur = x
    while cur.size(1) > 1:
        n = cur.size(1)
        even = n - (n % 2)
        pairs = cur[:, :even, :].reshape(B, even // 2, 2, D)
        cur = 0.5 * pairs[:, :, 0, :] + 0.5 * pairs[:, :, 1, :]
        levels.append(cur)
    if not levels:
        return None
    return torch.cat(levels, dim=1)


# ---------------------------------------------------------------------------
# Op level: parent nodes (3-way attention)
# ---------------------------------------------------------------------------

def build_parent_nodes(Q_p, K_p, V_p, K_c, V_c, compute_dtype=torch.float32):
    """out[b,i,h] = softmax_j(scale q.k_j) . v_j over (self, child 2i, child 2i+1).

    Layout [B, P, H, D] / [B, 2P, H, D]; math of
    hierarchical_attention/ops/triton/build_parents.py:43-99 and of the eager twin
    (Hierarchical_Attention_Triton_Test.py:239-251).  Differentiable; the result is in
    `compute_dtype` (callers cast to the storage dtype when they compare).
    """
    B, P, H, D = Q_p.shape
    assert K_c.shape[1] == 2 * P
    q = Q_p.to(compute_dtype)
    k = torch.stack([K_p.to(compute_dtype),
                     K_c.to(compute_dtype)[:, 0::2], K_c.to(compute_dtype)[:, 1::2]], dim=3)  # B,P,H,3,D
    v = torch.stack([V_p.to(compute_dtype),
                     V_c.to(compute_dtype)[:, 0::2], V_c.to(compute_dtype)[:, 1::2]], dim=3)
    logits = torch.einsum("bphd,bphjd->bphj", q, k) / math.sqrt(D)
    w = F.softmax(logits, dim=-1)
    return torch.einsum("bphj,bphjd->bphd", w, v)


# ---------------------------------------------------------------------------
# Op level: span attention (window + one sibling node per level)
# ---------------------------------------------------------------------------

@functools.lru_cache(maxsize=16)
def span_candidates(N: int, radius: int, is_causal: bool):
    """(rows [N, 2R+1+L] int64, valid [N, 2R+1+L] bool): candidate key rows per leaf.

    Window slots follow Hierarchical_Attention_Triton_Test.py:281-304, level slots
    :309-324 (tables from build_tree_topology above).
    """
    t = build_tree_topology(N, is_causal)
    n = np.arange(N)[:, None]
    win = n + np.arange(-radius, radius + 1)[None, :]
    win_valid = (win >= 0) & (win < N)
    if is_causal:
        win_valid &= win <= n
    win = np.clip(win, 0, N - 1)
    lvl = t["forward_idx"].astype(np.int64)
    lvl_valid = lvl >= 0
    if is_causal:
        lvl_valid &= ~t["forward_mask"]
    lvl = np.where(lvl >= 0, lvl, 0)
    rows = np.concatenate([win, lvl], axis=1)
    valid = np.concatenate([win_valid, lvl_valid], axis=1)
    return torch.from_numpy(rows), torch.from_numpy(valid)


def hierarchical_attention(Q, K, V, radius: int, is_causal: bool, compute_dtype=torch.float32,
                           return_lse: bool = False, leaves: Optional[torch.Tensor] = None):
    """Span attention on given Q [B,N,H,D], K,V [B,2N-1,H,D] (leaves then parents).

    `leaves` (int64 indices) restricts the evaluation to those query rows (each leaf is
    independent); the result then has len(leaves) rows.

    Joint softmax over the valid window slots and level slots
    (hierarchical_attention/ops/triton/sparse_attn.py:57-179; eager twin :277-339).
    The level-0 sibling also sits inside the window for R >= 1 and is counted twice,
    as in the reference.  Differentiable.
    """
    B, N, H, D = Q.shape
    assert K.shape[1] == 2 * N - 1
    rows, valid = span_candidates(N, radius, is_causal)
    q = Q.to(compute_dtype)
    if leaves is not None:
        rows, valid, q = rows[leaves], valid[leaves], q[:, leaves]
    k = K.to(compute_dtype)[:, rows]            # B,N,C,H,D
    v = V.to(compute_dtype)[:, rows]
    logits = torch.einsum("bnhd,bnchd->bnhc", q, k) / math.sqrt(D)
    logits = logits.masked_fill(~valid[None, :, None, :], float("-inf"))
    m = logits.max(dim=-1, keepdim=True)[0]
    w = F.softmax(logits - m, dim=-1)
    out = torch.einsum("bnhc,bnchd->bnhd", w, v)
    if return_lse:
        return out, torch.logsumexp(logits, dim=-1)
    return out


def span_logits(Q, K, radius: int, is_causal: bool, weights: bool = False):
    """Candidate logits [B, N, H, 2R+1+L] of span attention (window slots, then level slots): scaled q.k, -inf at
    masked slots; weights=True gives the softmax weights with zeros at masked slots, the `Weights` tensor of
    hierarchical_attention/ops/functional.py:131-132 (kernel ops/triton/sparse_attn.py:57-145)."""
    B, N, H, D = Q.shape
    rows, valid = span_candidates(N, radius, is_causal)
    k = K.float()[:, rows]                                       # B,N,C,H,D
    logits = torch.einsum("bnhd,bnchd->bnhc", Q.float(), k) / math.sqrt(D)
    logits = logits.masked_fill(~valid[None, :, None, :], float("-inf"))
    return F.softmax(logits, dim=-1) if weights else logits


def sibling_logits(ALL_Q, ALL_K, H: int, D: int, seq_len: int):
    """build_hierarchical_logits of the first prototype (Hierarchical_Attention_Triton.py:456-514):
    RES_SELF[b,t,h] = q_t.k_t / sqrt(D) for t < seq_len (:327-393, as its launcher and commented body state),
    RES_CROSS[b,r,h] = q_{r^1}.k_r / sqrt(D) for r < total_nodes-1 (:414-454)."""
    B, total, _ = ALL_Q.shape
    q = ALL_Q.float().view(B, total, H, D)
    k = ALL_K.float().view(B, total, H, D)
    res_self = (q[:, :seq_len] * k[:, :seq_len]).sum(-1) / math.sqrt(D)
    r = torch.arange(total - 1)
    res_cross = (q[:, r ^ 1] * k[:, r]).sum(-1) / math.sqrt(D)
    return res_self, res_cross


# ---------------------------------------------------------------------------
# Module level: the layer (restates HierarchicalSparseAttentionRef,
# Hierarchical_Attention_Triton_Test.py:107-374; same parameter names as the package
# module hierarchical_attention/modules/attention.py:20-29)
# ---------------------------------------------------------------------------

class HierarchicalAttentionOracle(nn.Module):
    def __init__(self, dim: int, num_heads: int, dropout: float = 0.1, window_size: int = 16):
        super().__init__()
        self.dim, self.num_heads, self.head_dim = dim, num_heads, dim // num_heads
        self.window_size = window_size
        self.Wq_y = nn.Linear(dim, dim, bias=False)
        self.Wk_y = nn.Linear(dim, dim, bias=False)
        self.Wv_y = nn.Linear(dim, dim, bias=False)
        self.out_proj_y = nn.Linear(dim, dim)
        # The eager twin owns an unused merge_layer at this point (Test.py:124); drawing and
        # dropping one keeps seeded initialisation identical to the twin's.
        nn.Linear(2 * dim, dim)
        self.Wq_x = nn.Linear(dim, dim, bias=False)
        self.Wk_x = nn.Linear(dim, dim, bias=False)
        self.Wv_x = nn.Linear(dim, dim, bias=False)
        self.out_proj_x = nn.Linear(dim, dim)
        self.dropout = nn.Dropout(dropout)

    @staticmethod
    def level_sizes(N: int) -> List[int]:
        sizes, cur = [], N
        while cur > 1:
            sizes.append(cur // 2)
            cur //= 2
        return sizes

    def cross_update_Y(self, x, y_in):
        """Bottom-up refresh of the parents (Test.py:201-256 / attention.py:79-162)."""
        B, N, D = x.shape
        H, Dh = self.num_heads, self.head_dim
        assert y_in is not None and y_in.size(1) == N - 1
        sizes = self.level_sizes(N)
        Qs = torch.split(self.Wq_y(y_in).view(B, -1, H, Dh), sizes, dim=1)
        Ks = torch.split(self.Wk_y(y_in).view(B, -1, H, Dh), sizes, dim=1)
        Vs = torch.split(self.Wv_y(y_in).view(B, -1, H, Dh), sizes, dim=1)
        prev = x
        outs = []
        for level, P in enumerate(sizes):
            K_c = self.Wk_y(prev).view(B, -1, H, Dh)
            V_c = self.dropout(self.Wv_y(prev).view(B, -1, H, Dh))
            o = build_parent_nodes(Qs[level], Ks[level], Vs[level], K_c, V_c, compute_dtype=x.dtype)
            prev = o.reshape(B, P, D)
            outs.append(prev)
        return self.out_proj_y(torch.cat(outs, dim=1))

    def update_X_from_Y(self, x, y, mask=None):
        """Top-down span attention (Test.py:258-341 / attention.py:165-220)."""
        B, N, D = x.shape
        H, Dh = self.num_heads, self.head_dim
        assert y is not None
        XY = torch.cat([x, y], dim=1)
        Q = self.Wq_x(x).view(B, N, H, Dh)
        K = self.Wk_x(XY).view(B, -1, H, Dh)
        V = self.dropout(self.Wv_x(XY).view(B, -1, H, Dh))
        o = hierarchical_attention(Q, K, V, self.window_size, mask is not None, compute_dtype=x.dtype)
        return self.out_proj_x(o.reshape(B, N, D))

    def forward(self, query, key, value, y=None, mask=None, return_attention=False):
        assert y is not None and query.size(1) == key.size(1) == value.size(1)
        out = self.update_X_from_Y(query, y, mask)
        return (out, None) if return_attention else out


def lm_loss_reference(model, tokens, label_smoothing: float = 0.1, ignore_index: int = -100):
    """The reference's criterion on a [B, N+1] token window: nn.CrossEntropyLoss(ignore_index, label_smoothing)
    on logits of window[:, :-1] against window[:, 1:]
    (hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:181-194, 514, 562-572)."""
    logits = model(tokens[:, :-1])
    return F.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), tokens[:, 1:].reshape(-1),
                           label_smoothing=label_smoothing, ignore_index=ignore_index)
