"""Decoder-only language model built on the hierarchical attention layer.

Restates the caller of the hot path in the reference project,
hierarchical_attention_project/Hierarchical_Transformer_Pretrain.py:331-481
(PositionwiseFeedForward, PositionalEncoding, DecoderLayer, TransformerLM), so the layer can be
measured inside the training step the reference measures.  Differences from the reference classes:
  * DecoderLayer does not create the `alpha_proj` / `beta_proj` Linear layers: the reference never
    uses them in forward (Pretrain.py:374-375, 391-399), and unused parameters break gradient
    all-reduce bookkeeping; load a reference checkpoint with strict=False;
  * the causal "mask" handed to the layers is a 1-element tensor: the layer only tests it for
    `is not None` (the reference builds an N x N boolean matrix per forward for that purpose);
  * the attention class and the span initialiser are constructor arguments, so tests can run the
    same model around the CPU oracle (which then also keeps nn.LayerNorm);
  * the three LayerNorms of a decoder layer run the library's kernels (`ops.norm.LayerNorm`, same parameters):
    nn.LayerNorm's backward was the single largest item of the training step on B200;
  * the tied embedding / output matrix is stored with its vocabulary dimension padded up to a multiple
    of 64 rows (50257 -> 50304).  The extra rows are never looked up and their logits are cut off before
    the loss, so the function computed is unchanged; the padding only lets the library GEMM of the LM
    head use aligned tensor-core tiles (an odd vocabulary size sends cuBLAS to its legacy kernels,
    about 9x slower on B200).  `vocab_size` rows of a reference checkpoint go into the first rows.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .modules.attention import HierarchicalAttention
from .ops.loss import cross_entropy
from .ops.norm import LayerNorm
from .ops.topology import generate_span_input_Y


class PositionwiseFeedForward(nn.Module):
    def __init__(self, d_model: int, d_ff: int, dropout: float = 0.1):
        super().__init__()
        self.fc1 = nn.Linear(d_model, d_ff)
        self.fc2 = nn.Linear(d_ff, d_model)
        self.dropout = nn.Dropout(p=dropout)

    def forward(self, x):
        return self.fc2(self.dropout(F.relu(self.fc1(x))))


class PositionalEncoding(nn.Module):
    def __init__(self, d_model: int, dropout: float, max_len: int = 5000):
        super().__init__()
        self.dropout = nn.Dropout(p=dropout)
        pe = torch.zeros(max_len, d_model)
        position = torch.arange(0.0, max_len).unsqueeze(1)
        div_term = torch.exp(torch.arange(0.0, d_model, 2) * -(math.log(10000.0) / d_model))
        pe[:, 0::2] = torch.sin(position * div_term)
        pe[:, 1::2] = torch.cos(position * div_term)
        self.register_buffer("pe", pe.unsqueeze(0))

    def forward(self, x):
        return self.dropout(x + self.pe[:, : x.size(1), :])


class DecoderLayer(nn.Module):
    """Pre-LN block: refresh the parents, span attention on the leaves, feed-forward."""

    def __init__(self, d_model: int, num_heads: int, d_ff: int, dropout: float = 0.1, window_size: int = 16,
                 attention_cls: Callable[..., nn.Module] = HierarchicalAttention):
        super().__init__()
        self.self_attn = attention_cls(d_model, num_heads, dropout, window_size=window_size)
        self.feed_forward = PositionwiseFeedForward(d_model, d_ff, dropout)
        norm_cls = LayerNorm if attention_cls is HierarchicalAttention else nn.LayerNorm
        self.norm1 = norm_cls(d_model)
        self.norm2 = norm_cls(d_model)
        self.norm_y = norm_cls(d_model)
        self.dropout = nn.Dropout(dropout)

    def forward(self, x, y, mask=None, return_attention: bool = False):
        y_delta = self.self_attn.cross_update_Y(x, y_in=self.norm_y(y))
        y_next = y + self.dropout(y_delta)
        norm_x = self.norm1(x)
        if return_attention:
            attn_output, weights = self.self_attn(norm_x, norm_x, norm_x, y=y_next, mask=mask, return_attention=True)
        else:
            attn_output, weights = self.self_attn(norm_x, norm_x, norm_x, y=y_next, mask=mask), None
        x = x + self.dropout(attn_output)
        x = x + self.dropout(self.feed_forward(self.norm2(x)))
        if return_attention:
            return x, y_next, weights
        return x, y_next


class TransformerLM(nn.Module):
    def __init__(self, vocab_size: int, d_model: int, num_heads: int, d_ff: int, num_layers: int,
                 dropout: float = 0.1, window_size: int = 16, max_len: int = 5000,
                 attention_cls: Callable[..., nn.Module] = HierarchicalAttention,
                 span_init: Callable[[torch.Tensor], Optional[torch.Tensor]] = generate_span_input_Y):
        super().__init__()
        self.vocab_size = vocab_size
        self.vocab_padded = (vocab_size + 63) // 64 * 64
        self.embedding = nn.Embedding(self.vocab_padded, d_model)
        self.pos_encoding = PositionalEncoding(d_model, dropout=dropout, max_len=max_len)
        self.layers = nn.ModuleList([
            DecoderLayer(d_model, num_heads, d_ff, dropout, window_size, attention_cls) for _ in range(num_layers)])
        self.fc_out = nn.Linear(d_model, self.vocab_padded)
        self.fc_out.weight = self.embedding.weight          # weight tying, as the reference
        self.d_model = d_model
        self._span_init = span_init
        self.apply(self._init_weights)

    @staticmethod
    def _init_weights(module):
        if isinstance(module, nn.Linear):
            torch.nn.init.normal_(module.weight, mean=0.0, std=0.02)
            if module.bias is not None:
                torch.nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            torch.nn.init.normal_(module.weight, mean=0.0, std=0.02)

    def forward(self, trg, return_attention: bool = False, padded_logits: bool = False):
        """Logits [B, N, vocab_size]; with padded_logits=True the [B, N, vocab_padded] tensor the LM head
        produces (columns >= vocab_size are padding), which `lm_loss` consumes without a copy."""
        x = self.embedding(trg) * math.sqrt(self.d_model)
        x = self.pos_encoding(x)
        y = self._span_init(x)
        causal_flag = torch.ones(1, dtype=torch.bool, device=trg.device)    # only `is not None` matters
        for layer in self.layers:
            if return_attention:
                x, y, _ = layer(x, y, mask=causal_flag, return_attention=True)
            else:
                x, y = layer(x, y, mask=causal_flag)
        logits = self.fc_out(x)
        return logits if padded_logits else logits[..., : self.vocab_size]


def zipf_tokens(batch: int, length: int, vocab: int, seed: int, s: float = 1.1, device="cpu") -> torch.Tensor:
    """[batch, length] token ids, rank r drawn with probability proportional to r^-s (id = r - 1)."""
    gen = torch.Generator().manual_seed(seed)
    pmf = torch.arange(1, vocab + 1, dtype=torch.float64).pow(-s)
    ids = torch.multinomial((pmf / pmf.sum()).float(), batch * length, replacement=True, generator=gen)
    return ids.view(batch, length).to(device)


def lm_loss(model: "TransformerLM", tokens: torch.Tensor, label_smoothing: float = 0.1,
            ignore_index: int = -100) -> torch.Tensor:
    """Next-token cross entropy on a [B, N+1] window: input = window[:, :-1], labels = window[:, 1:]
    (the reference's loader and criterion, Pretrain.py:181-194, 514), computed by the library's
    cross-entropy kernel straight on the padded logits."""
    logits = model(tokens[:, :-1], padded_logits=True)
    return cross_entropy(logits.reshape(-1, logits.size(-1)), tokens[:, 1:].reshape(-1), model.vocab_size,
                         label_smoothing=label_smoothing, ignore_index=ignore_index)
