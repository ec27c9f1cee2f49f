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
from .ops.loss import cross_entropy, linear_cross_entropy
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
        self.fused = True           # set False to force the eager path (the numerical reference of the fused one)

    def forward(self, x, y, mask=None, return_attention: bool = False):
        if self.fused and not return_attention and type(self.self_attn) is HierarchicalAttention:
            from .fused_layer import fused_decoder_layer, fused_layer_supported
            if fused_layer_supported(self, x, y, mask):
                # bf16 autocast on CUDA: the whole layer as one autograd node (tcgen05 products with fused tails)
                return fused_decoder_layer(self, x, y, mask)
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

    def _bf16_weights(self, x, y, mask):
        """The layers' bfloat16 weight copies, refreshed for this call, when every layer takes the fused path."""
        layers = list(self.layers)
        if not layers or not all(layer.fused and type(layer.self_attn) is HierarchicalAttention for layer in layers):
            return None
        from .fused_layer import Bf16Weights, fused_layer_supported
        if not fused_layer_supported(layers[0], x, y, mask):
            return None
        cache = getattr(self, "_w16_cache", None)
        if cache is None or not cache.matches(layers):
            cache = Bf16Weights(layers)
            object.__setattr__(self, "_w16_cache", cache)       # not a parameter, buffer or submodule
        cache.refresh()
        return cache

    def forward(self, trg, return_attention: bool = False, padded_logits: bool = False, hidden_only: bool = False):
        """Logits [B, N, vocab_size]; with padded_logits=True the [B, N, vocab_padded] tensor the LM head
        produces (columns >= vocab_size are padding), which `lm_loss` consumes without a copy; with
        hidden_only=True the last hidden states [B, N, d_model] (the LM head is then applied by the caller)."""
        x = self.embedding(trg) * math.sqrt(self.d_model)
        x = self.pos_encoding(x)
        y = self._span_init(x)
        causal_flag = torch.ones(1, dtype=torch.bool, device=trg.device)    # only `is not None` matters
        w16 = None if return_attention else self._bf16_weights(x, y, causal_flag)
        for i, layer in enumerate(self.layers):
            if return_attention:
                x, y, _ = layer(x, y, mask=causal_flag, return_attention=True)
            else:
                layer._w16 = None if w16 is None else w16.per_layer[i]
                try:
                    x, y = layer(x, y, mask=causal_flag)
                finally:
                    layer._w16 = None            # a layer called on its own converts its weights itself
        if hidden_only:
            return x
        logits = self.fc_out(x)
        return logits if padded_logits else logits[..., : self.vocab_size]


class IncrementalDecoder:
    """Token-by-token evaluation of a TransformerLM with per-layer caches, giving the logits the full forward
    would give at each position without re-running it (the reference's generate() re-runs the whole model for
    every new token: Hierarchical_Transformer_Pretrain.py:483-504).

    It rests on the layer being causal: leaf n attends to leaves <= n and to LEFT sibling nodes only, and a
    node's value depends only on the leaves under it.  So everything computed for position n stays valid, and
    a parent node is computed exactly once, when its last leaf arrives (node j of level l completes at
    n = (j+1) * 2^l - 1).  Per layer the decoder keeps, for every leaf and completed node: the child key/value
    projections the bottom-up pass consumes (Wk_y / Wv_y of the row's output), the parent stream y entering
    the layer, and the key/value rows of the top-down pass (Wk_x / Wv_x).  One step costs O(log N) rows per layer.

    `capacity` (a power of two) is the longest sequence the caches hold; logits at position n equal those of
    model(tokens[:, :M])[:, n] for any power-of-two M > n, in eval mode.
    """

    def __init__(self, model: "TransformerLM", batch: int, capacity: int, dtype: Optional[torch.dtype] = None):
        assert capacity >= 2 and capacity & (capacity - 1) == 0, "capacity must be a power of two"
        self.model = model.eval()
        p = next(model.parameters())
        self.dev, self.dtype = p.device, (dtype or p.dtype)
        self.B, self.N, self.d = batch, capacity, model.d_model
        rows = 2 * capacity - 1
        attn0 = model.layers[0].self_attn
        self.H, self.Dh = attn0.num_heads, attn0.head_dim
        new = lambda *shape: torch.zeros(*shape, dtype=self.dtype, device=self.dev)   # noqa: E731
        nl = len(model.layers)
        self.y0 = new(batch, rows, self.d)                       # row r: x0 of leaf r, or the initial value of node r
        self.y_in = [new(batch, rows, self.d) for _ in range(nl + 1)]      # parent stream entering layer i (node rows)
        self.kc = [new(batch, rows, self.H, self.Dh) for _ in range(nl)]   # Wk_y of each row's bottom-up output
        self.vc = [new(batch, rows, self.H, self.Dh) for _ in range(nl)]
        self.K = [new(batch, rows, self.H, self.Dh) for _ in range(nl)]    # top-down keys / values
        self.V = [new(batch, rows, self.H, self.Dh) for _ in range(nl)]
        self.n = 0

    @staticmethod
    def _row(N: int, level: int, j: int) -> int:
        return j if level == 0 else 2 * N - (N >> (level - 1)) + j

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """Consume the tokens [B] of position self.n; returns the logits [B, vocab_size] of that position."""
        from .ops.functional import build_parent_nodes, span_attention_decode
        m, n, N, B, H, Dh = self.model, self.n, self.N, self.B, self.H, self.Dh
        assert n < N, "cache capacity exhausted"
        x = m.embedding(tokens.view(B)) * math.sqrt(self.d) + m.pos_encoding.pe[0, n]
        x = x.to(self.dtype)
        # levels whose node completes with this leaf: 1 .. (number of trailing ones of n)
        done = 0
        while done < N.bit_length() - 1 and (n >> done) & 1:
            done += 1
        # initial parents (pairwise means of the level below; generate_span_input_Y)
        self.y0[:, n] = x
        for l in range(1, done + 1):
            j = n >> l
            c0 = self._row(N, l - 1, 2 * j)
            self.y0[:, self._row(N, l, j)] = 0.5 * self.y0[:, c0] + 0.5 * self.y0[:, c0 + 1]
            self.y_in[0][:, self._row(N, l, j)] = self.y0[:, self._row(N, l, j)]
        for i, layer in enumerate(m.layers):
            at = layer.self_attn
            lin = lambda w, t: F.linear(t, w.weight)               # noqa: E731
            heads = lambda t: t.view(B, 1, H, Dh)                  # noqa: E731
            # ---- bottom-up: this leaf's child projections, then every node that completes now
            self.kc[i][:, n] = lin(at.Wk_y, x).view(B, H, Dh)
            self.vc[i][:, n] = lin(at.Wv_y, x).view(B, H, Dh)
            for l in range(1, done + 1):
                j = n >> l
                r = self._row(N, l, j)
                c0 = self._row(N, l - 1, 2 * j)
                y_prev = self.y_in[i][:, r]
                y_norm = layer.norm_y(y_prev)
                out = build_parent_nodes(heads(lin(at.Wq_y, y_norm)), heads(lin(at.Wk_y, y_norm)), heads(lin(at.Wv_y, y_norm)),
                                         self.kc[i][:, c0:c0 + 2], self.vc[i][:, c0:c0 + 2]).reshape(B, self.d)
                self.kc[i][:, r] = lin(at.Wk_y, out).view(B, H, Dh)
                self.vc[i][:, r] = lin(at.Wv_y, out).view(B, H, Dh)
                y_next = y_prev + at.out_proj_y(out)
                self.y_in[i + 1][:, r] = y_next
                self.K[i][:, r] = lin(at.Wk_x, y_next).view(B, H, Dh)
                self.V[i][:, r] = lin(at.Wv_x, y_next).view(B, H, Dh)
            # ---- top-down: the new leaf against the caches
            xn = layer.norm1(x)
            self.K[i][:, n] = lin(at.Wk_x, xn).view(B, H, Dh)
            self.V[i][:, n] = lin(at.Wv_x, xn).view(B, H, Dh)
            ctx = span_attention_decode(lin(at.Wq_x, xn).view(B, H, Dh), self.K[i], self.V[i], n, at.window_size)
            x = x + at.out_proj_x(ctx.reshape(B, self.d))
            x = x + layer.feed_forward(layer.norm2(x))
        self.n += 1
        return m.fc_out(x)[:, : m.vocab_size]


@torch.no_grad()
def generate(model: "TransformerLM", prompt: torch.Tensor, max_len: int = 50, temperature: float = 1.0,
             eos_token: Optional[int] = 3, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Sampling loop of the reference's TransformerLM.generate (Hierarchical_Transformer_Pretrain.py:483-504:
    softmax(logits / temperature), multinomial, stop at the EOS id when the batch is a single sequence), run
    incrementally: the prompt is fed token by token, then one decoder step per generated token."""
    if prompt.dim() == 1:
        prompt = prompt.unsqueeze(0)
    dev = next(model.parameters()).device
    prompt = prompt.to(dev)
    B, P = prompt.shape
    assert P + max_len <= model.pos_encoding.pe.size(1), "prompt + max_len exceeds the positional table"
    capacity = 1 << max(1, (P + max_len - 1).bit_length())
    dec = IncrementalDecoder(model, B, capacity)
    logits = None
    for t in range(P):
        logits = dec.step(prompt[:, t])
    tokens = prompt
    for _ in range(max_len):
        probs = F.softmax(logits.float() / temperature, dim=-1)
        nxt = torch.multinomial(probs, 1, generator=generator)
        tokens = torch.cat([tokens, nxt], dim=1)
        if eos_token is not None and B == 1 and int(nxt) == eos_token:
            break
        if dec.n >= dec.N:
            break
        logits = dec.step(nxt.view(B))
    return tokens


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
    if (tokens.is_cuda and torch.is_autocast_enabled() and torch.get_autocast_dtype("cuda") == torch.bfloat16
            and model.d_model % 8 == 0 and getattr(model, "fused_head", True)):
        # bf16 autocast: LM head and loss in one pass (tcgen05 product whose epilogue keeps the softmax statistics)
        hidden = model(tokens[:, :-1], hidden_only=True)
        return linear_cross_entropy(hidden.reshape(-1, hidden.size(-1)), model.fc_out.weight, model.fc_out.bias,
                                    tokens[:, 1:].reshape(-1), model.vocab_size, label_smoothing=label_smoothing,
                                    ignore_index=ignore_index)
    logits = model(tokens[:, :-1], padded_logits=True)
    return cross_entropy(logits.reshape(-1, logits.size(-1)), tokens[:, 1:].reshape(-1), model.vocab_size,
                         label_smoothing=label_smoothing, ignore_index=ignore_index)
