"""BERT-large-shaped encoder with a masked-language-model head (24 layers, hidden 1024, 16 heads,
FFN 4096, vocab 30522, sequence 512 by default).

The reference does not contain the model (it trains TensorFlow models through its collective mode);
this is the second data-parallel benchmark workload.  Linear layers run on the tcgen05 GEMM with bias and
GELU fused into the epilogue, layer norms and the softmax cross-entropy are the fused kernels of this
package (the input embedding as well), the attention core is the library scaled-dot-product attention.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.attention import packed_attention
from ..ops.linear import Linear
from ..ops.norm import LayerNorm
from ..ops.pointwise import embed_sum, softmax_cross_entropy


import os

_TORCH_EMBED = os.environ.get("TIPS_BERT_TORCH_EMBED", "0") == "1"


class BertLayer(nn.Module):
    def __init__(self, hidden, heads, ffn):
        super().__init__()
        self.heads = heads
        self.qkv = Linear(hidden, 3 * hidden)
        self.proj = Linear(hidden, hidden)
        self.ln1 = LayerNorm(hidden, eps=1e-12)
        self.fc1 = Linear(hidden, ffn, act="gelu")
        self.fc2 = Linear(ffn, hidden)
        self.ln2 = LayerNorm(hidden, eps=1e-12)

    def forward(self, x):
        # the residual adds are fused into the layer norms; in backward the gradient of each block input is summed
        # inside the GEMM that produces its second term (the "passthrough" linears)
        qkv, x = self.qkv(x, passthrough=True)
        att = packed_attention(qkv, self.heads)
        x = self.ln1(self.proj(att), residual=x)
        h, x = self.fc1(x, passthrough=True)
        return self.ln2(self.fc2(h), residual=x)


class BertMLM(nn.Module):
    def __init__(self, vocab=30522, hidden=1024, layers=24, heads=16, ffn=4096, max_seq=512, type_vocab=2):
        super().__init__()
        self.vocab = vocab
        # rows padded to a multiple of 64 so the tied decoder GEMM writes 16-byte vectors (unused classes)
        self.vocab_padded = (vocab + 63) // 64 * 64
        self.tok = nn.Embedding(self.vocab_padded, hidden)
        self.pos = nn.Embedding(max_seq, hidden)
        self.typ = nn.Embedding(type_vocab, hidden)
        self.ln_emb = LayerNorm(hidden, eps=1e-12)
        self.layers = nn.ModuleList([BertLayer(hidden, heads, ffn) for _ in range(layers)])
        self.head_dense = Linear(hidden, hidden, act="gelu")
        self.head_ln = LayerNorm(hidden, eps=1e-12)
        self.decoder_bias = nn.Parameter(torch.zeros(self.vocab_padded))
        for m in self.modules():
            if isinstance(m, (nn.Embedding,)):
                nn.init.normal_(m.weight, std=0.02)
            if isinstance(m, Linear):
                nn.init.normal_(m.weight, std=0.02)

    def encode(self, ids):
        if _TORCH_EMBED:  # TIPS_BERT_TORCH_EMBED=1: torch's embedding kernels, kept for A/B measurements
            pos = torch.arange(ids.shape[1], device=ids.device)
            x = self.tok(ids) + self.pos(pos)[None] + self.typ.weight[0]
        else:
            x = embed_sum(ids, self.tok.weight, self.pos.weight, self.typ.weight[0])
        x = self.ln_emb(x)
        for layer in self.layers:
            x = layer(x)
        return x

    def loss(self, ids, masked_positions, masked_labels):
        """ids [B, S]; masked_positions [B, P] indices into S; masked_labels [B, P] (-100 = unused slot)."""
        x = self.encode(ids)
        b, p = masked_positions.shape
        picked = torch.gather(x, 1, masked_positions[..., None].expand(b, p, x.shape[-1])).reshape(b * p, -1)
        hcur = self.head_ln(self.head_dense(picked))
        from ..ops.linear import linear
        # tied decoder
        logits = linear(hcur, self.tok.weight, self.decoder_bias)
        return softmax_cross_entropy(logits, masked_labels.reshape(-1))


def bert_large(dtype=torch.bfloat16, device="cuda", **kw):
    return BertMLM(**kw).to(device=device, dtype=dtype)


def tiny_bert(dtype=torch.bfloat16, device="cuda"):
    return BertMLM(vocab=1024, hidden=128, layers=2, heads=4, ffn=512, max_seq=64).to(device=device, dtype=dtype)


def synthetic_mlm_batch(batch, seq, vocab, seed, mask_frac=0.15):
    """Token ids uniform over the vocabulary, 15% of positions masked uniformly."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (batch, seq), generator=g)
    p = max(1, int(round(seq * mask_frac)))
    pos = torch.stack([torch.randperm(seq, generator=g)[:p] for _ in range(batch)])
    labels = torch.gather(ids, 1, pos)
    return ids, pos, labels
