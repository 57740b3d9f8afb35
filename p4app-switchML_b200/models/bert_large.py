"""BERT-large for masked-language-model pre-training: 24 layers, hidden 1024, 16 heads,
FFN 4096, vocabulary 30522, ~335 M parameters. Attention uses
``scaled_dot_product_attention``; with ``fused_ffn=True`` the two FFN projections of
every layer compute their weight gradients with the tcgen05 GEMM fused with the cross-GPU
reduction (ops/wgrad.py)."""
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from ..ops.wgrad import FusedWgradLinear


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden: int = 1024
    layers: int = 24
    heads: int = 16
    ffn: int = 4096
    max_pos: int = 512
    type_vocab: int = 2
    dropout: float = 0.1
    fused_ffn: bool = False


class Layer(nn.Module):
    def __init__(self, c):
        super().__init__()
        lin = FusedWgradLinear if c.fused_ffn else nn.Linear
        self.heads = c.heads
        self.qkv = nn.Linear(c.hidden, 3 * c.hidden)
        self.proj = nn.Linear(c.hidden, c.hidden)
        self.ln1 = nn.LayerNorm(c.hidden, eps=1e-12)
        self.ffn1 = lin(c.hidden, c.ffn)
        self.ffn2 = lin(c.ffn, c.hidden)
        self.ln2 = nn.LayerNorm(c.hidden, eps=1e-12)
        self.drop = nn.Dropout(c.dropout)

    def forward(self, x):
        b, s, h = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.heads, h // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, dropout_p=self.drop.p if self.training else 0.0)
        a = a.transpose(1, 2).reshape(b, s, h)
        x = self.ln1(x + self.drop(self.proj(a)))
        return self.ln2(x + self.drop(self.ffn2(F.gelu(self.ffn1(x)))))


class BertForMaskedLM(nn.Module):
    def __init__(self, c=BertConfig()):
        super().__init__()
        self.c = c
        self.tok = nn.Embedding(c.vocab_size, c.hidden)
        self.pos = nn.Embedding(c.max_pos, c.hidden)
        self.typ = nn.Embedding(c.type_vocab, c.hidden)
        self.ln = nn.LayerNorm(c.hidden, eps=1e-12)
        self.drop = nn.Dropout(c.dropout)
        self.layers = nn.ModuleList([Layer(c) for _ in range(c.layers)])
        self.head_dense = nn.Linear(c.hidden, c.hidden)
        self.head_ln = nn.LayerNorm(c.hidden, eps=1e-12)
        self.head_bias = nn.Parameter(torch.zeros(c.vocab_size))
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def fused_layers(self):
        return [m for m in self.modules() if isinstance(m, FusedWgradLinear)]

    def forward(self, ids, labels=None):
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device)
        x = self.drop(self.ln(self.tok(ids) + self.pos(pos)[None] + self.typ.weight[0]))
        for layer in self.layers:
            x = layer(x)
        x = self.head_ln(F.gelu(self.head_dense(x)))
        logits = F.linear(x, self.tok.weight.to(x.dtype)) + self.head_bias.to(x.dtype)  # tied decoder
        if labels is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.view(-1), ignore_index=-100)


def bert_large(fused_ffn=False, **overrides):
    return BertForMaskedLM(BertConfig(fused_ffn=fused_ffn, **overrides))
