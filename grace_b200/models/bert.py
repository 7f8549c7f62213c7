"""BERT encoder for MLM + NSP pre-training (Devlin et al. 2018).

``bert_large()``: 24 layers, hidden 1024, 16 heads, FFN 4096, vocab 30522,
512 positions (about 335 M parameters).  Attention goes through
``torch.nn.functional.scaled_dot_product_attention`` (a library kernel: the
model is the workload here, the gradient exchange is the product).
"""

import torch
from torch import nn
import torch.nn.functional as F


class BertLayer(nn.Module):
    def __init__(self, hidden, heads, ffn, dropout):
        super().__init__()
        self.heads = heads
        self.qkv = nn.Linear(hidden, 3 * hidden)
        self.proj = nn.Linear(hidden, hidden)
        self.ln1 = nn.LayerNorm(hidden, eps=1e-12)
        self.fc1 = nn.Linear(hidden, ffn)
        self.fc2 = nn.Linear(ffn, hidden)
        self.ln2 = nn.LayerNorm(hidden, eps=1e-12)
        self.drop = nn.Dropout(dropout)

    def forward(self, x, mask=None):
        b, s, h = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.heads, h // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        a = a.transpose(1, 2).reshape(b, s, h)
        x = self.ln1(x + self.drop(self.proj(a)))
        y = self.fc2(F.gelu(self.fc1(x)))
        return self.ln2(x + self.drop(y))


class BertForPreTraining(nn.Module):
    def __init__(self, vocab=30522, hidden=1024, layers=24, heads=16, ffn=4096, max_pos=512, type_vocab=2,
                 dropout=0.1):
        super().__init__()
        self.tok = nn.Embedding(vocab, hidden)
        self.pos = nn.Embedding(max_pos, hidden)
        self.typ = nn.Embedding(type_vocab, hidden)
        self.ln = nn.LayerNorm(hidden, eps=1e-12)
        self.drop = nn.Dropout(dropout)
        self.layers = nn.ModuleList(BertLayer(hidden, heads, ffn, dropout) for _ in range(layers))
        self.pooler = nn.Linear(hidden, hidden)
        self.mlm_dense = nn.Linear(hidden, hidden)
        self.mlm_ln = nn.LayerNorm(hidden, eps=1e-12)
        self.mlm_bias = nn.Parameter(torch.zeros(vocab))
        self.nsp = nn.Linear(hidden, 2)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, ids, token_type=None, mlm_labels=None, nsp_labels=None):
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device).unsqueeze(0)
        if token_type is None:
            token_type = torch.zeros_like(ids)
        x = self.drop(self.ln(self.tok(ids) + self.pos(pos) + self.typ(token_type)))
        for layer in self.layers:
            x = layer(x)
        pooled = torch.tanh(self.pooler(x[:, 0]))
        h = self.mlm_ln(F.gelu(self.mlm_dense(x)))
        logits = F.linear(h, self.tok.weight, self.mlm_bias)  # tied decoder
        nsp_logits = self.nsp(pooled)
        if mlm_labels is None:
            return logits, nsp_logits
        loss = F.cross_entropy(logits.view(-1, logits.size(-1)).float(), mlm_labels.view(-1), ignore_index=-100)
        if nsp_labels is not None:
            loss = loss + F.cross_entropy(nsp_logits.float(), nsp_labels)
        return loss


def bert_large(**kw):
    return BertForPreTraining(30522, 1024, 24, 16, 4096, 512, **kw)


def bert_tiny(**kw):
    return BertForPreTraining(1000, 64, 2, 4, 128, 64, **kw)
