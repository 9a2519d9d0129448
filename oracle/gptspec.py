"""CPU oracle of the reference decoder model's board-only forward pass (TEST INFRASTRUCTURE).

Restates `GPT.get_move_from_fen_no_thinking` up to the logits (model_bis.py:358-370): FenEncoder
(utils/fen_encoder.py:52-67) + fixed sinusoid positions (model_bis.py:141-146), pre-LN causal blocks
(model_bis.py:36-113), final LayerNorm, LM head on the last of the 64 board tokens. Parameter names are
the reference's. Pinned bit for bit against the unmodified reference by tests/golden/make_golden.py.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPTConfig:          # model_bis.py:115-123
    block_size: int = 256
    vocab_size: int = 1929
    n_layer: int = 6
    n_head: int = 12
    n_embd: int = 768
    dropout: float = 0.0
    bias: bool = True


class _Gating(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.a = nn.Parameter(torch.zeros(64, d))
        self.b = nn.Parameter(torch.ones(64, d))


class _FenEncoder(nn.Module):
    def __init__(self, d, planes=19):
        super().__init__()
        self.linear1 = nn.Linear(planes, d)
        self.layernorm1 = nn.LayerNorm(d)
        self.ma_gating = _Gating(d)

    def forward(self, x):
        x = self.layernorm1(F.gelu(self.linear1(x.view(-1, 64, self.linear1.in_features))))
        return x * torch.exp(self.ma_gating.a) + self.ma_gating.b


class _LN(nn.Module):
    def __init__(self, d, bias):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.bias = nn.Parameter(torch.zeros(d)) if bias else None

    def forward(self, x):
        return F.layer_norm(x, self.weight.shape, self.weight, self.bias, 1e-5)


class _Attn(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.c_attn = nn.Linear(c.n_embd, 3 * c.n_embd, bias=c.bias)
        self.c_proj = nn.Linear(c.n_embd, c.n_embd, bias=c.bias)
        self.h, self.d = c.n_head, c.n_embd

    def forward(self, x):
        b, t, c = x.size()
        q, k, v = self.c_attn(x).split(self.d, dim=2)
        q, k, v = (z.view(b, t, self.h, c // self.h).transpose(1, 2) for z in (q, k, v))
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=True)
        return self.c_proj(y.transpose(1, 2).contiguous().view(b, t, c))


class _MLP(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.c_fc = nn.Linear(c.n_embd, 4 * c.n_embd, bias=c.bias)
        self.c_proj = nn.Linear(4 * c.n_embd, c.n_embd, bias=c.bias)

    def forward(self, x):
        return self.c_proj(F.gelu(self.c_fc(x)))


class _Block(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.ln_1, self.attn, self.ln_2, self.mlp = _LN(c.n_embd, c.bias), _Attn(c), _LN(c.n_embd, c.bias), _MLP(c)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class GPTSpec(nn.Module):
    def __init__(self, c: GPTConfig):
        super().__init__()
        self.config = c
        self.FenEncoder = _FenEncoder(c.n_embd)
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(c.vocab_size, c.n_embd),
            h=nn.ModuleList([_Block(c) for _ in range(c.n_layer)]),
            ln_f=_LN(c.n_embd, c.bias)))
        self.lm_head = nn.Linear(c.n_embd, c.vocab_size, bias=False)
        pos = torch.arange(c.block_size).unsqueeze(1)
        div = torch.exp(torch.arange(0, c.n_embd, 2).float() * (-math.log(10000.0) / c.n_embd))
        pe = torch.zeros(c.block_size, c.n_embd)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)
        self.register_buffer("pe", pe)
        self.transformer.wte.weight = self.lm_head.weight          # tied (model_bis.py:148)

    def board_logits(self, board):
        """board [B,8,8,19] f32 -> [B, vocab] logits of the last board token."""
        x = self.FenEncoder(board) + self.pe[:64]
        for blk in self.transformer.h:
            x = blk(x)
        x = self.transformer.ln_f(x)
        return self.lm_head(x[:, [-1], :])[:, 0]
