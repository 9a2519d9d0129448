"""CPU oracle of the board-transformer forward pass (TEST INFRASTRUCTURE: only tests, the smoke check
and the bench's CPU-baseline leg may import this package; the product never does).

`BT4Spec` is a plain fp32 PyTorch restatement of the reference encoder `BT4`
(new_paradigm/value_q.py:121-211, new_paradigm/value.py:121-212; attention
new_paradigm/attn.py:445-533; value heads value.py:402-435, value_q.py:430-464; input embedding
utils/fen_encoder.py:41-67) with the reference's parameter names, plus the features that only the
target specification names (they have no source in the reference, so they are defined HERE and the
CUDA engine follows this file): Mish, activation between ff1 and ff2, pre-LN blocks, a smolgen-style
per-board attention bias, and an attention-policy head gathered to the 1858 Leela moves.

Pinning: with the reference's flags (`SpecConfig.reference_value_q`) this module reproduces the
reference module's outputs bit for bit on CPU (tests/golden/make_golden.py generates the fixtures by
importing the reference; tests/test_oracle_golden.py checks them). The specification-only features
have no reference implementation: parity for those is UNPINNED beyond that shared trunk.
"""
import math
from dataclasses import dataclass, asdict

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import vocab

LN_POST, LN_PRE = 0, 1
ACT_GELU, ACT_MISH = 1, 2
FFN_ACT_END, FFN_ACT_MID = 0, 1
BIAS_NONE, BIAS_CAUSAL, BIAS_RELPOS, BIAS_SMOLGEN = 0, 1, 2, 3
POLICY_NONE, POLICY_DENSE4096, POLICY_GATHER1858 = 0, 1, 2
VALUE_NONE, VALUE_WDL, VALUE_WDL_Q = 0, 1, 2


@dataclass
class SpecConfig:
    planes: int = 112
    d_model: int = 512
    n_layers: int = 10
    n_heads: int = 8
    d_ff: int = 736
    ln_mode: int = LN_POST
    act: int = ACT_GELU
    ffn_act_pos: int = FFN_ACT_END
    bias_mode: int = BIAS_RELPOS
    policy_mode: int = POLICY_DENSE4096
    value_mode: int = VALUE_WDL_Q
    smolgen_compress: int = 32
    smolgen_hidden: int = 256
    smolgen_gen: int = 256

    @staticmethod
    def reference_value_q(n_layers=10, d_model=512, d_ff=736, n_heads=8):
        """The reference `value_q.BT4(num_layers, d_model, d_ff, num_heads)` (112 planes)."""
        return SpecConfig(112, d_model, n_layers, n_heads, d_ff)

    @staticmethod
    def reference_value(n_layers=10, d_model=512, d_ff=736, n_heads=8):
        """The reference `value.BT4` (19 planes, WDL head only)."""
        return SpecConfig(19, d_model, n_layers, n_heads, d_ff, value_mode=VALUE_WDL)

    @staticmethod
    def baseline(n_layers, d_model, d_ff, n_heads, smolgen=True, value_only=False):
        """The network of the target specification: post-LN, Mish between ff1 and ff2, smolgen bias,
        1858-move gather policy, WDL head."""
        return SpecConfig(112, d_model, n_layers, n_heads, d_ff, LN_POST, ACT_MISH, FFN_ACT_MID,
                          BIAS_SMOLGEN if smolgen else BIAS_NONE,
                          POLICY_NONE if value_only else POLICY_GATHER1858, VALUE_WDL)

    def to_dict(self):
        return asdict(self)


def activation(x, act):
    return F.mish(x) if act == ACT_MISH else F.gelu(x)


def sinusoid_table(d_model):
    """[64, d] table of value.py:77-88: even columns sin(pos / 10000^(2i/d)), odd columns cos."""
    pos = torch.arange(64).unsqueeze(1)
    two_i = torch.arange(0, d_model, step=2).float()
    pe = torch.zeros(1, 64, d_model)
    pe[:, :, 0::2] = torch.sin(pos / (10000 ** (two_i / d_model)))
    pe[:, :, 1::2] = torch.cos(pos / (10000 ** (two_i / d_model)))
    return pe


def rel_shift(pos_score):
    """attn.py:525-533: prepend a zero column, reinterpret [64,65] as [65,64], drop the first row."""
    b, h, t1, t2 = pos_score.size()
    padded = torch.cat([pos_score.new_zeros(b, h, t1, 1), pos_score], dim=-1)
    padded = padded.view(b, h, t2 + 1, t1)
    return padded[:, :, 1:].view_as(pos_score)


class MaGating(nn.Module):
    def __init__(self, d_model):
        super().__init__()
        self.a = nn.Parameter(torch.zeros(64, d_model))
        self.b = nn.Parameter(torch.ones(64, d_model))

    def forward(self, x):
        return x * torch.exp(self.a) + self.b


class Attention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d, h = cfg.d_model, cfg.n_heads
        self.cfg, self.h, self.hd = cfg, h, d // h
        self.query_proj = nn.Linear(d, d)
        self.key_proj = nn.Linear(d, d)
        self.value_proj = nn.Linear(d, d)
        if cfg.bias_mode == BIAS_RELPOS:
            self.pos_proj = nn.Linear(d, d, bias=False)
            self.u_bias = nn.Parameter(torch.zeros(h, self.hd))
            self.v_bias = nn.Parameter(torch.zeros(h, self.hd))
        self.out_proj = nn.Linear(d, d)

    def forward(self, x, pos_enc, bias=None):
        b = x.size(0)
        q = self.query_proj(x).view(b, -1, self.h, self.hd)
        k = self.key_proj(x).view(b, -1, self.h, self.hd).permute(0, 2, 1, 3)
        v = self.value_proj(x).view(b, -1, self.h, self.hd).permute(0, 2, 1, 3)
        if self.cfg.bias_mode == BIAS_RELPOS:
            p = self.pos_proj(pos_enc).view(b, -1, self.h, self.hd)
            content = torch.matmul((q + self.u_bias).transpose(1, 2), k.transpose(2, 3))
            pos = torch.matmul((q + self.v_bias).transpose(1, 2), p.permute(0, 2, 3, 1))
            score = (content + rel_shift(pos)) / math.sqrt(self.cfg.d_model)   # attn.py:476,511
        else:
            score = torch.matmul(q.transpose(1, 2), k.transpose(2, 3)) / math.sqrt(self.hd)
            if bias is not None:
                score = score + bias
            if self.cfg.bias_mode == BIAS_CAUSAL:
                t = score.size(-1)
                score = score.masked_fill(torch.ones(t, t, dtype=torch.bool).triu(1), float("-inf"))
        attn = F.softmax(score, -1)
        ctx = torch.matmul(attn, v).transpose(1, 2).contiguous().view(b, -1, self.cfg.d_model)
        return self.out_proj(ctx)


class Smolgen(nn.Module):
    """Per-board additive attention bias (specification-only; this file is its definition).

    tokens [B,64,d] -> compress (d->c, no bias) -> flatten [B,64c] -> dense1 (->hidden) -> act -> LN
    -> dense2 (-> H*gen) -> act -> view [B,H,gen] -> LN over gen -> shared (gen->4096, no bias, one
    matrix for all layers) -> [B,H,64,64], element [q,k] at flat index q*64+k."""

    def __init__(self, cfg, shared):
        super().__init__()
        self.cfg = cfg
        self.compress = nn.Linear(cfg.d_model, cfg.smolgen_compress, bias=False)
        self.dense1 = nn.Linear(64 * cfg.smolgen_compress, cfg.smolgen_hidden)
        self.ln1 = nn.LayerNorm(cfg.smolgen_hidden)
        self.dense2 = nn.Linear(cfg.smolgen_hidden, cfg.n_heads * cfg.smolgen_gen)
        self.ln2 = nn.LayerNorm(cfg.smolgen_gen)
        self._shared = [shared]          # not registered here: owned by the top-level module

    def forward(self, x):
        b = x.size(0)
        c = self.compress(x).reshape(b, -1)
        h1 = self.ln1(activation(self.dense1(c), self.cfg.act))
        h2 = activation(self.dense2(h1), self.cfg.act).view(b, self.cfg.n_heads, self.cfg.smolgen_gen)
        h2 = self.ln2(h2)
        return self._shared[0](h2).view(b, self.cfg.n_heads, 64, 64)


class EncoderLayer(nn.Module):
    def __init__(self, cfg, shared):
        super().__init__()
        self.cfg = cfg
        self.attention = Attention(cfg)
        self.norm1 = nn.LayerNorm(cfg.d_model)
        self.norm2 = nn.LayerNorm(cfg.d_model)
        self.ff1 = nn.Linear(cfg.d_model, cfg.d_ff)
        self.ff2 = nn.Linear(cfg.d_ff, cfg.d_model)
        if cfg.bias_mode == BIAS_SMOLGEN:
            self.smolgen = Smolgen(cfg, shared)

    def _ffn(self, x):
        y = self.ff1(x)
        if self.cfg.ffn_act_pos == FFN_ACT_MID:
            return self.ff2(activation(y, self.cfg.act))
        return activation(self.ff2(y), self.cfg.act)          # value.py:65-67: act after ff2

    def forward(self, x, pos_enc):
        if self.cfg.ln_mode == LN_POST:                       # value.py:58-75
            bias = self.smolgen(x) if self.cfg.bias_mode == BIAS_SMOLGEN else None
            x = self.norm1(self.attention(x, pos_enc, bias) + x)
            return self.norm2(self._ffn(x) + x)
        xn = self.norm1(x)                                    # model_bis.py:110-113
        bias = self.smolgen(xn) if self.cfg.bias_mode == BIAS_SMOLGEN else None
        x = x + self.attention(xn, pos_enc, bias)
        return x + self._ffn(self.norm2(x))


class ValueHead(nn.Module):
    def __init__(self, d_model, n_out):
        super().__init__()
        self.dense1 = nn.Linear(d_model, 128)
        self.dense2 = nn.Linear(128 * 64, 128)
        self.dense3 = nn.Linear(128, n_out)

    def forward(self, x):
        b = x.size(0)
        x = F.gelu(self.dense1(x)).view(b, -1)
        return self.dense3(F.gelu(self.dense2(x)))


def gather_tables():
    """(flat from*64+to index [1858], promotion piece [1858]: 0 none, 1 q, 2 r, 3 b) with token index
    = square index a1=0 ... h8=63, the row order of the 112-plane input (gen_TC.py:42-59)."""
    idx, promo = [], []
    for m in vocab.policy_leela:
        f, t, p = vocab.move_squares(m)
        idx.append(f * 64 + t)
        promo.append(p)
    return torch.tensor(idx, dtype=torch.long), torch.tensor(promo, dtype=torch.long)


class BT4Spec(nn.Module):
    def __init__(self, cfg: SpecConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        if cfg.bias_mode == BIAS_SMOLGEN:
            self.smolgen_shared = nn.Linear(cfg.smolgen_gen, 4096, bias=False)
        shared = getattr(self, "smolgen_shared", None)
        self.layers = nn.ModuleList([EncoderLayer(cfg, shared) for _ in range(cfg.n_layers)])
        self.linear1 = nn.Linear(cfg.planes, d)
        self.layernorm1 = nn.LayerNorm(d)
        self.ma_gating = MaGating(d)
        if cfg.ln_mode == LN_PRE:
            self.norm_f = nn.LayerNorm(d)
        if cfg.policy_mode != POLICY_NONE:
            self.policy_tokens_lin = nn.Linear(d, d)
            self.queries_pol = nn.Linear(d, d)
            self.keys_pol = nn.Linear(d, d)
        if cfg.policy_mode == POLICY_DENSE4096:
            self.policy_head = nn.Linear(64 * 64, 1929, bias=False)
        if cfg.policy_mode == POLICY_GATHER1858:
            self.policy_promo = nn.Linear(d, 3, bias=False)
            idx, promo = gather_tables()
            self._gather_idx, self._gather_promo = idx, promo
        if cfg.value_mode != VALUE_NONE:
            self.value_head = ValueHead(d, 3)
        if cfg.value_mode == VALUE_WDL_Q:
            self.value_head_q = ValueHead(d, 1)
        self._pe = sinusoid_table(d)

    # ---- pieces -------------------------------------------------------------------------------
    def trunk(self, tokens):
        """tokens [B,64,P] -> [B,64,d] (value_q.py:159-171)."""
        x = self.ma_gating(self.layernorm1(F.gelu(self.linear1(tokens))))
        pos_enc = self._pe.expand(x.size(0), -1, -1)
        for layer in self.layers:
            x = layer(x, pos_enc)
        if self.cfg.ln_mode == LN_PRE:
            x = self.norm_f(x)
        return x, pos_enc

    def policy_logits(self, x, pos_enc):
        """value_q.py:176-192, or the 1858-move gather of the specification."""
        pt = F.gelu(self.policy_tokens_lin(x)) + pos_enc
        q, k = self.queries_pol(pt), self.keys_pol(pt)
        s = torch.matmul(q, torch.transpose(k, -2, -1)) / torch.sqrt(torch.tensor(self.cfg.d_model))
        s = s.view(x.size(0), 64 * 64)
        if self.cfg.policy_mode == POLICY_DENSE4096:
            return self.policy_head(s)
        out = s[:, self._gather_idx]
        promo = self.policy_promo(pt)                                   # [B,64,3]
        is_p = self._gather_promo > 0
        to_sq = self._gather_idx[is_p] % 64
        out[:, is_p] = out[:, is_p] + promo[:, to_sq, self._gather_promo[is_p] - 1]
        return out

    def forward_all(self, tokens):
        """tokens [B,64,P] f32 -> dict(policy [B,V] raw logits, wdl [B,3] raw logits, q [B,1] tanh)."""
        x, pos_enc = self.trunk(tokens)
        out = {}
        if self.cfg.value_mode != VALUE_NONE:
            out["wdl"] = self.value_head(x)
        if self.cfg.value_mode == VALUE_WDL_Q:
            out["q"] = torch.tanh(self.value_head_q(x))
        if self.cfg.policy_mode != POLICY_NONE:
            out["policy"] = self.policy_logits(x, pos_enc)
        return out

    def forward(self, inp, compute_loss=False):
        """Reference signature (value_q.py:156): inp[0] is [b, seq, 8, 8, P]; returns [b, seq, V]."""
        x = inp[0]
        b, seq, _, _, emb = x.size()
        out = self.forward_all(x.view(b * seq, 64, emb))
        return out["policy"].view(b, seq, -1)


def seeded_state_dict(module, seed=0, std=0.02):
    """Every parameter ~ N(0, std) drawn in sorted key order from one seeded CPU generator; LayerNorm
    weights 1 / biases 0 and the gating a=0, b=1 keep their constructor values."""
    g = torch.Generator().manual_seed(seed)
    sd = module.state_dict()
    keep = ("norm1.", "norm2.", "layernorm1.", "ln1.", "ln2.", "norm_f.", "ma_gating.", "ln_1.", "ln_2.",
            "ln_f.")
    for k in sorted(sd.keys()):
        v = sd[k]
        if any(t in k for t in keep):
            continue
        sd[k] = torch.randn(v.shape, generator=g) * std
    return sd


def apply_policy_mask(logits, legal_bits=None, additive=None):
    """Reference conventions: `logits + (1-mask)*(-999)` (model_bis.py:383, value.py:231) for a 0/1
    mask, or `mask_vec + logits` with mask_vec in {0,-1000} (Leela/server.py:56)."""
    if legal_bits is not None:
        return logits + (1 - legal_bits.to(logits.dtype)) * -999
    if additive is not None:
        return additive + logits
    return logits
