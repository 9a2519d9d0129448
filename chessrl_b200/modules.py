"""Drop-in `nn.Module`s: the reference's constructors, `forward` signature and `state_dict` layout
(new_paradigm/value_q.py:121-211, value.py:121-212), with the arithmetic done by the CUDA engine.

The parameters are ordinary fp32 `nn.Parameter`s under the reference's names, so `state_dict()`,
`load_state_dict()` and `torch.save` files interchange with the reference. They are storage only: the
engine keeps its own repacked f16 / e4m3 device copies, refreshed whenever a parameter changed.
Inference only: `compute_loss=True` (training) is not provided.
"""
import numpy as np
import torch
import torch.nn as nn

from . import _lib as L
from .engine import Engine, EngineConfig


def _param_shapes(cfg: EngineConfig):
    d, ff, h, p = cfg.d_model, cfg.d_ff, cfg.n_heads, cfg.planes
    hd = d // h
    shapes = {}
    for i in range(cfg.n_layers):
        pre = f"layers.{i}."
        if cfg.bias_mode == L.BIAS_RELPOS:
            shapes[pre + "attention.u_bias"] = (h, hd)
            shapes[pre + "attention.v_bias"] = (h, hd)
        for n in ("query_proj", "key_proj", "value_proj"):
            shapes[pre + f"attention.{n}.weight"] = (d, d)
            shapes[pre + f"attention.{n}.bias"] = (d,)
        if cfg.bias_mode == L.BIAS_RELPOS:
            shapes[pre + "attention.pos_proj.weight"] = (d, d)
        shapes[pre + "attention.out_proj.weight"] = (d, d)
        shapes[pre + "attention.out_proj.bias"] = (d,)
        for n in ("norm1", "norm2"):
            shapes[pre + n + ".weight"] = (d,)
            shapes[pre + n + ".bias"] = (d,)
        shapes[pre + "ff1.weight"] = (ff, d)
        shapes[pre + "ff1.bias"] = (ff,)
        shapes[pre + "ff2.weight"] = (d, ff)
        shapes[pre + "ff2.bias"] = (d,)
        if cfg.bias_mode == L.BIAS_SMOLGEN:
            c, hid, gen = cfg.smolgen_compress, cfg.smolgen_hidden, cfg.smolgen_gen
            shapes[pre + "smolgen.compress.weight"] = (c, d)
            shapes[pre + "smolgen.dense1.weight"] = (hid, 64 * c)
            shapes[pre + "smolgen.dense1.bias"] = (hid,)
            shapes[pre + "smolgen.ln1.weight"] = (hid,)
            shapes[pre + "smolgen.ln1.bias"] = (hid,)
            shapes[pre + "smolgen.dense2.weight"] = (h * gen, hid)
            shapes[pre + "smolgen.dense2.bias"] = (h * gen,)
            shapes[pre + "smolgen.ln2.weight"] = (gen,)
            shapes[pre + "smolgen.ln2.bias"] = (gen,)
    shapes["linear1.weight"] = (d, p)
    shapes["linear1.bias"] = (d,)
    shapes["layernorm1.weight"] = (d,)
    shapes["layernorm1.bias"] = (d,)
    if cfg.policy_mode != L.POLICY_NONE:
        for n in ("policy_tokens_lin", "queries_pol", "keys_pol"):
            shapes[n + ".weight"] = (d, d)
            shapes[n + ".bias"] = (d,)
    shapes["ma_gating.a"] = (64, d)
    shapes["ma_gating.b"] = (64, d)
    if cfg.bias_mode == L.BIAS_SMOLGEN:
        shapes["smolgen_shared.weight"] = (4096, cfg.smolgen_gen)
    if cfg.ln_mode == L.LN_PRE:
        shapes["norm_f.weight"] = (d,)
        shapes["norm_f.bias"] = (d,)
    if cfg.policy_mode == L.POLICY_DENSE4096:
        shapes["policy_head.weight"] = (1929, 4096)
    if cfg.policy_mode == L.POLICY_GATHER1858:
        shapes["policy_promo.weight"] = (3, d)
    heads = []
    if cfg.value_mode != L.VALUE_NONE:
        heads.append(("value_head", 3))
    if cfg.value_mode == L.VALUE_WDL_Q:
        heads.append(("value_head_q", 1))
    for name, n_out in heads:
        shapes[name + ".dense1.weight"] = (128, d)
        shapes[name + ".dense1.bias"] = (128,)
        shapes[name + ".dense2.weight"] = (128, 128 * 64)
        shapes[name + ".dense2.bias"] = (128,)
        shapes[name + ".dense3.weight"] = (n_out, 128)
        shapes[name + ".dense3.bias"] = (n_out,)
    return shapes


class _Node(nn.Module):
    """Container so that dotted reference names (`layers.0.attention.query_proj.weight`) come out of
    `state_dict()` unchanged."""


def _attach(root, dotted, param):
    parts = dotted.split(".")
    node = root
    for part in parts[:-1]:
        if not hasattr(node, part):
            node.add_module(part, _Node())
        node = getattr(node, part)
    node.register_parameter(parts[-1], param)


def move_from_policy(eng, planes, bits, mirrored, T, force_legal, return_probs, generator):
    """Policy logits of one position, illegal moves pushed down by 999 (model_bis.py:373-383; knight promotions share
    the un-suffixed token), then the arg-max for T == 0 or one draw from softmax(logits / T) (model_bis.py:385-392).
    Mask, softmax and draw run on the GPU inside the engine call; `generator` (torch.Generator, CPU) makes the draw
    reproducible. With return_probs the distribution [1, V] comes back too (one-hot for T == 0, where the
    reference leaves it undefined)."""
    from . import positions
    if force_legal and not bool(bits.any()):
        raise ValueError("No legal moves available")
    u = torch.rand(1, generator=generator) if T != 0 else None
    out = eng.forward(planes.to(eng.device), legal_mask=bits.to(eng.device) if force_legal else None, wdl=False,
                      moves=True, temperature=float(T), uniforms=u.to(eng.device) if u is not None else None)
    index = int(out["move"][0])
    move = positions.vocab_move(index)
    if mirrored:
        move = positions.mirror_uci(move)
    if not return_probs:
        return move
    if T == 0:
        probs = torch.zeros_like(out["policy"])
        probs[0, index] = 1.0
    else:
        probs = torch.softmax(out["policy"] / T, dim=-1)
    return move, probs


class BoardTransformer(nn.Module):
    """Board transformer behind the reference's module protocol. `engine_device` is the GPU index."""

    def __init__(self, cfg: EngineConfig, engine_device=0):
        super().__init__()
        self.cfg = cfg
        self.d_model = cfg.d_model
        self.num_layers = cfg.n_layers
        self.is_thinking_model = False                       # value_q.py:124
        for name, shape in _param_shapes(cfg).items():
            if name.endswith("norm1.weight") or name.endswith("norm2.weight") or name.endswith("ln1.weight") \
                    or name.endswith("ln2.weight") or name in ("layernorm1.weight", "norm_f.weight", "ma_gating.b"):
                init = torch.ones(shape)
            elif name.endswith(".bias") or name == "ma_gating.a":
                init = torch.zeros(shape)
            else:
                init = torch.randn(shape) * 0.02
            _attach(self, name, nn.Parameter(init, requires_grad=False))
        self._engine_device = engine_device
        self._engine = None
        self._pushed_versions = None

    # -- engine plumbing ---------------------------------------------------------------------------
    def engine(self):
        if self._engine is None:
            self._engine = Engine(self.cfg, self._engine_device)
        versions = tuple((p.data_ptr(), p._version) for p in self.parameters())
        if versions != self._pushed_versions:
            self._engine.load_state_dict(self.state_dict())
            self._pushed_versions = versions
        return self._engine

    def calibrate(self, x):
        """FP8 engines: x is a batch of planes like the one `forward` takes."""
        eng = self.engine()
        eng.calibrate(x.to(eng.device))

    def infer(self, x, **kw):
        """x: [..., 8, 8, P] planes (any device). Returns the engine's output dict on the GPU."""
        eng = self.engine()
        return eng.forward(x.to(eng.device), **kw)

    # -- reference protocol ------------------------------------------------------------------------
    def forward(self, inp, compute_loss=False):
        """inp[0]: [b, seq, 8, 8, P] f32 -> policy logits [b, seq, V] (value_q.py:156-211)."""
        if compute_loss:
            raise NotImplementedError("inference engine: the training losses are not provided")
        x = inp[0]
        b, seq = x.shape[0], x.shape[1]
        out = self.infer(x, wdl=False)
        return out["policy"].view(b, seq, -1)

    def position_values(self, x, softmax=True):
        """Planes -> [B, 3] (black win, draw, white win) as in get_batch_position_values
        (value.py:275-317), which softmaxes the value logits (value.py:315)."""
        return self.infer(x, policy=False, wdl=True, wdl_softmax=softmax)["wdl"]

    # -- move choice from the policy (model_bis.py:358-398, new_paradigm/value.py:214-243) ------------------
    def _fen_inputs(self, fen):
        """(planes [1,8,8,P] host tensor, legal bitset [1,242] over the 1929 vocabulary in the network's view,
        whether the network sees the board rank-mirrored)."""
        from . import positions
        if self.cfg.planes == 19:
            return (torch.from_numpy(positions.fen_to_tensor(fen))[None],
                    torch.from_numpy(positions.legal_mask_1929(fen))[None], False)
        # 112-plane networks see the board from the mover's side: mask and move are mirrored for Black
        black = fen.split()[1] == "b"
        view = positions.mirror_fen(fen) if black else fen
        return (torch.from_numpy(positions.fen_to_planes112(fen))[None],
                torch.from_numpy(positions.legal_mask_1929(view))[None], black)

    def get_move_from_fen_no_thinking(self, fen, T=1, device="cuda", force_legal=True, return_probs=False,
                                      generator=None):
        """The reference's board-only move choice (new_paradigm/value.py:214-243), see `move_from_policy`.
        112-plane networks see Black's positions rank-mirrored; the move returned is in real board coordinates
        either way."""
        if self.cfg.policy_mode != L.POLICY_DENSE4096:
            raise ValueError("get_move_from_fen_no_thinking needs the 1929-move policy head")
        planes, bits, mirrored = self._fen_inputs(fen)
        return move_from_policy(self.engine(), planes, bits, mirrored, T, force_legal, return_probs, generator)

    def _select_by_value(self, ucis, values, T, return_probs, generator):
        """value.py:356-400 / value_q.py:349-397: arg-max for T == 0, else one draw from softmax(values / T)."""
        if not ucis:
            raise ValueError("No legal moves available")
        if T == 0:
            idx = int(torch.argmax(values))
            probs = torch.zeros_like(values)
            probs[idx] = 1.0
        else:
            probs = torch.softmax(values / T, dim=0)
            idx = int(torch.multinomial(probs, num_samples=1, generator=generator))
        return (ucis[idx], probs.cpu().numpy()) if return_probs else ucis[idx]

    def get_best_move_value(self, fen, T=1, device=None, return_probs=False, generator=None):
        """value.py:356-400: T == 0 picks the highest-valued move, otherwise one draw from softmax(values / T)
        (`generator`: optional torch.Generator on the engine's device for a reproducible draw)."""
        ucis, values = self.calculate_move_values(fen)
        return self._select_by_value(ucis, values, T, return_probs, generator)

    def calculate_move_values(self, fen, device=None):
        """Every legal move of `fen` with the mover's value of the position it leads to, all successors in one
        engine call. Returns (UCI strings, values [n] on the GPU)."""
        return self.calculate_move_values_many([fen])[0]

    def calculate_move_values_many(self, fens):
        """The evaluation loops of metrics/tactics_evaluation_improved.py:8-62 and metrics/endgame_evaluation.py:6-63
        call calculate_move_values once per position; this entry scores the successors of MANY positions in one
        engine call. Returns a list of (UCI strings, values [n_i] on the GPU), one per FEN, values as
        calculate_move_values defines them for this class."""
        from . import positions
        per, planes = [], []
        for fen in fens:
            ucis, succ_fens, p19 = positions.successors(fen, planes19=self.cfg.planes == 19)
            if self.cfg.planes != 19 and ucis:
                p19 = torch.from_numpy(np.stack([positions.fen_to_planes112(f) for f in succ_fens]))
            per.append((ucis, fen.split()[1] == "w"))
            if ucis:
                planes.append(p19)
        dev = self.engine().device
        if not planes:
            return [([], torch.empty(0, device=dev)) for _ in per]
        values = self._successor_values(torch.cat(planes))
        out, at = [], 0
        for ucis, white in per:
            v = values[at:at + len(ucis)]
            at += len(ucis)
            out.append((ucis, self._mover_value(v, white)))
        return out


class BT4(BoardTransformer):
    """`BT4(num_layers, d_model, d_ff, num_heads)` of new_paradigm/value_q.py:121-153: 112 input
    planes, relative attention, dense 4096 -> 1929 policy, WDL and Q value heads."""

    def __init__(self, num_layers=10, d_model=512, d_ff=736, num_heads=8, dtype=L.DTYPE_F16, engine_device=0):
        super().__init__(EngineConfig.reference_value_q(num_layers, d_model, d_ff, num_heads, dtype=dtype),
                         engine_device)

    # -- Q-value entry points (new_paradigm/value_q.py:244-347). The reference feeds `fen_to_tensor`'s 19 planes
    # into this class's 112-plane input layer there, which cannot run; the 112-plane encoding of the FEN with an
    # empty history (positions.fen_to_planes112) takes their place.
    def get_batch_position_values(self, fens, device=None):
        """FENs -> [B, 1] tanh Q of `value_head_q` (value_q.py:275-310)."""
        from . import positions
        dev = self.engine().device
        if len(fens) == 0:
            return torch.empty(0, 1, device=dev)
        x = torch.from_numpy(np.stack([positions.fen_to_planes112(f) for f in fens]))
        return self.infer(x, policy=False, wdl=False, q=True)["q"].view(-1, 1)

    def get_position_value(self, fen, device=None):
        """One FEN -> scalar tanh Q (value_q.py:244-273)."""
        return self.get_batch_position_values([fen]).squeeze()

    def _successor_values(self, planes):
        return self.infer(planes, policy=False, wdl=False, q=True)["q"].view(-1)

    @staticmethod
    def _mover_value(q, white_to_move):
        """value_q.py:338-347: the mover's value of a successor is -Q for White to move, +Q for Black."""
        return -q if white_to_move else q


class BT4Planes19(BoardTransformer):
    """`BT4` of new_paradigm/value.py:121-153: 19 input planes (utils/fen_encoder.py:5-38), WDL head."""

    def __init__(self, num_layers=10, d_model=512, d_ff=736, num_heads=8, dtype=L.DTYPE_F16, engine_device=0):
        super().__init__(EngineConfig.reference_value(num_layers, d_model, d_ff, num_heads, dtype=dtype),
                         engine_device)


    # -- value-driven move selection (new_paradigm/value.py:245-400) ------------------------------------
    def get_batch_position_values(self, fens, device=None):
        """FENs -> [B, 3] probabilities (black win, draw, white win), value.py:275-317."""
        from . import positions
        x = torch.stack([torch.from_numpy(positions.fen_to_tensor(f)) for f in fens]) if len(fens) else torch.empty(0, 8, 8, 19)
        return self.position_values(x) if len(fens) else torch.empty(0, 3, device=self.engine().device)

    def get_position_value(self, fen, device=None):
        """One FEN -> [3] probabilities, value.py:245-273."""
        return self.get_batch_position_values([fen])[0]

    def _successor_values(self, planes):
        return self.position_values(planes)

    @staticmethod
    def _mover_value(probs, white_to_move):
        """value.py:345-352: 0.5 * draw + the mover's own win probability."""
        return 0.5 * probs[:, 1] + (probs[:, 2] if white_to_move else probs[:, 0])


class BT4Baseline(BoardTransformer):
    """The network of the target specification (smolgen bias, Mish FFN, 1858-move gather policy)."""

    def __init__(self, num_layers=15, d_model=1024, d_ff=1536, num_heads=32, smolgen=True, value_only=False,
                 dtype=L.DTYPE_F16, engine_device=0, chunk=0):
        super().__init__(EngineConfig.baseline(num_layers, d_model, d_ff, num_heads, smolgen=smolgen,
                                               value_only=value_only, dtype=dtype, chunk=chunk), engine_device)


# ------------------------------------------------------------------------------------------------------
# Decoder model of model_bis.py, board-only inference path
# ------------------------------------------------------------------------------------------------------
from dataclasses import dataclass  # noqa: E402


@dataclass
class GPTConfig:
    """Same fields as the reference's GPTConfig (model_bis.py:115-123)."""
    block_size: int = 1024
    vocab_size: int = 50304
    n_layer: int = 6
    n_head: int = 12
    n_embd: int = 768
    dropout: float = 0.0
    bias: bool = True


def _gpt_param_shapes(c: GPTConfig):
    d = c.n_embd
    shapes = {"FenEncoder.linear1.weight": (d, 19), "FenEncoder.linear1.bias": (d,),
              "FenEncoder.layernorm1.weight": (d,), "FenEncoder.layernorm1.bias": (d,),
              "FenEncoder.ma_gating.a": (64, d), "FenEncoder.ma_gating.b": (64, d),
              "transformer.wte.weight": (c.vocab_size, d)}
    for i in range(c.n_layer):
        pre = f"transformer.h.{i}."
        shapes[pre + "ln_1.weight"] = (d,)
        shapes[pre + "attn.c_attn.weight"] = (3 * d, d)
        shapes[pre + "attn.c_proj.weight"] = (d, d)
        shapes[pre + "ln_2.weight"] = (d,)
        shapes[pre + "mlp.c_fc.weight"] = (4 * d, d)
        shapes[pre + "mlp.c_proj.weight"] = (d, 4 * d)
        if c.bias:
            for n, width in (("ln_1", d), ("attn.c_attn", 3 * d), ("attn.c_proj", d), ("ln_2", d), ("mlp.c_fc", 4 * d),
                             ("mlp.c_proj", d)):
                shapes[pre + n + ".bias"] = (width,)
    shapes["transformer.ln_f.weight"] = (d,)
    if c.bias:
        shapes["transformer.ln_f.bias"] = (d,)
    shapes["lm_head.weight"] = (c.vocab_size, d)
    return shapes


def gpt_to_engine_state_dict(sd, c: GPTConfig):
    """Rename the reference GPT's tensors to the keys the engine uses (fused c_attn split into q/k/v, missing
    biases of a bias=False model filled with zeros)."""
    d = c.n_embd
    out = {"linear1.weight": sd["FenEncoder.linear1.weight"], "linear1.bias": sd["FenEncoder.linear1.bias"],
           "layernorm1.weight": sd["FenEncoder.layernorm1.weight"], "layernorm1.bias": sd["FenEncoder.layernorm1.bias"],
           "ma_gating.a": sd["FenEncoder.ma_gating.a"], "ma_gating.b": sd["FenEncoder.ma_gating.b"],
           "pe": sd["pe"], "lm_head.weight": sd["lm_head.weight"],
           "norm_f.weight": sd["transformer.ln_f.weight"],
           "norm_f.bias": sd.get("transformer.ln_f.bias", torch.zeros(d))}
    for i in range(c.n_layer):
        src, dst = f"transformer.h.{i}.", f"layers.{i}."
        w = sd[src + "attn.c_attn.weight"]
        b = sd.get(src + "attn.c_attn.bias", torch.zeros(3 * d))
        for j, name in enumerate(("query_proj", "key_proj", "value_proj")):
            out[dst + f"attention.{name}.weight"] = w[j * d:(j + 1) * d]
            out[dst + f"attention.{name}.bias"] = b[j * d:(j + 1) * d]
        out[dst + "attention.out_proj.weight"] = sd[src + "attn.c_proj.weight"]
        out[dst + "attention.out_proj.bias"] = sd.get(src + "attn.c_proj.bias", torch.zeros(d))
        out[dst + "norm1.weight"] = sd[src + "ln_1.weight"]
        out[dst + "norm1.bias"] = sd.get(src + "ln_1.bias", torch.zeros(d))
        out[dst + "norm2.weight"] = sd[src + "ln_2.weight"]
        out[dst + "norm2.bias"] = sd.get(src + "ln_2.bias", torch.zeros(d))
        out[dst + "ff1.weight"] = sd[src + "mlp.c_fc.weight"]
        out[dst + "ff1.bias"] = sd.get(src + "mlp.c_fc.bias", torch.zeros(4 * d))
        out[dst + "ff2.weight"] = sd[src + "mlp.c_proj.weight"]
        out[dst + "ff2.bias"] = sd.get(src + "mlp.c_proj.bias", torch.zeros(d))
    return out


class GPT(nn.Module):
    """`GPT(GPTConfig)` of model_bis.py:125-156 for board-only inference: the path of
    `get_move_from_fen_no_thinking` (model_bis.py:358-398) up to the masked logits. The move-token part
    of the sequence (`idx` beyond length 0) and training are not provided."""

    def __init__(self, config: GPTConfig, dtype=L.DTYPE_F16, engine_device=0):
        super().__init__()
        self.config = config
        d = config.n_embd
        for name, shape in _gpt_param_shapes(config).items():
            if name == "transformer.wte.weight":
                continue
            if name.endswith("ln_1.weight") or name.endswith("ln_2.weight") or name.endswith("ln_f.weight") \
                    or name.endswith("layernorm1.weight") or name.endswith("ma_gating.b"):
                init = torch.ones(shape)
            elif name.endswith(".bias") or name.endswith("ma_gating.a"):
                init = torch.zeros(shape)
            else:
                init = torch.randn(shape) * 0.02
            _attach(self, name, nn.Parameter(init, requires_grad=False))
        self.transformer.add_module("wte", _Node())
        self.transformer.wte.register_parameter("weight", self.lm_head.weight)        # tied, both keys present
        pos = torch.arange(config.block_size).unsqueeze(1)
        import math
        div = torch.exp(torch.arange(0, d, 2).float() * (-math.log(10000.0) / d))
        pe = torch.zeros(config.block_size, d)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)
        self.register_buffer("pe", pe)
        self._cfg = EngineConfig.reference_gpt(config.n_layer, config.n_head, config.n_embd, config.vocab_size, dtype=dtype)
        self._engine_device = engine_device
        self._engine = None
        self._pushed_versions = None

    def engine(self):
        if self._engine is None:
            self._engine = Engine(self._cfg, self._engine_device)
        versions = tuple((p.data_ptr(), p._version) for p in self.parameters())
        if versions != self._pushed_versions:
            self._engine.load_state_dict(gpt_to_engine_state_dict(self.state_dict(), self.config))
            self._pushed_versions = versions
        return self._engine

    def board_logits(self, board, legal_mask=None, softmax=False):
        """board [B,8,8,19] -> [B, vocab] logits of the last board token, optionally masked
        (`logits + (1-mask)*(-999)`, model_bis.py:383) and soft-maxed."""
        eng = self.engine()
        return eng.forward(board.to(eng.device), legal_mask=legal_mask, policy_softmax=softmax, wdl=False)["policy"]

    def get_move_from_fen_no_thinking(self, fen, T=1, device="cuda", force_legal=True, return_probs=False,
                                      generator=None):
        """model_bis.py:358-398: last-token logits of the encoded board, `logits + (1 - mask) * -999`, arg-max for
        T == 0 or one draw from softmax(logits / T); returns the UCI string (and the distribution [1, vocab])."""
        from . import positions
        if self.config.vocab_size < 1929:
            raise ValueError("the legal-move mask spans the 1929-move vocabulary")
        bits = torch.zeros(1, (self.config.vocab_size + 7) // 8, dtype=torch.uint8)
        bits[0, :242] = torch.from_numpy(positions.legal_mask_1929(fen))
        planes = torch.from_numpy(positions.fen_to_tensor(fen))[None]
        return move_from_policy(self.engine(), planes, bits, False, T, force_legal, return_probs, generator)

    def forward(self, batch, compute_loss=False):
        """batch = (board [B,8,8,19], idx [B,0]) -> (logits [B,1,V], None, targets [B,64]) as model_bis.py:171-199."""
        board, idx = batch[0], batch[1]
        if compute_loss or idx.numel() != 0:
            raise NotImplementedError("inference engine: board-only path (empty move sequence) only")
        logits = self.board_logits(board).unsqueeze(1)
        targets = torch.roll(torch.full((board.shape[0], 64), 1928, dtype=torch.int64, device=logits.device), -1, 1)
        return logits, None, targets
