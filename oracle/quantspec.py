"""Quantised CPU reference of the board-transformer forward pass (TEST INFRASTRUCTURE, like the rest of
this package: only tests, the smoke check and the bench's checker / CPU-baseline legs import it).

`QuantSpec` wraps a `BT4Spec` (oracle/bt4spec.py) and re-runs its encoder with the operands of chosen
linears rounded to a low-precision grid and de-quantised again ("fake quantisation"); every product is
then an exact fp32 (int8: fp64) matmul of grid values, which is what a tensor core with a wide accumulator
computes. It restates the numerics contract of the reference's FP8 model, which has no arithmetic of its
own in the reference tree: `model_fp8.py:43-45,90-92,140` swaps the block linears (`c_attn`, `c_proj`,
`c_fc`, MLP `c_proj`) for Transformer-Engine linears and `pretrain_fp8.py:75-79` runs them under
`DelayedScaling(fp8_format=Format.E4M3, amax_history_len=16, amax_compute_algo="max")`, i.e. per-tensor
e4m3 operands scaled by 448 / amax with margin 0, high-precision outputs, LayerNorm / softmax / residual
stream outside FP8. Transformer-Engine itself is absent, so parity for the quantised paths is UNPINNED;
this file is their definition and the CUDA engine follows it.

Tap points ("sites") that can be switched one by one, named after the GEMM whose operands they round:
  qkv      input of the fused Q/K/V projection (the layer input) and its weight
  out      attention context and the out-projection weight
  ff1      FFN input and the ff1 weight
  ff2      FFN hidden activation (after the activation function) and the ff2 weight
  compress smolgen's per-token compression d -> 32 (shares the rounded layer input with qkv)
  bias_gemm the last smolgen product [B*H, gen] x [4096, gen]^T: the normalised generator rows and the shared weight
plus two storage roundings of the FP8 engine that are not GEMM operands:
  qkv_store  Q, K, V written as e4m3 with one scale and read back by attention
  bias_tile  the smolgen 64 x 64 bias written as e4m3 with one scale

Formats: "e4m3" (per-tensor or per-output-channel weight scale 448 / amax; activations per-tensor with a
static scale from `calibrate`, or per-token dynamic) and "int8" (symmetric, weights per output channel
amax / 127, activations per token dynamic, integer products accumulated exactly) - the W8A8 twin.
`bias_correct` adds (W - dequant(W8)) . mean(x) over the calibration batch to the bias of a rounded linear,
which cancels the mean effect of the weight rounding.
"""
import math

import torch
import torch.nn.functional as F

from . import bt4spec

E4M3_MAX = 448.0
ALL_GEMM_SITES = ("qkv", "out", "ff1", "ff2", "compress", "bias_gemm")
ALL_FP8_SITES = ALL_GEMM_SITES + ("qkv_store", "bias_tile")


def round_e4m3(x, mult):
    """x * mult rounded to the e4m3 grid (round to nearest even, saturating at +-448), divided by mult."""
    y = (x * mult).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).to(torch.float32)
    return y / mult


def e4m3_mult(amax):
    """Multiplier 448 / amax (1 where amax is 0); works on scalars and tensors."""
    amax = torch.as_tensor(amax, dtype=torch.float32)
    return torch.where(amax > 0, E4M3_MAX / amax, torch.ones_like(amax))


def round_int8_rows(x):
    """Per-row symmetric int8: scale = max|row| / 127, q = rint(x / scale) clamped to +-127. Returns (q, scale)
    with q holding integer values in the dtype of x."""
    amax = x.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(x * (1.0 / scale)).clamp(-127, 127)
    return q, scale


class QuantSpec:
    """Fake-quantised forward of a BT4Spec (post-LN or pre-LN blocks, any bias mode the spec supports).

    fmt            "e4m3" or "int8"
    sites          iterable of site names (see the module docstring); None = every site of the format
    weight_scale   "tensor" or "channel" (e4m3 only; int8 is always per output channel)
    act_scale      "static" (per tensor, from calibrate()) or "token" (dynamic per row; int8 is always that)
    bias_correct   apply the calibration-mean bias correction to the rounded linears (e4m3 only)
    layers         optional set of layer indices the rounding applies to (others run in fp32)
    """

    def __init__(self, spec, fmt="e4m3", sites=None, weight_scale="tensor", act_scale="static", bias_correct=True,
                 layers=None):
        assert fmt in ("e4m3", "int8")
        self.spec = spec.eval()
        self.cfg = spec.cfg
        self.fmt = fmt
        if sites is None:
            sites = ALL_FP8_SITES if fmt == "e4m3" else ("qkv", "out", "ff1", "ff2")
        self.sites = frozenset(sites)
        self.weight_scale = weight_scale if fmt == "e4m3" else "channel"
        self.act_scale = act_scale if fmt == "e4m3" else "token"
        self.bias_correct = bias_correct and fmt == "e4m3"
        self.layers = None if layers is None else frozenset(layers)
        self.amax = None          # per layer: dict tap -> float (static activation scales)
        self.mean = None          # per layer: dict site -> column means of the GEMM input
        self._wq = {}             # (layer, site) -> de-quantised weight (e4m3) or (int weight, scale) (int8)

    # ---- weights ------------------------------------------------------------------------------------
    def _weights(self, l, site):
        layer = self.spec.layers[l]
        if site == "qkv":
            a = layer.attention
            return (torch.cat([a.query_proj.weight, a.key_proj.weight, a.value_proj.weight], 0),
                    torch.cat([a.query_proj.bias, a.key_proj.bias, a.value_proj.bias], 0))
        if site == "out":
            return layer.attention.out_proj.weight, layer.attention.out_proj.bias
        if site == "ff1":
            return layer.ff1.weight, layer.ff1.bias
        if site == "ff2":
            return layer.ff2.weight, layer.ff2.bias
        if site == "compress":
            return layer.smolgen.compress.weight, None
        raise KeyError(site)

    def _active(self, l, site):
        return site in self.sites and (self.layers is None or l in self.layers)

    def _quant_weight(self, l, site):
        key = (l, site)
        if key not in self._wq:
            w, _ = self._weights(l, site)
            w = w.detach()
            if self.fmt == "int8":
                self._wq[key] = round_int8_rows(w.double())
            else:
                amax = w.abs().amax(-1, keepdim=True) if self.weight_scale == "channel" else w.abs().amax()
                self._wq[key] = round_e4m3(w, e4m3_mult(amax))
        return self._wq[key]

    def _linear(self, l, site, x, x_tap):
        """One nn.Linear of layer l, rounded if the site is active. x_tap names the static activation scale."""
        w, b = self._weights(l, site)
        if not self._active(l, site):
            return F.linear(x, w, b)
        if self.fmt == "int8":
            wq, ws = self._quant_weight(l, site)
            xq, xs = round_int8_rows(x.double())
            y = (xq @ wq.t()) * xs * ws.t()          # exact integer sums in fp64, then the two scales
            y = y.float()
            return y + b if b is not None else y
        wd = self._quant_weight(l, site)
        if self.act_scale == "token":
            xd = round_e4m3(x, e4m3_mult(x.abs().amax(-1, keepdim=True)))
        else:
            xd = round_e4m3(x, e4m3_mult(self.amax[l][x_tap]))
        y = F.linear(xd, wd)
        if b is not None:
            y = y + b
        if self.bias_correct and self.mean is not None and site != "compress":
            y = y + F.linear(self.mean[l][site], w.detach() - wd)
        return y

    # ---- one block ----------------------------------------------------------------------------------
    def _smolgen(self, l, x, record):
        sg = self.spec.layers[l].smolgen
        cfg = self.cfg
        b = x.size(0)
        c = self._linear(l, "compress", x, "in").reshape(b, -1)
        h1 = sg.ln1(bt4spec.activation(sg.dense1(c), cfg.act))
        h2 = bt4spec.activation(sg.dense2(h1), cfg.act).view(b, cfg.n_heads, cfg.smolgen_gen)
        gen = sg.ln2(h2)
        if record is not None:
            record["gen"] = max(record.get("gen", 0.0), gen.abs().max().item())
        if self._active(l, "bias_gemm") and self.fmt == "e4m3":
            if "shared" not in self._wq:
                w = self.spec.smolgen_shared.weight.detach()
                self._wq["shared"] = round_e4m3(w, e4m3_mult(w.abs().amax()))
            bias = F.linear(round_e4m3(gen, e4m3_mult(self.amax[l]["gen"])), self._wq["shared"])
        else:
            bias = self.spec.smolgen_shared(gen)
        if record is not None:
            record["bias"] = max(record.get("bias", 0.0), bias.abs().max().item())
        if self._active(l, "bias_tile") and self.fmt == "e4m3":
            bias = round_e4m3(bias, e4m3_mult(self.amax[l]["bias"]))
        return bias.view(b, cfg.n_heads, 64, 64)

    def _attention(self, l, x, pos_enc, bias, record):
        cfg = self.cfg
        att = self.spec.layers[l].attention
        b, h, hd, d = x.size(0), cfg.n_heads, cfg.d_model // cfg.n_heads, cfg.d_model
        qkv = self._linear(l, "qkv", x, "in")
        if record is not None:
            record["qkv"] = max(record.get("qkv", 0.0), qkv.abs().max().item())
        if self._active(l, "qkv_store") and self.fmt == "e4m3":
            qkv = round_e4m3(qkv, e4m3_mult(self.amax[l]["qkv"]))
        q, k, v = (t.view(b, 64, h, hd) for t in qkv.split(d, -1))
        k, v = k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3)
        if cfg.bias_mode == bt4spec.BIAS_RELPOS:
            p = att.pos_proj(pos_enc).view(b, -1, h, hd)
            content = torch.matmul((q + att.u_bias).transpose(1, 2), k.transpose(2, 3))
            pos = torch.matmul((q + att.v_bias).transpose(1, 2), p.permute(0, 2, 3, 1))
            score = (content + bt4spec.rel_shift(pos)) / math.sqrt(d)
        else:
            score = torch.matmul(q.transpose(1, 2), k.transpose(2, 3)) / math.sqrt(hd)
            if bias is not None:
                score = score + bias
            if cfg.bias_mode == bt4spec.BIAS_CAUSAL:
                score = score.masked_fill(torch.ones(64, 64, dtype=torch.bool).triu(1), float("-inf"))
        ctx = torch.matmul(F.softmax(score, -1), v).transpose(1, 2).contiguous().view(b, 64, d)
        if record is not None:
            record["ctx"] = max(record.get("ctx", 0.0), ctx.abs().max().item())
            record.setdefault("sum", {})["out"] = ctx.reshape(-1, d).sum(0)
        return self._linear(l, "out", ctx, "ctx")

    def _ffn(self, l, x, record):
        cfg = self.cfg
        if record is not None:
            record["ffn"] = max(record.get("ffn", 0.0), x.abs().max().item())
            record.setdefault("sum", {})["ff1"] = x.reshape(-1, x.size(-1)).sum(0)
        y = self._linear(l, "ff1", x, "ffn")
        if cfg.ffn_act_pos == bt4spec.FFN_ACT_MID:
            y = bt4spec.activation(y, cfg.act)
        if record is not None:
            record["hid"] = max(record.get("hid", 0.0), y.abs().max().item())
            record.setdefault("sum", {})["ff2"] = y.reshape(-1, y.size(-1)).sum(0)
        y = self._linear(l, "ff2", y, "hid")
        if cfg.ffn_act_pos != bt4spec.FFN_ACT_MID:
            y = bt4spec.activation(y, cfg.act)
        return y

    def _block(self, l, x, pos_enc, record):
        cfg = self.cfg
        layer = self.spec.layers[l]
        post = cfg.ln_mode == bt4spec.LN_POST
        a_in = x if post else layer.norm1(x)
        if record is not None:
            record["in"] = max(record.get("in", 0.0), a_in.abs().max().item())
            record.setdefault("sum", {})["qkv"] = a_in.reshape(-1, a_in.size(-1)).sum(0)
        bias = self._smolgen(l, a_in, record) if cfg.bias_mode == bt4spec.BIAS_SMOLGEN else None
        att = self._attention(l, a_in, pos_enc, bias, record)
        if post:
            x = layer.norm1(att + x)
            return layer.norm2(self._ffn(l, x, record) + x)
        x = x + att
        return x + self._ffn(l, layer.norm2(x), record)

    def _trunk(self, tokens, records=None):
        s = self.spec
        x = s.ma_gating(s.layernorm1(F.gelu(s.linear1(tokens))))
        pos_enc = s._pe.expand(x.size(0), -1, -1)
        for l in range(self.cfg.n_layers):
            x = self._block(l, x, pos_enc, None if records is None else records[l])
        if self.cfg.ln_mode == bt4spec.LN_PRE:
            x = s.norm_f(x)
        return x, pos_enc

    # ---- public -------------------------------------------------------------------------------------
    @torch.no_grad()
    def calibrate(self, tokens, chunk=64):
        """Static activation scales (per-tensor amax of every tap) and the column means of the four GEMM
        inputs, from an UNQUANTISED pass over `tokens` [B,64,P] - the engine's calibration pass likewise
        runs its 16-bit path."""
        saved = self.sites
        self.sites = frozenset()
        records = [dict() for _ in range(self.cfg.n_layers)]
        sums = [dict() for _ in range(self.cfg.n_layers)]
        rows = 0
        for b0 in range(0, tokens.size(0), chunk):
            part = tokens[b0:b0 + chunk]
            self._trunk(part, records)
            rows += part.size(0) * 64
            for l, r in enumerate(records):
                for k, v in r.pop("sum", {}).items():
                    sums[l][k] = sums[l].get(k, 0) + v
        self.sites = saved
        self.amax = records
        self.mean = [{k: v / rows for k, v in s.items()} for s in sums]
        return self

    @torch.no_grad()
    def forward_all(self, tokens, chunk=64):
        """tokens [B,64,P] f32 -> dict(policy raw logits, wdl raw logits, q tanh) like BT4Spec.forward_all."""
        if self.fmt == "e4m3" and self.act_scale == "static" and self.amax is None:
            raise RuntimeError("QuantSpec.calibrate(tokens) has to run before a static-scale e4m3 forward")
        outs = []
        for b0 in range(0, tokens.size(0), chunk):
            x, pos_enc = self._trunk(tokens[b0:b0 + chunk])
            out = {}
            s = self.spec
            if self.cfg.value_mode != bt4spec.VALUE_NONE:
                out["wdl"] = s.value_head(x)
            if self.cfg.value_mode == bt4spec.VALUE_WDL_Q:
                out["q"] = torch.tanh(s.value_head_q(x))
            if self.cfg.policy_mode != bt4spec.POLICY_NONE:
                out["policy"] = s.policy_logits(x, pos_enc)
            outs.append(out)
        return {k: torch.cat([o[k] for o in outs], 0) for k in outs[0]}


def agreement(pol, ref_masked, legal):
    """(top-1 agreement over legal moves, max-abs logit error over legal moves) of masked policy rows."""
    same = (pol.argmax(-1) == ref_masked.argmax(-1)).float().mean().item()
    err = (pol - ref_masked)[legal].abs().max().item()
    return same, err
