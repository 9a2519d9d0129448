"""Seeded synthetic weights and inputs with the shapes and value distributions of the real ones
(random-init N(0, 0.02) weights; sparse 0/1 piece planes, constant and fractional scalar planes;
a few dozen legal moves per position). Used by the benchmark and the examples; no dataset or
checkpoint of the reference is available offline."""
import numpy as np
import torch

_KEEP = ("norm1.", "norm2.", "layernorm1.", "ln1.", "ln2.", "norm_f.", "ma_gating.")


def seeded_state_dict(shapes, seed=0, std=0.02):
    """shapes: {key: shape} (e.g. from `modules._param_shapes`). Every tensor ~ N(0, std) drawn in sorted
    key order from one seeded CPU generator; LayerNorm weights 1 / biases 0, gating a = 0, b = 1."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for k in sorted(shapes):
        shape = tuple(shapes[k])
        if any(t in k for t in _KEEP):
            ones = k.endswith(".weight") or k == "ma_gating.b"
            sd[k] = torch.ones(shape) if ones else torch.zeros(shape)
        else:
            sd[k] = torch.randn(shape, generator=g) * std
    return sd


def synthetic_planes(batch, planes=112, seed=0, dtype=torch.float16, chunk=8192):
    """[batch, 8, 8, planes]: piece planes Bernoulli(32/(64*12)) per square (about 32 pieces per board
    step), castling / side planes constant per board, a rule-50 fraction plane, a plane of ones."""
    g = torch.Generator().manual_seed(seed)
    out = torch.empty(batch, 8, 8, planes, dtype=dtype)
    for b0 in range(0, batch, chunk):
        n = min(chunk, batch - b0)
        x = (torch.rand(n, 8, 8, planes, generator=g) < (32.0 / (64 * 12))).to(dtype)
        if planes >= 8:
            flags = (torch.rand(n, 1, 1, 5, generator=g) < 0.5).to(dtype)
            x[..., planes - 8:planes - 3] = flags.expand(n, 8, 8, 5)
            x[..., planes - 3] = (torch.rand(n, 1, 1, generator=g) * 0.5).to(dtype).expand(n, 8, 8)
            x[..., planes - 2] = 0
            x[..., planes - 1] = 1
        out[b0:b0 + n] = x
    return out


def synthetic_legal_bits(batch, n_moves=1858, seed=1, mean_legal=30):
    """uint8 bitset [batch, ceil(n_moves/8)], bit m (little-endian within the byte) = move m legal."""
    rng = np.random.default_rng(seed)
    legal = rng.random((batch, n_moves)) < (mean_legal / n_moves)
    legal[:, 0] = True
    return torch.from_numpy(np.packbits(legal, axis=1, bitorder="little"))
