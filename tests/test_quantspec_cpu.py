"""The quantised CPU reference (oracle/quantspec.py): grid roundings against hand-computed e4m3 / int8 values, the
identity with the fp32 oracle when no site is rounded, and the properties the GPU tests rely on."""
import numpy as np
import torch

from oracle import bt4spec, quantspec


def small_spec(layers=2, smolgen=True, seed=3):
    cfg = bt4spec.SpecConfig.baseline(layers, 128, 256, 4, smolgen=smolgen)
    spec = bt4spec.BT4Spec(cfg)
    spec.load_state_dict(bt4spec.seeded_state_dict(spec, seed=seed))
    return spec.eval()


def tokens(batch, seed=5):
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand(batch, 64, 112, generator=g) < 0.08).float()
    x[:, :, 111] = 1.0
    return x


def test_e4m3_grid_known_answers():
    """e4m3: 3 mantissa bits, largest finite 448, spacing 2^(e-3) inside [2^e, 2^(e+1)), subnormal spacing 2^-9;
    round to nearest, ties to the even mantissa; the multiplier follows the reference recipe's 448 / amax (margin 0,
    pretrain_fp8.py:75-79)."""
    x = torch.tensor([0.0, 1.0, 1.0625, 1.0626, 17.0, 19.0, 447.0, 448.0, 500.0, -1000.0, 2.0 ** -9, 2.0 ** -10, 0.0029])
    want = torch.tensor([0.0, 1.0, 1.0, 1.125, 16.0, 20.0, 448.0, 448.0, 448.0, -448.0, 2.0 ** -9, 0.0, 2.0 ** -9 * 1.0])
    got = quantspec.round_e4m3(x, torch.tensor(1.0))
    assert torch.equal(got[:-1], want[:-1])
    assert got[-1].item() in (2.0 ** -9, 2.0 ** -8)          # 0.0029 = 1.48 subnormal steps: rounds to one step
    assert quantspec.e4m3_mult(7.0).item() == 64.0 and quantspec.e4m3_mult(0.0).item() == 1.0
    # a multiplier moves the grid: 0.3 * 448 / 0.5 = 268.8 -> 256 (spacing 32) -> 0.2857...
    y = quantspec.round_e4m3(torch.tensor([0.3, -0.5]), quantspec.e4m3_mult(0.5))
    assert torch.allclose(y, torch.tensor([256.0 / 896.0, -0.5]), rtol=0, atol=1e-7)


def test_int8_rows_known_answers():
    x = torch.tensor([[1.0, -2.0, 0.5, 127.0], [0.0, 0.0, 0.0, 0.0], [0.3, -0.1, 0.05, 0.0]], dtype=torch.float64)
    q, s = quantspec.round_int8_rows(x)
    assert torch.equal(q[0], torch.tensor([1.0, -2.0, 0.0, 127.0], dtype=torch.float64))    # 0.5 ties to even
    assert s[0].item() == 1.0 and s[1].item() == 1.0 and torch.equal(q[1], torch.zeros(4, dtype=torch.float64))
    assert torch.equal(q[2], torch.tensor([127.0, -42.0, 21.0, 0.0], dtype=torch.float64))
    assert abs(s[2].item() - 0.3 / 127) < 1e-15


def test_no_sites_is_the_fp32_oracle_bit_for_bit():
    for smolgen in (True, False):
        spec = small_spec(smolgen=smolgen)
        x = tokens(3)
        with torch.no_grad():
            ref = spec.forward_all(x)
        out = quantspec.QuantSpec(spec, sites=()).calibrate(x).forward_all(x)
        for k in ref:
            assert torch.equal(out[k], ref[k]), k


def test_prelayernorm_blocks_and_reference_form_run_through_the_same_taps():
    cfg = bt4spec.SpecConfig(112, 128, 2, 4, 256, bt4spec.LN_PRE, bt4spec.ACT_GELU, bt4spec.FFN_ACT_END, bt4spec.BIAS_NONE,
                             bt4spec.POLICY_GATHER1858, bt4spec.VALUE_WDL)
    spec = bt4spec.BT4Spec(cfg)
    spec.load_state_dict(bt4spec.seeded_state_dict(spec, seed=1))
    spec.eval()
    x = tokens(2)
    with torch.no_grad():
        ref = spec.forward_all(x)
    same = quantspec.QuantSpec(spec, sites=()).calibrate(x).forward_all(x)
    assert torch.equal(same["policy"], ref["policy"])
    q = quantspec.QuantSpec(spec, sites=("qkv", "out", "ff1", "ff2")).calibrate(x).forward_all(x)
    err = (q["policy"] - ref["policy"]).abs().max().item()
    assert 0 < err < 0.1


def test_e4m3_rounding_stays_small_and_every_site_contributes():
    spec = small_spec()
    x = tokens(8)
    with torch.no_grad():
        ref = spec.forward_all(x)
    full = quantspec.QuantSpec(spec).calibrate(x).forward_all(x)
    e_full = (full["policy"] - ref["policy"]).pow(2).mean().sqrt().item()
    assert 1e-4 < e_full / ref["policy"].std().item() < 0.3          # small against the logits' own spread, not zero
    assert (torch.softmax(full["wdl"], -1) - torch.softmax(ref["wdl"], -1)).abs().max() < 3e-2
    for site in quantspec.ALL_FP8_SITES:
        one = quantspec.QuantSpec(spec, sites=(site,)).calibrate(x).forward_all(x)
        e_one = (one["policy"] - ref["policy"]).pow(2).mean().sqrt().item()
        assert 0 < e_one < e_full * 1.5, site
    # layers restricts the rounding to the named blocks
    first = quantspec.QuantSpec(spec, layers=(0,)).calibrate(x).forward_all(x)
    assert 0 < (first["policy"] - ref["policy"]).abs().max() and not torch.equal(first["policy"], full["policy"])


def test_bias_correction_cancels_the_mean_effect_of_weight_rounding():
    """With every activation row equal to the calibration mean, W8 x + (W - W8) mean = W x exactly: the corrected
    linear reproduces the unrounded one on the mean input (up to the activation rounding, switched off here by
    feeding grid values)."""
    spec = small_spec(smolgen=False)
    x = tokens(6)
    qs = quantspec.QuantSpec(spec, sites=("ff1",)).calibrate(x)
    layer = spec.layers[0]
    mean = qs.mean[0]["ff1"]
    row = quantspec.round_e4m3(mean, quantspec.e4m3_mult(qs.amax[0]["ffn"]))     # on the activation grid
    qs.mean[0]["ff1"] = row
    with torch.no_grad():
        want = torch.nn.functional.linear(row, layer.ff1.weight, layer.ff1.bias)
        got = qs._linear(0, "ff1", row[None], "ffn")[0]
    assert torch.allclose(got, want, atol=2e-6)
    plain = quantspec.QuantSpec(spec, sites=("ff1",), bias_correct=False).calibrate(x)
    with torch.no_grad():
        off = plain._linear(0, "ff1", row[None], "ffn")[0]
    assert (off - want).abs().max() > 10 * (got - want).abs().max()


def test_int8_twin_is_exact_on_representable_operands():
    """Weights that are integer multiples of their row scale and activations that are integers with row maximum 127
    pass through the W8A8 path unchanged: integer products, exact sums, two scales."""
    spec = small_spec(smolgen=False)
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        w = torch.randint(-127, 128, spec.layers[0].ff1.weight.shape, generator=g).float()
        w[:, 0] = 127.0
        spec.layers[0].ff1.weight.copy_(w * 2.0 ** -9)
    qs = quantspec.QuantSpec(spec, fmt="int8", sites=("ff1",))
    a = torch.randint(-127, 128, (5, 128), generator=g).float()
    a[:, 0] = 127.0
    with torch.no_grad():
        want = torch.nn.functional.linear(a.double(), spec.layers[0].ff1.weight.double(), spec.layers[0].ff1.bias.double())
        got = qs._linear(0, "ff1", a, "ffn")
    assert torch.allclose(got.double(), want, rtol=1e-6, atol=1e-6)
    out = qs.forward_all(tokens(2))                       # needs no calibration
    assert torch.isfinite(out["policy"]).all()


def test_agreement_helper():
    ref = torch.tensor([[0.0, 1.0, -999.0], [2.0, 0.5, 0.1]])
    pol = torch.tensor([[0.2, 0.9, -999.0], [0.4, 0.5, 0.1]])
    legal = torch.tensor([[True, True, False], [True, True, True]])
    same, err = quantspec.agreement(pol, ref, legal)
    assert same == 0.5 and abs(err - 1.6) < 1e-6
