"""Parity of the CUDA engine (through the C ABI) against the CPU oracle and the reference fixtures.

Tolerances are the ones the target states: FP16 policy-logit max-abs error <= 2e-2 and WDL
probabilities within 1e-2 of the FP32 reference; masks and indices are exact."""
import glob
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import bt4spec, vocab

pytestmark = pytest.mark.gpu

POLICY_TOL = 2e-2
WDL_TOL = 1e-2


def engine_cfg(spec_cfg, **kw):
    from chessrl_b200 import EngineConfig
    return EngineConfig(dtype=kw.pop("dtype", 0), chunk=kw.pop("chunk", 0), **spec_cfg.to_dict())


def random_tokens(batch, planes, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand(batch, 64, planes, generator=g) < 0.08).float()
    x[:, :, planes - 1] = 1.0
    x[:, :, planes - 3] = (torch.rand(batch, 1, generator=g) * 0.5).half().float().expand(batch, 64)
    return x


def oracle_out(spec_cfg, sd, tokens):
    spec = bt4spec.BT4Spec(spec_cfg)
    spec.load_state_dict(sd)
    spec.eval()
    with torch.no_grad():
        return spec.forward_all(tokens)


def run_engine(spec_cfg, sd, tokens, **fw):
    from chessrl_b200 import Engine
    eng = Engine(engine_cfg(spec_cfg, dtype=fw.pop("dtype", 0), chunk=fw.pop("chunk", 0)))
    eng.load_state_dict(sd)
    x = tokens.view(tokens.shape[0], 8, 8, -1).cuda()
    out = eng.forward(x, **fw)
    torch.cuda.synchronize()
    rc, st = eng.last_status()
    assert rc == 0 and st == 0, f"device status {st}"
    assert eng.last_launch_count() > 0
    return {k: v.float().cpu() for k, v in out.items()}, eng


CASES = sorted(glob.glob(os.path.join(GOLDEN, "ref_value*.npz")))


@pytest.mark.parametrize("path", CASES, ids=[os.path.basename(p)[:-4] for p in CASES])
def test_reference_fixture(path):
    """Engine vs outputs of the unmodified reference module (relative attention, dense 1929 policy)."""
    from test_oracle_golden import golden_state_dict, spec_for
    z = np.load(path)
    dims = [int(v) for v in z["dims"]]
    cfg = spec_for(os.path.basename(path), dims)
    sd = golden_state_dict(bt4spec.BT4Spec(cfg), int(z["seed"]))
    tokens = torch.from_numpy(z["tokens"]).float()
    out, _ = run_engine(cfg, sd, tokens, wdl_softmax=False, q="q" in z.files)
    assert (out["policy"] - torch.from_numpy(z["policy"])).abs().max() <= POLICY_TOL
    assert (out["wdl"] - torch.from_numpy(z["wdl"])).abs().max() <= POLICY_TOL
    probs = torch.softmax(out["wdl"], -1)
    assert (probs - torch.softmax(torch.from_numpy(z["wdl"]), -1)).abs().max() <= WDL_TOL
    if "q" in z.files:
        assert (out["q"].view(-1) - torch.from_numpy(z["q"]).view(-1)).abs().max() <= WDL_TOL


@pytest.mark.parametrize("name,cfg,batch", [
    ("c2_small_gather", bt4spec.SpecConfig.baseline(8, 256, 1024, 8, smolgen=False), 5),
    ("c2_small_smolgen", bt4spec.SpecConfig.baseline(2, 256, 1024, 8, smolgen=True), 3),
    ("bt4_shape_2layers", bt4spec.SpecConfig.baseline(2, 1024, 1536, 32, smolgen=True), 3),
    ("prelN_gelu_end", bt4spec.SpecConfig(112, 256, 2, 8, 512, bt4spec.LN_PRE, bt4spec.ACT_GELU, bt4spec.FFN_ACT_END,
                                          bt4spec.BIAS_NONE, bt4spec.POLICY_GATHER1858, bt4spec.VALUE_WDL), 2),
    ("hd64_relpos", bt4spec.SpecConfig.reference_value_q(2, 512, 736, 8), 2),
    ("value_only", bt4spec.SpecConfig.baseline(2, 256, 1024, 8, smolgen=True, value_only=True), 4),
])
def test_against_oracle(name, cfg, batch):
    torch.manual_seed(0)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=3)
    tokens = random_tokens(batch, cfg.planes, seed=5)
    ref = oracle_out(cfg, sd, tokens)
    out, _ = run_engine(cfg, sd, tokens, wdl_softmax=True)
    if "policy" in ref:
        assert (out["policy"] - ref["policy"]).abs().max() <= POLICY_TOL
        assert torch.equal(out["policy"].argmax(-1), ref["policy"].argmax(-1)) or \
            (out["policy"] - ref["policy"]).abs().max() <= 2e-3
    else:
        assert "policy" not in out
    assert (out["wdl"] - torch.softmax(ref["wdl"], -1)).abs().max() <= WDL_TOL


def test_chunking_and_ragged_batch_are_invisible():
    """A batch that is not a multiple of the chunk, processed in several passes, equals one pass."""
    cfg = bt4spec.SpecConfig.baseline(2, 256, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=4)
    tokens = random_tokens(11, cfg.planes, seed=6)
    one, _ = run_engine(cfg, sd, tokens, chunk=64)
    many, _ = run_engine(cfg, sd, tokens, chunk=4)
    assert torch.equal(one["policy"], many["policy"]) and torch.equal(one["wdl"], many["wdl"])


def test_legal_mask_conventions_exact():
    """logits + (1-mask)*(-999) for a bitset (model_bis.py:383) and mask_vec + logits with -1000/0
    (Leela/server.py:56): the masked index set is exact, softmax mass on illegal moves vanishes."""
    cfg = bt4spec.SpecConfig.baseline(2, 256, 512, 8, smolgen=False)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=7)
    b = 6
    tokens = random_tokens(b, cfg.planes, seed=8)
    g = torch.Generator().manual_seed(9)
    legal = torch.rand(b, 1858, generator=g) < 0.02
    legal[:, 0] = True
    bits = np.packbits(legal.numpy(), axis=1, bitorder="little")
    bits_t = torch.from_numpy(bits).cuda()
    raw, eng = run_engine(cfg, sd, tokens)
    x = tokens.view(b, 8, 8, -1).cuda()
    masked = eng.forward(x, legal_mask=bits_t)["policy"].cpu()
    expect = raw["policy"] + (1 - legal.float()) * -999
    assert torch.equal(masked, expect)
    additive = ((~legal).float() * -1000.0).cuda()
    probs = eng.forward(x, legal_mask=additive, policy_softmax=True)["policy"].cpu()
    ref = torch.softmax(raw["policy"] + additive.cpu(), -1)
    assert (probs - ref).abs().max() < 1e-5
    assert torch.equal(probs > 0, legal) or float(probs[~legal].max()) == 0.0
    assert torch.equal(probs.argmax(-1), ref.argmax(-1))


def test_input_layouts_agree():
    """[B,8,8,P] f32 (module signature), the same in f16, and [B,P,8,8] f16 (server) give one result."""
    cfg = bt4spec.SpecConfig.baseline(1, 256, 512, 8, smolgen=False)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=10)
    tokens = random_tokens(3, cfg.planes, seed=11)
    a, eng = run_engine(cfg, sd, tokens)
    x = tokens.view(3, 8, 8, -1).cuda()
    b = eng.forward(x.half())["policy"].cpu()
    c = eng.forward(x.half().permute(0, 3, 1, 2).contiguous(), layout="nchw")["policy"].cpu()
    assert torch.equal(a["policy"], b) and torch.equal(a["policy"], c)


def test_host_entry_point_matches_device_entry_point():
    cfg = bt4spec.SpecConfig.baseline(1, 256, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=12)
    tokens = random_tokens(4, cfg.planes, seed=13)
    dev, eng = run_engine(cfg, sd, tokens)
    host = eng.forward(tokens.view(4, 8, 8, -1).half().pin_memory(), host=True)
    assert torch.equal(dev["policy"], host["policy"]) and torch.equal(dev["wdl"], host["wdl"])


def test_module_drop_in_round_trips_state_dict():
    """The nn.Module keeps the reference's key names and shapes and serves `forward(inp)`."""
    from chessrl_b200 import BT4
    cfg = bt4spec.SpecConfig.reference_value_q(2, 256, 320, 8)
    spec = bt4spec.BT4Spec(cfg)
    sd = bt4spec.seeded_state_dict(spec, seed=14)
    model = BT4(2, 256, 320, 8)
    assert {k: tuple(v.shape) for k, v in model.state_dict().items()} == {k: tuple(v.shape) for k, v in sd.items()}
    model.load_state_dict(sd)
    tokens = random_tokens(2, 112, seed=15)
    pol = model([tokens.view(2, 1, 8, 8, 112), None])
    assert pol.shape == (2, 1, 1929)
    ref = oracle_out(cfg, sd, tokens)
    assert (pol.view(2, -1).cpu() - ref["policy"]).abs().max() <= POLICY_TOL
    vals = model.position_values(tokens.view(2, 8, 8, 112)).cpu()
    assert (vals - torch.softmax(ref["wdl"], -1)).abs().max() <= WDL_TOL


def test_errors_are_reported_not_thrown_across_the_abi():
    from chessrl_b200 import Engine, CrlError
    cfg = bt4spec.SpecConfig.baseline(1, 256, 512, 8, smolgen=False)
    eng = Engine(engine_cfg(cfg))
    with pytest.raises(CrlError) as e:
        eng.forward(torch.zeros(1, 8, 8, 112, device="cuda"))
    assert e.value.code == -5                      # not finalized
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=1)
    missing = dict(sd)
    del missing["ma_gating.a"]
    with pytest.raises(CrlError) as e:
        eng.load_state_dict(missing)
    assert e.value.code == -4 and "ma_gating.a" in str(e.value)
    eng.load_state_dict(sd)
    assert eng.forward(torch.zeros(0, 8, 8, 112, device="cuda"))["policy"].shape == (0, 1858)   # empty batch


def test_fp8_engine_tolerances():
    """FP8 e4m3 (per-tensor weight and calibrated activation scales on the QKV / out-proj / FFN GEMMs)
    against the FP32 oracle: top-1 move agreement >= 99 %, WDL within 3e-2. The move is the arg-max
    over the legal moves (a few dozen per position, seeded), which is how every caller of the reference
    picks it (model_bis.py:383-386, value.py:231-234, Leela/server.py:56)."""
    from chessrl_b200 import Engine, CrlError, synth
    cfg = bt4spec.SpecConfig.baseline(8, 256, 1024, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=21)
    b = 1024
    tokens = random_tokens(b, cfg.planes, seed=22)
    ref = oracle_out(cfg, sd, tokens)
    bits = synth.synthetic_legal_bits(b, 1858, seed=23)
    legal = torch.from_numpy(np.unpackbits(bits.numpy(), axis=1, bitorder="little")[:, :1858].astype(bool))
    eng = Engine(engine_cfg(cfg, dtype=1))
    eng.load_state_dict(sd)
    x = tokens.view(b, 8, 8, -1).cuda()
    with pytest.raises(CrlError):
        eng.forward(x)                                  # FP8 needs calibration first
    eng.calibrate(x[:256])
    out = eng.forward(x, legal_mask=bits.cuda())
    rc, st = eng.last_status()
    assert rc == 0 and st == 0
    pol, wdl = out["policy"].cpu(), out["wdl"].cpu()
    ref_masked = bt4spec.apply_policy_mask(ref["policy"], legal_bits=legal)
    agree = (pol.argmax(-1) == ref_masked.argmax(-1)).float().mean().item()
    agree_unmasked = ((pol - (1 - legal.float()) * -999).argmax(-1) == ref["policy"].argmax(-1)).float().mean().item()
    werr = (wdl - torch.softmax(ref["wdl"], -1)).abs().max().item()
    perr = (pol - ref_masked).abs().max().item()
    print(f"fp8: top-1 agreement over legal moves {agree:.4f} (over all 1858 logits {agree_unmasked:.4f}), "
          f"wdl err {werr:.3e}, policy max-abs err {perr:.3e}")
    assert agree >= 0.99 and werr <= 3e-2


def test_rl_vocabulary_scatter_matches_map_leela_to_rl():
    """1858 -> 1929 with rank mirroring for Black rows, fused into the policy kernel, against the oracle's
    restatement of Leela/compare_policy.py:493-523 (index map exact, values untouched)."""
    cfg = bt4spec.SpecConfig.baseline(1, 256, 512, 8, smolgen=False)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=16)
    tokens = random_tokens(7, cfg.planes, seed=17)
    native, eng = run_engine(cfg, sd, tokens, policy_softmax=True)
    x = tokens.view(7, 8, 8, -1).cuda()
    black = torch.tensor([0, 1, 0, 1, 0, 1, 0], dtype=torch.uint8)          # first_is_white=True
    got = eng.forward(x, policy_softmax=True, rl_vocab=True, black_rows=black.cuda())["policy"].cpu()
    want = torch.from_numpy(vocab.map_leela_to_rl(native["policy"].numpy(), first_is_white=True))
    assert got.shape == (7, 1929) and torch.equal(got, want)
    host = eng.forward(tokens.view(7, 8, 8, -1).half().pin_memory(), policy_softmax=True, rl_vocab=True,
                       black_rows=black.pin_memory(), host=True)["policy"]
    assert torch.equal(host, want)


def test_gpt_board_only_path_against_reference_fixture():
    """The decoder model's board-only forward (model_bis.py:358-370; pre-LN, causal, last-token LM head)
    through the nn.Module drop-in, against logits of the unmodified reference GPT."""
    from chessrl_b200 import GPT, GPTConfig
    from oracle import gptspec
    from test_oracle_golden import gpt_golden_state_dict
    z = np.load(os.path.join(GOLDEN, "ref_gpt_L2_d128_h2.npz"))
    n_layer, n_head, d = [int(v) for v in z["dims"]]
    sd = gpt_golden_state_dict(gptspec.GPTSpec(gptspec.GPTConfig(256, 1929, n_layer, n_head, d)), int(z["seed"]))
    model = GPT(GPTConfig(256, 1929, n_layer, n_head, d))
    assert {k: tuple(v.shape) for k, v in model.state_dict().items()} == {k: tuple(v.shape) for k, v in sd.items()}
    model.load_state_dict(sd)
    board = torch.from_numpy(z["board"]).float()
    logits, loss, targets = model((board, torch.zeros(board.shape[0], 0, dtype=torch.int64)))
    assert logits.shape == (3, 1, 1929) and loss is None and targets.shape == (3, 64)
    assert (logits[:, 0].cpu() - torch.from_numpy(z["logits"])).abs().max() <= POLICY_TOL
    # masked, temperature-1 softmax as in model_bis.py:383-389
    legal = torch.zeros(3, 1929, dtype=torch.bool)
    legal[:, [3, 77, 1500, 1900]] = True
    bits = torch.from_numpy(np.packbits(legal.numpy(), axis=1, bitorder="little")).cuda()
    probs = model.board_logits(board, legal_mask=bits, softmax=True).cpu()
    ref = torch.softmax(torch.from_numpy(z["logits"]) + (1 - legal.float()) * -999, -1)
    assert (probs - ref).abs().max() <= 1e-2 and torch.equal(probs.argmax(-1), ref.argmax(-1))


@pytest.mark.parametrize("value_only", [True, False])
def test_int8_w8a8_engine_tolerances(value_only):
    """INT8 W8A8 on the QKV / out-proj / FFN GEMMs (per-output-channel symmetric weights, per-token dynamic
    activations, int32 accumulation) against the FP32 oracle: WDL within 3e-2; with a policy head, top-1
    agreement over the legal moves >= 99 %. value_only is the WDL-only network of the target's config 5."""
    from chessrl_b200 import Engine, synth
    cfg = bt4spec.SpecConfig.baseline(8, 256, 1024, 8, smolgen=True, value_only=value_only)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=31)
    b = 1024 if not value_only else 256
    tokens = random_tokens(b, cfg.planes, seed=32)
    ref = oracle_out(cfg, sd, tokens)
    eng = Engine(engine_cfg(cfg, dtype=2))
    eng.load_state_dict(sd)
    x = tokens.view(b, 8, 8, -1).cuda()
    bits = synth.synthetic_legal_bits(b, 1858, seed=33)
    out = eng.forward(x, legal_mask=None if value_only else bits.cuda())
    rc, st = eng.last_status()
    assert rc == 0 and st == 0
    werr = (out["wdl"].cpu() - torch.softmax(ref["wdl"], -1)).abs().max().item()
    msg = f"int8: wdl err {werr:.3e}"
    if not value_only:
        legal = torch.from_numpy(np.unpackbits(bits.numpy(), axis=1, bitorder="little")[:, :1858].astype(bool))
        ref_masked = bt4spec.apply_policy_mask(ref["policy"], legal_bits=legal)
        agree = (out["policy"].cpu().argmax(-1) == ref_masked.argmax(-1)).float().mean().item()
        msg += f", top-1 agreement over legal moves {agree:.4f}"
        assert agree >= 0.99
    else:
        assert "policy" not in out
    print(msg)
    assert werr <= 3e-2


def test_config1_shape_on_playout_positions_with_real_legal_masks():
    """The 256-wide 8-layer encoder on 64 seeded random-playout positions (112-plane history input and legal
    masks from the library's move generator) against the FP32 oracle: logits within 2e-2, WDL within 1e-2,
    and the soft-maxed, masked policy puts exactly zero mass outside the legal moves."""
    from chessrl_b200 import positions
    cfg = bt4spec.SpecConfig.baseline(8, 256, 1024, 8, smolgen=False)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=41)
    pos = positions.playout_positions(64, seed=20240607, max_plies=80)
    tokens = pos["planes112"].float().view(64, 64, 112)
    ref = oracle_out(cfg, sd, tokens)
    out, eng = run_engine(cfg, sd, tokens)
    assert (out["policy"] - ref["policy"]).abs().max() <= POLICY_TOL
    assert (out["wdl"] - torch.softmax(ref["wdl"], -1)).abs().max() <= WDL_TOL
    legal = torch.from_numpy(np.unpackbits(pos["legal1858"].numpy(), axis=1, bitorder="little")[:, :1858].astype(bool))
    probs = eng.forward(pos["planes112"].cuda(), legal_mask=pos["legal1858"].cuda(), policy_softmax=True)["policy"].cpu()
    assert float(probs[~legal].max()) == 0.0 and torch.allclose(probs.sum(-1), torch.ones(64), atol=1e-4)
    want = torch.softmax(bt4spec.apply_policy_mask(ref["policy"], legal_bits=legal), -1)
    assert (probs - want).abs().max() <= 1e-2


def test_packed104_input_is_bit_identical_to_f16_planes():
    """The 840-byte bit-packed records expanded on the device give the same token rows as the f16 planes they
    were packed from: policy and WDL are bit-identical, through the device call (two chunks + a ragged tail),
    the host call and the allocation-free call, for the FP16 and the FP8 engine."""
    from chessrl_b200 import Engine, positions
    import chessrl_b200 as crl
    cfg = bt4spec.SpecConfig.baseline(2, 256, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=51)
    n = 150
    pos = positions.playout_positions(n, seed=3, max_plies=100)
    planes = pos["planes112"]
    packed = positions.pack_planes104(planes)
    for dtype in (crl.DTYPE_F16, crl.DTYPE_F8E4M3):
        eng = Engine(engine_cfg(cfg, dtype=dtype, chunk=64))
        eng.load_state_dict(sd)
        if dtype == crl.DTYPE_F8E4M3:
            eng.calibrate(packed[:64].cuda(), layout="packed104")
        kw = dict(legal_mask=pos["legal1858"].cuda(), policy_softmax=True)
        a = eng.forward(planes.cuda(), **kw)
        b = eng.forward(packed.cuda(), layout="packed104", **kw)
        assert torch.equal(a["policy"], b["policy"]) and torch.equal(a["wdl"], b["wdl"])
        c = eng.forward(packed.pin_memory(), layout="packed104", host=True, legal_mask=pos["legal1858"], policy_softmax=True)
        assert torch.equal(a["policy"].cpu(), c["policy"]) and torch.equal(a["wdl"].cpu(), c["wdl"])
        rc, st = eng.last_status()
        assert rc == 0 and st == 0
    with pytest.raises(ValueError):
        eng.forward(packed[:, :839].contiguous().cuda(), layout="packed104")
    eng19 = Engine(engine_cfg(bt4spec.SpecConfig.reference_value(1, 64, 96, 2)))
    eng19.load_state_dict(bt4spec.seeded_state_dict(bt4spec.BT4Spec(bt4spec.SpecConfig.reference_value(1, 64, 96, 2)), seed=1))
    with pytest.raises(crl.CrlError):
        eng19.forward(packed.cuda(), layout="packed104")


def test_move_choice_on_device_matches_oracle():
    """Arg-max and inverse-CDF draws made on the GPU from the policy rows (logits and probabilities, f32 and f16,
    temperatures 0 / 0.5 / 1 / 2, native and 1929-entry vocabulary) equal the numpy oracle applied to the rows
    the same call returned; a draw may differ only where u * total sits within rounding of a CDF step. The host
    entry point with policy=False returns the same indices while copying back 4 bytes per position."""
    from chessrl_b200 import Engine, positions
    cfg = bt4spec.SpecConfig.baseline(2, 256, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=61)
    n = 300
    pos = positions.playout_positions(n, seed=9, max_plies=100)
    planes, bits = pos["planes112"].cuda(), pos["legal1858"].cuda()
    eng = Engine(engine_cfg(cfg, chunk=128))
    eng.load_state_dict(sd)
    g = torch.Generator().manual_seed(5)
    u = torch.rand(n, generator=g)
    legal = np.unpackbits(pos["legal1858"].numpy(), axis=1, bitorder="little")[:, :1858].astype(bool)
    for softmax in (False, True):
        for dtype in (torch.float32, torch.float16):
            for temp in (0.0, 0.5, 1.0, 2.0):
                for rl in (False, True):
                    out = eng.forward(planes, legal_mask=bits, policy_softmax=softmax, policy_dtype=dtype, moves=True,
                                      temperature=temp, uniforms=u.cuda(), rl_vocab=rl,
                                      black_rows=pos["black"].cuda() if rl else None)
                    rows = out["policy"].float().cpu().numpy()
                    want, margin = vocab.choose_moves(rows, softmax, temp, u.numpy())
                    got = out["move"].cpu().numpy()
                    bad = got != want
                    assert not (bad & (margin > 1e-5)).any(), (softmax, dtype, temp, rl, int(bad.sum()))
                    assert bad.sum() <= 2
                    if not rl and temp <= 1.0:
                        assert legal[np.arange(n), got].all()          # a masked move is never chosen
    am = eng.forward(planes, legal_mask=bits, moves=True)["move"].cpu()
    assert torch.equal(am, eng.forward(planes, legal_mask=bits)["policy"].argmax(-1).int().cpu())
    host = eng.forward(pos["planes112"].pin_memory(), legal_mask=pos["legal1858"], policy=False, wdl=False, host=True,
                       policy_softmax=True, moves=True, temperature=1.0, uniforms=u)
    dev = eng.forward(planes, legal_mask=bits, policy_softmax=True, policy_dtype=torch.float16, moves=True,
                      temperature=1.0, uniforms=u.cuda())
    assert set(host) == {"move"} and torch.equal(host["move"], dev["move"].cpu())
    with pytest.raises(Exception):
        eng.forward(planes, moves=True, temperature=-1.0)


def test_legal_moves_generated_on_device_match_the_host_generator():
    """Legal-move bitsets generated on the GPU from the packed records equal, bit for bit, the host generator's
    (itself pinned by perft counts and the oracle) on 12 000 seeded playout positions up to 300 plies deep
    (castling, en passant from the history planes, promotions, checks and pins all occur), and a forward pass
    masking with them is bit-identical to one given the host bitsets."""
    from chessrl_b200 import Engine, positions
    cfg = bt4spec.SpecConfig.baseline(1, 256, 512, 8, smolgen=False)
    eng = Engine(engine_cfg(cfg))
    eng.load_state_dict(bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=71))
    seen_ep = seen_castle = seen_promo = 0
    for seed, plies in ((11, 300), (12, 120), (13, 40)):
        n = 4000
        pos = positions.playout_positions(n, seed=seed, max_plies=plies, fens=True)
        packed = positions.pack_planes104(pos["planes112"])
        got = eng.legal_masks(packed.cuda()).cpu()
        want = pos["legal1858"]
        bad = (got != want).any(dim=1).nonzero().flatten().tolist()
        assert not bad, (seed, bad[:5], [pos["fens"][i] for i in bad[:5]])
        bits = np.unpackbits(want.numpy(), axis=1, bitorder="little")[:, :1858]
        seen_promo += int(bits[:, 1792:].any(axis=1).sum())
        seen_ep += sum(1 for f in pos["fens"] if f.split()[3] != "-")
        seen_castle += int((bits[:, vocab.policy_index.index("e1g1")] | bits[:, vocab.policy_index.index("e1c1")]).sum())
    assert seen_ep > 0 and seen_castle > 0 and seen_promo > 0
    pos = positions.playout_positions(200, seed=14, max_plies=150)
    packed = positions.pack_planes104(pos["planes112"]).cuda()
    a = eng.forward(packed, layout="packed104", legal_mask=pos["legal1858"].cuda(), policy_softmax=True)["policy"]
    b = eng.forward(packed, layout="packed104", legal_mask="records", policy_softmax=True)["policy"]
    assert torch.equal(a, b)
    with pytest.raises(Exception):
        eng.forward(pos["planes112"].cuda(), legal_mask="records")      # needs the packed layout


def test_policy_server_end_to_end_equals_direct_engine_call():
    """The socket server (reference wire protocol) in front of a real engine: the arrays a client receives are the
    engine's own rows for the same records - masked with GPU-generated legal moves, soft-maxed, scattered into the
    1929 vocabulary with Black rows mirrored - and each row is a distribution over legal moves."""
    from chessrl_b200 import Engine, positions, server
    from test_server_cpu import SAN_A, UCI_B
    cfg = bt4spec.SpecConfig.baseline(2, 256, 512, 8, smolgen=True)
    eng = Engine(engine_cfg(cfg))
    eng.load_state_dict(bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=81))
    srv = server.PolicyServer(eng, port=0, linger_ms=1.0).start()
    try:
        req = [(SAN_A[:8], SAN_A[8:30]), (UCI_B[:9], UCI_B[9:])]
        ans = server.query(srv.address, req)
    finally:
        srv.close()
    assert len(ans) == 2
    for (pre, post), rows in zip(req, ans):
        g = positions.game_records(pre + post, first_ply=len(pre), count=len(post), legal=True, rule50_plane=False)
        direct = eng.forward(g["packed"].cuda(), layout="packed104", legal_mask=g["legal1858"].cuda(), policy_softmax=True,
                             policy_dtype=torch.float16, rl_vocab=True, black_rows=g["black"].cuda())["policy"].cpu().numpy()
        np.testing.assert_array_equal(rows, direct)
        np.testing.assert_allclose(rows.astype(np.float32).sum(-1), 1.0, atol=2e-3)
        legal = np.unpackbits(g["legal1858"].numpy(), axis=1, bitorder="little")[:, :1858].astype(bool)
        assert ((rows > 0).sum(-1) <= legal.sum(-1)).all()


def test_value_driven_move_selection_matches_oracle():
    """calculate_move_values / get_best_move_value of the 19-plane module (value.py:319-400): the mover's expected
    score of every successor equals the FP32 oracle's within the WDL tolerance, T = 0 picks its arg-max, and a
    seeded draw follows softmax(values / T)."""
    from chessrl_b200 import BT4Planes19, positions
    from oracle import chesspos
    spec_cfg = bt4spec.SpecConfig.reference_value(2, 128, 192, 4)
    spec = bt4spec.BT4Spec(spec_cfg)
    sd = bt4spec.seeded_state_dict(spec, seed=91)
    spec.load_state_dict(sd)
    spec.eval()
    model = BT4Planes19(2, 128, 192, 4)
    model.load_state_dict(sd)
    for fen in ("r3k2r/p1ppqpb1/bn2pnp1/3PN3/1p2P3/2N2Q1p/PPPBBPPP/R3K2R w KQkq - 0 1",
                "rnbqkbnr/ppp1pppp/8/8/3pP3/8/PPPP1PPP/RNBQKBNR b KQkq e3 0 2"):
        ucis, values = model.calculate_move_values(fen)
        pos = chesspos.Position(fen)
        planes = []
        for u in ucis:
            (m,) = [x for x in pos.legal_moves() if chesspos.uci(x) == u]
            c = pos.copy()
            c.push(m)
            planes.append(torch.from_numpy(chesspos.planes19(c)))
        with torch.no_grad():
            probs = torch.softmax(spec.forward_all(torch.stack(planes).view(len(ucis), 64, 19))["wdl"], -1)
        want = 0.5 * probs[:, 1] + (probs[:, 2] if fen.split()[1] == "w" else probs[:, 0])
        assert (values.cpu() - want).abs().max() <= WDL_TOL
        assert model.get_best_move_value(fen, T=0) == ucis[int(values.argmax())]
        move, p = model.get_best_move_value(fen, T=0.5, return_probs=True,
                                            generator=torch.Generator(device="cuda").manual_seed(3))
        assert move in ucis and abs(float(p.sum()) - 1.0) < 1e-5
        np.testing.assert_allclose(p, torch.softmax(values / 0.5, 0).cpu().numpy(), atol=1e-6)
        one = model.get_position_value(fen).cpu()
        assert one.shape == (3,) and abs(float(one.sum()) - 1.0) < 1e-4
    with pytest.raises(ValueError):
        model.get_best_move_value("1n1Rkb1r/p4ppp/4q3/4p1B1/4P3/8/PPP2PPP/2K5 b k - 1 17")


@pytest.mark.parametrize("gain", [8.0, 32.0])
def test_large_attention_scores_stay_finite_and_bounded(gain):
    """The fast attention kernels accumulate Q K^T in f16 and run the softmax on packed f16. With the query / key
    projections scaled up (raw scores in the tens to hundreds instead of O(1), as a trained network may have)
    nothing may overflow to inf / NaN, and the fp32-score kernel (CRL_PREC_ATTN_F32) must stay inside the FP16
    tolerance; the fast kernel's own error is printed and bounded at the looser figure it shows here."""
    from chessrl_b200 import Engine, EngineConfig
    import chessrl_b200 as crl
    cfg = bt4spec.SpecConfig.baseline(2, 256, 512, 8, smolgen=True)
    spec = bt4spec.BT4Spec(cfg)
    sd = bt4spec.seeded_state_dict(spec, seed=61)
    for l in range(2):
        for name in ("query_proj", "key_proj"):
            sd[f"layers.{l}.attention.{name}.weight"] = sd[f"layers.{l}.attention.{name}.weight"] * gain
    tokens = random_tokens(6, cfg.planes, seed=62)
    ref = oracle_out(cfg, sd, tokens)
    x = tokens.view(6, 8, 8, -1).cuda()
    errs = {}
    for label, prec in (("fast", 0), ("fp32 scores", crl.PREC_ATTN_F32)):
        eng = Engine(EngineConfig(dtype=0, precision=prec, **cfg.to_dict()))
        eng.load_state_dict(sd)
        out = eng.forward(x, wdl_softmax=True)
        torch.cuda.synchronize()
        pol, wdl = out["policy"].float().cpu(), out["wdl"].cpu()
        assert torch.isfinite(pol).all() and torch.isfinite(wdl).all(), label
        errs[label] = ((pol - ref["policy"]).abs().max().item(), (wdl - torch.softmax(ref["wdl"], -1)).abs().max().item())
        eng.close()
    print(f"Q/K weights x{gain}: policy / wdl max-abs error fast {errs['fast']}, fp32 scores {errs['fp32 scores']}")
    assert errs["fp32 scores"][0] <= POLICY_TOL and errs["fp32 scores"][1] <= WDL_TOL
    assert errs["fast"][0] <= 5 * POLICY_TOL and errs["fast"][1] <= 5 * WDL_TOL


FENS = ["r3k2r/p1ppqpb1/bn2pnp1/3PN3/1p2P3/2N2Q1p/PPPBBPPP/R3K2R w KQkq - 0 1",
        "rnbqkbnr/ppp1pppp/8/8/3pP3/8/PPPP1PPP/RNBQKBNR b KQkq e3 0 2",
        "8/P7/8/8/8/8/k6p/4K3 w - - 0 1", "8/P7/8/8/8/8/k6p/4K3 b - - 0 1"]


def _check_policy_move(model, logits_of, fen, planes, bits, mirrored):
    """get_move_from_fen_no_thinking against the oracle's masked logits of the same input (model_bis.py:373-392)."""
    from chessrl_b200 import positions
    ref = logits_of(planes)                                                     # [1, 1929] fp32 oracle logits
    legal = torch.from_numpy(np.unpackbits(bits.numpy(), axis=1, bitorder="little")[:, :1929].astype(bool))
    masked = ref + (1 - legal.float()) * -999
    unview = (lambda m: positions.mirror_uci(m)) if mirrored else (lambda m: m)
    legal_moves = {unview(vocab.policy_index[i]) for i in torch.nonzero(legal[0]).flatten().tolist()}
    # T = 0: the arg-max of the masked logits (a near-tie within the FP16 tolerance may resolve either way)
    move = model.get_move_from_fen_no_thinking(fen, T=0)
    best = masked[0].argmax().item()
    if move != unview(vocab.policy_index[best]):
        other = [i for i in range(1929) if unview(vocab.policy_index[i]) == move]
        assert other and masked[0, best] - masked[0, other[0]] <= 2 * POLICY_TOL
    assert move in legal_moves
    # T > 0: distribution = softmax(masked / T), the draw lands on a legal move and is reproducible
    for T in (0.5, 1.0):
        g = torch.Generator().manual_seed(11)
        m1, probs = model.get_move_from_fen_no_thinking(fen, T=T, return_probs=True, generator=g)
        m2 = model.get_move_from_fen_no_thinking(fen, T=T, generator=torch.Generator().manual_seed(11))
        assert m1 == m2 and m1 in legal_moves
        want = torch.softmax(masked / T, -1)
        assert probs.shape == (1, 1929) and (probs.cpu() - want).abs().max() <= 1e-2
        assert float(probs.cpu()[~legal].sum()) <= 1e-6
        u = torch.rand(1, generator=torch.Generator().manual_seed(11)).numpy()
        idx, margin = vocab.choose_moves(probs.cpu().numpy(), True, 1.0, u)
        assert m1 == unview(vocab.policy_index[int(idx[0])]) or margin[0] < 1e-3
    move, onehot = model.get_move_from_fen_no_thinking(fen, T=0, return_probs=True)
    assert float(onehot.sum()) == 1.0 and unview(vocab.policy_index[int(onehot.argmax())]) == move
    # force_legal=False: the raw arg-max, legal or not
    raw = model.get_move_from_fen_no_thinking(fen, T=0, force_legal=False)
    raw_best = ref[0].argmax().item()
    assert raw == unview(vocab.policy_index[raw_best]) or ref[0, raw_best] - ref[0].topk(2).values[1] <= 2 * POLICY_TOL


def test_get_move_from_fen_no_thinking_on_the_three_modules():
    """The board-only move choice every metrics script of the reference calls (model_bis.py:358-398,
    new_paradigm/value.py:214-243), on the 19-plane BT4, the decoder GPT and the 112-plane BT4: legal mask with
    knight promotions folded, -999 push-down, arg-max / temperature draw, UCI string out."""
    from chessrl_b200 import BT4, BT4Planes19, GPT, GPTConfig, positions
    from oracle import gptspec
    # 19-plane BT4 (value.py)
    c19 = bt4spec.SpecConfig.reference_value(2, 128, 192, 4)
    s19 = bt4spec.BT4Spec(c19)
    sd = bt4spec.seeded_state_dict(s19, seed=31)
    s19.load_state_dict(sd)
    s19.eval()
    m19 = BT4Planes19(2, 128, 192, 4)
    m19.load_state_dict(sd)
    # decoder GPT (model_bis.py)
    gcfg = gptspec.GPTConfig(256, 1929, 2, 2, 128)
    gs = gptspec.GPTSpec(gcfg)
    from test_oracle_golden import gpt_golden_state_dict
    gsd = gpt_golden_state_dict(gs, 32)
    gs.load_state_dict(gsd)
    gs.eval()
    gpt = GPT(GPTConfig(256, 1929, 2, 2, 128))
    gpt.load_state_dict(gsd)
    # 112-plane BT4 (value_q.py)
    c112 = bt4spec.SpecConfig.reference_value_q(2, 128, 192, 4)
    s112 = bt4spec.BT4Spec(c112)
    sd112 = bt4spec.seeded_state_dict(s112, seed=33)
    s112.load_state_dict(sd112)
    s112.eval()
    m112 = BT4(2, 128, 192, 4)
    m112.load_state_dict(sd112)
    for fen in FENS:
        p19 = torch.from_numpy(positions.fen_to_tensor(fen))[None]
        bits = torch.from_numpy(positions.legal_mask_1929(fen))[None]
        with torch.no_grad():
            _check_policy_move(m19, lambda x: s19.forward_all(x.view(1, 64, 19))["policy"], fen, p19, bits, False)
            _check_policy_move(gpt, lambda x: gs.board_logits(x), fen, p19, bits, False)
            black = fen.split()[1] == "b"
            view_bits = torch.from_numpy(positions.legal_mask_1929(positions.mirror_fen(fen) if black else fen))[None]
            p112 = torch.from_numpy(positions.fen_to_planes112(fen)).float()[None]
            _check_policy_move(m112, lambda x: s112.forward_all(x.view(1, 64, 112))["policy"], fen, p112, view_bits, black)
    with pytest.raises(ValueError):
        m19.get_move_from_fen_no_thinking("1n1Rkb1r/p4ppp/4q3/4p1B1/4P3/8/PPP2PPP/2K5 b k - 1 17")   # checkmate


def test_q_value_entry_points_and_many_position_scoring():
    """value_q.py:244-347 on the 112-plane module: tanh Q per FEN (shape [B, 1], scalar for one), successors scored
    as -Q for White to move / +Q for Black, and the many-position entry = the per-position calls, one engine call."""
    from chessrl_b200 import BT4, BT4Planes19, positions
    c112 = bt4spec.SpecConfig.reference_value_q(2, 128, 192, 4)
    s112 = bt4spec.BT4Spec(c112)
    sd = bt4spec.seeded_state_dict(s112, seed=41)
    s112.load_state_dict(sd)
    s112.eval()
    m = BT4(2, 128, 192, 4)
    m.load_state_dict(sd)
    x = torch.from_numpy(np.stack([positions.fen_to_planes112(f) for f in FENS])).float()
    with torch.no_grad():
        want = s112.forward_all(x.view(len(FENS), 64, 112))["q"]
    got = m.get_batch_position_values(FENS)
    assert got.shape == (len(FENS), 1) and (got.cpu() - want).abs().max() <= WDL_TOL
    one = m.get_position_value(FENS[1])
    assert one.dim() == 0 and abs(float(one) - float(want[1])) <= WDL_TOL
    assert m.get_batch_position_values([]).shape == (0, 1)
    for fen in FENS[:2]:
        ucis, values = m.calculate_move_values(fen)
        _, succ, _ = positions.successors(fen, planes19=False)
        sx = torch.from_numpy(np.stack([positions.fen_to_planes112(f) for f in succ])).float()
        with torch.no_grad():
            q = s112.forward_all(sx.view(len(succ), 64, 112))["q"].view(-1)
        sign = -1.0 if fen.split()[1] == "w" else 1.0
        assert (values.cpu() - sign * q).abs().max() <= WDL_TOL
        assert m.get_best_move_value(fen, T=0) == ucis[int(values.argmax())]
    many = m.calculate_move_values_many(FENS)
    assert len(many) == len(FENS)
    for fen, (ucis, values) in zip(FENS, many):
        u1, v1 = m.calculate_move_values(fen)
        assert ucis == u1 and (values - v1).abs().max() <= 1e-3
    eng = m.engine()
    before = eng.last_launch_count()
    m.calculate_move_values_many(FENS)
    assert eng.last_launch_count() == before                 # one engine call, whatever the number of positions
    # the 19-plane module shares the machinery (value.py:319-354)
    c19 = bt4spec.SpecConfig.reference_value(2, 128, 192, 4)
    s19 = bt4spec.BT4Spec(c19)
    sd19 = bt4spec.seeded_state_dict(s19, seed=42)
    m19 = BT4Planes19(2, 128, 192, 4)
    m19.load_state_dict(sd19)
    many19 = m19.calculate_move_values_many(FENS[:3])
    for fen, (ucis, values) in zip(FENS[:3], many19):
        u1, v1 = m19.calculate_move_values(fen)
        assert ucis == u1 and (values - v1).abs().max() <= 1e-3
    assert m19.calculate_move_values_many(["1n1Rkb1r/p4ppp/4q3/4p1B1/4P3/8/PPP2PPP/2K5 b k - 1 17"])[0][0] == []


@pytest.mark.parametrize("dtype", [0, 1])
def test_gemm_fused_layernorm_equals_separate_passes(dtype):
    """With crl_config.fuse_layernorm on, large passes of post-LN networks normalise inside the ff1 / QKV GEMM
    kernels. The fused warps use the arithmetic of the stand-alone LayerNorm kernel, so switching the fusion on
    must not change a single bit."""
    from chessrl_b200 import Engine, EngineConfig, positions
    import chessrl_b200 as crl
    cfg = bt4spec.SpecConfig.baseline(3, 256, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=13)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    b = 4 * sms + 37                                        # 64 b rows: more than two 256-row blocks per CTA pair, ragged
    pos = positions.playout_positions(b, seed=21)
    planes, bits = pos["planes112"].cuda(), pos["legal1858"].cuda()
    outs = []
    for fuse in (crl.FUSE_LN_ON, crl.FUSE_LN_OFF):
        eng = Engine(EngineConfig(dtype=dtype, fuse_layernorm=fuse, **cfg.to_dict()))
        eng.load_state_dict(sd)
        if dtype == crl.DTYPE_F8E4M3:
            eng.calibrate(planes[:256])
        out = eng.forward(planes, legal_mask=bits)
        torch.cuda.synchronize()
        rc, st = eng.last_status()
        assert rc == 0 and st == 0
        outs.append((out["policy"].cpu(), out["wdl"].cpu(), eng.last_launch_count()))
        eng.close()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert outs[0][2] == outs[1][2] - 2 * 3 + 1             # two LayerNorm launches fewer per block, the last block keeps its second
    if dtype == 0:
        ref = oracle_out(cfg, sd, pos["planes112"].float().view(b, 64, 112)[:64])
        legal = torch.from_numpy(np.unpackbits(pos["legal1858"].numpy()[:64], axis=1, bitorder="little")[:, :1858].astype(bool))
        assert (outs[0][0][:64] - bt4spec.apply_policy_mask(ref["policy"], legal_bits=legal))[legal].abs().max() <= POLICY_TOL


@pytest.mark.parametrize("dtype,d", [(0, 512), (1, 512), (1, 256), (2, 512)])
def test_layernorm_inside_the_producing_gemm_matches_separate_passes(dtype, d):
    """crl_config.fuse_layernorm = CRL_FUSE_LN_OUT: the out-projection and ff2 kernels of large post-LN passes
    normalise their own output rows (d = 512: two column tiles per row block, so two CTA pairs exchange row sums).
    The row statistics are summed in another order than the stand-alone kernel's, so the results agree within f16
    rounding rather than bit for bit; two fused runs are identical, and both LayerNorm launches of every block go."""
    from chessrl_b200 import Engine, EngineConfig, positions
    import chessrl_b200 as crl
    cfg = bt4spec.SpecConfig.baseline(3, d, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=17)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    b = 4 * sms + 37
    pos = positions.playout_positions(b, seed=23)
    planes, bits = pos["planes112"].cuda(), pos["legal1858"].cuda()
    outs = []
    for fuse in (crl.FUSE_LN_OUT, crl.FUSE_LN_OUT, crl.FUSE_LN_OFF):
        eng = Engine(EngineConfig(dtype=dtype, fuse_layernorm=fuse, **cfg.to_dict()))
        eng.load_state_dict(sd)
        if dtype == crl.DTYPE_F8E4M3:
            eng.calibrate(planes[:256])
        out = eng.forward(planes, legal_mask=bits)
        torch.cuda.synchronize()
        rc, st = eng.last_status()
        assert rc == 0 and st == 0
        outs.append((out["policy"].cpu(), out["wdl"].cpu(), eng.last_launch_count()))
        eng.close()
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert outs[0][2] == outs[2][2] - 2 * 3
    if d == 512 and dtype != 2:      # large enough for the library to choose this route by itself (FP16 / FP8 only)
        eng = Engine(EngineConfig(dtype=dtype, fuse_layernorm=crl.FUSE_LN_AUTO, **cfg.to_dict()))
        eng.load_state_dict(sd)
        if dtype == crl.DTYPE_F8E4M3:
            eng.calibrate(planes[:256])
        auto = eng.forward(planes, legal_mask=bits)
        torch.cuda.synchronize()
        assert torch.equal(auto["policy"].cpu(), outs[0][0]) and eng.last_launch_count() == outs[0][2]
        eng.close()
    tol = 2e-3 if dtype == 0 else 2e-2           # FP8 / INT8: a flipped f16 rounding can move an 8-bit rounding downstream
    assert (outs[0][0] - outs[2][0]).abs().max() <= tol and (outs[0][1] - outs[2][1]).abs().max() <= tol
    if dtype == 0:
        ref = oracle_out(cfg, sd, pos["planes112"].float().view(b, 64, 112)[:64])
        legal = torch.from_numpy(np.unpackbits(pos["legal1858"].numpy()[:64], axis=1, bitorder="little")[:, :1858].astype(bool))
        assert (outs[0][0][:64] - bt4spec.apply_policy_mask(ref["policy"], legal_bits=legal))[legal].abs().max() <= POLICY_TOL


def test_determinism_and_output_guards():
    """Two runs give identical bits, and nothing is written outside the rows and columns the call owns:
    outputs are carved out of larger buffers whose padding keeps its canary value."""
    import ctypes
    from chessrl_b200 import Engine, _lib as L, positions
    cfg = bt4spec.SpecConfig.baseline(2, 256, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=51)
    eng = Engine(engine_cfg(cfg, chunk=8))
    eng.load_state_dict(sd)
    b = 19                                                   # three chunks, the last one ragged
    pos = positions.playout_positions(b, seed=3)
    planes, bits = pos["planes112"].cuda(), pos["legal1858"].cuda()
    stride = 1858 + 6
    canary = 12345.0

    def run():
        policy = torch.full((b + 2, stride), canary, device="cuda")
        wdl = torch.full((b + 2, 3), canary, device="cuda")
        io = L.IO()
        io.planes, io.layout, io.batch = planes.data_ptr(), L.LAYOUT_NHWC_F16, b
        io.legal_mask, io.mask_mode, io.mask_stride = bits.data_ptr(), L.MASK_BITS, bits.shape[1]
        io.policy_out, io.policy_dtype, io.policy_softmax, io.policy_stride = policy[1:].data_ptr(), L.OUT_F32, 1, stride
        io.wdl_out, io.wdl_softmax = wdl[1:].data_ptr(), 1
        ws = eng.workspace(b)
        io.workspace, io.workspace_bytes = ws.data_ptr(), ws.numel()
        io.stream = torch.cuda.current_stream().cuda_stream
        assert eng.lib.crl_forward(eng._h, ctypes.byref(io)) == 0
        torch.cuda.synchronize()
        return policy.cpu(), wdl.cpu()

    p1, w1 = run()
    p2, w2 = run()
    assert torch.equal(p1, p2) and torch.equal(w1, w2)
    assert (p1[0] == canary).all() and (p1[-1] == canary).all() and (p1[1:-1, 1858:] == canary).all()
    assert (w1[0] == canary).all() and (w1[-1] == canary).all()
    assert torch.isfinite(p1[1:-1, :1858]).all() and torch.allclose(p1[1:-1, :1858].sum(-1), torch.ones(b), atol=1e-4)


def test_cuda_graph_of_a_pass_with_the_layernorm_inside_the_gemms():
    """A large pass (LayerNorms inside the out-projection / ff2 kernels: a memset of the exchange buffer plus a
    kernel whose CTAs wait for one another) captured into a CUDA graph replays to the bits of the eager call."""
    from chessrl_b200 import Engine, EngineConfig, positions
    import chessrl_b200 as crl
    cfg = bt4spec.SpecConfig.baseline(2, 512, 512, 8, smolgen=True)
    sd = bt4spec.seeded_state_dict(bt4spec.BT4Spec(cfg), seed=29)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    b = 4 * sms + 37
    pos = positions.playout_positions(b, seed=31)
    planes, bits = pos["planes112"].cuda(), pos["legal1858"].cuda()
    eng = Engine(EngineConfig(dtype=crl.DTYPE_F8E4M3, **cfg.to_dict()))
    eng.load_state_dict(sd)
    eng.calibrate(planes[:256])

    def call():
        return eng.forward(planes, legal_mask=bits)

    eager = call()
    torch.cuda.synchronize()
    want = {k: v.clone() for k, v in eager.items()}
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = call()
    for _ in range(3):
        for v in out.values():
            v.zero_()
        g.replay()
        torch.cuda.synchronize()
        rc, st = eng.last_status()
        assert rc == 0 and st == 0
        for k in want:
            assert torch.equal(out[k], want[k]), k
    eng.close()
