"""Generates tests/golden/*.npz by running the UNMODIFIED reference modules on CPU.

Run once in a container that has the reference checkout:
    python tests/golden/make_golden.py /path/to/reference
The fixtures are committed; tests and the GPU box only read the .npz files.

Import shim (no reference file is edited): the reference imports `chess` and `zstandard` at module
top but its forward passes do not use them, so empty stand-in modules are registered; constructors
hard-code `.to("cuda")` (new_paradigm/value.py:35-41,82), which is mapped to the CPU while they run.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import bt4spec  # noqa: E402


def import_reference(ref_root):
    for name in ("chess", "chess.pgn", "chess.engine", "zstandard"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["chess"].pgn = sys.modules["chess.pgn"]
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "new_paradigm"))
    cwd = os.getcwd()
    os.chdir(ref_root)
    tensor_to, module_to = torch.Tensor.to, torch.nn.Module.to

    def cpu_args(args):
        return tuple("cpu" if isinstance(a, str) and a.startswith("cuda") else a for a in args)

    torch.Tensor.to = lambda self, *a, **k: tensor_to(self, *cpu_args(a), **k)
    torch.nn.Module.to = lambda self, *a, **k: module_to(self, *cpu_args(a), **k)
    import io
    import contextlib
    with contextlib.redirect_stdout(io.StringIO()):
        from new_paradigm import value_q, value
    os.chdir(cwd)
    return value_q, value


def synthetic_tokens(batch, planes, seed):
    """Plane values with the distribution of real inputs: sparse 0/1 piece planes, a few constant
    planes, one fractional plane."""
    g = torch.Generator().manual_seed(seed)
    x = (torch.rand(batch, 64, planes, generator=g) < 0.08).float()
    x[:, :, planes - 1] = 1.0
    x[:, :, planes - 3] = torch.rand(batch, 1, generator=g).expand(batch, 64) * 0.5
    return x


def run_case(name, ref_cls, spec_cfg, dims, batch, seed, head_q):
    model = ref_cls(*dims)
    spec = bt4spec.BT4Spec(spec_cfg)
    assert sorted(model.state_dict().keys()) == sorted(spec.state_dict().keys()), "state_dict keys differ"
    sd = bt4spec.seeded_state_dict(spec, seed=seed)
    # non-trivial LayerNorm / gating parameters so that those code paths are pinned as well
    g = torch.Generator().manual_seed(seed + 1)
    for k in sorted(sd):
        if k.endswith("ma_gating.a"):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.1
        elif "norm" in k and k.endswith("weight"):
            sd[k] = 1.0 + torch.randn(sd[k].shape, generator=g) * 0.1
        elif "norm" in k and k.endswith("bias"):
            sd[k] = torch.randn(sd[k].shape, generator=g) * 0.1
    model.load_state_dict(sd)
    model.eval()
    tokens = synthetic_tokens(batch, spec_cfg.planes, seed + 2)
    x5 = tokens.view(batch, 1, 8, 8, spec_cfg.planes)
    with torch.no_grad():
        policy = model([x5, None]).view(batch, -1)
        # value heads: same body as the reference's get_batch_position_values (value.py:296-313)
        h = model.ma_gating(model.layernorm1(torch.nn.GELU()(model.linear1(tokens))))
        pos_enc = model.positional(h)
        for layer in model.layers:
            h = layer(h, pos_enc)
        wdl = model.value_head(h)
        out = dict(policy=policy.numpy(), wdl=wdl.numpy(), trunk=h.numpy())
        if head_q:
            out["q"] = model.value_head_q(h).numpy()
    out["tokens_u8"] = (tokens * 255).round().to(torch.uint8).numpy()   # exact for 0/1; see below
    out["tokens"] = tokens.numpy().astype(np.float16)                   # fractional plane in f16
    out["dims"] = np.array(dims)
    out["seed"] = np.array(seed)
    out["weight_abs_sum"] = np.array(sum(float(v.abs().sum()) for v in sd.values()))
    # the fixture's inputs are the f16-rounded tokens, so recompute the outputs from exactly those
    tokens16 = torch.from_numpy(out["tokens"]).float()
    with torch.no_grad():
        out["policy"] = model([tokens16.view(batch, 1, 8, 8, -1), None]).view(batch, -1).numpy()
        h = model.ma_gating(model.layernorm1(torch.nn.GELU()(model.linear1(tokens16))))
        for layer in model.layers:
            h = layer(h, pos_enc)
        out["trunk"] = h.numpy().astype(np.float32)
        out["wdl"] = model.value_head(h).numpy()
        if head_q:
            out["q"] = model.value_head_q(h).numpy()
    del out["tokens_u8"]
    # chain of trust, checked at generation time too: the oracle must agree bit for bit
    spec.load_state_dict(sd)
    spec.eval()
    with torch.no_grad():
        mine = spec.forward_all(tokens16)
    assert torch.equal(mine["policy"], torch.from_numpy(out["policy"])), "oracle policy differs"
    assert torch.equal(mine["wdl"], torch.from_numpy(out["wdl"])), "oracle wdl differs"
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, "ok", {k: getattr(v, "shape", None) for k, v in out.items()})


def run_gpt_case(name, ref_root, seed):
    """Board-only path of the reference GPT (body of get_move_from_fen_no_thinking, model_bis.py:358-370)."""
    import io
    import contextlib
    from oracle import gptspec
    cwd = os.getcwd()
    os.chdir(ref_root)
    with contextlib.redirect_stdout(io.StringIO()):
        import model_bis
        cfg = model_bis.GPTConfig(block_size=256, vocab_size=1929, n_layer=2, n_head=2, n_embd=128)
        model = model_bis.GPT(cfg)
    os.chdir(cwd)
    spec = gptspec.GPTSpec(gptspec.GPTConfig(256, 1929, 2, 2, 128))
    assert sorted(model.state_dict().keys()) == sorted(spec.state_dict().keys()), "GPT state_dict keys differ"
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for k in sorted(spec.state_dict().keys()):
        v = spec.state_dict()[k]
        if k == "pe":
            sd[k] = v.clone()
        elif k.endswith("ln_1.weight") or k.endswith("ln_2.weight") or k.endswith("ln_f.weight") or "layernorm1.weight" in k:
            sd[k] = 1.0 + torch.randn(v.shape, generator=g) * 0.1
        elif k.endswith("ma_gating.b"):
            sd[k] = torch.ones(v.shape)
        elif k.endswith("ma_gating.a"):
            sd[k] = torch.randn(v.shape, generator=g) * 0.1
        else:
            sd[k] = torch.randn(v.shape, generator=g) * (0.1 if k.endswith(".bias") else 0.02)
    sd["transformer.wte.weight"] = sd["lm_head.weight"]
    model.load_state_dict(sd)
    model.eval()
    batch = 3
    board = (torch.rand(batch, 8, 8, 19, generator=g) < 0.1).float()
    board[..., 18] = (torch.rand(batch, 1, 1, generator=g) * 0.5).half().float().expand(batch, 8, 8)
    with torch.no_grad():
        x = model.FenEncoder(board) + model.pe[torch.arange(0, 64)]
        for block in model.transformer.h:
            x = block(x)
        x = model.transformer.ln_f(x)
        logits = model.lm_head(x[:, [-1], :])[:, 0]
    spec.load_state_dict(sd)
    spec.eval()
    with torch.no_grad():
        mine = spec.board_logits(board)
    assert torch.equal(mine, logits), "GPT oracle differs from the reference"
    np.savez_compressed(os.path.join(HERE, name + ".npz"), board=board.numpy().astype(np.float16), logits=logits.numpy(),
                        seed=np.array(seed), dims=np.array([2, 2, 128]))
    print(name, "ok", tuple(logits.shape))


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference repository>")
    ref_root = sys.argv[1]
    value_q, value = import_reference(ref_root)
    torch.set_num_threads(1)   # one thread: summation order independent of the machine
    run_case("ref_value_q_L2_d64_ff96_h2", value_q.BT4, bt4spec.SpecConfig.reference_value_q(2, 64, 96, 2),
             (2, 64, 96, 2), batch=3, seed=11, head_q=True)
    run_case("ref_value_q_L2_d256_ff320_h8", value_q.BT4, bt4spec.SpecConfig.reference_value_q(2, 256, 320, 8),
             (2, 256, 320, 8), batch=2, seed=12, head_q=True)
    run_case("ref_value_L1_d64_ff64_h2", value.BT4, bt4spec.SpecConfig.reference_value(1, 64, 64, 2),
             (1, 64, 64, 2), batch=2, seed=13, head_q=False)
    run_gpt_case("ref_gpt_L2_d128_h2", ref_root, seed=14)


if __name__ == "__main__":
    main()
