"""Single-kernel and per-kernel-breakdown cases for profiling the engine.

    python -m chessrl_b200.kernel_cases gemm <kind> <M> <N> <K> <out> [act] [residual]
        three launches of one linear layer through `crl_linear` (kind: 0 f16, 1 e4m3, 2 int8 operands;
        out: 0 f16, 1 f32, 2 e4m3), timed with CUDA events over 20 more launches.
    python -m chessrl_b200.kernel_cases forward <f16|f8|i8> <positions> [chunk]
        the BT4-shaped forward pass (15 blocks, d 1024, 32 heads, d_ff 1536, smolgen): plain timing of three
        passes, then one pass with the library's per-launch CUDA events, grouped by kernel and shape.

Both need a GPU and the built library; they exist so that a profiler capture (`-k regex:<kernel>`) has a
small, repeatable program to attach to.
"""
import collections
import sys

import torch

from . import _lib
from . import synth
from ._lib import DTYPE_F16, DTYPE_F8E4M3, DTYPE_I8
from .engine import Engine, EngineConfig
from .modules import _param_shapes


def gemm_case(kind, M, N, K, out, act=0, residual=0, launches=20):
    lib = _lib.load()
    dev = "cuda"
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(0)
    if kind == 1:
        a = torch.randn(M, K, device=dev, generator=g).to(torch.float8_e4m3fn)
        w = torch.randn(N, K, device=dev, generator=g).to(torch.float8_e4m3fn)
    elif kind == 2:
        a = torch.randint(-127, 128, (M, K), device=dev, generator=g, dtype=torch.int8)
        w = torch.randint(-127, 128, (N, K), device=dev, generator=g, dtype=torch.int8)
    else:
        a = torch.randn(M, K, device=dev, generator=g).half()
        w = torch.randn(N, K, device=dev, generator=g).half()
    c = torch.empty(M, N, device=dev, dtype={0: torch.float16, 1: torch.float32, 2: torch.uint8}[out])
    b = torch.randn(N, device=dev, generator=g)
    r = torch.randn(M, N, device=dev, generator=g).half() if residual else None

    def launch():
        return lib.crl_linear(kind, a.data_ptr(), K, w.data_ptr(), K, c.data_ptr(), N, out, M, N, K, b.data_ptr(),
                              r.data_ptr() if r is not None else None, N, 0.01, act, status.data_ptr(), None)

    for _ in range(3):
        rc = launch()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        rc = launch()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / launches * 1e3
    print(f"rc {rc} status {status[0].item()}  {us:.1f} us/launch  {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
    return us


def forward_case(which, B, chunk=0):
    dtype = {"f16": DTYPE_F16, "f8": DTYPE_F8E4M3, "i8": DTYPE_I8}[which]
    cfg = EngineConfig.baseline(15, 1024, 1536, 32, smolgen=True, dtype=dtype, chunk=chunk)
    eng = Engine(cfg, 0)
    eng.load_state_dict(synth.seeded_state_dict(_param_shapes(cfg), seed=0))
    planes = synth.synthetic_planes(B, 112, seed=1).cuda()
    bits = synth.synthetic_legal_bits(B).cuda()
    if dtype == DTYPE_F8E4M3:
        eng.calibrate(planes[:2048])

    def step():
        eng.forward(planes, legal_mask=bits, policy_softmax=True, policy_dtype=torch.float16)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 3
    print(f"B={B} chunk={chunk}: {ms:.2f} ms/step, {B / ms * 1e3:.0f} pos/s")
    eng.profile(True)
    step()
    agg = collections.OrderedDict()
    for e in eng.profile_entries():
        a = agg.setdefault((e["cat"], e["m"], e["n"], e["k"], e["kind"]), [0, 0.0, 0.0, 0.0])
        a[0] += 1
        a[1] += e["ms"]
        a[2] += e["flops"]
        a[3] += e["bytes"]
    tot = sum(a[1] for a in agg.values())
    print(f"profiled total {tot:.2f} ms")
    for (cat, m, n, k, kind), a in sorted(agg.items(), key=lambda kv: -kv[1][1]):
        name = ["gemm", "attn", "ln", "policy"][cat]
        tf = a[2] / a[1] / 1e9 if a[1] else 0.0
        gb = a[3] / a[1] / 1e6 if a[1] else 0.0
        print(f"{name:6s} M={m:7d} N={n:5d} K={k:5d} kind={kind} x{a[0]:3d}  {a[1]:8.3f} ms "
              f"({a[1] / tot * 100:5.1f}%)  {tf:8.1f} TFLOP/s  {gb:8.1f} GB/s")


def main(argv):
    if len(argv) >= 6 and argv[0] == "gemm":
        nums = [int(x) for x in argv[1:]]
        gemm_case(*nums[:7])
    elif len(argv) >= 3 and argv[0] == "forward":
        forward_case(argv[1], int(argv[2]), int(argv[3]) if len(argv) > 3 else 0)
    else:
        print(__doc__)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
