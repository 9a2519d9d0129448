"""crl_forward_static, the forward call for callers that cannot allocate device memory (a worker that
shares the GPU with a framework owning all of its memory, or a loop that cannot afford the device-wide
stall inside cudaMalloc): called through the C ABI, twice in a row, and compared with crl_forward on the
same inputs. The file name keeps this test last in collection order, and it builds its own engine, so it
passes both alone in a fresh process and after the rest of the suite."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_forward_matches_forward_twice(lib):
    from chessrl_b200 import Engine, EngineConfig, _lib as L, synth
    from chessrl_b200.modules import _param_shapes
    cfg = EngineConfig.baseline(2, 256, 512, 8, smolgen=True)
    eng = Engine(cfg, 0)
    eng.load_state_dict(synth.seeded_state_dict(_param_shapes(cfg), seed=31))
    static_bytes = 64 << 20

    def run_static(planes, bits):
        b = planes.shape[0]
        policy = torch.full((b, 1858), float("nan"), device="cuda")
        wdl = torch.full((b, 3), float("nan"), device="cuda")
        io = L.IO()
        io.planes, io.layout, io.batch = planes.data_ptr(), L.LAYOUT_NHWC_F16, b
        io.legal_mask, io.mask_mode, io.mask_stride = bits.data_ptr(), L.MASK_BITS, bits.shape[1]
        io.policy_out, io.policy_dtype, io.policy_softmax, io.policy_stride = policy.data_ptr(), L.OUT_F32, 1, 1858
        io.wdl_out, io.wdl_softmax = wdl.data_ptr(), 1
        io.stream = torch.cuda.current_stream().cuda_stream
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.crl_forward_static(eng._h, ctypes.byref(io))
        torch.cuda.synchronize()
        return rc, policy, wdl, free_before - torch.cuda.mem_get_info()[0]

    # two calls in a row with different inputs: the second must not see anything of the first
    for seed, batch in ((41, 9), (42, 5)):
        planes = synth.synthetic_planes(batch, 112, seed=seed).cuda()
        bits = synth.synthetic_legal_bits(batch, 1858, seed=seed + 100).cuda()
        assert lib.crl_workspace_bytes(eng._h, batch) <= static_bytes
        rc, policy, wdl, grew = run_static(planes, bits)
        assert rc == 0, lib.crl_error_detail(eng._h).decode()
        ref = eng.forward(planes, legal_mask=bits, policy_softmax=True)
        torch.cuda.synchronize()
        rc2, st = eng.last_status()
        assert rc2 == 0 and st == 0
        # same kernels on the same inputs: identical bits; the suite's FP16 tolerances are the formal bound
        assert (policy - ref["policy"]).abs().max().item() <= 2e-2 and (wdl - ref["wdl"]).abs().max().item() <= 1e-2
        assert torch.equal(policy, ref["policy"]) and torch.equal(wdl, ref["wdl"])
        if seed == 42:
            # second call: the device's free memory is what it was before the call (the first call may
            # still see the driver load the library's device image, which holds the static scratch)
            assert grew == 0

    # beyond the static scratch: refused with a message, nothing launched
    big = 1
    while lib.crl_workspace_bytes(eng._h, big) <= static_bytes:
        big *= 2
    planes = synth.synthetic_planes(big, 112, seed=43).cuda()
    bits = synth.synthetic_legal_bits(big, 1858, seed=44).cuda()
    rc, _, _, _ = run_static(planes, bits)
    assert rc == -7
    assert "static scratch" in lib.crl_error_detail(eng._h).decode()
