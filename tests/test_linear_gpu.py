"""The tcgen05 GEMM through crl_linear against torch fp32 matmul of the same (rounded) operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def call(lib, kind, a, w, out_dtype, bias=None, res=None, alpha=1.0, act=0):
    m, k = a.shape
    n = w.shape[0]
    tdt = {0: torch.float16, 1: torch.float32, 2: torch.uint8}[out_dtype]
    c = torch.full((m, n), 7.0 if out_dtype != 2 else 0, device="cuda").to(tdt)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = lib.crl_linear(kind, a.data_ptr(), k, w.data_ptr(), k, c.data_ptr(), n, out_dtype, m, n, k,
                        bias.data_ptr() if bias is not None else None, res.data_ptr() if res is not None else None,
                        n, alpha, act, status.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0 and int(status[0]) == 0
    return c


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (64, 32, 1024), (200, 1929, 4096), (320, 256, 112), (1, 128, 8192),
                                   (4096, 3072, 1024), (777, 1536, 1024), (130, 8200, 256), (19001, 520, 200), (9473, 1929, 512)])
def test_f16_gemm(lib, m, n, k):
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda").half()
    w = (torch.randn(n, k, device="cuda") * 0.05).half()
    ref = a.float() @ w.float().t()
    c = call(lib, 0, a, w, 1)
    assert (c - ref).abs().max() <= 1e-3 * max(1.0, ref.abs().max().item())
    c16 = call(lib, 0, a, w, 0)
    assert (c16.float() - ref).abs().max() <= 2e-3 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_epilogue_bias_activation_residual(lib, act):
    torch.manual_seed(act)
    m, n, k = 300, 520, 256
    a = torch.randn(m, k, device="cuda").half()
    w = (torch.randn(n, k, device="cuda") * 0.05).half()
    bias = torch.randn(n, device="cuda")
    res = torch.randn(m, n, device="cuda").half()
    x = 0.5 * (a.float() @ w.float().t()) + bias
    x = [lambda t: t, torch.nn.functional.gelu, torch.nn.functional.mish, torch.relu][act](x) + res.float()
    c = call(lib, 0, a, w, 1, bias=bias, res=res, alpha=0.5, act=act)
    assert (c - x).abs().max() <= 2e-3


def test_e4m3_gemm_exact_products(lib):
    torch.manual_seed(1)
    m, n, k = 512, 768, 1024
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    w = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    ref = a.float() @ w.float().t()
    c = call(lib, 1, a, w, 1)
    assert (c - ref).abs().max() <= 1e-3 * ref.abs().max().item()


def test_int8_gemm_is_integer_exact(lib):
    torch.manual_seed(2)
    m, n, k = 256, 384, 512
    a = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8)
    ref = a.double() @ w.double().t()
    c = call(lib, 2, a, w, 1)
    # products sum to < 2^24 in magnitude here, so the f32 conversion of the int32 accumulator is exact
    assert ref.abs().max() < 2 ** 24 and torch.equal(c.double(), ref)
