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


# ---- the kernel variants that carry the benchmark pass (CTA pairs on 256 x 256 tiles, slab epilogue) ------------
def call_ex(lib, kind, a, w, out_dtype, bias=None, res=None, res_mod=0, alpha=1.0, act=0, out_scale=1.0,
            row_scale=None, col_scale=None, ldc=None, ldr=None):
    import ctypes
    from chessrl_b200 import _lib as L
    m, k = a.shape
    n = w.shape[0]
    ldc = n if ldc is None else ldc
    tdt = {0: torch.float16, 1: torch.float32, 2: torch.uint8}[out_dtype]
    c = torch.full((m + 3, ldc), 7.0 if out_dtype != 2 else 0x55, device="cuda").to(tdt)   # 3 canary rows
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    x = L.LinearArgs()
    x.kind, x.out_dtype = kind, out_dtype
    x.a, x.lda, x.w, x.ldw, x.c, x.ldc = a.data_ptr(), k, w.data_ptr(), k, c.data_ptr(), ldc
    x.m, x.n, x.k = m, n, k
    x.bias = bias.data_ptr() if bias is not None else None
    x.residual = res.data_ptr() if res is not None else None
    x.ldr = (res.shape[1] if res is not None else n) if ldr is None else ldr
    x.res_mod = res_mod
    x.alpha, x.act, x.out_scale = alpha, act, out_scale
    x.row_scale = row_scale.data_ptr() if row_scale is not None else None
    x.col_scale = col_scale.data_ptr() if col_scale is not None else None
    x.device_status = status.data_ptr()
    rc = lib.crl_linear_ex(ctypes.byref(x))
    torch.cuda.synchronize()
    assert rc == 0 and int(status[0]) == 0, (rc, int(status[0]))
    canary = c[m:]
    assert bool((canary == canary[0, 0]).all()), "rows beyond M were written"
    if ldc > n:
        assert bool((c[:m, n:] == canary[0, 0]).all()), "columns beyond N were written"
    return c[:m, :n]


def e4m3_decode(u8):
    return u8.view(torch.float8_e4m3fn).float()


def e4m3_step(x):
    """Spacing of the e4m3 grid around |x| (normal numbers: 2^(floor(log2|x|) - 3); subnormal spacing 2^-9)."""
    e = torch.floor(torch.log2(x.abs().clamp_min(2.0 ** -6)))
    return torch.exp2(e - 3)


FP8_SHAPES = [(4096, 3072, 1024), (16384, 1024, 1536), (19001, 520, 1024), (130 * 64, 8200, 256)]


@pytest.mark.parametrize("m,n,k", FP8_SHAPES)
def test_e4m3_pair_kernel_f16_out(lib, m, n, k):
    """e4m3 x e4m3 on the pair kernel (>= 74 tiles of 256 x 256), f16 output + bias, ragged M and N."""
    torch.manual_seed(n)
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    w = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    bias = torch.randn(n, device="cuda")
    alpha = 1.0 / 16
    ref = alpha * (a.float() @ w.float().t()) + bias
    c = call_ex(lib, 1, a, w, 0, bias=bias, alpha=alpha, ldc=n + 8)
    assert (c.float() - ref).abs().max() <= 2e-3 * ref.abs().max().item()


@pytest.mark.parametrize("m,n,k", FP8_SHAPES[:3])
def test_e4m3_pair_kernel_e4m3_out_with_out_scale(lib, m, n, k):
    """The QKV form: e4m3 operands, bias, e4m3 output with the next GEMM's input multiplier. The stored byte is
    the nearest e4m3 value of the scaled result: error at most half a grid step (+ fp32 accumulation noise)."""
    torch.manual_seed(k)
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    w = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    bias = torch.randn(n, device="cuda")
    alpha, out_scale = 1.0 / 32, 37.5
    ref = (alpha * (a.float() @ w.float().t()) + bias) * out_scale
    c = e4m3_decode(call_ex(lib, 1, a, w, 2, bias=bias, alpha=alpha, out_scale=out_scale, ldc=n + (16 - n % 16) % 16 + 16))
    ref = ref.clamp(-448, 448)
    assert bool(((c - ref).abs() <= 0.5 * e4m3_step(ref) + 1e-3 * ref.abs() + 1e-6).all())


def test_e4m3_pair_kernel_mish_packed_epilogue(lib):
    """The ff1 form: e4m3 operands, bias, Mish, e4m3 output (Mish on packed f16 pairs: <= 4.2e-3 relative, then
    one rounding to the e4m3 grid)."""
    torch.manual_seed(5)
    m, n, k = 8192, 1536, 1024
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    w = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    bias = torch.randn(n, device="cuda")
    alpha, out_scale = 1.0 / 32, 60.0
    ref = torch.nn.functional.mish(alpha * (a.float() @ w.float().t()) + bias) * out_scale
    c = e4m3_decode(call_ex(lib, 1, a, w, 2, bias=bias, alpha=alpha, act=2, out_scale=out_scale))
    ref = ref.clamp(-448, 448)
    tol = 0.5 * e4m3_step(ref) + 6e-3 * ref.abs() + 2e-3     # f16 arithmetic around zero: 2e-3 absolute after scaling
    assert bool(((c - ref).abs() <= tol).all())


@pytest.mark.parametrize("m,n,k,kind", [(16384, 1024, 1024, 1), (16384 + 77, 1024, 1536, 1), (16384, 1024, 1024, 0),
                                        (9000, 2056, 1024, 0)])
def test_pair_kernel_residual_by_tma(lib, m, n, k, kind):
    """The out-projection / ff2 form: residual slab fetched by TMA into the staging buffer, f16 output."""
    torch.manual_seed(m)
    if kind == 1:
        a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
        w = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    else:
        a = torch.randn(m, k, device="cuda").half()
        w = torch.randn(n, k, device="cuda").half()
    bias = torch.randn(n, device="cuda")
    res = torch.randn(m, n, device="cuda").half()
    alpha = 1.0 / 64
    ref = alpha * (a.float() @ w.float().t()) + bias + res.float()
    c = call_ex(lib, kind, a, w, 0, bias=bias, res=res, alpha=alpha)
    assert (c.float() - ref).abs().max() <= 2e-3 * ref.abs().max().item()


def test_pair_kernel_broadcast_residual_table(lib):
    """Policy-token form: GELU, then a [64, N] table added to every board (residual row = row % 64)."""
    torch.manual_seed(11)
    m, n, k = 64 * 200, 1024, 1024
    a = torch.randn(m, k, device="cuda").half()
    w = (torch.randn(n, k, device="cuda") * 0.03).half()
    bias = torch.randn(n, device="cuda")
    table = torch.randn(64, n, device="cuda").half()
    ref = torch.nn.functional.gelu(a.float() @ w.float().t() + bias) + table.float().repeat(200, 1)
    c = call_ex(lib, 0, a, w, 0, bias=bias, res=table, res_mod=64, act=1)
    assert (c.float() - ref).abs().max() <= 4e-3 * ref.abs().max().item()


@pytest.mark.parametrize("m,n,k,out", [(16384, 3072, 1024, 0), (19001, 1024, 1536, 0), (8192, 1536, 1024, 1)])
def test_int8_row_and_column_scales(lib, m, n, k, out):
    """W8A8: int32 accumulation exact, then per-token x per-channel scales, bias, f16 / f32 output (pair kernel for
    f16, single-CTA kernel for f32)."""
    torch.manual_seed(k + out)
    a = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8)
    rs = torch.rand(m, device="cuda") * 1e-3 + 1e-4
    cs = torch.rand(n, device="cuda") * 1e-2 + 1e-3
    bias = torch.randn(n, device="cuda")
    acc = (a.double() @ w.double().t())
    ref = (acc * rs.double()[:, None] * cs.double()[None, :] + bias.double()).float()
    c = call_ex(lib, 2, a, w, out, bias=bias, row_scale=rs, col_scale=cs)
    tol = 1e-3 if out == 0 else 2e-6
    assert (c.float() - ref).abs().max() <= tol * ref.abs().max().item()


def test_f16_pair_kernel_to_e4m3(lib):
    """The smolgen bias form: f16 operands, K = 256, e4m3 output with a scale."""
    torch.manual_seed(3)
    m, n, k = 32 * 300, 4096, 256
    a = torch.randn(m, k, device="cuda").half()
    w = (torch.randn(n, k, device="cuda") * 0.05).half()
    out_scale = 100.0
    ref = ((a.float() @ w.float().t()) * out_scale).clamp(-448, 448)
    c = e4m3_decode(call_ex(lib, 0, a, w, 2, out_scale=out_scale))
    assert bool(((c - ref).abs() <= 0.5 * e4m3_step(ref) + 1e-3 * ref.abs() + 1e-6).all())
