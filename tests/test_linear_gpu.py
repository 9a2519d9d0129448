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


def assert_close_elementwise(got, want, tol):
    """Every element within its own tolerance; on failure name the worst offenders (row, column, got, want)."""
    bad = ~((got - want).abs() <= tol)
    if bool(bad.any()):
        idx = torch.nonzero(bad)[:6].tolist()
        rows = sorted({i for i, _ in torch.nonzero(bad)[:20000].tolist()})
        raise AssertionError(f"{int(bad.sum())} of {bad.numel()} elements off; first: "
                             + ", ".join(f"[{i},{j}] got {float(got[i, j]):.5g} want {float(want[i, j]):.5g}" for i, j in idx)
                             + f"; rows touched (first 12): {rows[:12]} ... {len(rows)} rows")


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
    order = 1e-6 * alpha * out_scale * (a.float().abs() @ w.float().abs().t())
    assert_close_elementwise(c, ref, 0.5 * e4m3_step(ref) + 1e-3 * ref.abs() + order)


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
    assert_close_elementwise(c, ref, tol)


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
    # fp32 sums of 256 products of either sign: two summation orders differ by ~1e-6 of the sum of magnitudes, which
    # decides the rounding of results next to zero
    order = 1e-6 * (a.float().abs() @ w.float().abs().t()) * out_scale
    assert_close_elementwise(c, ref, 0.5 * e4m3_step(ref) + 1e-3 * ref.abs() + order)


@pytest.mark.parametrize("kind,out,n", [(1, 2, 1536), (1, 2, 3072), (0, 0, 1536), (1, 0, 512)])
def test_layernorm_fused_into_the_gemm(lib, kind, out, n):
    """LNA kernels: the rows of A are LayerNorm(y) computed by the GEMM kernel's own warps a row block ahead of the
    MMAs. Checked in two steps: the normalised rows it writes (f16, and e4m3 with a scale) against torch's
    layer_norm, then the product against an fp32 matmul of exactly those written rows (so the second check is as
    tight as for a plain GEMM). M is ragged and large enough for every CTA pair to own several row blocks."""
    import ctypes
    from chessrl_b200 import _lib as L
    torch.manual_seed(n + kind)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    m, k = 256 * sms + 256 * 40 + 77, 1024
    y = (torch.randn(m, k, device="cuda") * 1.3 + 0.2).half()
    gamma = (1.0 + 0.1 * torch.randn(k, device="cuda")).half()
    beta = (0.1 * torch.randn(k, device="cuda")).half()
    w = torch.randn(n, k, device="cuda")
    w = w.to(torch.float8_e4m3fn) if kind == 1 else (w * 0.05).half()
    bias = torch.randn(n, device="cuda")
    x16 = torch.zeros(m, k, device="cuda", dtype=torch.float16)
    x8 = torch.zeros(m, k, device="cuda", dtype=torch.uint8)
    s8 = 448.0 / 6.0
    c = torch.zeros(m + 2, n, device="cuda", dtype=torch.uint8 if out == 2 else torch.float16)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = L.LinearArgs()
    a.kind, a.out_dtype = kind, out
    a.a, a.lda = (x8 if kind == 1 else x16).data_ptr(), k
    a.w, a.ldw, a.c, a.ldc = w.data_ptr(), k, c.data_ptr(), n
    a.m, a.n, a.k = m, n, k
    a.bias = bias.data_ptr()
    a.alpha = 1.0 / (s8 * 8.0) if kind == 1 else 1.0
    a.out_scale = 20.0
    a.device_status = status.data_ptr()
    a.ln_y, a.ln_weight, a.ln_bias = y.data_ptr(), gamma.data_ptr(), beta.data_ptr()
    a.ln_x, a.ln_x8, a.ln_out8_scale = x16.data_ptr(), x8.data_ptr(), s8
    rc = lib.crl_linear_ex(ctypes.byref(a))
    torch.cuda.synchronize()
    assert rc == 0 and int(status[0]) == 0, (rc, int(status[0]))
    want_x = torch.nn.functional.layer_norm(y.float(), (k,), gamma.float(), beta.float(), 1e-5)
    assert (x16.float() - want_x).abs().max() <= 6e-3                       # f16 affine: a few f16 steps at |x| ~ 4
    got8 = e4m3_decode(x8)
    ref8 = (x16.float() * s8).clamp(-448, 448)
    assert_close_elementwise(got8, ref8, 0.5 * e4m3_step(ref8) + 2e-3 * ref8.abs() + 1e-6)
    a_used = got8 if kind == 1 else x16.float()
    ref = a.alpha * (a_used @ w.float().t()) + bias
    assert bool((c[m:] == 0).all()), "rows beyond M were written"
    if out == 2:
        ref = (ref * 20.0).clamp(-448, 448)
        order = 1e-6 * a.alpha * 20.0 * (a_used.abs() @ w.float().abs().t())          # summation-order slack, see above
        assert_close_elementwise(e4m3_decode(c[:m]), ref, 0.5 * e4m3_step(ref) + 1e-3 * ref.abs() + order)
    else:
        assert_close_elementwise(c[:m].float(), ref, torch.full_like(ref, 2e-3 * ref.abs().max().item()))


def test_layernorm_fusion_is_refused_where_it_cannot_run(lib):
    """Too few row blocks for the CTA pairs, or int8 operands: CRL_ERR_UNSUPPORTED, nothing launched."""
    import ctypes
    from chessrl_b200 import _lib as L
    m, n, k = 4096, 1024, 1024
    y = torch.zeros(m, k, device="cuda", dtype=torch.float16)
    g = torch.ones(k, device="cuda", dtype=torch.float16)
    x16 = torch.zeros_like(y)
    w = torch.zeros(n, k, device="cuda", dtype=torch.float16)
    c = torch.full((m, n), 3.0, device="cuda", dtype=torch.float16)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    a = L.LinearArgs()
    a.kind, a.out_dtype, a.a, a.lda, a.w, a.ldw, a.c, a.ldc = 0, 0, x16.data_ptr(), k, w.data_ptr(), k, c.data_ptr(), n
    a.m, a.n, a.k, a.alpha, a.device_status = m, n, k, 1.0, status.data_ptr()
    a.ln_y, a.ln_weight, a.ln_bias, a.ln_x = y.data_ptr(), g.data_ptr(), g.data_ptr(), x16.data_ptr()
    assert lib.crl_linear_ex(ctypes.byref(a)) == -8
    torch.cuda.synchronize()
    assert bool((c == 3.0).all())


@pytest.mark.parametrize("kind,n,k,in_place,want8", [(1, 1024, 1024, True, True), (1, 1024, 1536, True, True),
                                                     (0, 1024, 1024, False, False), (1, 512, 1024, False, True),
                                                     (0, 256, 512, True, True), (1, 768, 768, True, True)])
def test_layernorm_of_the_output_rows_inside_the_gemm(lib, kind, n, k, in_place, want8):
    """LNO kernels: c = LayerNorm(a @ w.T * alpha + bias + residual) over the n columns, the row sums exchanged between
    the CTAs that hold the row block's column tiles. Checked against torch on the GPU: the pre-norm sum in fp32 from
    the same operands, rounded to f16 (what the kernel normalises), then layer_norm. M is ragged (the last row block
    is partial) and gives every CTA pair several tiles; `in_place` writes the result over the residual."""
    import ctypes
    from chessrl_b200 import _lib as L
    torch.manual_seed(n + k + kind)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    m = 256 * ((3 * sms) // (n // 256)) + 256 * 5 + 77
    a = torch.randn(m, k, device="cuda")
    w = torch.randn(n, k, device="cuda")
    if kind == 1:
        a, w, alpha = a.to(torch.float8_e4m3fn), w.to(torch.float8_e4m3fn), 1.0 / 32.0
    else:
        a, w, alpha = a.half(), (w * 0.05).half(), 1.0
    bias = torch.randn(n, device="cuda")
    res = (torch.randn(m, n, device="cuda") * 1.5 + 0.3).half()
    gamma = (1.0 + 0.1 * torch.randn(n, device="cuda")).half()
    beta = (0.1 * torch.randn(n, device="cuda")).half()
    s8 = 448.0 / 6.0
    pre = (alpha * (a.float() @ w.float().t()) + bias + res.float()).half().float()
    want = torch.nn.functional.layer_norm(pre, (n,), gamma.float(), beta.float(), 1e-5)
    c = res.clone() if in_place else torch.full((m + 2, n), 7.0, device="cuda", dtype=torch.float16)
    x8 = torch.full((m + 2, n), 0x55, device="cuda", dtype=torch.uint8)
    scratch = torch.zeros(4096 * ((m + 255) // 256), device="cuda", dtype=torch.int64)          # 32 KiB per 256 rows
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    x = L.LinearArgs()
    x.kind, x.out_dtype = kind, 0
    x.a, x.lda, x.w, x.ldw, x.c, x.ldc = a.data_ptr(), k, w.data_ptr(), k, c.data_ptr(), n
    x.m, x.n, x.k = m, n, k
    x.bias, x.residual, x.ldr = bias.data_ptr(), (c if in_place else res).data_ptr(), n
    x.alpha, x.out_scale = alpha, 1.0
    x.device_status = status.data_ptr()
    x.lno_weight, x.lno_bias, x.lno_scratch = gamma.data_ptr(), beta.data_ptr(), scratch.data_ptr()
    x.lno_x8, x.lno_out8_scale = (x8.data_ptr() if want8 else None), s8
    for _ in range(2):      # the second call finds the exchange buffer used
        if in_place:
            c.copy_(res)
        rc = lib.crl_linear_ex(ctypes.byref(x))
        torch.cuda.synchronize()
        assert rc == 0 and int(status[0]) == 0, (rc, int(status[0]))
    got = c[:m].float()
    # one f16 rounding of the pre-norm sum may fall the other way (fp32 summation order): a step of it times rstd ~ 1
    assert_close_elementwise(got, want, 6e-3 + 2e-3 * want.abs())
    assert (got - want).abs().mean().item() < 6e-4
    if not in_place:
        assert bool((c[m:] == 7.0).all()), "rows beyond M were written"
    if want8:
        ref8 = (got * s8).clamp(-448, 448)
        assert_close_elementwise(e4m3_decode(x8[:m]), ref8, 0.5 * e4m3_step(ref8) + 2e-3 * ref8.abs() + 1e-6)
        assert bool((x8[m:] == 0x55).all()), "e4m3 rows beyond M were written"
    else:
        assert bool((x8 == 0x55).all())


@pytest.mark.parametrize("k,want_copy", [(1024, True), (1536, True), (1024, False)])
def test_layernorm_of_the_output_rows_with_int8_operands(lib, k, want_copy):
    """LNO kernels on int8 operands (per-token and per-channel scales in, W8A8): the normalised rows in f16 and their
    per-token int8 copy - scale = row maximum / 127, exchanged between the CTAs that hold the row's column tiles -
    as the stand-alone LayerNorm kernel of the INT8 engine writes them. The copy and the scales are checked
    against the f16 rows the kernel wrote (the int8 values up to the rounding of the reciprocal scale)."""
    import ctypes
    from chessrl_b200 import _lib as L
    torch.manual_seed(k + int(want_copy))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    m, n = 256 * (sms // 4 + 9) + 77, 1024
    a = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8)
    rs = (torch.rand(m, device="cuda") * 0.02 + 0.005)
    cs = (torch.rand(n, device="cuda") * 0.02 + 0.005) / 40.0
    bias = torch.randn(n, device="cuda")
    res = (torch.randn(m, n, device="cuda") * 1.5 + 0.3).half()
    gamma = (1.0 + 0.1 * torch.randn(n, device="cuda")).half()
    beta = (0.1 * torch.randn(n, device="cuda")).half()
    acc = (a.double() @ w.double().t()).float()                      # exact: |sums| < 2^53
    pre = (acc * rs[:, None] * cs[None, :] + bias + res.float()).half().float()
    want = torch.nn.functional.layer_norm(pre, (n,), gamma.float(), beta.float(), 1e-5)
    c = res.clone()
    q8 = torch.full((m + 2, n), 0x55, device="cuda", dtype=torch.int8)
    qs = torch.full((m + 2,), -1.0, device="cuda")
    scratch = torch.zeros(4096 * ((m + 255) // 256), device="cuda", dtype=torch.int64)          # 32 KiB per 256 rows
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    x = L.LinearArgs()
    x.kind, x.out_dtype = 2, 0
    x.a, x.lda, x.w, x.ldw, x.c, x.ldc = a.data_ptr(), k, w.data_ptr(), k, c.data_ptr(), n
    x.m, x.n, x.k = m, n, k
    x.bias, x.residual, x.ldr = bias.data_ptr(), c.data_ptr(), n
    x.alpha, x.out_scale = 1.0, 1.0
    x.row_scale, x.col_scale = rs.data_ptr(), cs.data_ptr()
    x.device_status = status.data_ptr()
    x.lno_weight, x.lno_bias, x.lno_scratch = gamma.data_ptr(), beta.data_ptr(), scratch.data_ptr()
    if want_copy:
        x.lno_x8, x.lno_qscale = q8.data_ptr(), qs.data_ptr()
    rc = lib.crl_linear_ex(ctypes.byref(x))
    torch.cuda.synchronize()
    assert rc == 0 and int(status[0]) == 0, (rc, int(status[0]))
    got = c.float()
    assert_close_elementwise(got, want, 6e-3 + 2e-3 * want.abs())
    assert (got - want).abs().mean().item() < 6e-4
    if want_copy:
        amax = got.abs().amax(dim=1)
        want_qs = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
        assert torch.allclose(qs[:m], want_qs, rtol=1e-6, atol=0.0) and bool((qs[m:] == -1.0).all())
        want_q = torch.round(got * (1.0 / qs[:m])[:, None]).clamp(-127, 127)
        dq = (q8[:m].float() - want_q).abs()         # a product within a rounding error of .5 may land on either side
        assert dq.max().item() <= 1 and (dq > 0).float().mean().item() < 1e-4
        assert bool((q8[m:] == 0x55).all()), "int8 rows beyond M were written"
    else:
        assert bool((q8 == 0x55).all()) and bool((qs == -1.0).all())


def test_output_layernorm_is_refused_where_it_cannot_run(lib):
    """Too few tiles for the CTA pairs, a width that is no multiple of 256, int8 operands: CRL_ERR_UNSUPPORTED."""
    import ctypes
    from chessrl_b200 import _lib as L
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for kind, m, n in ((0, 2048, 1024), (0, 65536, 768 + 64), (2, 65536, 1024)):
        k = 256
        a = torch.zeros(m, k, device="cuda", dtype=torch.int8 if kind == 2 else torch.float16)
        w = torch.zeros(n, k, device="cuda", dtype=a.dtype)
        g = torch.ones(n, device="cuda", dtype=torch.float16)
        c = torch.full((m, n), 3.0, device="cuda", dtype=torch.float16)
        scratch = torch.zeros(4096 * ((m + 255) // 256), device="cuda", dtype=torch.int64)
        x = L.LinearArgs()
        x.kind, x.out_dtype, x.a, x.lda, x.w, x.ldw, x.c, x.ldc = kind, 0, a.data_ptr(), k, w.data_ptr(), k, c.data_ptr(), n
        x.m, x.n, x.k, x.alpha, x.device_status = m, n, k, 1.0, status.data_ptr()
        x.residual, x.ldr = c.data_ptr(), n
        x.lno_weight, x.lno_bias, x.lno_scratch = g.data_ptr(), g.data_ptr(), scratch.data_ptr()
        if kind == 2:
            x.lno_x8 = a.data_ptr()          # int8 copy asked for, lno_qscale missing
        assert lib.crl_linear_ex(ctypes.byref(x)) == -8, (kind, m, n)
        torch.cuda.synchronize()
        assert bool((c == 3.0).all())


_AB_SCRIPT = r'''
import ctypes, hashlib, sys, torch
sys.path.insert(0, %(root)r)
from chessrl_b200 import _lib as L
lib = L.load()
torch.manual_seed(1)
sms = torch.cuda.get_device_properties(0).multi_processor_count
m = 256 * (sms // 2 + 3) + 64
h = hashlib.sha256()

def run(kind, n, k, out, bias=True, act=0, res=False, scales=False, lno=False, copy=False):
    if kind == 1:
        a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn); w = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    elif kind == 2:
        a = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8); w = torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8)
    else:
        a = torch.randn(m, k, device="cuda").half(); w = (torch.randn(n, k, device="cuda") * 0.05).half()
    c = torch.zeros(m, n, device="cuda", dtype=torch.uint8 if out == 2 else torch.float16)
    b = torch.randn(n, device="cuda")
    r = torch.randn(m, n, device="cuda").half()
    rs = torch.rand(m, device="cuda") * 0.01 + 0.001; cs = torch.rand(n, device="cuda") * 0.01 + 0.001
    g = (1.0 + 0.1 * torch.randn(n, device="cuda")).half(); be = (0.1 * torch.randn(n, device="cuda")).half()
    x8 = torch.zeros(m, n, device="cuda", dtype=torch.uint8)
    scratch = torch.zeros(4096 * ((m + 255) // 256), device="cuda", dtype=torch.int64)
    st = torch.zeros(4, dtype=torch.int32, device="cuda")
    x = L.LinearArgs()
    x.kind, x.out_dtype = kind, out
    x.a, x.lda, x.w, x.ldw, x.c, x.ldc = a.data_ptr(), k, w.data_ptr(), k, c.data_ptr(), n
    x.m, x.n, x.k = m, n, k
    x.bias = b.data_ptr() if bias else None
    if res or lno:
        x.residual, x.ldr = r.data_ptr(), n
    x.alpha, x.act, x.out_scale = (1.0 / 64.0 if kind == 1 else 1.0), act, 3.0
    if scales:
        x.row_scale, x.col_scale = rs.data_ptr(), cs.data_ptr()
    x.device_status = st.data_ptr()
    if lno:
        x.lno_weight, x.lno_bias, x.lno_scratch = g.data_ptr(), be.data_ptr(), scratch.data_ptr()
        if copy:
            x.lno_x8, x.lno_out8_scale = x8.data_ptr(), 50.0
    rc = lib.crl_linear_ex(ctypes.byref(x))
    torch.cuda.synchronize()
    assert rc == 0 and int(st[0]) == 0, (rc, int(st[0]))
    h.update(c.cpu().numpy().tobytes()); h.update(x8.cpu().numpy().tobytes())

run(1, 3072, 1024, 2)                       # e4m3 out, bias
run(1, 4096, 256, 2, bias=False)            # e4m3 out, no bias
run(1, 1536, 1024, 2, act=2)                # e4m3 out, bias + Mish on packed pairs
run(1, 1024, 1536, 0, res=True)             # f16 out, residual by TMA
run(0, 3072, 1024, 0)                       # f16 operands
run(0, 1536, 1024, 0, act=2)                # f16 operands, Mish in fp32
run(2, 3072, 1024, 0, scales=True)          # int8 operands with both scale vectors
run(2, 1024, 1024, 0, scales=True, res=True)
run(1, 1024, 1024, 0, lno=True, copy=True)  # output LayerNorm with the e4m3 copy
run(0, 1024, 1024, 0, lno=True)             # ... without
print(h.hexdigest())
'''


def test_specialised_epilogues_equal_the_generic_one():
    """The instantiations with compile-time epilogue switches against the generic epilogue (CRL_GEMM_GENERIC keeps every
    launch on it; the library reads the variable once, hence two processes): every output byte of ten launches that
    cover each specialised kernel family must agree."""
    import os
    import subprocess
    import sys
    from conftest import ROOT
    script = _AB_SCRIPT % {"root": ROOT}
    digests = []
    for generic in (False, True):
        env = dict(os.environ)
        env.pop("CRL_GEMM_GENERIC", None)
        if generic:
            env["CRL_GEMM_GENERIC"] = "1"
        out = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr[-2000:]
        digests.append(out.stdout.strip().splitlines()[-1])
    assert digests[0] == digests[1]
