"""Numerics of every CUDA kernel against the plain fp32 PyTorch statement of the same op.

The reference math is the CPU branch of `oa_b200.ops.kernels` (run on fp32 copies of the inputs), so
a kernel and its oracle share one definition of the contract.
"""
import math

import pytest
import torch

from oa_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, ref, rtol, atol=None, what=""):
    got = got.float().cpu()
    ref = ref.float().cpu()
    scale = ref.abs().max().item() + 1e-12
    err = (got - ref).abs().max().item()
    tol = rtol * scale + (atol or 0.0)
    assert math.isfinite(err) and err <= tol, f"{what}: max err {err:.4g} > tol {tol:.4g} (ref scale {scale:.4g})"


BF16_EPS = 2.0 ** -8          # half an ulp of a bf16 result, relative


def _close_elem(got, ref, atol, rtol, what=""):
    """Every element on its own: |got - ref| <= atol + rtol * |ref| (a max-norm bound alone hides relative errors on
    small entries)."""
    got, ref = got.float().cpu(), ref.float().cpu()
    err = (got - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = err > bound
    assert torch.isfinite(got).all() and not bad.any(), \
        f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance, worst {float((err - bound).max()):.4g} over the bound"


def _close_gemm_bf16(got, ref, k_total, what="", out_bf16=True):
    """The reference's GEMM tier (Test/OaTest.h:118-127): absolute bound 2e-2 * sqrt(K / 16) for unit-variance bf16 operands
    accumulated in fp32, plus the rounding of a bf16 result; checked per element."""
    _close_elem(got, ref, 2.0e-2 * math.sqrt(k_total / 16.0), BF16_EPS if out_bf16 else 1e-6, what)


@pytest.fixture(autouse=True)
def _status():
    yield
    torch.cuda.synchronize()
    K.check_status()


def _rand(*shape, dtype=torch.bfloat16, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(dtype)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K_", [(128, 128, 64), (256, 512, 256), (300, 520, 264), (1024, 256, 2048)])
def test_gemm_bf16_layouts(a_mn, b_mn, M, N, K_):
    torch.manual_seed(0)
    if a_mn and M % 8:
        M = (M + 7) // 8 * 8
    a = _rand(K_, M) if a_mn else _rand(M, K_)
    b = _rand(K_, N) if b_mn else _rand(N, K_)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn)
    _close(out, ref, 1e-2, what=f"gemm a_mn={a_mn} b_mn={b_mn} {M}x{N}x{K_}")
    _close_gemm_bf16(out, ref, K_, what=f"gemm (per element) a_mn={a_mn} b_mn={b_mn} {M}x{N}x{K_}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_bf16_cta_pair_kernel(a_mn, b_mn):
    """Shapes with at least 74 tiles of 256 x 256 take the CTA-pair (cta_group::2) kernel; ragged M, N and K edges."""
    torch.manual_seed(3)
    M, N, K_ = 2200, 2624, 328
    a = _rand(K_, M) if a_mn else _rand(M, K_)
    b = _rand(K_, N, scale=0.05) if b_mn else _rand(N, K_, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, residual=res, act=K.ACT_GELU)
    ref = K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn, bias=bias.cpu().float(), residual=res.cpu().float(), act=K.ACT_GELU)
    _close(out, ref, 1e-2, what=f"pair gemm a_mn={a_mn} b_mn={b_mn}")
    out32 = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out32)
    K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out32, accumulate=True)
    ref32 = 2 * K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn)
    _close(out32, ref32, 1e-2, what="pair gemm fp32 accumulate")
    _close_gemm_bf16(out32, ref32, K_, what="pair gemm fp32 accumulate (per element)", out_bf16=False)
    # bf16 outputs (they leave through TMA stores): pre-activation copy out, saved pre-activation in, plain store
    aux = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    out = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, act=K.ACT_GELU, aux_out=aux)
    aux_ref = torch.empty(M, N)
    ref = K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn, bias=bias.cpu().float(), act=K.ACT_GELU, aux_out=aux_ref)
    _close(out, ref, 1e-2, what="pair gemm bias+gelu with pre-activation copy")
    _close(aux, aux_ref, 1e-2, what="pair gemm pre-activation copy")
    z = _rand(M, N)
    for act in (K.ACT_GELU_BWD, K.ACT_RELU_BWD):
        got = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, act=act, aux_in=z)
        want = K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn, act=act, aux_in=z.cpu().float())
        _close(got, want, 1e-2, what=f"pair gemm activation backward {act}")
    plain = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, alpha=0.5)
    _close(plain, 0.5 * K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn), 1e-2, what="pair gemm plain bf16 store")
    # the specialised epilogue forms (no bias): + residual; GELU with the pre-activation copy
    got = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, residual=res)
    _close(got, K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn, residual=res.cpu().float()), 1e-2, what="pair gemm + residual")
    aux2 = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=DEV)
    got = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, act=K.ACT_GELU, aux_out=aux2)
    aux2_ref = torch.empty(M, N)
    want = K.gemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn, act=K.ACT_GELU, aux_out=aux2_ref)
    _close(got, want, 1e-2, what="pair gemm gelu with pre-activation copy, no bias")
    _close(aux2, aux2_ref, 1e-2, what="pair gemm pre-activation copy, no bias")
    # N a multiple of 8 but not of the 32-column store box, output a column slice of a wider matrix (row pitch != N):
    # the boxes at the right and bottom edges are clipped, the columns beside the slice stay untouched
    N2 = 2632
    b2 = _rand(K_, N2, scale=0.05) if b_mn else _rand(N2, K_, scale=0.05)
    wide = torch.full((M, N2 + 64), 3.0, dtype=torch.bfloat16, device=DEV)
    K.gemm(a, b2, a_mn=a_mn, b_mn=b_mn, out=wide[:, 32:32 + N2])
    _close(wide[:, 32:32 + N2], K.gemm(a.cpu().float(), b2.cpu().float(), a_mn=a_mn, b_mn=b_mn), 1e-2, what="pair gemm into a column slice")
    assert bool((wide[:, :32] == 3.0).all()) and bool((wide[:, 32 + N2:] == 3.0).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fill_large_and_unaligned(dtype):
    """Large aligned fills use 16-byte stores for the bulk and the element kernel for the remainder; a view that does not start
    on a 16-byte boundary takes the element kernel; the guard elements around the filled range stay untouched."""
    n = (1 << 20) + 3
    buf = torch.full((n + 16,), 7.0, dtype=dtype, device=DEV)
    for off in (8, 9):                                   # 8 elements: 16-byte aligned for both types; 9: not aligned
        buf.fill_(7.0)
        K.fill_(buf[off:off + n], -1.5)
        torch.cuda.synchronize()
        assert bool((buf[off:off + n] == -1.5).all()), off
        assert bool((buf[:off] == 7.0).all()) and bool((buf[off + n:] == 7.0).all()), off


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_bf16_epilogues(bn):
    torch.manual_seed(1)
    M, N, K_ = 384, 768, 320
    a, b = _rand(M, K_), _rand(N, K_, scale=0.05)
    bias, res = _rand(N), _rand(M, N)
    aux = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    out = K.gemm(a, b, bias=bias, residual=res, act=K.ACT_GELU, aux_out=aux, force_bn=bn)
    aux_ref = torch.empty(M, N)
    ref = K.gemm(a.cpu().float(), b.cpu().float(), bias=bias.cpu().float(), residual=res.cpu().float(), act=K.ACT_GELU,
                 aux_out=aux_ref)
    _close(out, ref, 1e-2, what="bias+gelu+residual")
    _close(aux, aux_ref, 1e-2, what="pre-activation copy")
    # backward-style epilogue: multiply by gelu'(z) and accumulate into fp32
    z = _rand(M, N)
    acc = torch.randn(M, N, device=DEV)
    acc_ref = acc.cpu().clone()
    K.gemm(a, b, act=K.ACT_GELU_BWD, aux_in=z, out=acc, accumulate=True, force_bn=bn)
    K.gemm(a.cpu().float(), b.cpu().float(), act=K.ACT_GELU_BWD, aux_in=z.cpu().float(), out=acc_ref, accumulate=True)
    _close(acc, acc_ref, 1e-2, what="gelu_bwd+accumulate fp32")


def test_gemm_bf16_split_k():
    torch.manual_seed(2)
    M, N, K_ = 512, 512, 8192  # weight-gradient shape: few tiles, long reduction -> split-K path
    a, b = _rand(K_, M), _rand(K_, N)
    out = K.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    ref = K.gemm(a.cpu().float(), b.cpu().float(), a_mn=True, b_mn=True)
    _close(out, ref, 5e-3, what="split-k")
    out2 = K.gemm(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    assert torch.equal(out, out2), "split-K reduction must be deterministic"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
def test_gemm_bf16_batched(a_mn, b_mn):
    torch.manual_seed(12)
    nb, M, N, K_ = 5, 200, 136, 96
    a = _rand(nb, K_, M) if a_mn else _rand(nb, M, K_)
    b = _rand(nb, K_, N) if b_mn else _rand(nb, N, K_)
    out = K.bgemm(a, b, a_mn=a_mn, b_mn=b_mn)
    ref = K.bgemm(a.cpu().float(), b.cpu().float(), a_mn=a_mn, b_mn=b_mn)
    _close(out, ref, 1e-2, what="batched gemm")
    # strided batch view (e.g. heads inside a packed activation) and fp32 accumulate
    big = _rand(nb, 256, 2 * K_)
    a2 = big[:, :M, K_:]
    if not a_mn and not b_mn:
        acc = torch.randn(nb, M, N, device=DEV)
        ref2 = acc.cpu() + torch.bmm(a2.cpu().float(), b.cpu().float().transpose(1, 2))
        K.bgemm(a2, b, out=acc, accumulate=True)
        _close(acc, ref2, 1e-2, what="batched strided accumulate")


def test_gemm_f32():
    torch.manual_seed(3)
    a, b = torch.randn(70, 50, device=DEV), torch.randn(33, 50, device=DEV)
    bias = torch.randn(33, device=DEV)
    out = K.gemm(a, b, bias=bias, act=K.ACT_GELU)
    ref = K.gemm(a.cpu(), b.cpu(), bias=bias.cpu(), act=K.ACT_GELU)
    _close(out, ref, 1e-5, what="f32 gemm")
    out = K.gemm(a.t().contiguous(), b.t().contiguous(), a_mn=True, b_mn=True)
    _close(out, a.cpu() @ b.cpu().t(), 1e-5, what="f32 gemm mn")
    x, y = torch.randn(5, 40, 24, device=DEV), torch.randn(5, 24, 36, device=DEV)
    _close(K.bmm_f32(x, y, b_mn=True), torch.bmm(x.cpu(), y.cpu()), 1e-5, what="bmm")
    # whole 64 x 64 tiles next to edge tiles, both layouts, epilogues, accumulation
    for (M, N, Kk) in [(256, 192, 128), (200, 136, 64), (128, 64, 1024)]:      # the last one takes the split-K path
        a, b = torch.randn(M, Kk, device=DEV), torch.randn(N, Kk, device=DEV)
        bias = torch.randn(N, device=DEV)
        ref = a.cpu().double() @ b.cpu().double().t()
        _close(K.gemm(a, b), ref.float(), 2e-5, what=f"f32 gemm {M}x{N}x{Kk} K-major")
        _close(K.gemm(a.t().contiguous(), b.t().contiguous(), a_mn=True, b_mn=True), ref.float(), 2e-5, what=f"f32 gemm {M}x{N}x{Kk} MN-major")
        _close(K.gemm(a, b.t().contiguous(), b_mn=True, bias=bias, act=K.ACT_RELU), torch.relu(ref + bias.cpu().double()).float(), 2e-5,
               what=f"f32 gemm {M}x{N}x{Kk} mixed layouts, bias + relu")
        acc = torch.randn(M, N, device=DEV)
        want = acc.cpu().double() + 0.5 * ref
        K.gemm(a, b, out=acc, accumulate=True, alpha=0.5)
        _close(acc, want.float(), 2e-5, what=f"f32 gemm {M}x{N}x{Kk} accumulate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_elementwise(dtype):
    torch.manual_seed(4)
    x = _rand(37, 96, dtype=dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for op in ["neg", "abs", "exp", "sin", "cos", "relu", "gelu", "silu", "tanh", "sigmoid", "softplus", "mish", "square"]:
        _close(K.unary(op, x), K.unary(op, x.cpu().float()), tol, what=op)
        # the reference's elementwise tier (Test/OaTest.h:108-110: 5e-4 absolute) plus the rounding of the stored result
        _close_elem(K.unary(op, x), K.unary(op, x.cpu().float()), 5e-4 if dtype == torch.bfloat16 else 2e-6,
                    BF16_EPS if dtype == torch.bfloat16 else 2e-6, what=op + " (per element)")
    xp = x.abs() + 0.5
    for op in ["log", "sqrt", "recip"]:
        _close(K.unary(op, xp), K.unary(op, xp.cpu().float()), tol, what=op)
    _close(K.unary("scale", x, 2.5), x.cpu().float() * 2.5, tol)
    y = _rand(37, 96, dtype=dtype)
    for op in ["add", "sub", "mul", "relu_bwd", "gelu_bwd", "silu_bwd", "silu_mul"]:
        _close(K.binary(op, x, y), K.binary(op, x.cpu().float(), y.cpu().float()), tol, what=op)
    row = _rand(96, dtype=dtype)
    _close(K.binary("add", x, row), x.cpu().float() + row.cpu().float(), tol, what="row bcast")
    col = _rand(37, 1, dtype=dtype)
    _close(K.binary("mul", x, col), x.cpu().float() * col.cpu().float(), tol, what="col bcast")
    _close(K.cast(x, torch.float32), x.cpu().float(), 1e-6)
    xt = x.t()
    assert torch.equal(K.contiguous(xt).cpu(), xt.cpu().contiguous())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_rope_embedding(dtype):
    torch.manual_seed(5)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    gu, d = _rand(50, 256, dtype=dtype), _rand(50, 128, dtype=dtype)
    _close(K.swiglu_fwd(gu), K.swiglu_fwd(gu.cpu().float()), tol)
    _close(K.swiglu_bwd(gu, d), K.swiglu_bwd(gu.cpu().float(), d.cpu().float()), tol)
    x = _rand(2 * 24, 3 * 4 * 32, dtype=dtype)
    ref = K.rope_(x.cpu().float().clone()[:, : 4 * 32], 4, 32, 24, pos_offset=3)
    got = x.clone()
    K.rope_(got[:, : 4 * 32], 4, 32, 24, pos_offset=3)
    _close(got[:, : 4 * 32], ref, tol, what="rope")
    _close(got[:, 4 * 32:], x[:, 4 * 32:], 0.0, atol=0.0, what="rope must not touch k,v columns")
    back = got.clone()
    K.rope_(back[:, : 4 * 32], 4, 32, 24, pos_offset=3, backward=True)
    _close(back, x, 2 * tol, what="rope inverse")
    table, pos = _rand(100, 64, dtype=dtype), _rand(24, 64, dtype=dtype)
    ids = torch.randint(0, 100, (48,), device=DEV, dtype=torch.int32)
    _close(K.embedding_fwd(table, ids, pos, 24), K.embedding_fwd(table.cpu().float(), ids.cpu(), pos.cpu().float(), 24), tol)
    do = _rand(48, 64, dtype=dtype)
    _close(K.embedding_bwd(do, ids, 100), K.embedding_bwd(do.cpu().float(), ids.cpu(), 100), tol)
    _close(K.col_sum(do), do.cpu().float().sum(0), tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(33, 128), (300, 512), (1000, 1024)])
def test_norms(dtype, rows, cols):
    torch.manual_seed(6)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    x, w, b, dy, res = (_rand(rows, cols, dtype=dtype), _rand(cols, dtype=dtype), _rand(cols, dtype=dtype),
                        _rand(rows, cols, dtype=dtype), _rand(rows, cols, dtype=dtype))
    c = lambda t: t.cpu().float()
    y, rstd, _ = K.rmsnorm_fwd(x, w, 1e-5)
    yr, rstdr, _ = K.rmsnorm_fwd(c(x), c(w), 1e-5)
    _close(y, yr, tol, what="rmsnorm")
    _close(rstd, rstdr, 1e-3)
    y2, _, ro = K.rmsnorm_fwd(x, w, 1e-5, residual=res)
    y2r, _, ror = K.rmsnorm_fwd(c(x), c(w), 1e-5, residual=c(res))
    _close(y2, y2r, tol, what="residual rmsnorm")
    _close(ro, ror, tol)
    dx, dw = K.rmsnorm_bwd(x, w, dy, rstd, dres=res)
    dxr, dwr = K.rmsnorm_bwd(c(x), c(w), c(dy), rstdr, dres=c(res))
    _close(dx, dxr, tol, what="rmsnorm dx")
    _close(dw, dwr, tol, what="rmsnorm dw")
    y, mean, rstd = K.layernorm_fwd(x, w, b, 1e-5)
    yr, meanr, rstdr = K.layernorm_fwd(c(x), c(w), c(b), 1e-5)
    _close(y, yr, tol, what="layernorm")
    dx, dw, db = K.layernorm_bwd(x, w, dy, mean, rstd)
    dxr, dwr, dbr = K.layernorm_bwd(c(x), c(w), c(dy), meanr, rstdr)
    _close(dx, dxr, tol, what="layernorm dx")
    _close(dw, dwr, tol, what="layernorm dw")
    _close(db, dbr, tol, what="layernorm db")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_xent(dtype):
    torch.manual_seed(7)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    x = _rand(64, 1000, dtype=dtype, scale=3.0)
    c = lambda t: t.cpu().float()
    for log in (False, True):
        y = K.softmax(x, log=log, scale=0.5)
        _close(y, K.softmax(c(x), log=log, scale=0.5), tol)
        dy = _rand(64, 1000, dtype=dtype)
        _close(K.softmax_bwd(y, dy, log=log, scale=0.5), K.softmax_bwd(c(y), c(dy), log=log, scale=0.5), tol)
    tg = torch.randint(0, 1000, (64,), device=DEV)
    tg[3] = -100   # ignored
    tg[5] = 5000   # out of range -> NaN loss row, zero onehot
    loss, dl = K.xent_fwd_bwd(x, tg, grad_scale=1.0 / 64)
    lossr, dlr = K.xent_fwd_bwd(c(x), tg.cpu(), grad_scale=1.0 / 64)
    assert math.isnan(loss[5].item()) and loss[3].item() == 0.0
    ok = torch.ones(64, dtype=torch.bool)
    ok[5] = False
    _close(loss.cpu()[ok], lossr[ok], 1e-2 if dtype == torch.bfloat16 else 1e-5, what="xent loss")
    _close(dl, dlr, tol, what="xent grad")
    xin = x.clone()
    K.xent_fwd_bwd(xin, tg, grad_scale=1.0 / 64, dlogits=xin)  # in place
    _close(xin, dlr, tol, what="xent in-place grad")
    _close(K.row_reduce("sum", x), c(x).sum(1), tol)
    assert torch.equal(K.row_reduce("argmax", x).cpu().long(), c(x).argmax(1))


@pytest.mark.parametrize("pdt,gdt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32)])
def test_adam_sgd(pdt, gdt):
    torch.manual_seed(8)
    n = 10007
    w0 = torch.randn(n, device=DEV)
    p = w0.to(pdt)
    master = w0.clone() if pdt == torch.bfloat16 else None
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    state = torch.tensor([0, 1e-2, 0.9, 0.999, 1e-8, 0.1, 1.0, 0], dtype=torch.float32, device=DEV)
    pr, mr_, vr = w0.cpu().clone(), torch.zeros(n), torch.zeros(n)
    master_r = w0.cpu().clone() if master is not None else None
    state_r = state.cpu().clone()
    for _ in range(3):
        g = torch.randn(n, device=DEV).to(gdt)
        K.optim_advance(state)
        K.adam_step(p, g, master, m, v, state, decoupled=True)
        K.optim_advance(state_r)
        K.adam_step(pr, g.cpu().float(), master_r, mr_, vr, state_r, decoupled=True)
    _close(master if master is not None else p, master_r if master_r is not None else pr, 1e-5, what="adamw")
    _close(p, pr, 1e-2 if pdt == torch.bfloat16 else 1e-5)
    ss = torch.zeros(1, device=DEV)
    K.sumsq(p, ss)
    _close(ss, p.float().pow(2).sum().reshape(1), 1e-4)


@pytest.mark.parametrize("hd,heads,seq,batch,causal", [(64, 2, 256, 2, True), (64, 3, 384, 1, False), (128, 2, 256, 2, True),
                                                       (64, 2, 200, 2, True), (128, 1, 520, 1, True)])
def test_flash_fwd_bwd(hd, heads, seq, batch, causal):
    torch.manual_seed(9)
    D = heads * hd
    qkv = _rand(batch * seq, 3 * D)
    q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
    o, lse = K.flash_fwd(q, k, v, batch, seq, heads, hd, causal=causal)
    c = lambda t: t.cpu().float()
    orf, lser = K.flash_fwd(c(q), c(k), c(v), batch, seq, heads, hd, causal=causal)
    _close(o, orf, 2e-2, what="flash fwd o")
    _close(lse, lser, 1e-2, what="flash lse")
    do = _rand(batch * seq, D)
    dq, dk, dv = K.flash_bwd(q, k, v, o, do, lse, batch, seq, heads, hd, causal=causal)
    dqr, dkr, dvr = K.flash_bwd(c(q), c(k), c(v), orf, c(do), lser, batch, seq, heads, hd, causal=causal)
    _close(dv, dvr, 3e-2, what="flash dv")
    _close(dk, dkr, 3e-2, what="flash dk")
    _close(dq, dqr, 3e-2, what="flash dq")


@pytest.mark.parametrize("hd,seq,causal", [(32, 70, True), (16, 33, False), (64, 200, True), (128, 130, True), (48, 64, False)])
def test_attn_f32(hd, seq, causal):
    torch.manual_seed(10)
    batch, heads = 2, 4
    D = heads * hd
    qkv = torch.randn(batch * seq, 3 * D, device=DEV)
    q, k, v = qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:]
    o, lse = K.flash_fwd(q, k, v, batch, seq, heads, hd, causal=causal)
    orf, lser = K.flash_fwd(q.cpu(), k.cpu(), v.cpu(), batch, seq, heads, hd, causal=causal)
    _close(o, orf, 1e-5)
    _close(lse, lser, 1e-5)
    do = torch.randn(batch * seq, D, device=DEV)
    got = K.flash_bwd(q, k, v, o, do, lse, batch, seq, heads, hd, causal=causal)
    ref = K.flash_bwd(q.cpu(), k.cpu(), v.cpu(), orf, do.cpu(), lser, batch, seq, heads, hd, causal=causal)
    for g, r, nm in zip(got, ref, "qkv"):
        _close(g, r, 1e-4, what="attn_f32 d" + nm)


def test_philox_dropout():
    x = torch.empty(100000, device=DEV)
    K.philox_(x, 1234, 0, normal=False, a=0.0, b=1.0)
    assert 0.49 < x.mean().item() < 0.51 and x.min().item() >= 0 and x.max().item() < 1
    K.philox_(x, 1234, 0, normal=True, a=0.0, b=1.0)
    assert abs(x.mean().item()) < 0.02 and 0.97 < x.std().item() < 1.03
    y = torch.empty_like(x)
    K.philox_(y, 1234, 0, normal=True, a=0.0, b=1.0)
    assert torch.equal(x, y)
    d = K.dropout(torch.ones(100000, device=DEV), 0.25, 7, 0)
    assert 0.73 < (d > 0).float().mean().item() < 0.77


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_xent_rows_not_16_byte_aligned(dtype):
    """A vocabulary of 27 (the character tokenizer) gives rows that start off a 16-byte boundary: the scalar loops run."""
    torch.manual_seed(8)
    x = _rand(96, 27, dtype=dtype, scale=2.0)
    tg = torch.randint(0, 27, (96,), device=DEV)
    loss, dl = K.xent_fwd_bwd(x, tg, grad_scale=1.0 / 96)
    lossr, dlr = K.xent_fwd_bwd(x.cpu().float(), tg.cpu(), grad_scale=1.0 / 96)
    _close(loss, lossr, 1e-2 if dtype == torch.bfloat16 else 1e-5, what="xent loss, vocab 27")
    _close(dl, dlr, 2e-2 if dtype == torch.bfloat16 else 1e-6, what="xent grad, vocab 27")


@pytest.mark.parametrize("terms,tol", [(2, 4e-5), (3, 2e-6)])
@pytest.mark.parametrize("layout", [(False, False), (True, True)])
def test_gemm_f32_on_the_tensor_cores(terms, tol, layout):
    """fp32 GEMM as bf16 part products on tcgen05 (2 parts: 3 products, 3 parts: 6 products) against an fp64 statement of the
    product; the FMA kernel is the control.  Error is measured against |A| |B|^T, the scale rounding errors live on."""
    from oa_b200.ops import kernels as K
    a_mn, b_mn = layout
    M, N, Kd = 1024, 512, 768
    torch.manual_seed(4)
    a = torch.randn((Kd, M) if a_mn else (M, Kd), device="cuda")
    b = torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda")
    A = (a.t() if a_mn else a).double()
    B = (b.t() if b_mn else b).double()
    want = A @ B.t()
    scale = A.abs() @ B.abs().t()
    exact = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    K.set_f32_tensor_terms(terms)
    try:
        got = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
        acc = K.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=exact.clone(), accumulate=True, alpha=0.5)
    finally:
        K.set_f32_tensor_terms(0)
    assert got.dtype == torch.float32
    err = ((got.double() - want).abs() / scale).max().item()
    assert err <= tol, err
    assert ((exact.double() - want).abs() / scale).max().item() <= 1e-6
    assert ((acc.double() - 1.5 * want).abs() / scale).max().item() <= 2 * tol + 1e-6
    K.check_status()
