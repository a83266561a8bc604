"""GPU parity: the CUDA forward through the module / C ABI against the oracle and the
golden outputs of the reference.  Tolerance: max|y - y_ref| / max|y_ref| <= 1e-3 with
y_ref the reference forward evaluated in fp32 on the same (already rounded) inputs."""
import numpy as np
import pytest
import torch

from oracle import bqq_oracle as O
from tests.helpers import LAYER_CASES, load_golden, oracle_forward_t, synth_layer
from tests.test_gpu_pack import _module_from_golden

pytestmark = pytest.mark.gpu
TOL = 1e-3        # contract
# what the decode kernel should reach with fp32 outputs: x is quantised to 16-bit block fixed
# point per col patch (error <= 2^-16 of the patch maximum per element), everything else is exact
# integer arithmetic or fp32
TOL_FP32 = 1e-4


def _run(bq, X):
    with torch.no_grad():
        y = bq(X)
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize('name', LAYER_CASES)
def test_golden_cases(name):
    g = load_golden(name)
    bq = _module_from_golden(g)
    X = torch.from_numpy(g['X'])
    if bool(g['x_is_bf16']):
        X = X.to(torch.bfloat16)
    y = _run(bq, X.cuda())
    assert y.dtype == X.dtype and tuple(y.shape) == tuple(g['y_ref_fp32'].shape)
    err = O.max_rel_err(y.float().cpu().numpy(), g['y_ref_fp32'])
    # bf16 outputs carry their own rounding (2^-9 relative) on top of the compute error
    assert err < (4e-3 if X.dtype == torch.bfloat16 else TOL_FP32), err
    if X.dtype == torch.bfloat16:
        y32 = _run(bq, X.float().cuda())
        assert O.max_rel_err(y32.cpu().numpy(), g['y_ref_fp32']) < TOL_FP32


def test_config1_golden():
    g = load_golden('config1_4096')
    Y, Z, A, _, X = synth_layer(2, 128, 128, 32, 32, 32, 1, seed=0)
    assert np.array_equal(X.numpy(), g['X'])
    from bqq_b200.bqq_modules import BinaryQuadratic
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    y = _run(bq, X.cuda())
    assert O.max_rel_err(y.cpu().numpy(), g['y_ref_fp64']) < TOL_FP32


DECODE_SHAPES = [
    # bw, rw, cw, P, Q, r
    (2, 16, 24, 32, 32, 32), (3, 8, 8, 32, 32, 32), (4, 8, 4, 32, 32, 32),
    (2, 8, 8, 64, 64, 32), (3, 4, 6, 64, 64, 64), (2, 2, 3, 128, 128, 64),
    (2, 4, 4, 16, 16, 16), (2, 2, 2, 32, 32, 12), (1, 3, 5, 96, 40, 33), (5, 2, 3, 32, 64, 7),
]


@pytest.mark.parametrize('shape', DECODE_SHAPES)
@pytest.mark.parametrize('M', [1, 2, 4, 5, 16])
def test_decode_against_oracle(shape, M):
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, X = synth_layer(*shape, M, seed=sum(shape) + M, bias=(M % 2 == 0))
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    ref = oracle_forward_t(Y, Z, A, bias, X)
    y = _run(bq, X.cuda())
    assert O.max_rel_err(y.cpu().numpy(), ref) < TOL_FP32
    Xb = X.to(torch.bfloat16)
    refb = oracle_forward_t(Y, Z, A, bias, Xb)
    yb = _run(bq, Xb.cuda())
    assert yb.dtype == torch.bfloat16
    # compare before the final bf16 rounding dominates: |err| <= 1e-3 of max plus bf16 output rounding
    assert O.max_rel_err(yb.float().cpu().numpy(), refb) < TOL + 2 ** -8
    yh = _run(bq, X.half().cuda())
    assert O.max_rel_err(yh.float().cpu().numpy(), oracle_forward_t(Y, Z, A, bias, X.half())) < TOL + 2 ** -10


@pytest.mark.parametrize('shape,M', [((2, 8, 8, 32, 32, 32), 64), ((2, 16, 8, 32, 32, 32), 200),
                                     ((3, 4, 6, 64, 64, 64), 130), ((2, 3, 2, 64, 64, 32), 17),
                                     ((2, 40, 16, 32, 32, 32), 300)])
def test_prefill_against_oracle(shape, M):
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, X = synth_layer(*shape, M, seed=sum(shape) + M, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        Xd = X.to(dt)
        ref = oracle_forward_t(Y, Z, A, bias, Xd)
        y = _run(bq, Xd.cuda())
        assert y.dtype == dt
        out_round = {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -10, torch.float32: 0.0}[dt]
        err = O.max_rel_err(y.float().cpu().numpy(), ref)
        assert err < TOL + out_round, (dt, err)


@pytest.mark.parametrize('M', [1024, 512, 256, 128, 40])
def test_prefill_every_tile_width(M):
    """4096 outputs: the GEMM picks its tile width (256, 128, 64, 32 columns) by the number of tiles the batch gives."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, X = synth_layer(2, 128, 8, 32, 32, 32, M, seed=M, x_dtype=torch.bfloat16, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    y = _run(bq, X.cuda())
    assert O.max_rel_err(y.float().cpu().numpy(), oracle_forward_t(Y, Z, A, bias, X)) < TOL + 2 ** -8
    y32 = _run(bq, X.float().cuda())
    assert O.max_rel_err(y32.cpu().numpy(), oracle_forward_t(Y, Z, A, bias, X)) < TOL


@pytest.mark.parametrize('M,rw', [(512, 896), (2048, 160)])
def test_prefill_column_panels(M, rw):
    """Enough GEMM tiles for several waves: W is rebuilt and multiplied in column panels (the rebuild of a panel runs
    beside the GEMM of the previous one), with two row halves per CTA.  Every output is checked."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, X = synth_layer(2, rw, 8, 32, 32, 32, M, seed=rw + M, x_dtype=torch.bfloat16, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    ref = oracle_forward_t(Y, Z, A, bias, X)
    for _ in range(2):                                   # twice: the workspace is reused
        y = _run(bq, X.cuda())
        assert O.max_rel_err(y.float().cpu().numpy(), ref) < TOL + 2 ** -8
    y32 = _run(bq, X.float().cuda())
    assert O.max_rel_err(y32.cpu().numpy(), ref) < TOL


def test_prefill_fp32_output_tolerance():
    """Config-3-like contraction (K = 4096) with fp32 outputs so only compute error remains."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, _, X = synth_layer(2, 8, 128, 32, 32, 32, 256, seed=5, x_dtype=torch.bfloat16)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    ref = oracle_forward_t(Y, Z, A, None, X)
    st = bq._ensure_packed()
    from bqq_b200 import _cabi
    from bqq_b200.bqq_modules import _workspace
    xg = X.cuda()
    y = torch.empty(256, 256, dtype=torch.float32, device='cuda')
    ws = _workspace(xg.device, 'prefill', _cabi.lib.bqq_prefill_workspace_bytes(st.dims, 256))
    layer = bq._layer(st)
    rc = _cabi.lib.bqq_forward_prefill(layer, xg.data_ptr(), _cabi.BF16, 256, xg.stride(0), y.data_ptr(),
                                       _cabi.F32, y.stride(0), ws.data_ptr(), ws.numel(),
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 0          # no bounded wait gave up
    assert O.max_rel_err(y.cpu().numpy(), ref) < TOL


def test_prefill_row_strided_bf16_inputs():
    """bf16 rows longer than one pass of the staging block keeps in registers, read through row-strided views whose
    pitch does (16-byte accesses) and does not (2-byte accesses) allow the vector path: all three give the same bits."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, P, Q, r, M = 2, 2, 144, 32, 32, 32, 40
    Y, Z, A, _, X = synth_layer(bw, rw, cw, P, Q, r, M, seed=11, x_dtype=torch.bfloat16)
    K = cw * Q
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    y = _run(bq, X.cuda())
    assert O.max_rel_err(y.float().cpu().numpy(), oracle_forward_t(Y, Z, A, None, X)) < TOL + 2 ** -8
    for pad in (16, 12):
        big = torch.zeros(M, K + pad, dtype=torch.bfloat16, device='cuda')
        big[:, :K] = X.cuda()
        view = big[:, :K]
        assert view.stride(0) == K + pad
        assert torch.equal(_run(bq, view), y)


def test_leading_dims_and_strides():
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, _, _ = synth_layer(2, 4, 4, 32, 32, 32, 1, seed=3)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    X = torch.randn(2, 3, 128, generator=torch.Generator().manual_seed(1))
    y = _run(bq, X.cuda())
    assert tuple(y.shape) == (2, 3, 128)
    ref = oracle_forward_t(Y, Z, A, None, X.reshape(6, 128)).reshape(2, 3, 128)
    assert O.max_rel_err(y.cpu().numpy(), ref) < TOL_FP32
    # X on the host is moved to the layer's device, as the reference does with X.to(device)
    y2 = _run(bq, X)
    assert y2.is_cuda and torch.equal(y2, y)
    # row-strided view
    big = torch.randn(6, 256, generator=torch.Generator().manual_seed(2)).cuda()
    view = big[:, :128]
    y3 = _run(bq, view)
    ref3 = oracle_forward_t(Y, Z, A, None, view.cpu())
    assert O.max_rel_err(y3.cpu().numpy(), ref3) < TOL_FP32
    assert _run(bq, torch.empty(0, 128).cuda()).shape == (0, 128)


def test_get_weight_gpu():
    for name in ('layer_0', 'layer_2', 'extend_3bit', 'fused_s123'):
        g = load_golden(name)
        bq = _module_from_golden(g)
        W = bq.get_weight(torch.float32).cpu().numpy()
        Wref = O.dense_weight(g['Y'], g['Z'], g['a'], g['b'], g['c'], g['d'])
        assert np.abs(W - Wref).max() <= 1e-5 * max(1.0, np.abs(Wref).max())
        Wb = bq.get_weight(torch.bfloat16)
        assert Wb.dtype == torch.bfloat16
        assert np.abs(Wb.float().cpu().numpy() - Wref).max() <= 2 ** -8 * np.abs(Wref).max()


@pytest.mark.parametrize('shape', DECODE_SHAPES + [(2, 3, 4, 9, 7, 5), (2, 2, 3, 33, 31, 40)])
def test_get_weight_all_geometries(shape):
    """Dense weight from the planes for padded, ragged, odd-width and two-rank-block patches, in every element type."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, P, Q, r = shape
    Y, Z, A, _, _ = synth_layer(bw, rw, cw, P, Q, r, 1, seed=21)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    a, b, c, d = O.split_coefficients(A.numpy())
    Wref = O.dense_weight(Y.numpy(), Z.numpy(), a, b, c, d)
    scale = max(1.0, np.abs(Wref).max())
    W = bq.get_weight(torch.float32)
    assert tuple(W.shape) == (rw * P, cw * Q)
    assert np.abs(W.cpu().numpy() - Wref).max() <= 1e-5 * scale
    for dt, eps in ((torch.bfloat16, 2 ** -8), (torch.float16, 2 ** -10)):
        Wd = bq.get_weight(dt)
        assert Wd.dtype == dt
        assert np.abs(Wd.float().cpu().numpy() - Wref).max() <= eps * scale


def test_decode_is_deterministic_and_workspace_reusable():
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, _, X = synth_layer(2, 32, 64, 32, 32, 32, 4, seed=9)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    xg = X.cuda()
    y0 = _run(bq, xg)
    for _ in range(5):
        assert torch.equal(_run(bq, xg), y0)


def test_linearity_full_size():
    """Size-independent property at a full configuration size (4096 x 14336, 2 bit layers):
    f(x1 + x2) = f(x1) + f(x2) and f(0) = 0, plus parity of a random output subset rebuilt by the oracle."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, P, Q, r = 2, 128, 448, 32, 32, 32
    gen = torch.Generator(device='cuda').manual_seed(4)
    Y = torch.rand(bw, rw, cw, P, r, generator=gen, device='cuda') > 0.5
    Z = torch.rand(bw, rw, cw, r, Q, generator=gen, device='cuda') > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=gen, device='cuda') * 0.02
    bq = BinaryQuadratic(Y, Z, A)
    x1 = torch.randn(1, cw * Q, generator=gen, device='cuda')
    x2 = torch.randn(1, cw * Q, generator=gen, device='cuda')
    y1, y2, y12 = _run(bq, x1), _run(bq, x2), _run(bq, x1 + x2)
    scale = y12.abs().max().item()
    assert (y12 - (y1 + y2)).abs().max().item() < 1e-4 * scale
    assert _run(bq, torch.zeros_like(x1)).abs().max().item() == 0.0
    # oracle on 3 row patches only (the rest of the layer does not influence them)
    for i in (0, 57, 127):
        a, b, c, d = O.split_coefficients(A[:, i:i + 1].cpu().numpy())
        ref = O.forward(Y[:, i:i + 1].cpu().numpy(), Z[:, i:i + 1].cpu().numpy(), a, b, c, d, x1.cpu().numpy())
        got = y1[:, i * P:(i + 1) * P].cpu().numpy()
        assert np.abs(got - ref).max() < TOL_FP32 * scale


@pytest.mark.parametrize('geom,M,dtype', [((2, 6, 5, 32, 32, 32), 1, torch.bfloat16),     # all bit layers per CTA
                                          ((3, 4, 40, 32, 32, 32), 1, torch.float32),     # preparation kernel
                                          ((2, 4, 6, 64, 64, 32), 5, torch.float16),
                                          ((2, 3, 9, 32, 32, 32), 16, torch.bfloat16)])
def test_fused_prologue_and_residual(geom, M, dtype):
    """bqq_forward_decode_fused: RMS normalisation or SwiGLU applied to x on the way in, residual added on the
    way out, against the fp32 oracle on the same (fp32) prologue arithmetic."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, P, Q, r = geom
    Y, Z, A, bias, _ = synth_layer(bw, rw, cw, P, Q, r, M, seed=41, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    g = torch.Generator().manual_seed(7)
    in_f, out_f = cw * Q, rw * P
    w = (1.0 + 0.1 * torch.randn(in_f, generator=g)).to(dtype)
    res = torch.randn(M, out_f, generator=g).to(dtype)
    tol = TOL if dtype == torch.float32 else TOL + 2 ** -8

    def oracle(H):
        return oracle_forward_t(Y, Z, A, bias, H)

    with torch.no_grad():
        # RMS normalisation + residual
        X = (3.0 * torch.randn(M, in_f, generator=g)).to(dtype)
        got = bq.forward_fused(X.cuda(), rms_weight=w.cuda(), eps=1e-5, residual=res.cuda())
        Xf = X.float()
        H = Xf * torch.rsqrt(Xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
        want = oracle(H) + res.float().numpy()
        assert O.max_rel_err(got.float().cpu().numpy(), want) < tol
        # SwiGLU, no residual
        GU = torch.randn(M, 2 * in_f, generator=g).to(dtype)
        got = bq.forward_fused(GU.cuda(), swiglu=True)
        H = torch.nn.functional.silu(GU.float()[:, :in_f]) * GU.float()[:, in_f:]
        assert O.max_rel_err(got.float().cpu().numpy(), oracle(H)) < tol
        # residual alone
        h = res.cuda().clone()
        X = torch.randn(M, in_f, generator=g).to(dtype)
        got = bq.forward_fused(X.cuda(), residual=h)
        assert O.max_rel_err(got.float().cpu().numpy(), oracle(X.float()) + res.float().numpy()) < tol
        # no fusion at all equals the plain forward bit for bit
        assert torch.equal(bq.forward_fused(X.cuda()), bq(X.cuda()))


@pytest.mark.parametrize('M', [1, 4])
@pytest.mark.parametrize('sign', [1.0, -1.0])
def test_u_at_its_bound(M, sign):
    """Every rank's u sits exactly on the bound its fixed-point scale is derived from (Z all ones, x of one
    sign, a and b of one sign), on the upper and on the lower edge: the digits must not wrap.  With narrow
    patches this happens by chance (a Z row of ones, 8 inputs of one sign)."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, P, Q, r = 2, 3, 9, 32, 8, 48
    g = torch.Generator().manual_seed(3)
    Y = torch.rand(bw, rw, cw, P, r, generator=g) > 0.5
    Z = torch.ones(bw, rw, cw, r, Q, dtype=torch.bool)
    A = torch.rand(bw, rw, cw, 4, generator=g) * 0.02 + 0.001
    A[..., :2] *= sign
    X = torch.rand(M, cw * Q, generator=g) + 0.1
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    with torch.no_grad():
        y = bq(X.cuda())
    ref = oracle_forward_t(Y, Z, A, None, X)
    assert O.max_rel_err(y.cpu().numpy(), ref) < TOL_FP32


def test_narrow_patch_regression():
    """Seeded case found by a random sweep (P=32, Q=8, r=48, 33 col patches): one rank of one patch exceeded
    the bound by the rounding of the x digits and its u digits wrapped (3.6e-2 error in one row)."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, P, Q, r, M = 2, 5, 33, 32, 8, 48, 8
    g = torch.Generator().manual_seed(106)
    Y = torch.rand(bw, rw, cw, P, r, generator=g) > 0.5
    Z = torch.rand(bw, rw, cw, r, Q, generator=g) > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=g) * 0.02
    X = torch.randn(M, cw * Q, generator=g)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    ref = oracle_forward_t(Y, Z, A, None, X)
    with torch.no_grad():
        assert O.max_rel_err(bq(X.cuda()).cpu().numpy(), ref) < TOL_FP32
        assert O.max_rel_err(bq(X[6:7].cuda()).cpu().numpy(), ref[6:7]) < TOL_FP32
