"""GPU parity at the full sizes of the benchmark configurations.

The layers are generated on the GPU (seeded), run through the module, and compared with the CPU
oracle on sampled output-row patches: a row patch of the output depends only on its own slice of
Y, Z and the coefficients, so the oracle rebuilds exactly those slices (seconds), for every row
of X.  Tolerance: max|y - y_ref| / max|y_ref| <= 1e-3 (contract), 1e-4 where the output is fp32
and only the compute error remains; 16-bit outputs add their own rounding (2^-8 bf16, 2^-10 fp16)."""
import numpy as np
import pytest
import torch

from oracle import bqq_oracle as O

pytestmark = pytest.mark.gpu
TOL, TOL_FP32 = 1e-3, 1e-4


def _layer(bw, rw, cw, P, Q, r, seed, ext_bit_scale=None):
    from bqq_b200.bqq_modules import BinaryQuadratic
    gen = torch.Generator(device='cuda').manual_seed(seed)
    Y = torch.rand(bw, rw, cw, P, r, generator=gen, device='cuda') > 0.5
    Z = torch.rand(bw, rw, cw, r, Q, generator=gen, device='cuda') > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=gen, device='cuda') * 0.02
    if ext_bit_scale is not None:                      # the bit layer added by a depth extension is smaller
        A[-1] *= ext_bit_scale / 0.02
    return BinaryQuadratic(Y, Z, A), Y, Z, A, gen


def _oracle_rows(Y, Z, A, i, X32):
    a, b, c, d = O.split_coefficients(A[:, i:i + 1].cpu().numpy())
    return O.forward(Y[:, i:i + 1].cpu().numpy(), Z[:, i:i + 1].cpu().numpy(), a, b, c, d, X32, dtype=np.float64)


def _check_sampled(y, Y, Z, A, X, rows, tol, what):
    """y [M, out] against the oracle on the row patches `rows`; the error is relative to the
    largest |y| over the whole output, the reference's own metric."""
    P = Y.shape[3]
    X32 = X.float().cpu().numpy()
    y32 = y.float()
    scale = y32.abs().max().item()
    assert np.isfinite(scale) and scale > 0
    worst = 0.0
    for i in rows:
        ref = _oracle_rows(Y, Z, A, i, X32)
        got = y32[:, i * P:(i + 1) * P].cpu().numpy()
        worst = max(worst, float(np.abs(got - ref).max()))
    assert worst < tol * scale, (what, worst / scale)


def _forward_fp32_out(bq, X):
    """The forward with 16-bit activations and fp32 outputs, straight through the C ABI (the module
    returns X's dtype): what remains is the compute error alone."""
    from bqq_b200 import _cabi
    from bqq_b200.bqq_modules import _DTYPE_CODE, _workspace
    st = bq._ensure_packed()
    M, out_f = X.shape[0], bq.row_width * bq.y_row
    y = torch.empty(M, out_f, dtype=torch.float32, device='cuda')
    layer = bq._layer(st)
    stream = torch.cuda.current_stream().cuda_stream
    if M <= _cabi.DECODE_MAX_M:
        ws = _workspace(X.device, 'decode', _cabi.lib.bqq_decode_workspace_bytes(st.dims, M))
        fn = _cabi.lib.bqq_forward_decode
    else:
        ws = _workspace(X.device, 'prefill', _cabi.lib.bqq_prefill_workspace_bytes(st.dims, M))
        fn = _cabi.lib.bqq_forward_prefill
    _cabi.check(fn(layer, X.data_ptr(), _DTYPE_CODE[X.dtype], M, X.stride(0), y.data_ptr(), _cabi.F32, y.stride(0),
                   ws.data_ptr(), ws.numel(), stream), 'forward')
    torch.cuda.synchronize()
    return y


def _run(bq, X):
    with torch.no_grad():
        y = bq(X)
    torch.cuda.synchronize()
    return y


# ---- decode sweep: every shape x number of bit layers x batch of the sweep ---------------------
SWEEP_SHAPES = [(2048, 2048), (2048, 6144), (6144, 2048), (4096, 14336)]      # (out, in)


@pytest.mark.parametrize('out_f,in_f', SWEEP_SHAPES)
@pytest.mark.parametrize('bw', [2, 3, 4])
def test_decode_sweep_shapes_full_size(out_f, in_f, bw):
    rw, cw = out_f // 32, in_f // 32
    bq, Y, Z, A, gen = _layer(bw, rw, cw, 32, 32, 32, seed=out_f + in_f + bw)
    rows = sorted({0, rw // 3, rw - 1})
    for M in (1, 4, 16):
        X = torch.randn(M, in_f, generator=gen, device='cuda').to(torch.bfloat16)
        y = _run(bq, X)
        assert y.dtype == torch.bfloat16 and tuple(y.shape) == (M, out_f)
        _check_sampled(y, Y, Z, A, X, rows, TOL + 2 ** -8, (out_f, in_f, bw, M, 'bf16'))
        _check_sampled(_forward_fp32_out(bq, X), Y, Z, A, X, rows, TOL_FP32, (out_f, in_f, bw, M, 'bf16->f32'))


# ---- prefill: 2048 tokens x 4096 on a 4096 x 4096 layer with 2 bit layers ----------------------
def test_prefill_2048_tokens_full_size():
    bq, Y, Z, A, gen = _layer(2, 128, 128, 32, 32, 32, seed=3)
    X = torch.randn(2048, 4096, generator=gen, device='cuda').to(torch.bfloat16)
    # row patches on both sides of the 256-column tile borders of the GEMM, first and last tile
    rows = (0, 7, 8, 63, 64, 100, 127)
    y = _run(bq, X)
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (2048, 4096)
    _check_sampled(y, Y, Z, A, X, rows, TOL + 2 ** -8, 'bf16')
    _check_sampled(_forward_fp32_out(bq, X), Y, Z, A, X, rows, TOL, 'bf16->f32')
    # linearity at full size: f(2x) = 2 f(x) exactly (power-of-two scaling commutes with every rounding)
    y2 = _run(bq, X * 2)
    assert torch.equal(y2.float(), y.float() * 2)


# ---- bit-depth-extended large layers: 2 + 1 bit layers, P = Q = r = 64 --------------------------
@pytest.mark.parametrize('out_f,in_f', [(8192, 28672), (28672, 8192)])
def test_extended_large_layer_full_size(out_f, in_f):
    rw, cw = out_f // 64, in_f // 64
    bq, Y, Z, A, gen = _layer(3, rw, cw, 64, 64, 64, seed=out_f // 64, ext_bit_scale=0.005)
    rows = (0, rw // 2 + 1, rw - 1)
    # the sampled row patches also go through the patch-dict route of a depth extension
    # (bit_idx 0..2 per patch, src/bqq_modules.py:485-507), restated by the oracle's get_matrices
    i = rows[1]
    patches = [dict(patch_row=0, patch_col=j, bit_idx=k, coeff=A[k, i, j].cpu().numpy(),
                    mat1=Y[k, i, j].cpu().numpy().astype(np.float32), mat2=Z[k, i, j].cpu().numpy().astype(np.float32))
               for k in range(3) for j in range(cw)]
    A1, Y1, Z1 = O.get_matrices(patches, 3)
    for M in (1, 32):
        X = torch.randn(M, in_f, generator=gen, device='cuda').to(torch.bfloat16)
        y = _run(bq, X)
        assert tuple(y.shape) == (M, out_f)
        _check_sampled(y, Y, Z, A, X, rows, TOL + 2 ** -8, (out_f, in_f, M, 'bf16'))
        y32 = _forward_fp32_out(bq, X)
        _check_sampled(y32, Y, Z, A, X, rows, TOL_FP32 if M == 1 else TOL, (out_f, in_f, M, 'bf16->f32'))
        a, b, c, d = O.split_coefficients(A1)
        ref = O.forward(O.threshold(Y1), O.threshold(Z1), a, b, c, d, X.float().cpu().numpy(), dtype=np.float64)
        got = y32[:, i * 64:(i + 1) * 64].cpu().numpy()
        assert np.abs(got - ref).max() < (TOL_FP32 if M == 1 else TOL) * y32.abs().max().item()
