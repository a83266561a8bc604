"""GPU: drop-in behaviour of the module (pickles, construction without __init__,
in-place parameter updates, dtype casts, error behaviour)."""
import io

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import bqq_oracle as O
from tests.helpers import oracle_forward_t, synth_layer

pytestmark = pytest.mark.gpu


def _fwd(m, X):
    with torch.no_grad():
        return m(X)


def test_pickle_round_trip_and_install():
    import bqq_b200
    from bqq_b200.bqq_modules import BinaryQuadratic
    bqq_b200.install()
    Y, Z, A, bias, X = synth_layer(2, 4, 4, 32, 32, 32, 3, seed=1, bias=True)
    model = nn.Sequential(BinaryQuadratic(Y.float(), Z.float(), A, bias=bias)).cuda()
    y0 = _fwd(model, X.cuda())
    buf = io.BytesIO()
    torch.save(model, buf)                      # whole-module pickle, as the reference saves models
    assert b'bqq_modules' in buf.getvalue() and b'_bqq_state' not in buf.getvalue()
    buf.seek(0)
    model2 = torch.load(buf, weights_only=False)
    assert torch.equal(_fwd(model2, X.cuda()), y0)
    # state_dict route
    m3 = BinaryQuadratic(torch.zeros_like(Y).float(), torch.zeros_like(Z).float(), torch.zeros_like(A),
                         bias=torch.zeros_like(bias)).cuda()
    m3.load_state_dict(model[0].state_dict())
    assert torch.equal(_fwd(m3, X.cuda()), y0)


def test_construct_without_init():
    """The reference benchmark builds layers with __new__ and fills attributes by hand."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, gs = 2, 4, 6, 32
    g = torch.Generator().manual_seed(2)
    Y = torch.randint(0, 2, (bw, rw, cw, gs, gs), generator=g).bool()
    Z = torch.randint(0, 2, (bw, rw, cw, gs, gs), generator=g).bool()
    A = torch.randn(bw, rw, cw, 4, generator=g) * 0.01
    bq = BinaryQuadratic.__new__(BinaryQuadratic)
    nn.Module.__init__(bq)
    bq.bit_width, bq.row_width, bq.col_width = bw, rw, cw
    bq.y_row, bq.inter_dimension, bq.z_col = gs, gs, gs
    bq.register_buffer('Y', Y)
    bq.register_buffer('Z', Z)
    bq.a = nn.Parameter(A[..., 0].unsqueeze(-1).unsqueeze(-1))
    bq.b = nn.Parameter(A[..., 1].unsqueeze(-1).unsqueeze(-1))
    bq.c = nn.Parameter(A[..., 2].unsqueeze(-1).unsqueeze(-1))
    bq.d = nn.Parameter(A[..., 3].unsqueeze(-1).unsqueeze(-1).sum(dim=0))
    bq.bias = None
    bq = bq.cuda()
    X = torch.randn(1, cw * gs, generator=g)
    assert O.max_rel_err(_fwd(bq, X.cuda()).cpu().numpy(), oracle_forward_t(Y, Z, A, None, X)) < 1e-4


def test_in_place_coefficient_update_is_seen():
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, _, X = synth_layer(2, 4, 4, 32, 32, 32, 2, seed=3)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    y0 = _fwd(bq, X.cuda())
    with torch.no_grad():
        bq.a.data[...] = bq.a.data * 2.0        # scale refinement rewrites .data in place
        bq.d.data.add_(0.5)
    A2 = A.clone()
    A2[..., 0] *= 2.0
    A2[0, ..., 3] += 0.5
    y1 = _fwd(bq, X.cuda())
    assert not torch.equal(y0, y1)
    assert O.max_rel_err(y1.cpu().numpy(), oracle_forward_t(Y, Z, A2, None, X)) < 1e-4


def test_bfloat16_cast_and_device_moves():
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, X = synth_layer(2, 4, 4, 64, 64, 32, 4, seed=4, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias)
    bq = bq.cuda().bfloat16()                   # model.bfloat16() casts the coefficient parameters
    assert bq.a.dtype == torch.bfloat16 and bq.Y.dtype == torch.bool
    Ab = A.to(torch.bfloat16).float()
    Ab[0, ..., 3] = A[..., 3].sum(0).to(torch.bfloat16).float()
    Ab[1:, ..., 3] = 0
    Xb = X.to(torch.bfloat16)
    ref = oracle_forward_t(Y, Z, Ab, bias.to(torch.bfloat16).float(), Xb)
    y = _fwd(bq, Xb.cuda())
    assert O.max_rel_err(y.float().cpu().numpy(), ref) < 1e-3 + 2 ** -8


def test_errors():
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, _, X = synth_layer(1, 2, 2, 32, 32, 32, 1, seed=6)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    with pytest.raises(RuntimeError, match='inference-only'):
        bq(X.cuda())
    with torch.no_grad():
        with pytest.raises(RuntimeError, match='last dim'):
            bq(torch.randn(1, 65).cuda())
        with pytest.raises(RuntimeError, match='unsupported activation dtype'):
            bq(X.long().cuda())


def test_sharded_rows_equal_unsharded():
    """Column-parallel shards (output-row patches) reproduce the full layer bit for bit: the
    decode kernel's work split never depends on the number of row patches."""
    from bqq_b200.bqq_modules import BinaryQuadratic, shard_rows
    Y, Z, A, bias, X = synth_layer(2, 8, 6, 32, 32, 32, 4, seed=8, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    full = _fwd(bq, X.cuda())
    for world in (2, 4, 8):
        parts = [_fwd(shard_rows(bq, r, world), X.cuda()) for r in range(world)]
        assert torch.equal(torch.cat(parts, dim=-1), full)
    # a tall layer takes one CTA per bit layer, its shards one CTA for all bit layers: still identical bits
    from bqq_b200 import _cabi
    Y, Z, A, bias, X = synth_layer(2, 512, 4, 32, 32, 32, 1, seed=9, bias=False)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    assert _cabi.lib.bqq_decode_launches(bq._dims(), 1) == 2
    assert _cabi.lib.bqq_decode_launches(shard_rows(bq, 0, 2)._dims(), 1) == 1
    full = _fwd(bq, X.cuda())
    for world in (2, 4):
        parts = [_fwd(shard_rows(bq, r, world), X.cuda()) for r in range(world)]
        assert torch.equal(torch.cat(parts, dim=-1), full)


@pytest.mark.parametrize('M,dtype', [(1, torch.bfloat16), (3, torch.float32), (40, torch.float16)])
def test_forward_host_equals_device_forward(M, dtype):
    """bqq_forward_host (host buffers in and out, one C call) gives the values of the device forward,
    for the decode path (M <= 16) and the prefill path, also with a strided host input."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, _ = synth_layer(2, 6, 5, 32, 32, 32, 1, seed=21, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    g = torch.Generator().manual_seed(5)
    wide = torch.randn(M, 5 * 32 + 8, generator=g).to(dtype).pin_memory()
    xh = wide[:, :5 * 32]                                   # row stride larger than in_features
    want = _fwd(bq, xh.cuda())
    out = torch.empty(M, 6 * 32, dtype=dtype).pin_memory()
    with torch.no_grad():
        got = bq.forward_host(xh, out)
        torch.cuda.current_stream().synchronize()
        assert got is out and torch.equal(out.cuda(), want)
        got2 = bq.forward_host(xh)                          # allocates a pinned output
        torch.cuda.current_stream().synchronize()
        assert got2.is_pinned() and torch.equal(got2.cuda(), want)
        with pytest.raises(RuntimeError, match='CPU tensor'):
            bq.forward_host(xh.cuda())


def test_decode_launch_count():
    """Short single-chunk layers at batch 1 take one kernel, everything else two."""
    from bqq_b200 import _cabi
    lib = _cabi.lib
    assert lib.bqq_decode_launches(_cabi.dims(2, 64, 64, 32, 32, 32), 1) == 1
    assert lib.bqq_decode_launches(_cabi.dims(2, 64, 64, 32, 32, 32), 4) == 2
    assert lib.bqq_decode_launches(_cabi.dims(2, 128, 448, 32, 32, 32), 1) == 2
    assert lib.bqq_decode_launches(_cabi.dims(2, 64, 64, 64, 64, 32), 1) == 2
    assert lib.bqq_decode_launches(_cabi.dims(2, 896, 128, 32, 32, 32), 1) == 2      # tall: one CTA per bit layer
    assert lib.bqq_decode_launches(_cabi.dims(2, 64, 64, 32, 32, 32), 17) < 0


def test_bind_host_reads_current_contents():
    """A host binding is one C call per run and sees in-place changes of its input buffer."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, X = synth_layer(2, 4, 4, 32, 32, 32, 1, seed=22, bias=False)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    xh = X.to(torch.bfloat16).pin_memory()
    with torch.no_grad():
        run, out = bq.bind_host(xh)
        for scale in (1.0, -0.5):
            xh.copy_((X * scale).to(torch.bfloat16))
            assert run() is out
            torch.cuda.current_stream().synchronize()
            assert torch.equal(out.cuda(), _fwd(bq, xh.cuda()))


def test_forward_host_with_pageable_buffers():
    """Host buffers that are not pinned take the copy-engine route and give the same values."""
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, bias, X = synth_layer(2, 4, 40, 32, 32, 32, 2, seed=23, bias=False)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    xh = X.to(torch.bfloat16)
    out = torch.empty(2, 4 * 32, dtype=torch.bfloat16)
    with torch.no_grad():
        bq.forward_host(xh, out)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(out.cuda(), _fwd(bq, xh.cuda()))


def test_plane_layer_from_patches_equals_dense_route():
    """Patch files packed patch by patch (no dense Y / Z) give the forward and the weight of
    get_matrices + BinaryQuadratic bit for bit."""
    from bqq_b200.bqq_modules import BinaryQuadratic, PlaneBinaryQuadratic, get_matrices
    from tests.test_cabi_cpu import _patch_list
    patches = _patch_list(3, 4, 6, 32, 32, 32, seed=9)
    A, Y, Z = get_matrices(patches, 3)
    dense = BinaryQuadratic(Y, Z, A).cuda()
    planes = PlaneBinaryQuadratic.from_patches(patches, 3).cuda()
    g = torch.Generator().manual_seed(4)
    for M, dt in ((1, torch.bfloat16), (7, torch.float32), (33, torch.float16)):
        X = torch.randn(M, 6 * 32, generator=g).to(dt).cuda()
        assert torch.equal(_fwd(planes, X), _fwd(dense, X))
    assert torch.equal(planes.get_weight(torch.float32), dense.get_weight(torch.float32))
    Yb, Zb = planes.unpack_planes()
    assert torch.equal(Yb, dense.Y) and torch.equal(Zb, dense.Z)
    buf = io.BytesIO()
    torch.save(planes, buf)
    buf.seek(0)
    again = torch.load(buf, weights_only=False)
    X = torch.randn(2, 6 * 32, generator=g).cuda()
    assert torch.equal(_fwd(again, X), _fwd(dense, X))


def test_reference_made_pickles_run_on_the_gpu():
    """Whole-module pickles written by the reference's own builder and classes
    (tests/golden/make_pickles.py: replace_linear_with_bqq + torch.save, pack_existing_model) load onto
    this package's classes and reproduce the reference's stored fp32 outputs."""
    import os

    import bqq_b200
    from tests.helpers import GOLDEN
    bqq_b200.install()
    io = np.load(os.path.join(GOLDEN, 'ref_model_io.npz'))
    X = torch.from_numpy(io['X'])
    for fname, cls in (('ref_model_bq.pth', bqq_b200.BinaryQuadratic),
                       ('ref_model_bq-packed.pth', bqq_b200.PackedBinaryQuadratic)):
        model = torch.load(os.path.join(GOLDEN, fname), weights_only=False)
        assert type(model.fc1) is cls and type(model.fc2) is cls
        model = model.cuda()
        y = _fwd(model, X.cuda())
        assert O.max_rel_err(y.cpu().numpy(), io['y_ref_fp32']) < 1e-4, fname
        W = model.fc1.get_weight(torch.float32)
        assert np.abs(W.cpu().numpy() - io['fc1_weight']).max() < 1e-6


@pytest.mark.parametrize('geom,lead', [((2, 4, 4, 32, 32, 32), (1,)), ((2, 2, 2, 32, 32, 12), (3,)),
                                       ((3, 2, 8, 32, 32, 16), (2, 20))])
def test_extension_call_signature(geom, lead):
    """bqq_cuda_ext._get_ext().bqq_forward(Y_packed, Z_packed, X, a, b, c, d, bias): the call the
    reference's packed layer makes (src/bqq_modules.py:217-230; src/bqq_cuda.cu:289-297)."""
    from bqq_b200 import bqq_cuda_ext
    from bqq_b200.bqq_modules import BinaryQuadratic, PackedBinaryQuadratic
    Y, Z, A, bias, _ = synth_layer(*geom, 1, seed=21, bias=True)
    pk = PackedBinaryQuadratic.from_unpacked(BinaryQuadratic(Y.float(), Z.float(), A, bias=bias)).cuda()
    g = torch.Generator().manual_seed(5)
    X = torch.randn(*lead, geom[2] * geom[4], generator=g)
    ext = bqq_cuda_ext._get_ext()
    y = ext.bqq_forward(pk.Y_packed, pk.Z_packed, X.cuda(), pk.a, pk.b, pk.c, pk.d, pk.bias)
    assert tuple(y.shape) == (*lead, geom[1] * geom[3]) and y.dtype == torch.float32
    ref = oracle_forward_t(Y, Z, A, bias, X.reshape(-1, X.shape[-1])).reshape(y.shape)
    tol = 1e-4 if X.numel() // X.shape[-1] <= 16 else 1e-3
    assert O.max_rel_err(y.cpu().numpy(), ref) < tol
    # "no bias" is an empty tensor in the reference's call; coefficients are read on every call
    y0 = bqq_cuda_ext.bqq_forward(pk.Y_packed, pk.Z_packed, X.cuda(), pk.a, pk.b, pk.c, pk.d,
                                  torch.empty(0, device='cuda'))
    ref0 = oracle_forward_t(Y, Z, A, None, X.reshape(-1, X.shape[-1])).reshape(y.shape)
    assert O.max_rel_err(y0.cpu().numpy(), ref0) < tol
    y2 = ext.bqq_forward(pk.Y_packed, pk.Z_packed, X.cuda(), pk.a * 2, pk.b * 2, pk.c * 2, pk.d * 2, None)
    assert O.max_rel_err(y2.cpu().numpy(), 2 * ref0) < tol
    assert len(ext._engines) >= 1


def test_fp64_activations_go_through_fp32():
    from bqq_b200.bqq_modules import BinaryQuadratic
    Y, Z, A, _, X = synth_layer(2, 4, 4, 32, 32, 32, 3, seed=13)
    bq = BinaryQuadratic(Y.float(), Z.float(), A).cuda()
    y = _fwd(bq, X.double().cuda())
    assert y.dtype == torch.float64
    assert O.max_rel_err(y.cpu().numpy(), oracle_forward_t(Y, Z, A, None, X)) < 1e-4
    with pytest.raises(RuntimeError, match='floating point'):
        _fwd(bq, torch.zeros(1, 128, dtype=torch.int32, device='cuda'))
