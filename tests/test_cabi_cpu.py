"""CPU: the C-ABI library loads, exports every declared symbol, and its host-side
code (sizes, argument checks, host packer) agrees with the oracle.  No GPU work."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import bqq_oracle as O
from tests.helpers import LAYER_CASES, load_golden

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def cabi():
    from bqq_b200 import _cabi
    return _cabi


def test_exports_match_header(cabi):
    hdr = open(os.path.join(ROOT, 'include', 'bqq_b200.h')).read()
    hdr = re.sub(r'/\*.*?\*/', '', hdr, flags=re.S)
    declared = set(re.findall(r'\b(bqq_[a-z0-9_]+)\s*\(', hdr))
    assert declared, 'no declarations parsed'
    for name in declared:
        assert hasattr(cabi.lib, name), f'{name} declared in the header but not exported'
    assert declared == set(cabi.EXPORTS)
    assert cabi.lib.bqq_abi_version() == 2


def test_strerror_and_codes(cabi):
    assert cabi.strerror(0) == 'ok'
    for code in range(-9, 0):
        assert 'unknown bqq error' not in cabi.strerror(code)
    assert 'unknown bqq error' in cabi.strerror(-99)


@pytest.mark.parametrize('shape', [(2, 128, 128, 32, 32, 32), (2, 4, 4, 64, 64, 32), (3, 2, 8, 32, 32, 16),
                                   (2, 2, 2, 32, 32, 12), (3, 3, 5, 64, 64, 64), (1, 1, 3, 16, 48, 20)])
def test_sizes(cabi, shape):
    bw, rw, cw, P, Q, r = shape
    d = cabi.dims(*shape)
    g = O.plane_geometry(bw, rw, cw, P, Q, r)
    assert cabi.lib.bqq_zplane_words(d) == rw * g['NS'] * g['RT'] * g['QT'] * 32 * 4
    assert cabi.lib.bqq_yplane_words(d) == rw * g['NS'] * g['PT'] * g['RT'] * 32 * 4
    assert cabi.lib.bqq_algorithmic_bytes(d) == O.algorithmic_bytes(bw, rw, cw, P, Q, r)


def test_bad_arguments_rejected_without_gpu(cabi):
    lib = cabi.lib
    bad = cabi.dims(0, 1, 1, 32, 32, 32)
    assert lib.bqq_zplane_words(bad) == 0
    big = cabi.dims(1, 1, 1, 256, 32, 32)
    assert lib.bqq_zplane_words(big) == 0
    ok = cabi.dims(1, 1, 1, 32, 32, 32)
    buf = np.zeros(4096, np.uint8)
    p = buf.ctypes.data
    assert lib.bqq_pack_planes(None, p, ok, p, p, None, None, None) == -1          # NULL
    assert lib.bqq_pack_planes(p, p, bad, p, p, None, None, None) == -2            # bad shape
    assert lib.bqq_pack_planes(p, p, big, p, p, None, None, None) == -3            # unsupported
    layer = cabi.BqqLayer(ok, p, p, p, p, p, p, None, 0, 0)
    assert lib.bqq_forward_decode(layer, None, 0, 1, 32, p, 0, 32, None, 0, None) == -1
    assert lib.bqq_forward_decode(layer, p, 0, 0, 32, p, 0, 32, None, 0, None) == -2
    assert lib.bqq_forward_decode(layer, p, 0, 17, 32, p, 0, 32, None, 0, None) == -3
    assert lib.bqq_forward_decode(layer, p, 9, 1, 32, p, 0, 32, None, 0, None) == -6
    assert lib.bqq_forward_decode(layer, p, 0, 1, 16, p, 0, 32, None, 0, None) == -2   # ldx < in_features
    mis = cabi.BqqLayer(ok, p + 4, p, p, p, p, p, None, 0, 0)
    assert lib.bqq_forward_decode(mis, p, 0, 1, 32, p, 0, 32, None, 0, None) == -4
    assert lib.bqq_forward_prefill(layer, p, 0, 64, 32, p, 0, 32, None, 0, None) == -5  # workspace
    baddt = cabi.BqqLayer(ok, p, p, p, p, p, p, None, 5, 0)
    assert lib.bqq_forward_decode(baddt, p, 0, 1, 32, p, 0, 32, None, 0, None) == -6    # coefficient dtype


@pytest.mark.parametrize('name', LAYER_CASES)
def test_host_packer_bit_exact(cabi, name):
    g = load_golden(name)
    bw, rw, cw, P, Q, r = g['dims']
    d = cabi.dims(bw, rw, cw, P, Q, r)
    Y = np.ascontiguousarray(g['Y'].astype(np.uint8))
    Z = np.ascontiguousarray(g['Z'].astype(np.uint8))
    zp = np.empty(cabi.lib.bqq_zplane_words(d), np.uint32)
    yp = np.empty(cabi.lib.bqq_yplane_words(d), np.uint32)
    ys = np.empty(bw * rw * cw * P, np.uint8)
    zs = np.empty(bw * rw * cw * Q, np.uint8)
    rc = cabi.lib.bqq_pack_planes_host(Y.ctypes.data, Z.ctypes.data, d, zp.ctypes.data, yp.ctypes.data,
                                       ys.ctypes.data, zs.ctypes.data)
    assert rc == 0
    zo, yo, yso, zso = O.pack_planes_u32(g['Y'], g['Z'])
    assert np.array_equal(zp, zo.reshape(-1)) and np.array_equal(yp, yo.reshape(-1))
    assert np.array_equal(ys, yso.reshape(-1)) and np.array_equal(zs, zso.reshape(-1))
    assert np.array_equal(ys.reshape(bw, rw, cw, P), g['Y_sum_i16'][..., 0])
    Y2 = np.empty_like(Y)
    Z2 = np.empty_like(Z)
    assert cabi.lib.bqq_unpack_planes_host(zp.ctypes.data, yp.ctypes.data, d, Y2.ctypes.data, Z2.ctypes.data) == 0
    assert np.array_equal(Y2, Y) and np.array_equal(Z2, Z)


def test_host_packer_ragged_geometry(cabi):
    rng = np.random.default_rng(3)
    for shape in [(1, 1, 3, 16, 48, 20), (3, 2, 5, 96, 40, 33), (2, 1, 1, 128, 128, 64), (5, 2, 3, 32, 32, 7)]:
        bw, rw, cw, P, Q, r = shape
        Y = rng.integers(0, 2, (bw, rw, cw, P, r)).astype(np.uint8)
        Z = rng.integers(0, 2, (bw, rw, cw, r, Q)).astype(np.uint8)
        d = cabi.dims(*shape)
        zp = np.empty(cabi.lib.bqq_zplane_words(d), np.uint32)
        yp = np.empty(cabi.lib.bqq_yplane_words(d), np.uint32)
        assert cabi.lib.bqq_pack_planes_host(Y.ctypes.data, Z.ctypes.data, d, zp.ctypes.data, yp.ctypes.data,
                                             None, None) == 0
        zo, yo, _, _ = O.pack_planes_u32(Y, Z)
        assert np.array_equal(zp, zo.reshape(-1)) and np.array_equal(yp, yo.reshape(-1))


def test_module_api_surface_on_cpu():
    """Constructor, attributes, state_dict layout and pickling work without a GPU;
    forward on a CPU module fails loudly (no fallback)."""
    import io
    import torch
    import bqq_b200
    from bqq_b200.bqq_modules import BinaryQuadratic
    bqq_b200.install()
    torch.manual_seed(0)
    Y = (torch.rand(2, 3, 4, 32, 16) > 0.5).float()
    Z = (torch.rand(2, 3, 4, 16, 32) > 0.5).float()
    A = torch.randn(2, 3, 4, 4)
    bq = BinaryQuadratic(Y, Z, A, bias=torch.randn(96))
    sd = bq.state_dict()
    assert list(sd.keys()) == ['a', 'b', 'c', 'd', 'bias', 'Y', 'Z']
    assert sd['a'].shape == (2, 3, 4, 1, 1) and sd['d'].shape == (3, 4, 1, 1)
    assert sd['Y'].dtype == torch.bool and sd['Z'].shape == (2, 3, 4, 16, 32)
    assert torch.allclose(sd['d'][..., 0, 0], A[..., 3].sum(0))
    assert (bq.bit_width, bq.row_width, bq.col_width, bq.y_row, bq.inter_dimension, bq.z_col) == (2, 3, 4, 32, 16, 32)
    buf = io.BytesIO()
    torch.save(bq, buf)
    assert b'bqq_modules' in buf.getvalue()
    buf.seek(0)
    bq2 = torch.load(buf, weights_only=False)
    assert type(bq2).__name__ == 'BinaryQuadratic' and torch.equal(bq2.Y, bq.Y)
    a, b, c, d = (sd[k].numpy() for k in 'abcd')
    W = O.dense_weight(sd['Y'].numpy(), sd['Z'].numpy(), a, b, c, d)
    assert np.abs(bq.get_weight().detach().numpy() - W).max() < 1e-5
    with torch.no_grad(), pytest.raises(RuntimeError, match='no CPU fallback'):
        bq(torch.randn(1, 128))
    with pytest.raises(RuntimeError, match='inference-only'):
        bq(torch.randn(1, 128))


def _patch_list(bw_total, rw, cw, P, Q, r, seed):
    """Patch dicts as the reference's consolidated files hold them, in a shuffled order."""
    import torch
    g = torch.Generator().manual_seed(seed)
    patches = []
    for b in range(bw_total):
        for i in range(rw):
            for j in range(cw):
                patches.append({'patch_row': i, 'patch_col': j, 'bit_idx': b,
                                'coeff': torch.randn(4, generator=g) * 0.02,
                                'mat1': (torch.rand(P, r, generator=g) > 0.5).float(),
                                'mat2': (torch.rand(r, Q, generator=g) > 0.5).float()})
    order = torch.randperm(len(patches), generator=g).tolist()
    return [patches[k] for k in order]


@pytest.mark.parametrize('geom', [(3, 3, 5, 32, 32, 32), (2, 2, 3, 64, 48, 20)])
def test_patches_straight_into_planes(geom):
    """PlaneBinaryQuadratic.from_patches (bqq_pack_patch_host, one patch at a time) builds the planes and
    coefficients that get_matrices + the whole-layer packer build, including the skipping of
    bit_idx >= bit_width and last-entry-wins for repeated patches."""
    import torch
    from bqq_b200.bqq_modules import PlaneBinaryQuadratic, get_matrices
    bw_total, rw, cw, P, Q, r = geom
    bit_width = bw_total - 1                                  # the last bit layer of the file is ignored
    patches = _patch_list(bw_total, rw, cw, P, Q, r, seed=3)
    dup = dict(patches[0])
    dup['mat1'] = 1.0 - dup['mat1']
    dup['coeff'] = dup['coeff'] * 2
    patches.append(dup)                                       # repeated (bit, row, col): the later entry wins
    layer = PlaneBinaryQuadratic.from_patches(patches, bit_width)
    A, Y, Z = get_matrices(patches, bit_width)
    zp, yp, _, _ = O.pack_planes_u32(Y.numpy() > 0.5, Z.numpy() > 0.5)
    assert np.array_equal(layer.zplanes.numpy().view(np.uint32), zp.reshape(-1))
    assert np.array_equal(layer.yplanes.numpy().view(np.uint32), yp.reshape(-1))
    a, b, c, d = O.split_coefficients(A.numpy())
    for name, want in zip('abcd', (a, b, c, d)):
        assert np.array_equal(getattr(layer, name).detach().numpy(), want), name
    assert (layer.bit_width, layer.row_width, layer.col_width, layer.y_row, layer.z_col, layer.inter_dimension) == \
        (bit_width, rw, cw, P, Q, r)
    sd = layer.state_dict()
    assert list(sd) == ['a', 'b', 'c', 'd', 'zplanes', 'yplanes']
