"""CPU: the oracle restatement against fixtures produced by the unmodified reference."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import bqq_oracle as O
from tests.helpers import LAYER_CASES, load_golden


@pytest.mark.parametrize('name', LAYER_CASES)
def test_forward_matches_reference(name):
    g = load_golden(name)
    y = O.forward(g['Y'], g['Z'], g['a'], g['b'], g['c'], g['d'], g['X'], g.get('bias'))
    assert O.max_rel_err(y, g['y_ref_fp32']) < 2e-6
    yf = O.forward_factored(g['Y'], g['Z'], g['a'], g['b'], g['c'], g['d'], g['X'], g.get('bias'))
    assert O.max_rel_err(yf, g['y_ref_fp32']) < 2e-6


@pytest.mark.parametrize('name', LAYER_CASES)
def test_dense_weight_matches_reference(name):
    g = load_golden(name)
    W = O.dense_weight(g['Y'], g['Z'], g['a'], g['b'], g['c'], g['d'])
    # sums of fp32 entries: compare against the magnitude that was summed (order-of-summation noise)
    assert np.abs(W.sum(1, dtype=np.float64) - g['W_rowsum']).max() <= 1e-6 * np.abs(W).sum(1).max()
    assert np.abs(W.sum(0, dtype=np.float64) - g['W_colsum']).max() <= 1e-6 * np.abs(W).sum(0).max()
    sub = W[:: max(1, W.shape[0] // 16), :: max(1, W.shape[1] // 16)]
    np.testing.assert_allclose(sub, g['W_sample'], rtol=1e-5, atol=1e-6)
    assert float(g['W_packed_maxdiff']) < 1e-5          # the reference's own packed == unpacked check


@pytest.mark.parametrize('name', LAYER_CASES)
def test_reference_u8_packing_bit_exact(name):
    g = load_golden(name)
    Yp, Zp, Ys, Zs = O.pack_u8_reference(g['Y'], g['Z'])
    assert (Yp == g['Y_packed']).all() and (Zp == g['Z_packed']).all()
    assert (Ys == g['Y_sum_i16']).all() and (Zs == g['Z_sum_i16']).all()


def test_big_endian_byte_layout():
    # element 0 of the rank axis is the MSB of byte 0; bits {0, 9} -> bytes [128, 64, 0, 0]
    Y = np.zeros((1, 1, 1, 1, 32), bool)
    Y[..., 0] = True
    Y[..., 9] = True
    Yp, _, _, _ = O.pack_u8_reference(Y, np.zeros((1, 1, 1, 32, 1), bool))
    assert Yp.reshape(-1).tolist() == [128, 64, 0, 0]


def test_popcount_golden():
    g = load_golden('popcount')
    assert (O.popcount_matmul_u8(g['Yp'], g['Zp']) == g['ref']).all()


@pytest.mark.parametrize('name', LAYER_CASES)
def test_plane_layout_round_trip(name):
    g = load_golden(name)
    bw, rw, cw, P, Q, r = g['dims']
    zp, yp, ys, zs = O.pack_planes_u32(g['Y'], g['Z'])
    Y2, Z2 = O.unpack_planes_u32(zp, yp, bw, rw, cw, P, Q, r)
    assert (Y2 == g['Y']).all() and (Z2 == g['Z']).all()
    assert (ys.astype(np.int16) == g['Y_sum_i16'][..., 0]).all()
    assert (zs.astype(np.int16) == g['Z_sum_i16'][..., 0, :]).all()


def test_extension_bits_through_patch_dicts():
    g = load_golden('extend_3bit')
    # a 2-bit build of the same patch list keeps only bit_idx 0 and 1
    assert np.array_equal(g['A'][:2], g['A_2bit'])
    assert g['dims'][0] == 3


def test_config1_outputs_and_input_digests():
    """The 4096x4096 configuration: inputs are regenerated from seed 0 and must hash
    to what the reference run saw; the oracle must reproduce the reference output."""
    g = load_golden('config1_4096')
    bw, rw, cw, P, r, Q = (int(v) for v in g['shape'])
    gen = torch.Generator().manual_seed(0)
    Y = torch.rand(bw, rw, cw, P, r, generator=gen) > 0.5
    Z = torch.rand(bw, rw, cw, r, Q, generator=gen) > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=gen) * 0.02
    X = torch.randn(1, cw * Q, generator=gen)
    assert hashlib.sha256(np.packbits(Y.numpy())).hexdigest() == str(g['Y_sha256'])
    assert hashlib.sha256(np.packbits(Z.numpy())).hexdigest() == str(g['Z_sha256'])
    assert hashlib.sha256(A.numpy().tobytes()).hexdigest() == str(g['A_sha256'])
    np.testing.assert_array_equal(X.numpy(), g['X'])
    a, b, c, d = O.split_coefficients(A.numpy())
    y = O.forward_factored(Y.numpy(), Z.numpy(), a, b, c, d, X.numpy())
    assert O.max_rel_err(y, g['y_ref_fp64']) < 1e-9
    assert O.max_rel_err(g['y_ref_fp32'], g['y_ref_fp64']) < 1e-5
    assert O.algorithmic_bytes(bw, rw, cw, P, Q, r) == 8388608 + 458752


@pytest.mark.parametrize('name', LAYER_CASES)
def test_c_restatement_matches_reference(name):
    from oracle import c_oracle
    g = load_golden(name)
    y = c_oracle.forward(g['Y'], g['Z'], g['a'], g['b'], g['c'], g['d'], g['X'], g.get('bias'))
    assert O.max_rel_err(y.reshape(g['y_ref_fp32'].shape), g['y_ref_fp32']) < 2e-6
    y2 = c_oracle.forward(g['Y'], g['Z'], g['a'], g['b'], g['c'], g['d'], g['X'], g.get('bias'),
                          use_double=True, nthreads=2)
    assert O.max_rel_err(y2.reshape(g['y_ref_fp32'].shape), g['y_ref_fp32']) < 2e-6
