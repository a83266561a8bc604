"""GPU: packer / unpacker / coefficient records through the C ABI, bit-exact
against the numpy layout oracle and the reference's uint8 packs."""
import numpy as np
import pytest
import torch

from oracle import bqq_oracle as O
from tests.helpers import LAYER_CASES, load_golden

pytestmark = pytest.mark.gpu


def _module_from_golden(g, device='cuda', coef_dtype=torch.float32):
    from bqq_b200.bqq_modules import BinaryQuadratic
    bw, rw, cw, P, Q, r = g['dims']
    A = np.zeros((bw, rw, cw, 4), np.float32)
    A[..., 0], A[..., 1], A[..., 2] = g['a'][..., 0, 0], g['b'][..., 0, 0], g['c'][..., 0, 0]
    A[0, ..., 3] = g['d'][..., 0, 0]
    bias = torch.from_numpy(g['bias']) if 'bias' in g else None
    bq = BinaryQuadratic(torch.from_numpy(g['Y']).float(), torch.from_numpy(g['Z']).float(),
                         torch.from_numpy(A), bias=bias)
    return bq.to(device)


@pytest.mark.parametrize('name', LAYER_CASES)
def test_planes_bit_exact(name):
    g = load_golden(name)
    bq = _module_from_golden(g)
    st = bq._ensure_packed()
    zo, yo, yso, zso = O.pack_planes_u32(g['Y'], g['Z'])
    assert np.array_equal(st.zplanes.cpu().numpy().view(np.uint32), zo.reshape(-1))
    assert np.array_equal(st.yplanes.cpu().numpy().view(np.uint32), yo.reshape(-1))
    assert np.array_equal(st.ysum.cpu().numpy(), yso.reshape(-1))
    assert np.array_equal(st.zsum.cpu().numpy(), zso.reshape(-1))
    # row sums equal what the reference stores as Y_sum_i16 / Z_sum_i16
    assert np.array_equal(st.ysum.cpu().numpy().reshape(g['Y_sum_i16'].shape[:-1]), g['Y_sum_i16'][..., 0])
    Y2, Z2 = bq.unpack_planes()
    assert np.array_equal(Y2.cpu().numpy(), g['Y']) and np.array_equal(Z2.cpu().numpy(), g['Z'])


@pytest.mark.parametrize('name', ['layer_0', 'layer_2', 'fused_s123', 'extend_3bit'])
def test_reference_u8_checkpoint_repack(name):
    """Planes built from the reference's PackedBinaryQuadratic buffers equal planes built from bools."""
    from bqq_b200.bqq_modules import PackedBinaryQuadratic
    g = load_golden(name)
    bq = _module_from_golden(g)
    st = bq._ensure_packed()
    pk = PackedBinaryQuadratic(
        torch.from_numpy(g['Y_packed']), torch.from_numpy(g['Z_packed']),
        torch.from_numpy(g['a']), torch.from_numpy(g['b']), torch.from_numpy(g['c']), torch.from_numpy(g['d']),
        torch.from_numpy(g['Y_sum_i16']), torch.from_numpy(g['Z_sum_i16']),
        g['dims'][5], g['dims'][3], g['dims'][4]).cuda()
    st2 = pk._ensure_packed()
    assert torch.equal(st.zplanes, st2.zplanes) and torch.equal(st.yplanes, st2.yplanes)
    assert torch.equal(st.ysum, st2.ysum) and torch.equal(st.zsum, st2.zsum)
    # our from_unpacked reproduces the reference's big-endian bytes
    pk2 = PackedBinaryQuadratic.from_unpacked(bq)
    assert np.array_equal(pk2.Y_packed.cpu().numpy(), g['Y_packed'])
    assert np.array_equal(pk2.Z_packed.cpu().numpy(), g['Z_packed'])
    assert np.array_equal(pk2.Y_sum_i16.cpu().numpy(), g['Y_sum_i16'])


def test_ragged_geometry_round_trip():
    from bqq_b200.bqq_modules import BinaryQuadratic
    gen = torch.Generator().manual_seed(11)
    for (bw, rw, cw, P, Q, r) in [(1, 1, 3, 16, 48, 20), (3, 2, 5, 96, 40, 33), (2, 1, 1, 128, 128, 64),
                                  (5, 2, 3, 32, 32, 7)]:
        Y = torch.rand(bw, rw, cw, P, r, generator=gen) > 0.5
        Z = torch.rand(bw, rw, cw, r, Q, generator=gen) > 0.5
        bq = BinaryQuadratic(Y.float(), Z.float(), torch.randn(bw, rw, cw, 4, generator=gen)).cuda()
        st = bq._ensure_packed()
        zo, yo, _, _ = O.pack_planes_u32(Y.numpy(), Z.numpy())
        assert np.array_equal(st.zplanes.cpu().numpy().view(np.uint32), zo.reshape(-1))
        assert np.array_equal(st.yplanes.cpu().numpy().view(np.uint32), yo.reshape(-1))
        Y2, Z2 = bq.unpack_planes()
        assert torch.equal(Y2.cpu(), Y) and torch.equal(Z2.cpu(), Z)
