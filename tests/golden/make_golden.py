"""Generate the golden fixtures in this directory from the UNMODIFIED reference.

Run once, in a container that has the reference checkout, as

    python tests/golden/make_golden.py /path/to/reference

It imports BinaryQuadratic / PackedBinaryQuadratic from the reference's
neural_network_compression/src/bqq_modules.py, re-runs the seeded generators of
the reference's own self-tests and stores inputs and reference outputs as
small .npz files.  The test-suite reads only the .npz files, never the
reference checkout.

Cases (reference file:line of the generator each one re-runs):
  fused_s42 / fused_s123 / fused_s7   src/bqq_triton_kernel.py:578-582 (+ :541-553)
  fused_bias_s99                      src/bqq_triton_kernel.py:611-613
  layer_0 / layer_1 / layer_2         lm/scripts/test_packed_layer.py:15-23,128-134
  popcount                            src/bqq_triton_kernel.py:511-530
  extend_3bit                         get_matrices with bit_idx 0..2 (src/bqq_modules.py:485-507)
  config1_4096                        4096x4096, 2 bit layers, P=Q=r=32, seed 0 (outputs + input digests only)
"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def ref_import(ref_root):
    sys.path.insert(0, os.path.join(ref_root, 'neural_network_compression', 'src'))
    import bqq_modules  # noqa
    bqq_modules.PackedBinaryQuadratic.use_packed_kernel = False  # no GPU/Triton here
    return bqq_modules


def new_like_triton_test(bm, bit, row, col, yr, zc, inter, with_bias):
    """Same draw order as the reference helper: Y, Z (randint), A (randn), bias."""
    import torch.nn as nn
    Y = torch.randint(0, 2, (bit, row, col, yr, inter)).bool()
    Z = torch.randint(0, 2, (bit, row, col, inter, zc)).bool()
    A = torch.randn(bit, row, col, 4)
    bq = bm.BinaryQuadratic.__new__(bm.BinaryQuadratic)
    nn.Module.__init__(bq)
    bq.bit_width, bq.row_width, bq.col_width = bit, row, col
    bq.y_row, bq.inter_dimension, bq.z_col = yr, inter, zc
    bq.register_buffer('Y', Y)
    bq.register_buffer('Z', Z)
    bq.a = nn.Parameter(A[..., 0].unsqueeze(-1).unsqueeze(-1))
    bq.b = nn.Parameter(A[..., 1].unsqueeze(-1).unsqueeze(-1))
    bq.c = nn.Parameter(A[..., 2].unsqueeze(-1).unsqueeze(-1))
    bq.d = nn.Parameter(A[..., 3].unsqueeze(-1).unsqueeze(-1).sum(dim=0))
    bq.bias = nn.Parameter(torch.randn(row * yr)) if with_bias else None
    return bq


def dump(name, bm, bq, X, extra=None):
    """Store bits (reference uint8 packing), coefficients, X and reference outputs."""
    pk = bm.PackedBinaryQuadratic.from_unpacked(bq)
    with torch.no_grad():
        y32 = bq(X.float())
        y_native = bq(X)
        W = bq.get_weight(torch.float32)
        Wp = pk.get_weight(torch.float32)
    rec = dict(
        shape=np.array([bq.bit_width, bq.row_width, bq.col_width, bq.y_row,
                        bq.inter_dimension, bq.z_col], np.int64),
        Y_packed=pk.Y_packed.numpy(), Z_packed=pk.Z_packed.numpy(),
        Y_sum_i16=pk.Y_sum_i16.numpy(), Z_sum_i16=pk.Z_sum_i16.numpy(),
        a=bq.a.detach().numpy(), b=bq.b.detach().numpy(),
        c=bq.c.detach().numpy(), d=bq.d.detach().numpy(),
        X=X.float().numpy(), x_is_bf16=np.array(X.dtype == torch.bfloat16),
        y_ref_fp32=y32.numpy(), y_ref_native=y_native.float().numpy(),
        W_rowsum=W.sum(1).numpy(), W_colsum=W.sum(0).numpy(),
        W_sample=W[:: max(1, W.shape[0] // 16), :: max(1, W.shape[1] // 16)].numpy(),
        W_packed_maxdiff=np.array((W - Wp).abs().max().item()),
    )
    if bq.bias is not None:
        rec['bias'] = bq.bias.detach().numpy()
    if extra:
        rec.update(extra)
    np.savez_compressed(os.path.join(HERE, name + '.npz'), **rec)
    print(name, {k: getattr(v, 'shape', None) for k, v in rec.items() if k in ('X', 'y_ref_fp32')})


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else '/root/reference'
    bm = ref_import(ref_root)

    # --- fused kernel self-test generators --------------------------------
    for seed, (bit, row, col, yr, zc, inter, bshape) in [
        (42, (4, 8, 8, 32, 32, 32, (2,))),
        (123, (2, 4, 4, 16, 16, 16, (4, 8))),
        (7, (3, 6, 6, 32, 32, 32, (1,))),
    ]:
        torch.manual_seed(seed)
        bq = new_like_triton_test(bm, bit, row, col, yr, zc, inter, False)
        X = torch.randn(*bshape, col * zc, dtype=torch.float32)
        dump(f'fused_s{seed}', bm, bq, X)

    torch.manual_seed(99)
    bq = new_like_triton_test(bm, 4, 6, 6, 32, 32, 32, True)
    X = torch.randn(3, 6 * 32, dtype=torch.float32)
    dump('fused_bias_s99', bm, bq, X)

    # --- packed-vs-unpacked layer test generators ---------------------------
    torch.manual_seed(0)
    for idx, (bw, rw, cw, yr, inter, zc) in enumerate([
        (2, 4, 4, 64, 32, 64), (3, 2, 8, 32, 16, 32), (2, 2, 2, 32, 12, 32)]):
        Y = (torch.rand(bw, rw, cw, yr, inter) > 0.5)
        Z = (torch.rand(bw, rw, cw, inter, zc) > 0.5)
        A = torch.randn(bw, rw, cw, 4)
        bq = bm.BinaryQuadratic(Y.float(), Z.float(), A)
        X = torch.randn(2, 8, cw * zc, dtype=torch.bfloat16)
        dump(f'layer_{idx}', bm, bq, X)

    # --- exact AND+popcount check ------------------------------------------
    rng = np.random.default_rng(0)
    B, y_row, z_col, inter = 6, 32, 32, 64
    k8 = (inter + 7) // 8
    Yp = rng.integers(0, 256, (B, y_row, k8), dtype=np.uint8)
    Zp = rng.integers(0, 256, (B, z_col, k8), dtype=np.uint8)
    ref = np.zeros((B, y_row, z_col), np.int32)
    for b in range(B):
        for i in range(y_row):
            for j in range(z_col):
                for k in range(k8):
                    ref[b, i, j] += bin(int(Yp[b, i, k]) & int(Zp[b, j, k])).count('1')
    np.savez_compressed(os.path.join(HERE, 'popcount.npz'), Yp=Yp, Zp=Zp, ref=ref)

    # --- bit-depth extension through patch dicts ----------------------------
    g = torch.Generator().manual_seed(5)
    rw, cw, P, r, Q = 3, 2, 64, 64, 64
    patches = []
    for k in range(3):
        for i in range(rw):
            for j in range(cw):
                scale = 0.02 if k < 2 else 0.005
                patches.append(dict(
                    patch_row=i, patch_col=j, bit_idx=k,
                    coeff=torch.randn(4, generator=g) * scale,
                    mat1=(torch.rand(P, r, generator=g) > 0.5).float(),
                    mat2=(torch.rand(r, Q, generator=g) > 0.5).float()))
    # out-of-range bit index must be ignored by a 3-bit build
    patches.append(dict(patch_row=0, patch_col=0, bit_idx=3, coeff=torch.ones(4),
                        mat1=torch.ones(P, r), mat2=torch.ones(r, Q)))
    A, Y, Z = bm.get_matrices(patches, bit_width=3)
    bq = bm.BinaryQuadratic(Y, Z, A)
    X = torch.randn(5, cw * Q, generator=g).to(torch.bfloat16)
    A2, _, _ = bm.get_matrices(patches, bit_width=2)
    dump('extend_3bit', bm, bq, X, extra=dict(A=A.numpy(), A_2bit=A2.numpy()))

    # --- config 1: too large to store inputs; keep digests + outputs --------
    g = torch.Generator().manual_seed(0)
    bw, rw, cw, P, r, Q = 2, 128, 128, 32, 32, 32
    Y = torch.rand(bw, rw, cw, P, r, generator=g) > 0.5
    Z = torch.rand(bw, rw, cw, r, Q, generator=g) > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=g) * 0.02
    X = torch.randn(1, cw * Q, generator=g)
    bq = bm.BinaryQuadratic(Y.float(), Z.float(), A)
    with torch.no_grad():
        y = bq(X)
        y64 = bq.double()(X.double())
    np.savez_compressed(
        os.path.join(HERE, 'config1_4096.npz'),
        shape=np.array([bw, rw, cw, P, r, Q], np.int64),
        y_ref_fp32=y.numpy(), y_ref_fp64=y64.numpy(), X=X.numpy(),
        Y_sha256=np.array(hashlib.sha256(np.packbits(Y.numpy())).hexdigest()),
        Z_sha256=np.array(hashlib.sha256(np.packbits(Z.numpy())).hexdigest()),
        A_sha256=np.array(hashlib.sha256(A.numpy().tobytes()).hexdigest()))
    print('config1_4096 done')


if __name__ == '__main__':
    main()
