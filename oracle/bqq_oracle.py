"""CPU oracle for the BinaryQuadratic linear forward (TEST INFRASTRUCTURE ONLY).

This file is a plain numpy restatement of the reference algorithm.  It is the
checker that the CUDA path is compared against; it is never the product path.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
may import it.

Parity status: PINNED.  The functions here are checked (tests/test_oracle.py)
against fixtures under tests/golden/ that were produced by running the
unmodified reference classes (BinaryQuadratic / PackedBinaryQuadratic) on the
seeded generators the reference's own self-tests use.

Reference citations use paths inside the reference project:
  src/  = neural_network_compression/src/
  lm/   = neural_network_compression/lm/

Tensor conventions (src/bqq_modules.py:21-32):
  Y  bool [bw, rw, cw, P, r]     binary left factors
  Z  bool [bw, rw, cw, r, Q]     binary right factors
  a,b,c   [bw, rw, cw, 1, 1]     per (bit, patch) scalars
  d       [rw, cw, 1, 1]         per patch offset (sum over bits of A[...,3])
  out feature o = i*P + p, in feature n = j*Q + q  (src/bqq_modules.py:42)
"""
from __future__ import annotations

import numpy as np


# ---------------------------------------------------------------------------
# constructor semantics
# ---------------------------------------------------------------------------

def split_coefficients(A):
    """A [bw,rw,cw,4] -> a,b,c [bw,rw,cw,1,1], d [rw,cw,1,1].

    Follows BinaryQuadratic.__init__ (src/bqq_modules.py:28-31): the first
    three coefficient columns stay per bit layer, the fourth is summed over
    the bit-layer axis.
    """
    A = np.asarray(A)
    a = A[..., 0][..., None, None].copy()
    b = A[..., 1][..., None, None].copy()
    c = A[..., 2][..., None, None].copy()
    d = A[..., 3][..., None, None].sum(axis=0)
    return a, b, c, d


def threshold(M):
    """Binary factors are stored as `M > 0.5` (src/bqq_modules.py:26-27)."""
    return np.asarray(M) > 0.5


# ---------------------------------------------------------------------------
# dense weight and forward (the reference's definition of the result)
# ---------------------------------------------------------------------------

def dense_weight(Y, Z, a, b, c, d, dtype=np.float32):
    """W [rw*P, cw*Q] exactly as get_weight builds it (src/bqq_modules.py:48-55).

    W_core = Y @ Z per (bit, patch); W = a*W_core + b*rowsum(Y) + c*colsum(Z),
    summed over bits, plus d, then patches are laid out row-major.
    """
    Yf = np.asarray(Y).astype(dtype)
    Zf = np.asarray(Z).astype(dtype)
    core = np.matmul(Yf, Zf)                                  # [bw,rw,cw,P,Q]
    ysum = Yf.sum(axis=-1, keepdims=True)                     # [bw,rw,cw,P,1]
    zsum = Zf.sum(axis=-2, keepdims=True)                     # [bw,rw,cw,1,Q]
    W = (np.asarray(a, dtype) * core + np.asarray(b, dtype) * ysum
         + np.asarray(c, dtype) * zsum)
    W = W.sum(axis=0) + np.asarray(d, dtype)                  # [rw,cw,P,Q]
    rw, cw, P, Q = W.shape
    return np.ascontiguousarray(W.transpose(0, 2, 1, 3)).reshape(rw * P, cw * Q)


def forward(Y, Z, a, b, c, d, X, bias=None, dtype=np.float32):
    """y = X @ W.T (+ bias), evaluated in `dtype` (src/bqq_modules.py:34-46).

    X may have any leading dims; the last one is in_features.
    """
    W = dense_weight(Y, Z, a, b, c, d, dtype)
    X = np.asarray(X, dtype)
    y = X.reshape(-1, X.shape[-1]) @ W.T
    if bias is not None:
        y = y + np.asarray(bias, dtype)
    return y.reshape(*X.shape[:-1], W.shape[0])


def forward_factored(Y, Z, a, b, c, d, X, bias=None, dtype=np.float64):
    """Same result without building W: the fused identity the reference's
    decode kernel uses (src/bqq_cuda.cu:82-84,134-156).

    Per (patch i,j, bit): xsum = sum_q x[j,q]; t_k = sum_q Z[k,q] x[j,q];
    y[i,p] += sum_k Y[p,k] (a t_k + b xsum) + c sum_k t_k, and once per patch
    y[i,p] += d xsum.  Used to cross-check dense_weight/forward.
    """
    Yf = np.asarray(Y).astype(dtype)
    Zf = np.asarray(Z).astype(dtype)
    bw, rw, cw, P, r = Yf.shape
    Q = Zf.shape[-1]
    X = np.asarray(X, dtype)
    lead = X.shape[:-1]
    x = X.reshape(-1, cw, Q)                                  # [M,cw,Q]
    xsum = x.sum(axis=-1)                                     # [M,cw]
    t = np.einsum('bijkq,mjq->mbijk', Zf, x)                  # [M,bw,rw,cw,r]
    a_ = np.asarray(a, dtype)[..., 0, 0]
    b_ = np.asarray(b, dtype)[..., 0, 0]
    c_ = np.asarray(c, dtype)[..., 0, 0]
    d_ = np.asarray(d, dtype)[..., 0, 0]
    u = a_[None, ..., None] * t + (b_[None] * xsum[:, None, None, :])[..., None]
    y = np.einsum('bijpk,mbijk->mip', Yf, u)                  # [M,rw,P]
    y += np.einsum('bij,mbij->mi', c_, t.sum(axis=-1))[..., None]
    y += np.einsum('ij,mj->mi', d_, xsum)[..., None]
    y = y.reshape(-1, rw * P)
    if bias is not None:
        y = y + np.asarray(bias, dtype)
    return y.reshape(*lead, rw * P)


def max_rel_err(y, y_ref):
    """max|y - y_ref| / max|y_ref|: the reference's own error metric
    (src/bqq_triton_kernel.py:595)."""
    y = np.asarray(y, np.float64)
    y_ref = np.asarray(y_ref, np.float64)
    return float(np.abs(y - y_ref).max() / max(np.abs(y_ref).max(), 1e-30))


# ---------------------------------------------------------------------------
# patch list -> dense tensors
# ---------------------------------------------------------------------------

def get_matrices(patch_list, bit_width):
    """Scatter patch dicts {patch_row, patch_col, coeff[4], mat1[P,r],
    mat2[r,Q], bit_idx} into A, Y, Z; entries with bit_idx >= bit_width are
    dropped; patch geometry comes from the first entry
    (src/bqq_modules.py:485-507)."""
    rw = max(int(p['patch_row']) for p in patch_list) + 1
    cw = max(int(p['patch_col']) for p in patch_list) + 1
    P, r = np.asarray(patch_list[0]['mat1']).shape
    Q = np.asarray(patch_list[0]['mat2']).shape[1]
    A = np.zeros((bit_width, rw, cw, 4), np.asarray(patch_list[0]['coeff']).dtype)
    Y = np.zeros((bit_width, rw, cw, P, r), np.asarray(patch_list[0]['mat1']).dtype)
    Z = np.zeros((bit_width, rw, cw, r, Q), np.asarray(patch_list[0]['mat1']).dtype)
    for p in patch_list:
        k = int(p['bit_idx'])
        if k >= bit_width:
            continue
        i, j = int(p['patch_row']), int(p['patch_col'])
        A[k, i, j] = np.asarray(p['coeff'])
        Y[k, i, j] = np.asarray(p['mat1'])
        Z[k, i, j] = np.asarray(p['mat2'])
    return A, Y, Z


# ---------------------------------------------------------------------------
# the reference's uint8 packing (PackedBinaryQuadratic)
# ---------------------------------------------------------------------------

def pack_u8_reference(Y, Z):
    """Big-endian uint8 packs along the rank axis, Z transposed first, plus
    int16 sums (src/bqq_modules.py:99-148).

    Returns Y_packed [bw,rw,cw,P,ceil(r/8)], Z_packed [bw,rw,cw,Q,ceil(r/8)],
    Y_sum [bw,rw,cw,P,1] int16, Z_sum [bw,rw,cw,1,Q] int16.
    """
    Y = np.asarray(Y).astype(bool)
    Z = np.asarray(Z).astype(bool)
    Yp = np.packbits(Y.astype(np.uint8), axis=-1)
    Zp = np.packbits(np.swapaxes(Z, -1, -2).astype(np.uint8), axis=-1)
    Ys = Y.sum(axis=-1, keepdims=True).astype(np.int16)
    Zs = Z.sum(axis=-2, keepdims=True).astype(np.int16)
    return Yp, Zp, Ys, Zs


def unpack_u8_reference(Y_packed, Z_packed, r):
    """Inverse of pack_u8_reference (src/bqq_modules.py:159-169): element 0 is
    the MSB of byte 0, trailing pad bits dropped; Z comes back as [.., r, Q]."""
    Y = np.unpackbits(np.asarray(Y_packed, np.uint8), axis=-1)[..., :r].astype(bool)
    Zt = np.unpackbits(np.asarray(Z_packed, np.uint8), axis=-1)[..., :r].astype(bool)
    return Y, np.swapaxes(Zt, -1, -2)


def popcount_matmul_u8(Yp, Zp):
    """W_core[b,i,j] = sum_k popcount(Yp[b,i,k] & Zp[b,j,k]) on uint8 packs,
    the exact check of src/bqq_triton_kernel.py:511-530."""
    Yp = np.asarray(Yp, np.uint8)
    Zp = np.asarray(Zp, np.uint8)
    anded = Yp[:, :, None, :] & Zp[:, None, :, :]
    return np.unpackbits(anded, axis=-1).sum(axis=-1).astype(np.int32)


# ---------------------------------------------------------------------------
# 32-bit bit-plane layout of this library (layout oracle for the GPU packer)
# ---------------------------------------------------------------------------

GROUP = 4  # patch-bits interleaved per 128-bit lane load


def plane_geometry(bw, rw, cw, P, Q, r):
    """Sizes of the packed planes.

    A "patch-bit" is one (col patch j, bit b) pair of a row patch i, numbered
    n = j*bw + b.  GROUP consecutive patch-bits form a super-group.
    """
    QW = (Q + 31) // 32           # words per Z row (bits over q)
    RW = (r + 31) // 32           # words per Y row (bits over k)
    RP = ((r + 31) // 32) * 32    # Z rows, padded to a lane multiple
    PP = ((P + 31) // 32) * 32    # Y rows, padded to a lane multiple
    NPB = cw * bw
    NS = (NPB + GROUP - 1) // GROUP
    return dict(QW=QW, RW=RW, RP=RP, PP=PP, NPB=NPB, NS=NS)


def pack_planes_u32(Y, Z):
    """Bit planes as the GPU packer must produce them.

    Zp uint32 [rw, NS, QW, RP, 4]: word = bits q%32 (LSB first) of Z row k,
        word index qw = q//32, for the 4 patch-bits of super-group s.
    Yp uint32 [rw, NS, RW, PP, 4]: word = bits k%32 (LSB first) of Y row p.
    ysum uint8 [bw,rw,cw,P], zsum uint8 [bw,rw,cw,Q]: row sums of Y over k and
        column sums of Z over k (equal the reference's Y_sum_i16 / Z_sum_i16).
    Padding rows/bits/patch-bits are zero.
    """
    Y = np.asarray(Y).astype(bool)
    Z = np.asarray(Z).astype(bool)
    bw, rw, cw, P, r = Y.shape
    Q = Z.shape[-1]
    g = plane_geometry(bw, rw, cw, P, Q, r)
    QW, RW, RP, PP, NS = g['QW'], g['RW'], g['RP'], g['PP'], g['NS']

    def to_words(bits, nwords):
        # bits [..., L] -> uint32 [..., nwords], LSB-first
        L = bits.shape[-1]
        padded = np.zeros(bits.shape[:-1] + (nwords * 32,), np.uint8)
        padded[..., :L] = bits
        by = np.packbits(padded, axis=-1, bitorder='little')
        return np.ascontiguousarray(by).view('<u4').reshape(bits.shape[:-1] + (nwords,))

    Zw = to_words(Z, QW)                      # [bw,rw,cw,r,QW]
    Yw = to_words(Y, RW)                      # [bw,rw,cw,P,RW]
    Zp = np.zeros((rw, NS * GROUP, QW, RP), np.uint32)
    Yp = np.zeros((rw, NS * GROUP, RW, PP), np.uint32)
    # n = j*bw + b
    Zn = Zw.transpose(1, 2, 0, 4, 3).reshape(rw, cw * bw, QW, r)
    Yn = Yw.transpose(1, 2, 0, 4, 3).reshape(rw, cw * bw, RW, P)
    Zp[:, :cw * bw, :, :r] = Zn
    Yp[:, :cw * bw, :, :P] = Yn
    Zp = Zp.reshape(rw, NS, GROUP, QW, RP).transpose(0, 1, 3, 4, 2)
    Yp = Yp.reshape(rw, NS, GROUP, RW, PP).transpose(0, 1, 3, 4, 2)
    ysum = Y.sum(axis=-1).astype(np.uint8)
    zsum = Z.sum(axis=-2).astype(np.uint8)
    return np.ascontiguousarray(Zp), np.ascontiguousarray(Yp), ysum, zsum


def unpack_planes_u32(Zp, Yp, bw, rw, cw, P, Q, r):
    """Inverse of pack_planes_u32 -> bool Y [bw,rw,cw,P,r], Z [bw,rw,cw,r,Q]."""
    g = plane_geometry(bw, rw, cw, P, Q, r)
    QW, RW, RP, PP, NS = g['QW'], g['RW'], g['RP'], g['PP'], g['NS']
    Zp = np.asarray(Zp, np.uint32).reshape(rw, NS, QW, RP, GROUP)
    Yp = np.asarray(Yp, np.uint32).reshape(rw, NS, RW, PP, GROUP)
    Zn = Zp.transpose(0, 1, 4, 2, 3).reshape(rw, NS * GROUP, QW, RP)[:, :cw * bw, :, :r]
    Yn = Yp.transpose(0, 1, 4, 2, 3).reshape(rw, NS * GROUP, RW, PP)[:, :cw * bw, :, :P]

    def to_bits(words, L):
        # words [..., nwords] -> bits [..., L]
        by = np.ascontiguousarray(words.astype('<u4')).view(np.uint8)
        bits = np.unpackbits(by, axis=-1, bitorder='little')
        return bits[..., :L].astype(bool)

    # Zn [rw, n, QW, r] -> [rw, cw, bw, r, QW]
    Zw = Zn.reshape(rw, cw, bw, QW, r).transpose(2, 0, 1, 4, 3)
    Yw = Yn.reshape(rw, cw, bw, RW, P).transpose(2, 0, 1, 4, 3)
    Z = to_bits(np.ascontiguousarray(Zw), Q)
    Y = to_bits(np.ascontiguousarray(Yw), r)
    return Y, Z


def pack_coefficients(a, b, c, d):
    """float32 [rw, NS*4, 4]: (a, b, c, d if bit==0 else 0) per patch-bit
    n = j*bw + b; padding patch-bits are all-zero."""
    a = np.asarray(a, np.float32)[..., 0, 0]
    b = np.asarray(b, np.float32)[..., 0, 0]
    c = np.asarray(c, np.float32)[..., 0, 0]
    d = np.asarray(d, np.float32)[..., 0, 0]
    bw, rw, cw = a.shape
    NS = (cw * bw + GROUP - 1) // GROUP
    out = np.zeros((rw, NS * GROUP, 4), np.float32)
    co = np.zeros((rw, cw, bw, 4), np.float32)
    co[..., 0] = a.transpose(1, 2, 0)
    co[..., 1] = b.transpose(1, 2, 0)
    co[..., 2] = c.transpose(1, 2, 0)
    co[:, :, 0, 3] = d
    out[:, :cw * bw] = co.reshape(rw, cw * bw, 4)
    return out


def algorithmic_bytes(bw, rw, cw, P, Q, r):
    """Packed information per forward: one bit per binary entry plus fp32
    a,b,c per (bit, patch) and d per patch."""
    bits = bw * rw * cw * (P * r + r * Q)
    return bits // 8 + 4 * rw * cw * (3 * bw + 1)
