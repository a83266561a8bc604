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
#
# Patches are padded to multiples of 32 in P, Q and r (PT, QT, RT blocks of 32).
# For one row patch i the patch-bits are ordered bit layer first: super-group
# s = b*JG + jg holds the 4 col patches j = 4*jg + sub (JG = ceil(cw/4)); the 4
# words of a super-group are adjacent so that one 128-bit load fetches them.
#
# Inside a 32x32 block a word belongs to a lane = 4*g + t (g = 0..7, t = 0..3)
# and holds a 4-row x 8-column fragment arranged for the int8 tensor-core
# operand that the decode kernel builds with byte masks:
#   Z word bit 8*e + 4*qh + rr  =  Z[k = 32*rt + 4*g + rr][q = 32*qt + 16*qh + 4*t + e]
#   Y word bit 8*e + 4*kh + rr  =  Y[p = 32*pt + g + 8*rr][k = 32*rt + 16*kh + 4*t + e]
# Word order: Z [rw][NS][RT][QT][32 lanes][4 sub], Y [rw][NS][PT][RT][32][4].

GROUP = 4  # col patches interleaved per 128-bit lane load


def plane_geometry(bw, rw, cw, P, Q, r):
    PT, QT, RT = (P + 31) // 32, (Q + 31) // 32, (r + 31) // 32
    JG = (cw + GROUP - 1) // GROUP
    return dict(PT=PT, QT=QT, RT=RT, JG=JG, NS=bw * JG)


_BITW = (1 << (8 * np.arange(4)[:, None, None] + 4 * np.arange(2)[None, :, None]
               + np.arange(4)[None, None, :])).astype(np.uint64)      # [e][half][rr]


def pack_planes_u32(Y, Z):
    """Bit planes as the GPU packer must produce them (see the layout note above).

    Returns Zp uint32 [rw,NS,RT,QT,32,4], Yp uint32 [rw,NS,PT,RT,32,4],
    ysum uint8 [bw,rw,cw,P] (row sums of Y over k) and zsum uint8 [bw,rw,cw,Q]
    (column sums of Z over k; the reference's Y_sum_i16 / Z_sum_i16).
    """
    Y = np.asarray(Y).astype(bool)
    Z = np.asarray(Z).astype(bool)
    bw, rw, cw, P, r = Y.shape
    Q = Z.shape[-1]
    g = plane_geometry(bw, rw, cw, P, Q, r)
    PT, QT, RT, JG = g['PT'], g['QT'], g['RT'], g['JG']
    Zf = np.zeros((bw, rw, JG * GROUP, RT * 32, QT * 32), np.uint64)
    Yf = np.zeros((bw, rw, JG * GROUP, PT * 32, RT * 32), np.uint64)
    Zf[:, :, :cw, :r, :Q] = Z
    Yf[:, :, :cw, :P, :r] = Y
    # Z rows (ranks) = 32*blk + 4*g + rr ; Y rows = 32*blk + 8*rr + g ; cols = 32*blk + 16*half + 4*t + e
    Zf = Zf.reshape(bw, rw, JG, GROUP, RT, 8, 4, QT, 2, 4, 4)     # b i jg sub rt g rr qt qh t e
    Zf = Zf.transpose(1, 0, 2, 4, 7, 5, 9, 3, 10, 8, 6)           # i b jg rt qt g t sub e qh rr
    Zp = (Zf * _BITW).sum(axis=(-1, -2, -3)).astype(np.uint32)
    Yf = Yf.reshape(bw, rw, JG, GROUP, PT, 4, 8, RT, 2, 4, 4)     # b i jg sub pt rr g rt kh t e
    Yf = Yf.transpose(1, 0, 2, 4, 7, 6, 9, 3, 10, 8, 5)           # i b jg pt rt g t sub e kh rr
    Yp = (Yf * _BITW).sum(axis=(-1, -2, -3)).astype(np.uint32)
    Zp = np.ascontiguousarray(Zp.reshape(rw, bw * JG, RT, QT, 32, GROUP))
    Yp = np.ascontiguousarray(Yp.reshape(rw, bw * JG, PT, RT, 32, GROUP))
    return Zp, Yp, Y.sum(axis=-1).astype(np.uint8), Z.sum(axis=-2).astype(np.uint8)


def unpack_planes_u32(Zp, Yp, bw, rw, cw, P, Q, r):
    """Inverse of pack_planes_u32 -> bool Y [bw,rw,cw,P,r], Z [bw,rw,cw,r,Q]."""
    g = plane_geometry(bw, rw, cw, P, Q, r)
    PT, QT, RT, JG = g['PT'], g['QT'], g['RT'], g['JG']
    shifts = (8 * np.arange(4)[:, None, None] + 4 * np.arange(2)[None, :, None]
              + np.arange(4)[None, None, :]).astype(np.uint32)    # [e][half][rr]
    Zw = np.asarray(Zp, np.uint32).reshape(rw, bw, JG, RT, QT, 8, 4, GROUP)
    Zb = (Zw[..., None, None, None] >> shifts) & 1                # i b jg rt qt g t sub e qh rr
    Zb = Zb.transpose(1, 0, 2, 7, 3, 5, 10, 4, 9, 6, 8)           # b i jg sub rt g rr qt qh t e
    Z = Zb.reshape(bw, rw, JG * GROUP, RT * 32, QT * 32)[:, :, :cw, :r, :Q].astype(bool)
    Yw = np.asarray(Yp, np.uint32).reshape(rw, bw, JG, PT, RT, 8, 4, GROUP)
    Yb = (Yw[..., None, None, None] >> shifts) & 1                # i b jg pt rt g t sub e kh rr
    Yb = Yb.transpose(1, 0, 2, 7, 3, 10, 5, 4, 9, 6, 8)           # b i jg sub pt rr g rt kh t e
    Y = Yb.reshape(bw, rw, JG * GROUP, PT * 32, RT * 32)[:, :, :cw, :P, :r].astype(bool)
    return Y, Z


def algorithmic_bytes(bw, rw, cw, P, Q, r):
    """Packed information per forward: one bit per binary entry plus fp32
    a,b,c per (bit, patch) and d per patch."""
    bits = bw * rw * cw * (P * r + r * Q)
    return bits // 8 + 4 * rw * cw * (3 * bw + 1)
