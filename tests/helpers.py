"""Shared test helpers: golden loading and seeded synthetic layers."""
import glob
import os

import numpy as np
import torch

from oracle import bqq_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
LAYER_CASES = ['fused_s42', 'fused_s123', 'fused_s7', 'fused_bias_s99', 'layer_0', 'layer_1', 'layer_2',
               'extend_3bit']


def load_golden(name):
    g = np.load(os.path.join(GOLDEN, name + '.npz'))
    rec = {k: g[k] for k in g.files}
    if 'Y_packed' in rec:
        bw, rw, cw, P, r, Q = (int(v) for v in rec['shape'])
        rec['dims'] = (bw, rw, cw, P, Q, r)
        rec['Y'], rec['Z'] = O.unpack_u8_reference(rec['Y_packed'], rec['Z_packed'], r)
    return rec


def synth_layer(bw, rw, cw, P, Q, r, M, seed=0, coef_scale=0.02, x_dtype=torch.float32, bias=False):
    """Seeded synthetic layer; draw order Y, Z, A, (bias), X on one CPU generator."""
    g = torch.Generator().manual_seed(seed)
    Y = torch.rand(bw, rw, cw, P, r, generator=g) > 0.5
    Z = torch.rand(bw, rw, cw, r, Q, generator=g) > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=g) * coef_scale
    b = torch.randn(rw * P, generator=g) if bias else None
    X = torch.randn(M, cw * Q, generator=g).to(x_dtype)
    return Y, Z, A, b, X


def oracle_forward_t(Y, Z, A, bias, X):
    """fp32 oracle result for torch inputs (X already rounded to its dtype)."""
    a, b, c, d = O.split_coefficients(A.numpy())
    return O.forward(Y.numpy(), Z.numpy(), a, b, c, d, X.float().numpy(),
                     None if bias is None else bias.numpy())
