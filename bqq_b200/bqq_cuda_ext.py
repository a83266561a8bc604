"""Stand-in for the reference's extension loader neural_network_compression/src/bqq_cuda_ext.py.

The reference's packed layer calls `bqq_cuda_ext._get_ext().bqq_forward(Y_packed, Z_packed, X, a, b,
c, d, bias)` (src/bqq_modules.py:217-230), a pybind function of its JIT-compiled src/bqq_cuda.cu
(:289-297, 452-457).  This module offers the same two names - `_get_ext()` and `bqq_forward` -
on top of this package's C-ABI library, so that code written against the reference's extension
(its PackedBinaryQuadratic.forward included) runs on the B200 kernels.  Nothing is compiled at
import time and there is no other backend behind it.

The uint8 bit-packs are re-packed into 32-bit planes the first time a (Y_packed, Z_packed) pair is
seen; the planes are cached per pair (keyed on storage address and version counter, at most
`MAX_CACHED_LAYERS` pairs, least recently used dropped first).  Coefficients and bias are read
from the tensors passed in on every call.
"""
from __future__ import annotations

from collections import OrderedDict

import torch

from .bqq_modules import _BqqForwardMixin, _cabi, check, lib

MAX_CACHED_LAYERS = 4096


class _PackedEngine(_BqqForwardMixin):
    """Forward engine over the reference's packed buffers, without being an nn.Module: the tensors
    of the current call are plain attributes."""

    def __init__(self, Y_packed, Z_packed):
        self.bit_width, self.row_width, self.col_width, self.y_row, k8 = Y_packed.shape
        self.z_col = Z_packed.shape[3]
        # the rank itself is not passed; padding bits are zero, so the padded rank gives the same sums
        self.inter_dimension = 8 * k8
        self.Y_packed, self.Z_packed = Y_packed, Z_packed
        self.a = self.b = self.c = self.d = self.bias = None

    def _plane_sources(self):
        return self.Y_packed, self.Z_packed

    def _build_planes(self, st, device):
        check(lib.bqq_repack_u8_planes(self.Y_packed.contiguous().data_ptr(), self.Z_packed.contiguous().data_ptr(),
                                       st.dims, st.zplanes.data_ptr(), st.yplanes.data_ptr(), st.ysum.data_ptr(),
                                       st.zsum.data_ptr(), torch.cuda.current_stream(device).cuda_stream),
              'bqq_repack_u8_planes')


class _Extension:
    """What `_get_ext()` returns: an object with the pybind module's `bqq_forward`."""

    def __init__(self):
        self._engines: OrderedDict = OrderedDict()

    def bqq_forward(self, Y_packed, Z_packed, X, a, b, c, d, bias):
        """y = X W' (+ bias) for the packed layer; X [..., in] -> [..., out] in X's dtype, as
        src/bqq_cuda.cu:289-393.  `bias` may be None or an empty tensor for "no bias"."""
        if Y_packed.dtype != torch.uint8 or Z_packed.dtype != torch.uint8 or Y_packed.dim() != 5 or Z_packed.dim() != 5:
            raise RuntimeError('bqq_forward: Y_packed / Z_packed must be uint8 [bit, row, col, rows, ceil(r/8)]')
        key = (Y_packed.data_ptr(), Y_packed._version, tuple(Y_packed.shape), Z_packed.data_ptr(), Z_packed._version,
               tuple(Z_packed.shape), Y_packed.device)
        engine = self._engines.get(key)
        if engine is None:
            engine = _PackedEngine(Y_packed, Z_packed)
            self._engines[key] = engine
            while len(self._engines) > MAX_CACHED_LAYERS:
                self._engines.popitem(last=False)
        else:
            self._engines.move_to_end(key)
        engine.a, engine.b, engine.c, engine.d = a, b, c, d
        engine.bias = bias if bias is not None and bias.numel() > 0 else None
        with torch.no_grad():
            return engine.forward(X)


_ext = None


def _get_ext():
    global _ext
    if _ext is None:
        _ext = _Extension()
    return _ext


def bqq_forward(Y_packed, Z_packed, X, a, b, c, d, bias):
    return _get_ext().bqq_forward(Y_packed, Z_packed, X, a, b, c, d, bias)


cuda_bqq_forward = bqq_forward      # the name the reference's README uses for the same call

__all__ = ['_get_ext', 'bqq_forward', 'cuda_bqq_forward', 'MAX_CACHED_LAYERS', '_cabi']
