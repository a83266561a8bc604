"""Drop-in `bqq_modules` for the B200 path.

Same names, constructor arguments, attributes and state_dict layout as the
reference module neural_network_compression/src/bqq_modules.py, so that
saved whole-model pickles (which record the class path
`bqq_modules.BinaryQuadratic`), the reference's own lm/build_bqq_model.py
(it imports BinaryQuadratic, PackedBinaryQuadratic, PartialBQQLinear,
get_matrices, merge_binary_quadratic, merge_binaryquadratic_recursive and
pack_binaryquadratic_model from here, lm/build_bqq_model.py:57-65) and the
`__new__`-and-fill construction of lm/benchmark_inference.py:24-41 keep
working.  Put this package's directory on sys.path in place of the reference's
`src/`, or call `bqq_b200.install()`.  The {-1,+1} vision layers of the
reference (BQQLinear and friends) are not implemented; see the end of the file.

What differs is only how forward() computes: instead of rebuilding the dense
weight with torch ops on every call (src/bqq_modules.py:34-46) it calls the
C-ABI CUDA library through ctypes.  There is no Triton path, no backend switch
and no CPU fallback: a module whose buffers are not on an sm_100 GPU raises.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn as nn

from . import _cabi
from ._cabi import BqqLayer, check, lib

_DTYPE_CODE = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


# ---------------------------------------------------------------------------
# workspace cache: one growing buffer per (device, stream, kind)
# ---------------------------------------------------------------------------
_WORKSPACES: dict = {}
_RETIRED_WORKSPACES: list = []


def _workspace(device: torch.device, kind: str, nbytes: int) -> torch.Tensor:
    """Scratch buffer for the kernels.  Decode scratch must start zeroed (the
    kernel leaves it zeroed); calls that share a buffer must not overlap on the
    GPU, hence one buffer per stream.

    A buffer that has to grow is replaced, but the old one is kept alive for the life of the
    process: a CUDA graph captured earlier holds its raw address and would otherwise read and
    write memory that the allocator has handed to another tensor.  Growth while the stream is
    being captured is refused (the allocation would land in the capture's private pool)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, kind)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                'bqq_b200: the scratch buffer of this stream has to grow during a CUDA graph capture; run the '
                'largest layer / batch of the captured region once before capturing')
        if buf is not None:
            _RETIRED_WORKSPACES.append(buf)
        size = max(int(nbytes), 256)
        buf = torch.zeros(size, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = buf
    return buf


def check_status(device=None) -> None:
    """Synchronise and raise if a bounded device-side wait gave up in any forward that used this
    process's scratch buffers on `device` (all devices when None); the outputs of such a forward
    are invalid.  The kernels never hang on such a wait: they record it and return."""
    index = None if device is None else torch.device(device).index
    for (dev, stream, kind), buf in list(_WORKSPACES.items()):
        if index is not None and dev != index:
            continue
        with torch.cuda.device(dev):
            fn = lib.bqq_prefill_status if kind.endswith('prefill') else lib.bqq_decode_status
            check(fn(buf.data_ptr(), stream), f'bqq_b200 {kind} scratch on cuda:{dev}')


class _PackedState:
    """Derived, non-persistent device state of one layer: bit planes and row sums,
    rebuilt when the source buffers change.  Coefficients are not cached: the
    kernels read the parameter tensors themselves on every call."""

    __slots__ = ('plane_key', 'dims', 'zplanes', 'yplanes', 'ysum', 'zsum')

    def __init__(self):
        self.plane_key = None


def _tensor_key(t: torch.Tensor):
    return (t.data_ptr(), t._version, t.dtype, t.device, tuple(t.shape))


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f'bqq_b200: {what} lives on {t.device}; the BinaryQuadratic forward of this package '
            'runs only on an sm_100 GPU (move the module with .cuda()); there is no CPU fallback')


class _BqqForwardMixin:
    """Shared engine of BinaryQuadratic and PackedBinaryQuadratic."""

    # -- packed state -------------------------------------------------------
    def _state(self) -> _PackedState:
        st = self.__dict__.get('_bqq_state')
        if st is None:
            st = _PackedState()
            self.__dict__['_bqq_state'] = st
        return st

    def __getstate__(self):
        state = self.__dict__.copy()
        state.pop('_bqq_state', None)      # derived GPU state never enters a pickle
        return state

    def _dims(self):
        return _cabi.dims(self.bit_width, self.row_width, self.col_width, self.y_row, self.z_col,
                          self.inter_dimension)

    def _build_planes(self, st: _PackedState, device) -> None:
        raise NotImplementedError

    def _ensure_packed(self) -> _PackedState:
        st = self._state()
        src_y, src_z = self._plane_sources()
        _require_cuda(src_y, 'the binary factor buffer')
        device = src_y.device
        pkey = (_tensor_key(src_y), _tensor_key(src_z))
        if st.plane_key != pkey:
            with torch.cuda.device(device):
                if not lib.bqq_device_supported():
                    raise RuntimeError('bqq_b200: the current GPU is not an sm_100 device')
                st.dims = self._dims()
                nz, ny = lib.bqq_zplane_words(st.dims), lib.bqq_yplane_words(st.dims)
                if nz == 0 or ny == 0:
                    raise RuntimeError('bqq_b200: unsupported patch geometry '
                                       f'(P={self.y_row}, Q={self.z_col}, r={self.inter_dimension})')
                st.zplanes = torch.empty(nz, dtype=torch.int32, device=device)
                st.yplanes = torch.empty(ny, dtype=torch.int32, device=device)
                n = self.bit_width * self.row_width * self.col_width
                st.ysum = torch.empty(n * self.y_row, dtype=torch.uint8, device=device)
                st.zsum = torch.empty(n * self.z_col, dtype=torch.uint8, device=device)
                self._build_planes(st, device)
            st.plane_key = pkey
        return st

    def _layer(self, st: _PackedState) -> BqqLayer:
        """Descriptor handed to the C ABI; coefficient pointers are the live parameters."""
        coefs = []
        dt = self.a.dtype
        if dt not in _DTYPE_CODE:
            raise RuntimeError(f'bqq_b200: coefficients must be fp32, bf16 or fp16, got {dt}')
        for n in 'abcd':
            t = getattr(self, n).detach()
            _require_cuda(t, f'coefficient {n}')
            if t.dtype != dt:
                raise RuntimeError('bqq_b200: coefficients a, b, c, d must share one dtype')
            if not t.is_contiguous():
                t = t.contiguous()
            coefs.append(t)
        bias = getattr(self, 'bias', None)
        if bias is not None:
            bias = bias.detach()
            _require_cuda(bias, 'the bias')
            if bias.dtype not in _DTYPE_CODE:
                raise RuntimeError(f'bqq_b200: unsupported bias dtype {bias.dtype}')
            if not bias.is_contiguous():
                bias = bias.contiguous()
        layer = BqqLayer(st.dims, st.zplanes.data_ptr(), st.yplanes.data_ptr(),
                         coefs[0].data_ptr(), coefs[1].data_ptr(), coefs[2].data_ptr(), coefs[3].data_ptr(),
                         bias.data_ptr() if bias is not None else None,
                         _DTYPE_CODE[dt], _DTYPE_CODE[bias.dtype] if bias is not None else 0)
        layer._keepalive = (coefs, bias)
        return layer

    # -- forward ------------------------------------------------------------
    def _check_inference_only(self, X) -> None:
        if torch.is_grad_enabled():
            needs = X.requires_grad or any(
                p is not None and p.requires_grad
                for p in (self.a, self.b, self.c, self.d, getattr(self, 'bias', None)))
            if needs:
                raise RuntimeError(
                    'bqq_b200: this BinaryQuadratic forward is inference-only and records no autograd '
                    'graph; call it under torch.no_grad() (training workflows need the reference module)')

    def forward(self, X):
        self._check_inference_only(X)
        if X.dtype not in _DTYPE_CODE:
            # the reference computes in whatever float type X has (src/bqq_modules.py:35); the kernels
            # take fp32 / bf16 / fp16, so any other float type (fp64) goes through fp32 and back
            if not X.is_floating_point():
                raise RuntimeError(f'bqq_b200: unsupported activation dtype {X.dtype} (floating point only)')
            return self.forward(X.to(torch.float32)).to(X.dtype)
        st = self._ensure_packed()
        device = st.zplanes.device
        in_f = self.col_width * self.z_col
        out_f = self.row_width * self.y_row
        if X.shape[-1] != in_f:
            raise RuntimeError(f'bqq_b200: last dim of X is {X.shape[-1]}, layer expects {in_f}')
        X = X.to(device)
        x2 = X.reshape(-1, in_f)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        M = x2.shape[0]
        y = torch.empty((M, out_f), dtype=X.dtype, device=device)
        if M == 0:
            return y.reshape(*X.shape[:-1], out_f)
        code = _DTYPE_CODE[X.dtype]
        layer = self._layer(st)
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            # up to 16 rows: bit-streaming decode kernel; more: tensor-core prefill path
            if M <= _cabi.DECODE_MAX_M:
                nbytes = lib.bqq_decode_workspace_bytes(st.dims, M)
                ws = _workspace(device, 'decode', nbytes)
                check(lib.bqq_forward_decode(layer, x2.data_ptr(), code, M, x2.stride(0), y.data_ptr(), code,
                                             y.stride(0), ws.data_ptr(), ws.numel(), stream),
                      'bqq_forward_decode')
            else:
                nbytes = lib.bqq_prefill_workspace_bytes(st.dims, M)
                ws = _workspace(device, 'prefill', nbytes)
                check(lib.bqq_forward_prefill(layer, x2.data_ptr(), code, M, x2.stride(0), y.data_ptr(),
                                              code, y.stride(0), ws.data_ptr(), ws.numel(), stream),
                      'bqq_forward_prefill')
        return y.reshape(*X.shape[:-1], out_f)

    def _fusion(self, M, rms_weight, eps, swiglu, res2d):
        """BqqFusion descriptor for bqq_forward_decode_fused / _gathered; res2d is [M, out] (any row pitch)."""
        in_f = self.col_width * self.z_col
        out_f = self.row_width * self.y_row
        fusion = _cabi.BqqFusion()
        keep = []
        if rms_weight is not None:
            w = rms_weight.detach()
            _require_cuda(w, 'the normalisation weight')
            if w.dtype not in _DTYPE_CODE or w.numel() != in_f:
                raise RuntimeError('bqq_b200: rms_weight must be an fp32/bf16/fp16 vector of in_features elements')
            w = w.contiguous()
            keep.append(w)
            fusion.prologue, fusion.norm_weight, fusion.norm_dtype, fusion.eps = (
                _cabi.PRO_RMSNORM, w.data_ptr(), _DTYPE_CODE[w.dtype], float(eps))
        elif swiglu:
            fusion.prologue = _cabi.PRO_SWIGLU
        if res2d is not None:
            if (not res2d.is_cuda or tuple(res2d.shape) != (M, out_f) or res2d.stride(-1) != 1
                    or res2d.dtype not in _DTYPE_CODE):
                raise RuntimeError('bqq_b200: residual must be a CUDA tensor [..., out_features] with unit inner stride')
            keep.append(res2d)
            fusion.residual, fusion.ld_residual, fusion.residual_dtype = (
                res2d.data_ptr(), res2d.stride(0), _DTYPE_CODE[res2d.dtype])
        return fusion, keep

    def forward_fused(self, X, rms_weight=None, eps: float = 1e-5, swiglu: bool = False, residual=None):
        """Forward with the neighbouring element-wise operations of a decoder block folded into the
        kernels (bqq_forward_decode_fused):

            rms_weight:  the layer sees  rms_norm(X, weight=rms_weight, eps)
            swiglu:      X is [..., 2*in] = [gate | up]; the layer sees  silu(gate) * up
            residual:    [..., out] added to the output (pass the tensor the result replaces)

        The prologue runs in fp32 on the unrounded values.  Up to 16 rows this is one decode call; larger
        batches apply the same operations with torch ops and call forward()."""
        self._check_inference_only(X)
        if rms_weight is not None and swiglu:
            raise RuntimeError('bqq_b200: rms_weight and swiglu cannot be combined')
        in_f = self.col_width * self.z_col
        out_f = self.row_width * self.y_row
        width = 2 * in_f if swiglu else in_f
        if X.shape[-1] != width:
            raise RuntimeError(f'bqq_b200: last dim of X is {X.shape[-1]}, expected {width}')
        M = X.numel() // width
        if M > _cabi.DECODE_MAX_M or M == 0 or X.dtype not in _DTYPE_CODE:
            H = X
            if rms_weight is not None:
                H = torch.nn.functional.rms_norm(X, (in_f,), rms_weight, eps)
            elif swiglu:
                H = torch.nn.functional.silu(X[..., :in_f]) * X[..., in_f:]
            Yo = self.forward(H)
            return Yo if residual is None else residual + Yo
        st = self._ensure_packed()
        device = st.zplanes.device
        X = X.to(device)
        x2 = X.reshape(-1, width)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        y = torch.empty((M, out_f), dtype=X.dtype, device=device)
        fusion, keep = self._fusion(M, rms_weight, eps, swiglu,
                                    None if residual is None else residual.reshape(-1, out_f))
        code = _DTYPE_CODE[X.dtype]
        layer = self._layer(st)
        with torch.cuda.device(device):
            ws = _workspace(device, 'decode', lib.bqq_decode_workspace_bytes(st.dims, M))
            check(lib.bqq_forward_decode_fused(layer, x2.data_ptr(), code, M, x2.stride(0), y.data_ptr(), code,
                                               y.stride(0), C.byref(fusion), ws.data_ptr(), ws.numel(),
                                               torch.cuda.current_stream(device).cuda_stream),
                  'bqq_forward_decode_fused')
        return y.reshape(*X.shape[:-1], out_f)

    def forward_gathered(self, X, peer, out=None, rms_weight=None, eps: float = 1e-5, swiglu: bool = False,
                         residual=None, out_segments: int = 1):
        """Forward of a row-patch shard with the column gather built in: every rank calls it on its
        shard with the full activation X [..., in] and gets the full output [..., world*out_local]
        (columns in rank order).  `peer` is a bqq_b200.peer.PeerGatherGroup of the ranks.

        Up to 16 rows the decode kernel itself stores each finished row patch into the peers' gather
        regions (bqq_forward_decode_gathered); larger batches run the forward and then the gather kernel.
        rms_weight / swiglu / residual as in forward_fused; `residual` is the full [..., world*out_local]
        tensor, of which this rank adds its own columns before sending.  `out_segments=2`: the local
        output is two halves [h0 | h1] (a stacked gate / up layer) and the result is
        [h0 of all ranks | h1 of all ranks], the [gate | up] rows a SwiGLU consumer expects."""
        self._check_inference_only(X)
        if X.dtype not in _DTYPE_CODE:
            raise RuntimeError(f'bqq_b200: unsupported activation dtype {X.dtype} (fp32, bf16, fp16 only)')
        st = self._ensure_packed()
        device = st.zplanes.device
        in_f = self.col_width * self.z_col
        out_f = self.row_width * self.y_row
        width = 2 * in_f if swiglu else in_f
        if X.shape[-1] != width:
            raise RuntimeError(f'bqq_b200: last dim of X is {X.shape[-1]}, expected {width}')
        X = X.to(device)
        x2 = X.reshape(-1, width)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        M = x2.shape[0]
        esize = X.element_size()
        res_local = None
        if residual is not None:
            res_local = residual.reshape(M, peer.world * out_f)[:, peer.rank * out_f:(peer.rank + 1) * out_f]
        fused = (0 < M <= _cabi.DECODE_MAX_M and (out_f * esize) % 4 == 0
                 and (esize == 4 or self.y_row % 2 == 0)
                 and M * out_f * peer.world * esize <= peer.max_bytes)
        if out_segments not in (1, 2) or (out_segments == 2 and (out_f % 2 or residual is not None)):
            raise RuntimeError('bqq_b200: out_segments must be 1 or 2 (2: even out_features, no residual)')
        if not fused:
            y_local = self.forward_fused(X, rms_weight=rms_weight, eps=eps, swiglu=swiglu,
                                         residual=None if res_local is None else res_local.contiguous())
            if out_segments == 2:
                h = out_f // 2
                both = torch.cat([peer.gather(y_local[..., :h].contiguous()), peer.gather(y_local[..., h:].contiguous())],
                                 dim=-1)
                return both if out is None else out.copy_(both.reshape(out.shape))
            return peer.gather(y_local, out=out)
        fusion, keep = self._fusion(M, rms_weight, eps, swiglu, res_local)
        fusion.out_segments = out_segments
        if out is None:
            out = torch.empty((M, peer.world * out_f), dtype=X.dtype, device=device)
        o2 = out.reshape(M, peer.world * out_f)
        if o2.data_ptr() != out.data_ptr() or o2.stride(-1) != 1 or out.dtype != X.dtype:
            raise RuntimeError('bqq_b200: `out` must be a [rows, world*out] tensor of the input dtype with unit inner stride')
        y = torch.empty((M, out_f), dtype=X.dtype, device=device)
        code = _DTYPE_CODE[X.dtype]
        layer = self._layer(st)
        with torch.cuda.device(device):
            nbytes = lib.bqq_decode_workspace_bytes(st.dims, M)
            ws = _workspace(device, 'decode', nbytes)
            check(lib.bqq_forward_decode_gathered(layer, x2.data_ptr(), code, M, x2.stride(0), y.data_ptr(), code,
                                                  y.stride(0), C.byref(fusion), peer.descriptor(), o2.data_ptr(),
                                                  o2.stride(0),
                                                  ws.data_ptr(), ws.numel(),
                                                  torch.cuda.current_stream(device).cuda_stream),
                  'bqq_forward_decode_gathered')
        return o2.reshape(*X.shape[:-1], peer.world * out_f)

    def bind_host(self, X_host, out=None):
        """Prepare the forward for activations that live in HOST memory and return `(run, out)`.

        `X_host` [..., in] is a CPU tensor (pinned for asynchronous copies), `out` [..., out] a CPU tensor
        of X's dtype (pinned; allocated when None).  Each `run()` is one C call (bqq_forward_host) that
        enqueues the host->device copy of X_host's current contents, the kernels and the device->host
        copy into `out` on the stream that was current when bind_host was called; nothing is
        synchronised: synchronise that stream before reading `out`.  The binding holds raw pointers: it
        stays valid while X_host, out and the layer's parameters and buffers are not reallocated
        (in-place updates are fine)."""
        self._check_inference_only(X_host)
        if X_host.is_cuda:
            raise RuntimeError('bqq_b200: host forward expects a CPU tensor; use forward() for device tensors')
        if X_host.dtype not in _DTYPE_CODE:
            raise RuntimeError(f'bqq_b200: unsupported activation dtype {X_host.dtype} (fp32, bf16, fp16 only)')
        st = self._ensure_packed()
        device = st.zplanes.device
        in_f = self.col_width * self.z_col
        out_f = self.row_width * self.y_row
        if X_host.shape[-1] != in_f:
            raise RuntimeError(f'bqq_b200: last dim of X is {X_host.shape[-1]}, layer expects {in_f}')
        x2 = X_host.reshape(-1, in_f)
        if x2.stride(-1) != 1 or x2.data_ptr() != X_host.data_ptr():
            raise RuntimeError('bqq_b200: X_host must be viewable as [M, in_features] rows with unit inner stride')
        M = x2.shape[0]
        if out is None:
            out = torch.empty((*X_host.shape[:-1], out_f), dtype=X_host.dtype, pin_memory=True)
        y2 = out.reshape(-1, out_f)
        if (out.is_cuda or out.dtype != X_host.dtype or y2.shape[0] != M or y2.stride(-1) != 1
                or y2.data_ptr() != out.data_ptr()):
            raise RuntimeError("bqq_b200: `out` must be a CPU tensor [..., out_features] of X's dtype with unit inner stride")
        if M == 0:
            return (lambda: out), out
        code = _DTYPE_CODE[X_host.dtype]
        layer = self._layer(st)
        with torch.cuda.device(device):
            nbytes = lib.bqq_forward_host_workspace_bytes(st.dims, M, code, code)
            ws = _workspace(device, 'host_decode' if M <= _cabi.DECODE_MAX_M else 'host_prefill', nbytes)
            stream = torch.cuda.current_stream(device).cuda_stream
        args = (layer, x2.data_ptr(), code, M, x2.stride(0), y2.data_ptr(), code, y2.stride(0),
                ws.data_ptr(), ws.numel(), stream)
        call = lib.bqq_forward_host
        index = device.index
        keep = (x2, y2, ws, layer, st)                  # keeps the bound memory alive with the closure
        result = out

        def run():
            if torch.cuda.current_device() != index:
                with torch.cuda.device(index):
                    rc = call(*args)
            else:
                rc = call(*args)
            if rc:
                check(rc, 'bqq_forward_host')
            return result

        return run, out

    def forward_host(self, X_host, out=None):
        """One-shot form of bind_host: enqueue the forward of host activations `X_host` into the host
        tensor `out` (allocated pinned when None) and return `out`; synchronise the current stream of
        the layer's GPU before reading it.  The values are those of forward(X_host.to(device)).cpu()."""
        if not X_host.is_cuda and X_host.dim() >= 1 and X_host.stride(-1) != 1:
            X_host = X_host.contiguous()
        run, out = self.bind_host(X_host, out)
        run()
        return out

    def _weight_gpu(self, dtype):
        st = self._ensure_packed()
        device = st.zplanes.device
        out_f = self.row_width * self.y_row
        in_f = self.col_width * self.z_col
        W = torch.empty((out_f, in_f), dtype=dtype, device=device)
        with torch.cuda.device(device):
            check(lib.bqq_reconstruct_weight(self._layer(st), W.data_ptr(), _DTYPE_CODE[dtype], 1.0,
                                             torch.cuda.current_stream(device).cuda_stream),
                  'bqq_reconstruct_weight')
        return W


def _dense_weight(Y, Z, a, b, c, d, dtype):
    """W [rw*P, cw*Q] from the factors with torch ops (src/bqq_modules.py:37-42):
    sum over bit layers of a*YZ + b*(Y1)1' + c*1(1'Z), plus d, patches laid out row-major.
    Differentiable in a, b, c, d; used where autograd or a CPU tensor is wanted, never by forward()."""
    Yd, Zd = Y.to(dtype), Z.to(dtype)
    per_bit = (a.to(dtype) * (Yd @ Zd) + b.to(dtype) * Yd.sum(-1, keepdim=True)
               + c.to(dtype) * Zd.sum(-2, keepdim=True))
    tiles = per_bit.sum(0) + d.to(dtype)                      # [rw, cw, P, Q]
    rw, cw, P, Q = tiles.shape
    return tiles.transpose(1, 2).reshape(rw * P, cw * Q)


# ---------------------------------------------------------------------------
# BinaryQuadratic
# ---------------------------------------------------------------------------

class BinaryQuadratic(_BqqForwardMixin, nn.Module):
    """BQQ layer with {0,1} factors.  Constructor, buffers (`Y`, `Z` bool),
    parameters (`a`, `b`, `c` [bw,rw,cw,1,1], `d` [rw,cw,1,1], `bias`) and the
    attributes bit_width/row_width/col_width/y_row/inter_dimension/z_col match
    the reference class (src/bqq_modules.py:18-32)."""

    def __init__(self, Y, Z, A, bias=None):
        super().__init__()
        self.bit_width, self.row_width, self.col_width, self.y_row, self.inter_dimension = Y.shape
        self.z_col = Z.shape[-1]
        self.register_buffer('Y', Y > 0.5)
        self.register_buffer('Z', Z > 0.5)
        coef = [A[..., n].unsqueeze(-1).unsqueeze(-1) for n in range(4)]
        self.a = nn.Parameter(coef[0].clone())
        self.b = nn.Parameter(coef[1].clone())
        self.c = nn.Parameter(coef[2].clone())
        self.d = nn.Parameter(coef[3].sum(dim=0))       # one offset per patch: summed over bit layers
        self.bias = nn.Parameter(bias) if bias is not None else None

    def _plane_sources(self):
        return self.Y, self.Z

    def _build_planes(self, st, device):
        Y = self.Y.contiguous()
        Z = self.Z.contiguous()
        if Y.dtype != torch.bool or Z.dtype != torch.bool:
            Y, Z = Y > 0.5, Z > 0.5
        check(lib.bqq_pack_planes(Y.data_ptr(), Z.data_ptr(), st.dims, st.zplanes.data_ptr(),
                                  st.yplanes.data_ptr(), st.ysum.data_ptr(), st.zsum.data_ptr(),
                                  torch.cuda.current_stream(device).cuda_stream), 'bqq_pack_planes')

    def get_weight(self, dtype=torch.float32):
        """Dense W [out, in] (src/bqq_modules.py:48-55).  On the GPU it comes from
        the popcount reconstruction kernel; before the module is moved to a GPU
        it is evaluated with torch ops (not a forward path)."""
        if self.Y.is_cuda and dtype in _DTYPE_CODE:
            return self._weight_gpu(dtype)
        return _dense_weight(self.Y, self.Z, self.a, self.b, self.c, self.d, dtype)

    def unpack_planes(self):
        """Bit planes back to bool Y, Z (bit-exact round-trip check)."""
        st = self._ensure_packed()
        device = st.zplanes.device
        Y = torch.empty(self.Y.shape, dtype=torch.uint8, device=device)
        Z = torch.empty(self.Z.shape, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            check(lib.bqq_unpack_planes(st.zplanes.data_ptr(), st.yplanes.data_ptr(), st.dims, Y.data_ptr(),
                                        Z.data_ptr(), torch.cuda.current_stream(device).cuda_stream),
                  'bqq_unpack_planes')
        return Y.bool(), Z.bool()


# ---------------------------------------------------------------------------
# PackedBinaryQuadratic: the reference's uint8-packed checkpoints
# ---------------------------------------------------------------------------

class PackedBinaryQuadratic(_BqqForwardMixin, nn.Module):
    """Accepts the reference's packed layer (src/bqq_modules.py:62-97): buffers
    Y_packed [bw,rw,cw,P,ceil(r/8)], Z_packed [bw,rw,cw,Q,ceil(r/8)] (big-endian
    uint8, Z transposed), Y_sum_i16, Z_sum_i16 and the same parameters.  The
    bytes are re-packed on the GPU into this library's 32-bit planes at first
    use; forward then runs the same kernels as BinaryQuadratic."""

    def __init__(self, Y_packed, Z_packed, a, b, c, d, Y_sum_i16, Z_sum_i16,
                 inter_dimension, y_row, z_col, bias=None):
        super().__init__()
        self.bit_width, self.row_width, self.col_width = Y_packed.shape[:3]
        self.y_row, self.z_col, self.inter_dimension = y_row, z_col, inter_dimension
        self._k8 = Y_packed.shape[-1]
        self.register_buffer('Y_packed', Y_packed)
        self.register_buffer('Z_packed', Z_packed)
        self.register_buffer('Y_sum_i16', Y_sum_i16)
        self.register_buffer('Z_sum_i16', Z_sum_i16)
        self.a, self.b = nn.Parameter(a), nn.Parameter(b)
        self.c, self.d = nn.Parameter(c), nn.Parameter(d)
        self.bias = nn.Parameter(bias) if bias is not None else None

    @classmethod
    def from_unpacked(cls, bq: BinaryQuadratic) -> 'PackedBinaryQuadratic':
        """BinaryQuadratic -> packed layer with the reference's byte layout
        (src/bqq_modules.py:115-148): element 0 of the rank axis is the MSB."""
        Y, Z = bq.Y, bq.Z
        r = Y.shape[-1]
        k8 = (r + 7) // 8
        weights = (2 ** torch.arange(7, -1, -1, device=Y.device)).to(torch.int32)

        def pack_last(bits):
            pad = k8 * 8 - bits.shape[-1]
            if pad:
                bits = torch.nn.functional.pad(bits, (0, pad))
            grouped = bits.reshape(*bits.shape[:-1], k8, 8).to(torch.int32)
            return (grouped * weights).sum(-1).to(torch.uint8)

        return cls(pack_last(Y), pack_last(Z.transpose(-1, -2)),
                   bq.a.data.clone(), bq.b.data.clone(), bq.c.data.clone(), bq.d.data.clone(),
                   Y.sum(-1, keepdim=True).to(torch.int16), Z.sum(-2, keepdim=True).to(torch.int16),
                   r, Y.shape[-2], Z.shape[-1],
                   bias=bq.bias.data.clone() if bq.bias is not None else None)

    def _plane_sources(self):
        return self.Y_packed, self.Z_packed

    def _build_planes(self, st, device):
        check(lib.bqq_repack_u8_planes(self.Y_packed.contiguous().data_ptr(),
                                       self.Z_packed.contiguous().data_ptr(), st.dims,
                                       st.zplanes.data_ptr(), st.yplanes.data_ptr(),
                                       st.ysum.data_ptr(), st.zsum.data_ptr(),
                                       torch.cuda.current_stream(device).cuda_stream), 'bqq_repack_u8_planes')

    def get_weight(self, dtype=torch.float32):
        if not self.Y_packed.is_cuda or dtype not in _DTYPE_CODE:
            raise RuntimeError('bqq_b200: PackedBinaryQuadratic.get_weight needs the module on an sm_100 GPU '
                               'and an fp32/bf16/fp16 dtype')
        return self._weight_gpu(dtype)


# ---------------------------------------------------------------------------
# PlaneBinaryQuadratic: patch files straight into this library's bit planes
# ---------------------------------------------------------------------------

class PlaneBinaryQuadratic(_BqqForwardMixin, nn.Module):
    """BQQ layer that holds only this library's 32-bit bit planes (buffers `zplanes`, `yplanes`,
    int32) and the coefficients: what BinaryQuadratic derives at first use is here the stored form.
    The reference has no such class; `from_patches` replaces get_matrices + BinaryQuadratic
    (src/bqq_modules.py:485-507, 21-32) for loaders that want to skip the dense bool Y / Z
    (32 times the planes' size as bytes on the host)."""

    def __init__(self, zplanes, yplanes, a, b, c, d, dims, bias=None):
        super().__init__()
        (self.bit_width, self.row_width, self.col_width, self.y_row, self.z_col,
         self.inter_dimension) = (int(v) for v in dims)
        self.register_buffer('zplanes', zplanes)
        self.register_buffer('yplanes', yplanes)
        self.a, self.b = nn.Parameter(a), nn.Parameter(b)
        self.c, self.d = nn.Parameter(c), nn.Parameter(d)
        self.bias = nn.Parameter(bias) if bias is not None else None

    @classmethod
    def from_patches(cls, patch_list, bit_width, bias=None) -> 'PlaneBinaryQuadratic':
        """Patch dicts {patch_row, patch_col, coeff, mat1, mat2, bit_idx} -> layer, one patch at a
        time on the host (bqq_pack_patch_host).  Same rules as get_matrices: entries with
        bit_idx >= bit_width are skipped, the geometry comes from the first entry, a later entry for
        the same (bit, row, col) replaces the earlier one, missing patches are zero."""
        rw = max(int(p['patch_row']) for p in patch_list) + 1
        cw = max(int(p['patch_col']) for p in patch_list) + 1
        first = patch_list[0]
        P, r = first['mat1'].shape
        Q = first['mat2'].shape[1]
        dims = _cabi.dims(bit_width, rw, cw, P, Q, r)
        nz, ny = lib.bqq_zplane_words(dims), lib.bqq_yplane_words(dims)
        if nz == 0 or ny == 0:
            raise RuntimeError(f'bqq_b200: unsupported patch geometry (P={P}, Q={Q}, r={r})')
        zp = torch.zeros(nz, dtype=torch.int32)
        yp = torch.zeros(ny, dtype=torch.int32)
        A = torch.zeros((bit_width, rw, cw, 4), dtype=first['coeff'].dtype)
        for p in patch_list:
            k = int(p['bit_idx'])
            if k >= bit_width:
                continue
            i, j = int(p['patch_row']), int(p['patch_col'])
            A[k, i, j] = p['coeff']
            m1 = (p['mat1'] > 0.5).to(torch.uint8).contiguous()
            m2 = (p['mat2'] > 0.5).to(torch.uint8).contiguous()
            if tuple(m1.shape) != (P, r) or tuple(m2.shape) != (r, Q):
                raise RuntimeError('bqq_b200: patches of one layer must share one geometry')
            check(lib.bqq_pack_patch_host(m1.data_ptr(), m2.data_ptr(), dims, k, i, j, zp.data_ptr(), yp.data_ptr()),
                  'bqq_pack_patch_host')
        coef = [A[..., n].unsqueeze(-1).unsqueeze(-1) for n in range(4)]
        return cls(zp, yp, coef[0].clone(), coef[1].clone(), coef[2].clone(), coef[3].sum(dim=0),
                   (bit_width, rw, cw, P, Q, r), bias=bias)

    def _plane_sources(self):
        return self.yplanes, self.zplanes

    def _ensure_packed(self) -> _PackedState:
        """The buffers are the packed state: nothing is derived or copied."""
        st = self._state()
        _require_cuda(self.zplanes, 'the bit plane buffer')
        pkey = (_tensor_key(self.yplanes), _tensor_key(self.zplanes))
        if st.plane_key != pkey:
            with torch.cuda.device(self.zplanes.device):
                if not lib.bqq_device_supported():
                    raise RuntimeError('bqq_b200: the current GPU is not an sm_100 device')
            st.dims = self._dims()
            if (self.zplanes.numel() != lib.bqq_zplane_words(st.dims) or self.yplanes.numel() != lib.bqq_yplane_words(st.dims)
                    or self.zplanes.dtype != torch.int32 or self.yplanes.dtype != torch.int32):
                raise RuntimeError('bqq_b200: plane buffers do not match the layer geometry')
            st.zplanes, st.yplanes = self.zplanes.contiguous(), self.yplanes.contiguous()
            st.ysum = st.zsum = None
            st.plane_key = pkey
        return st

    def get_weight(self, dtype=torch.float32):
        if not self.zplanes.is_cuda or dtype not in _DTYPE_CODE:
            raise RuntimeError('bqq_b200: PlaneBinaryQuadratic.get_weight needs the module on an sm_100 GPU '
                               'and an fp32/bf16/fp16 dtype')
        return self._weight_gpu(dtype)

    def unpack_planes(self):
        """Bit planes back to bool Y [bw,rw,cw,P,r], Z [bw,rw,cw,r,Q]."""
        st = self._ensure_packed()
        device = st.zplanes.device
        shape = (self.bit_width, self.row_width, self.col_width)
        Y = torch.empty(shape + (self.y_row, self.inter_dimension), dtype=torch.uint8, device=device)
        Z = torch.empty(shape + (self.inter_dimension, self.z_col), dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            check(lib.bqq_unpack_planes(st.zplanes.data_ptr(), st.yplanes.data_ptr(), st.dims, Y.data_ptr(),
                                        Z.data_ptr(), torch.cuda.current_stream(device).cuda_stream),
                  'bqq_unpack_planes')
        return Y.bool(), Z.bool()


def pack_binaryquadratic_model(model: nn.Module) -> nn.Module:
    """Replace every BinaryQuadratic by its packed twin (src/bqq_modules.py:435-442)."""
    for name, module in list(model.named_children()):
        if isinstance(module, BinaryQuadratic):
            setattr(model, name, PackedBinaryQuadratic.from_unpacked(module))
        else:
            pack_binaryquadratic_model(module)
    return model


# ---------------------------------------------------------------------------
# patch list -> tensors, Linear -> BinaryQuadratic replacement
# ---------------------------------------------------------------------------

def get_matrices(patch_list, bit_width):
    """Patch dicts {patch_row, patch_col, coeff, mat1, mat2, bit_idx} to dense
    A [bw,rw,cw,4], Y [bw,rw,cw,P,r], Z [bw,rw,cw,r,Q]; entries whose bit_idx is
    >= bit_width are skipped and patch geometry is taken from the first entry,
    as in the reference (src/bqq_modules.py:485-507)."""
    rw = max(int(p['patch_row']) for p in patch_list) + 1
    cw = max(int(p['patch_col']) for p in patch_list) + 1
    first = patch_list[0]
    P, r = first['mat1'].shape
    Q = first['mat2'].shape[1]
    A = torch.zeros((bit_width, rw, cw, 4), dtype=first['coeff'].dtype)
    Y = torch.zeros((bit_width, rw, cw, P, r), dtype=first['mat1'].dtype)
    Z = torch.zeros((bit_width, rw, cw, r, Q), dtype=first['mat1'].dtype)
    for p in patch_list:
        k = int(p['bit_idx'])
        if k >= bit_width:
            continue
        i, j = int(p['patch_row']), int(p['patch_col'])
        A[k, i, j] = p['coeff']
        Y[k, i, j] = p['mat1']
        Z[k, i, j] = p['mat2']
    return A, Y, Z


def _patch_loader(source):
    """`source` of replace_linear_with_bqq -> function weight_key -> patch list.

    A callable is used as it is.  A directory is read in the reference's on-disk formats
    (lm/compressed_data.py:40-58, 152-191): `<dir>/_consolidated/<weight_key>.pth` holds the whole
    list of patch dicts of one tensor; otherwise the files `<dir>/<weight_key>_row*.pth` each hold a
    list of patch dicts and are concatenated in sorted order."""
    if callable(source):
        return source
    import os
    root = os.fspath(source)
    if not os.path.isdir(root):
        raise FileNotFoundError(f'bqq_b200: patch directory does not exist: {root}')
    merged_dir = os.path.join(root, '_consolidated')
    per_patch: dict = {}
    for entry in os.scandir(root):
        if entry.name.endswith('.pth') and '_row' in entry.name:
            per_patch.setdefault(entry.name[:-4].rsplit('_row', 1)[0], []).append(entry.path)

    def load(weight_key):
        merged = os.path.join(merged_dir, weight_key + '.pth')
        if os.path.exists(merged):
            return torch.load(merged, weights_only=False, map_location='cpu')
        patches = []
        for path in sorted(per_patch.get(weight_key, ())):
            patches.extend(torch.load(path, weights_only=False, map_location='cpu'))
        return patches

    return load


def replace_linear_with_bqq(model: nn.Module, weights_dir, bit_width: int, prefix: str = '',
                            device=None, show_tqdm: bool = False, patch_index=None,
                            planes_only: bool = False) -> nn.Module:
    """Walk the module tree and replace nn.Linear by BinaryQuadratic, skipping any name that
    contains 'head'; argument order and meaning follow lm/build_bqq_model.py:79-112.

    `weights_dir` is the directory of patch files written by the quantiser (see _patch_loader for
    the two layouts) or, as an extension, a callable `weight_key -> patch list`.  `patch_index`
    (the reference's name -> path(s) dictionary) is honoured when given; `device` and `show_tqdm`
    are accepted for call compatibility (patches are read on the host; no progress bar is drawn).
    With `planes_only` the new layers are PlaneBinaryQuadratic, packed patch by patch without the
    dense Y / Z tensors.  Linears without patches are left in place, as in the reference."""
    if patch_index is not None and not callable(weights_dir):
        index = patch_index

        def load_patches(weight_key):
            entry = index.get(weight_key)
            if entry is None:
                return []
            paths = [entry] if not isinstance(entry, (list, tuple)) else list(entry)
            out = []
            for path in paths:
                out.extend(torch.load(path, weights_only=False, map_location='cpu'))
            return out
    else:
        load_patches = _patch_loader(weights_dir)
    return _replace_linears(model, load_patches, bit_width, prefix, planes_only)


def _replace_linears(model, load_patches, bit_width, prefix, planes_only):
    for name, module in list(model.named_children()):
        full = f'{prefix}.{name}' if prefix else name
        if 'head' in full:
            continue
        if isinstance(module, nn.Linear):
            patches = load_patches(f'{full}.weight')
            if not patches:
                continue
            if planes_only:
                bias = module.bias.data.clone() if module.bias is not None else None
                setattr(model, name, PlaneBinaryQuadratic.from_patches(patches, bit_width, bias=bias))
            else:
                A, Y, Z = get_matrices(patches, bit_width)
                setattr(model, name, BinaryQuadratic(Y, Z, A, bias=module.bias))
        else:
            _replace_linears(module, load_patches, bit_width, full, planes_only)
    return model


# ---------------------------------------------------------------------------
# Layers and helpers of the reference's quantisation workflows (not on the forward path)
# ---------------------------------------------------------------------------

def _binaryquadratic_from_parts(Y, Z, a, b, c, d, bias):
    """BinaryQuadratic from already split coefficients, without the (Y, Z, A) constructor - the
    route lm/benchmark_inference.py:30-40 and src/bqq_modules.py:416-432 take."""
    layer = BinaryQuadratic.__new__(BinaryQuadratic)
    nn.Module.__init__(layer)
    (layer.bit_width, layer.row_width, layer.col_width, layer.y_row, layer.inter_dimension) = Y.shape
    layer.z_col = Z.shape[-1]
    layer.register_buffer('Y', Y.clone() if Y.dtype == torch.bool else Y > 0.5)
    layer.register_buffer('Z', Z.clone() if Z.dtype == torch.bool else Z > 0.5)
    for name, value in (('a', a), ('b', b), ('c', c), ('d', d)):
        setattr(layer, name, nn.Parameter(value.detach().clone()))
    layer.bias = nn.Parameter(bias.detach().clone()) if bias is not None else None
    return layer


class PartialBQQLinear(nn.Module):
    """Linear layer whose patches are quantised one group at a time during block-wise training
    (src/bqq_modules.py:246-432; used by lm/blockwise_quant.py:540-632 and imported by
    lm/build_bqq_model.py:57-65).

    State, names as in the reference so that its pickles and training loops work: `float_weight`
    [out, in] fp32 (trainable, stands for every patch not yet quantised), `bias_param`, bool buffer
    `quantized_mask` [rw, cw], and - created by the first quantize_patch, when the rank is known -
    bool buffers `Y`, `Z` and parameters `a, b, c, d` shaped as in BinaryQuadratic.

    This is a training-time layer: forward() is plain differentiable torch code (W is assembled per
    call; gradients reach a..d through the quantised patches and float_weight through the others).
    It is not a forward path of the CUDA library; to_binaryquadratic() hands the finished layer to
    it."""

    def __init__(self, weight: torch.Tensor, bias, group_size: int, bit_width: int):
        super().__init__()
        out_f, in_f = weight.shape
        for what, n in (('out_features', out_f), ('in_features', in_f)):
            if n % group_size:
                raise ValueError(f'{what}={n} is not divisible by group_size={group_size}.')
        self.group_size, self.bit_width = group_size, bit_width
        self.row_width, self.y_row = out_f // group_size, group_size
        self.col_width, self.z_col = in_f // group_size, group_size
        self.inter_dimension = None                      # known once the first patch arrives
        self.float_weight = nn.Parameter(weight.detach().clone().float())
        self.bias_param = nn.Parameter(bias.detach().clone().float()) if bias is not None else None
        self.register_buffer('quantized_mask', torch.zeros(self.row_width, self.col_width, dtype=torch.bool))

    def _init_bqq_tensors(self, inter_dimension: int) -> None:
        dev = self.float_weight.device
        grid = (self.bit_width, self.row_width, self.col_width)
        self.inter_dimension = inter_dimension
        self.register_buffer('Y', torch.zeros(*grid, self.y_row, inter_dimension, dtype=torch.bool, device=dev))
        self.register_buffer('Z', torch.zeros(*grid, inter_dimension, self.z_col, dtype=torch.bool, device=dev))
        for name in 'abc':
            setattr(self, name, nn.Parameter(torch.zeros(*grid, 1, 1, device=dev)))
        self.d = nn.Parameter(torch.zeros(self.row_width, self.col_width, 1, 1, device=dev))

    def quantize_patch(self, i: int, j: int, A_ij, Y_ij, Z_ij) -> None:
        """Patch (i, j) becomes quantised: A_ij [bw, 4], Y_ij [bw, P, r], Z_ij [bw, r, Q]."""
        if self.inter_dimension is None:
            self._init_bqq_tensors(Y_ij.shape[-1])
        dev = self.float_weight.device
        with torch.no_grad():
            self.Y[:, i, j] = (Y_ij > 0.5).to(dev)
            self.Z[:, i, j] = (Z_ij > 0.5).to(dev)
            for n, name in enumerate('abc'):
                getattr(self, name).data[:, i, j, 0, 0] = A_ij[:, n].to(dev)
            self.d.data[i, j, 0, 0] = A_ij[:, 3].sum().to(dev)      # one offset per patch, as BinaryQuadratic
            self.quantized_mask[i, j] = True

    def _bqq_weight(self, dtype):
        return _dense_weight(self.Y, self.Z, self.a, self.b, self.c, self.d, dtype)

    def forward(self, X):
        dtype, dev = X.dtype, self.float_weight.device
        none_done = self.inter_dimension is None or not bool(self.quantized_mask.any())
        if none_done:
            W = self.float_weight.to(dtype)
        else:
            W = self._bqq_weight(dtype)
            if not bool(self.quantized_mask.all()):
                per_entry = self.quantized_mask.repeat_interleave(self.y_row, 0).repeat_interleave(self.z_col, 1)
                W = torch.where(per_entry, W, self.float_weight.to(dtype))
        out = X.to(dev) @ W.T
        if self.bias_param is not None:
            out = out + self.bias_param.to(dtype=dtype, device=dev)
        return out

    def to_binaryquadratic(self) -> BinaryQuadratic:
        """The finished layer as this package's BinaryQuadratic; raises while patches are missing."""
        missing = int((~self.quantized_mask).sum())
        if missing:
            raise RuntimeError(f'to_binaryquadratic() called but {missing} patches are still unquantized')
        return _binaryquadratic_from_parts(self.Y, self.Z, self.a.data, self.b.data, self.c.data, self.d.data,
                                           self.bias_param.data if self.bias_param is not None else None)


def merge_binary_quadratic(diff_layer: BinaryQuadratic, quant_layer: BinaryQuadratic) -> BinaryQuadratic:
    """Bit-depth extension: the bit layers of `diff_layer` (fitted to the residual) are appended to
    those of `quant_layer`; d adds up; the bias is quant_layer's (src/bqq_modules.py:449-463).

    The reference builds the result through the (Y, Z, A) constructor and concatenates a 4-D with a
    5-D tensor on the way, so its version raises for every input.  This one returns the layer that
    code describes: bit layers [quant..., diff...] and d = quant.d + diff.d."""
    if (quant_layer.Y.shape[1:] != diff_layer.Y.shape[1:]) or (quant_layer.Z.shape[1:] != diff_layer.Z.shape[1:]):
        raise ValueError('merge_binary_quadratic: layers differ in patch grid or patch geometry')
    cat = lambda name: torch.cat([getattr(quant_layer, name).data, getattr(diff_layer, name).data], dim=0)  # noqa: E731
    return _binaryquadratic_from_parts(torch.cat([quant_layer.Y, diff_layer.Y], 0),
                                       torch.cat([quant_layer.Z, diff_layer.Z], 0),
                                       cat('a'), cat('b'), cat('c'), quant_layer.d.data + diff_layer.d.data,
                                       quant_layer.bias.data if quant_layer.bias is not None else None)


def merge_binaryquadratic_recursive(model_q: nn.Module, model_d: nn.Module, prefix=''):
    """Merge every BinaryQuadratic of `model_d` into its namesake in `model_q`, in place
    (src/bqq_modules.py:466-479)."""
    for (name_q, child_q), (name_d, child_d) in zip(list(model_q.named_children()), list(model_d.named_children())):
        if name_q != name_d:
            raise AssertionError(f'Module name mismatch: {name_q} != {name_d}')
        full = f'{prefix}.{name_q}' if prefix else name_q
        if isinstance(child_q, BinaryQuadratic) and isinstance(child_d, BinaryQuadratic):
            setattr(model_q, name_q, merge_binary_quadratic(child_d, child_q))
        else:
            merge_binaryquadratic_recursive(child_q, child_d, prefix=full)
    return model_q


# The {-1,+1} layers of the reference's vision workflow (src/bqq_modules.py:514-736: transform_A,
# SymQuantSTE, BQQLinear, BQQLinearInference) are a different layer family with its own training
# code and are not implemented here.  So that scripts which import them beside BinaryQuadratic
# still run, they are taken from a checkout of the reference when BQQ_REFERENCE_SRC names its
# `src` directory; without it the import fails with a message that says so.
_REFERENCE_ONLY = ('transform_A', 'SymQuantSTE', 'BQQLinear', 'BQQLinearInference')
_reference_module = None


def _load_reference_module():
    global _reference_module
    if _reference_module is None:
        import importlib.util
        import os
        src = os.environ.get('BQQ_REFERENCE_SRC', '')
        path = os.path.join(src, 'bqq_modules.py')
        if not src or not os.path.exists(path):
            raise ImportError(
                'bqq_b200: ' + ', '.join(_REFERENCE_ONLY) + ' belong to the reference\'s {-1,+1} vision layers, '
                'which this package does not implement; set BQQ_REFERENCE_SRC to the reference\'s '
                'neural_network_compression/src directory to have them loaded from there')
        spec = importlib.util.spec_from_file_location('_bqq_reference_modules', path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        _reference_module = module
    return _reference_module


def __getattr__(name):
    if name in _REFERENCE_ONLY:
        return getattr(_load_reference_module(), name)
    raise AttributeError(f'module {__name__!r} has no attribute {name!r}')


def shard_rows(bq: BinaryQuadratic, rank: int, world: int) -> BinaryQuadratic:
    """Column-parallel shard: rank `rank` of `world` keeps the output-row patches
    i in [rank*rw/world, (rank+1)*rw/world).  Row patches never interact, so the
    concatenation of the shard outputs equals the unsharded output exactly."""
    rw = bq.row_width
    if rw % world != 0:
        raise ValueError(f'row_width {rw} is not divisible by world size {world}')
    per = rw // world
    lo, hi = rank * per, (rank + 1) * per
    out = BinaryQuadratic.__new__(BinaryQuadratic)
    nn.Module.__init__(out)
    out.bit_width, out.row_width, out.col_width = bq.bit_width, per, bq.col_width
    out.y_row, out.inter_dimension, out.z_col = bq.y_row, bq.inter_dimension, bq.z_col
    out.register_buffer('Y', bq.Y[:, lo:hi].contiguous())
    out.register_buffer('Z', bq.Z[:, lo:hi].contiguous())
    out.a = nn.Parameter(bq.a.data[:, lo:hi].contiguous())
    out.b = nn.Parameter(bq.b.data[:, lo:hi].contiguous())
    out.c = nn.Parameter(bq.c.data[:, lo:hi].contiguous())
    out.d = nn.Parameter(bq.d.data[lo:hi].contiguous())
    out.bias = (nn.Parameter(bq.bias.data[lo * bq.y_row:hi * bq.y_row].contiguous())
                if bq.bias is not None else None)
    return out
