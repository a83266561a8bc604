"""ctypes binding of libbqq_b200.so (the C ABI declared in include/bqq_b200.h).

The library is built in-tree by bqq_b200/build.py.  There is no fallback: if the
shared object is missing, importing this module raises, and every wrapper turns a
non-zero return code into RuntimeError(bqq_strerror(rc)).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libbqq_b200.so')

F32, BF16, F16 = 0, 1, 2
DECODE_MAX_M = 16

EXPORTS = [
    'bqq_abi_version', 'bqq_strerror', 'bqq_device_supported',
    'bqq_zplane_words', 'bqq_yplane_words', 'bqq_algorithmic_bytes',
    'bqq_pack_planes', 'bqq_unpack_planes', 'bqq_pack_planes_host', 'bqq_unpack_planes_host', 'bqq_pack_patch_host',
    'bqq_repack_u8_planes',
    'bqq_decode_workspace_bytes', 'bqq_forward_decode', 'bqq_forward_decode_fused',
    'bqq_prefill_workspace_bytes', 'bqq_forward_prefill',
    'bqq_forward_workspace_bytes', 'bqq_forward', 'bqq_reconstruct_weight',
    'bqq_decode_launches', 'bqq_instruction_rate', 'bqq_attention_decode_workspace_bytes', 'bqq_attention_decode', 'bqq_attention_decode_gathered', 'bqq_forward_host_workspace_bytes', 'bqq_forward_host',
    'bqq_noalloc_scratch_bytes', 'bqq_forward_decode_noalloc', 'bqq_noalloc_status',
    'bqq_decode_status', 'bqq_prefill_status',
    'bqq_peer_region_bytes', 'bqq_peer_alloc', 'bqq_peer_open', 'bqq_peer_close', 'bqq_peer_free',
    'bqq_peer_gather', 'bqq_peer_status', 'bqq_forward_decode_gathered',
]


class BqqDims(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ('bw', 'rw', 'cw', 'P', 'Q', 'r')]


class BqqLayer(C.Structure):
    _fields_ = [('dims', BqqDims), ('zplanes', C.c_void_p), ('yplanes', C.c_void_p),
                ('a', C.c_void_p), ('b', C.c_void_p), ('c', C.c_void_p), ('d', C.c_void_p),
                ('bias', C.c_void_p), ('coef_dtype', C.c_int32), ('bias_dtype', C.c_int32)]


PRO_NONE, PRO_RMSNORM, PRO_SWIGLU = 0, 1, 2


class BqqFusion(C.Structure):
    _fields_ = [('prologue', C.c_int32), ('norm_dtype', C.c_int32), ('norm_weight', C.c_void_p), ('eps', C.c_float),
                ('residual_dtype', C.c_int32), ('residual', C.c_void_p), ('ld_residual', C.c_int64),
                ('out_segments', C.c_int32)]


MAX_PEERS = 8
PEER_HANDLE_BYTES = 64


class BqqPeerGroup(C.Structure):
    _fields_ = [('rank', C.c_int32), ('world', C.c_int32), ('regions', C.c_void_p * MAX_PEERS),
                ('gather_bytes', C.c_uint64), ('wait_cycles', C.c_uint64)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f'{LIB_PATH} is missing: build it with `python -m bqq_b200.build` '
            '(needs nvcc); bqq_b200 has no fallback path')
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, sz, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float
    dp, lp = C.POINTER(BqqDims), C.POINTER(BqqLayer)
    sig = {
        'bqq_abi_version': (C.c_int, []),
        'bqq_strerror': (C.c_char_p, [i32]),
        'bqq_device_supported': (C.c_int, []),
        'bqq_zplane_words': (sz, [dp]), 'bqq_yplane_words': (sz, [dp]),
        'bqq_algorithmic_bytes': (sz, [dp]),
        'bqq_pack_planes': (i32, [vp, vp, dp, vp, vp, vp, vp, vp]),
        'bqq_unpack_planes': (i32, [vp, vp, dp, vp, vp, vp]),
        'bqq_pack_planes_host': (i32, [vp, vp, dp, vp, vp, vp, vp]),
        'bqq_unpack_planes_host': (i32, [vp, vp, dp, vp, vp]),
        'bqq_pack_patch_host': (i32, [vp, vp, dp, i32, i32, i32, vp, vp]),
        'bqq_repack_u8_planes': (i32, [vp, vp, dp, vp, vp, vp, vp, vp]),
        'bqq_decode_workspace_bytes': (sz, [dp, i32]),
        'bqq_prefill_workspace_bytes': (sz, [dp, i32]),
        'bqq_forward_workspace_bytes': (sz, [dp, i32]),
        'bqq_forward_decode': (i32, [lp, vp, i32, i32, i64, vp, i32, i64, vp, sz, vp]),
        'bqq_forward_decode_fused': (i32, [lp, vp, i32, i32, i64, vp, i32, i64, C.POINTER(BqqFusion), vp, sz, vp]),
        'bqq_forward_prefill': (i32, [lp, vp, i32, i32, i64, vp, i32, i64, vp, sz, vp]),
        'bqq_forward': (i32, [lp, vp, i32, i32, i64, vp, i32, i64, vp, sz, vp]),
        'bqq_reconstruct_weight': (i32, [lp, vp, i32, f32, vp]),
        'bqq_decode_launches': (i32, [dp, i32]),
        'bqq_instruction_rate': (i32, [i32, i32, C.POINTER(C.c_double), vp]),
        'bqq_attention_decode_workspace_bytes': (C.c_size_t, [i32, i32, i32]),
        'bqq_attention_decode': (i32, [vp, i64, vp, vp, i64, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp, i64, vp,
                                       C.c_size_t, vp]),
        'bqq_attention_decode_gathered': (i32, [vp, vp, i64, vp, vp, i64, i32, vp, vp, vp, i32, i32, i32, i32, i32, vp,
                                                i64, vp, i64, vp, C.c_size_t, vp]),
        'bqq_forward_host_workspace_bytes': (sz, [dp, i32, i32, i32]),
        'bqq_forward_host': (i32, [lp, vp, i32, i32, i64, vp, i32, i64, vp, sz, vp]),
        'bqq_peer_region_bytes': (sz, [sz]),
        'bqq_peer_alloc': (i32, [sz, C.POINTER(vp), C.c_char_p]),
        'bqq_peer_open': (i32, [C.c_char_p, C.POINTER(vp)]),
        'bqq_peer_close': (i32, [vp]),
        'bqq_peer_free': (i32, [vp]),
        'bqq_peer_gather': (i32, [C.POINTER(BqqPeerGroup), vp, i32, i32, i64, i64, vp, i64, vp]),
        'bqq_peer_status': (i32, [C.POINTER(BqqPeerGroup), vp]),
        'bqq_forward_decode_gathered': (i32, [lp, vp, i32, i32, i64, vp, i32, i64, C.POINTER(BqqFusion),
                                            C.POINTER(BqqPeerGroup), vp, i64, vp, sz, vp]),
        'bqq_noalloc_scratch_bytes': (sz, []),
        'bqq_forward_decode_noalloc': (i32, [lp, vp, i32, i32, i64, vp, i32, i64, vp]),
        'bqq_noalloc_status': (i32, [vp]),
        'bqq_decode_status': (i32, [vp, vp]),
        'bqq_prefill_status': (i32, [vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def strerror(rc: int) -> str:
    return lib.bqq_strerror(rc).decode()


def check(rc: int, what: str = 'bqq call') -> None:
    if rc != 0:
        raise RuntimeError(f'{what} failed: {strerror(rc)} (code {rc})')


def dims(bw, rw, cw, P, Q, r) -> BqqDims:
    return BqqDims(int(bw), int(rw), int(cw), int(P), int(Q), int(r))
