"""GPU: the decode entry point that brings its own scratch (bqq_forward_decode_noalloc).

Some callers cannot hand the library a workspace because they cannot allocate device memory
where the call happens (an operator hosted by a runtime that passes only inputs and outputs,
code in a section where allocation is forbidden).  The variant keeps its scratch in a fixed
8 MiB array inside the library.  This test calls it through the C ABI twice in a row, with
different inputs, and compares each result with the regular entry point; it also checks that
a layer needing more than the fixed array is rejected with the dedicated error code.

Collected last on purpose (file name), so a run that stops at the first failure has already
run every other test; it does not depend on them and also passes alone in a fresh process.
"""
import pytest
import torch

from tests.helpers import synth_layer

pytestmark = pytest.mark.gpu


def _call(fn, layer, x, out_f, *extra):
    from bqq_b200 import _cabi
    y = torch.empty((x.shape[0], out_f), dtype=x.dtype, device=x.device)
    code = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16}[x.dtype]
    rc = fn(layer, x.data_ptr(), code, x.shape[0], x.stride(0), y.data_ptr(), code, y.stride(0), *extra,
            torch.cuda.current_stream().cuda_stream)
    return rc, y


def test_noalloc_matches_workspace_entry_point_twice():
    from bqq_b200 import _cabi
    from bqq_b200.bqq_modules import BinaryQuadratic
    lib = _cabi.lib
    assert lib.bqq_noalloc_scratch_bytes() == 8 << 20
    Y, Z, A, bias, _ = synth_layer(2, 16, 24, 32, 32, 32, 1, seed=31, bias=True)
    bq = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias).cuda()
    st = bq._ensure_packed()
    layer = bq._layer(st)
    out_f = 16 * 32
    gen = torch.Generator().manual_seed(77)
    for M, dt in ((1, torch.float32), (5, torch.bfloat16)):          # two calls in a row, different shapes
        x = torch.randn(M, 24 * 32, generator=gen).to(dt).cuda()
        need = lib.bqq_decode_workspace_bytes(st.dims, M)
        assert need <= lib.bqq_noalloc_scratch_bytes()
        ws = torch.zeros(need, dtype=torch.uint8, device='cuda')
        rc_ref, y_ref = _call(lib.bqq_forward_decode, layer, x, out_f, ws.data_ptr(), ws.numel())
        rc_new, y_new = _call(lib.bqq_forward_decode_noalloc, layer, x, out_f)
        torch.cuda.synchronize()
        assert rc_ref == 0 and rc_new == 0, (_cabi.strerror(rc_ref), _cabi.strerror(rc_new))
        scale = y_ref.float().abs().max().item()
        # same kernels, same reduction order: identical up to the tolerance the other decode tests use
        assert (y_new.float() - y_ref.float()).abs().max().item() <= 1e-4 * scale
        assert torch.equal(y_new, y_ref)
    # no bounded wait gave up in either call; the report synchronises the stream
    assert lib.bqq_noalloc_status(torch.cuda.current_stream().cuda_stream) == 0


def test_noalloc_rejects_oversized_request():
    from bqq_b200 import _cabi
    lib = _cabi.lib
    big = _cabi.dims(4, 1024, 448, 32, 32, 32)                        # 16 rows of X need > 8 MiB of partial sums
    assert lib.bqq_decode_workspace_bytes(big, 16) > lib.bqq_noalloc_scratch_bytes()
    dummy = torch.zeros(1024, dtype=torch.uint8, device='cuda')
    p = dummy.data_ptr()
    layer = _cabi.BqqLayer(big, p, p, p, p, p, p, None, 0, 0)
    rc = lib.bqq_forward_decode_noalloc(layer, p, _cabi.BF16, 16, 448 * 32, p, _cabi.BF16, 1024 * 32, None)
    assert rc == -10 and 'scratch' in _cabi.strerror(rc)
    # a bad argument is refused before anything is enqueued (here: a NULL activation pointer)
    small = _cabi.dims(2, 4, 4, 32, 32, 32)
    layer = _cabi.BqqLayer(small, p, p, p, p, p, p, None, 0, 0)
    assert lib.bqq_forward_decode_noalloc(layer, None, _cabi.BF16, 1, 128, p, _cabi.BF16, 128, None) == -1
    assert lib.bqq_noalloc_status(None) == 0
