"""GPU: the peer-to-peer column gather (bqq_peer_gather).  A one-rank group runs the whole protocol
(own slots) on a single GPU; with two or more GPUs a two-process run checks the gathered values against
every rank's slice, repeated gathers, and CUDA-graph replay.  The time-out path is exercised in one
process against a region that nobody writes."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _slice(rank, step, rows, n, dtype):
    g = torch.Generator().manual_seed(1000 * step + rank)
    return torch.randn(rows, n, generator=g).to(dtype)


def _worker(rank, world, port, result_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)      # host channel for the handles only
    try:
        from bqq_b200.peer import PeerGatherGroup
        dev = torch.device('cuda', rank)
        torch.cuda.set_device(dev)
        grp = PeerGatherGroup(16 * world * 1024 * 4, dev)
        step = 0
        for rows, n, dtype in [(1, 512, torch.bfloat16), (4, 1024, torch.float32), (3, 130, torch.float16),
                               (16, 1024, torch.bfloat16)]:
            for _ in range(3):                                        # back-to-back gathers reuse the buffers
                step += 1
                y = _slice(rank, step, rows, n, dtype).to(dev)
                got = grp.gather(y)
                want = torch.cat([_slice(q, step, rows, n, dtype) for q in range(world)], dim=-1)
                assert torch.equal(got.cpu(), want), (rank, step)
        # strided input, leading dims, caller-provided output
        step += 1
        wide = torch.zeros(2, 3, 96, dtype=torch.bfloat16, device=dev)
        wide[..., :64] = _slice(rank, step, 6, 64, torch.bfloat16).view(2, 3, 64).to(dev)
        out = torch.empty(6, world * 64, dtype=torch.bfloat16, device=dev)
        got = grp.gather(wide[..., :64], out=out)
        want = torch.cat([_slice(q, step, 6, 64, torch.bfloat16) for q in range(world)], dim=-1).view(2, 3, -1)
        assert got.data_ptr() == out.data_ptr() and torch.equal(got.cpu(), want)
        # graph capture and replay: the sequence number lives on the device
        y = torch.zeros(1, 256, dtype=torch.bfloat16, device=dev)
        out = torch.empty(1, world * 256, dtype=torch.bfloat16, device=dev)
        st = torch.cuda.Stream(dev)
        with torch.cuda.stream(st):
            grp.gather(y, out=out)
            st.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                grp.gather(y, out=out)
            for rep in range(4):
                step += 1
                y.copy_(_slice(rank, step, 1, 256, torch.bfloat16))
                graph.replay()
                st.synchronize()
                want = torch.cat([_slice(q, step, 1, 256, torch.bfloat16) for q in range(world)], dim=-1)
                assert torch.equal(out.cpu(), want), (rank, 'replay', rep)
            graph.reset()
            grp.status()
        # the forward with the gather built in: every rank's shard sends its row patches from the decode
        # kernel's epilogue; the result equals the unsharded layer bit for bit
        from bqq_b200.bqq_modules import BinaryQuadratic, shard_rows
        from tests.helpers import synth_layer
        for (bw, rw, cw, M, dtype, bias) in [(2, 8, 6, 1, torch.bfloat16, True), (3, 4, 136, 1, torch.float32, False),
                                             (2, 8, 6, 5, torch.float16, True), (2, 6, 40, 16, torch.bfloat16, False)]:
            Y, Z, A, b, X = synth_layer(bw, rw, cw, 32, 32, 32, M, seed=31, bias=bias)
            full = BinaryQuadratic(Y.float(), Z.float(), A, bias=b if bias else None).to(dev)
            Xd = X.to(dtype).to(dev)
            with torch.no_grad():
                want = full(Xd)
                shard = shard_rows(full, rank, world)
                for _ in range(2):
                    got = shard.forward_gathered(Xd, grp)
                    assert torch.equal(got, want), (rank, bw, rw, cw, M)
                # fused normalisation on the way in and residual on the way out, against the unsharded fused call
                gen = torch.Generator().manual_seed(77)
                w = (1 + 0.1 * torch.randn(cw * 32, generator=gen)).to(dtype).to(dev)
                h = torch.randn(M, rw * 32, generator=gen).to(dtype).to(dev)
                want = full.forward_fused(Xd, rms_weight=w, residual=h)
                got = shard.forward_gathered(Xd, grp, rms_weight=w, residual=h)
                assert torch.equal(got, want), (rank, 'fused', bw, rw, cw, M)
        # a stacked [gate ; up] layer: every rank holds [gate rows of its slice ; up rows of its slice]; gathered in two
        # segments the result is the unsharded layer's [gate | up] row
        bw, rw, cw = 2, 8 * world, 6
        Y, Z, A, _, X = synth_layer(bw, rw, cw, 32, 32, 32, 3, seed=47)
        full = BinaryQuadratic(Y.float(), Z.float(), A).to(dev)
        half, per = rw // 2, rw // 2 // world
        idx = torch.cat([torch.arange(rank * per, (rank + 1) * per), half + torch.arange(rank * per, (rank + 1) * per)])
        shard = BinaryQuadratic(Y[:, idx].float(), Z[:, idx].float(), A[:, idx]).to(dev)
        Xd = X.to(torch.bfloat16).to(dev)
        with torch.no_grad():
            want = full(Xd)
            got = shard.forward_gathered(Xd, grp, out_segments=2)
            assert torch.equal(got, want), (rank, 'two segments')
        # single-token attention with heads sharded over the ranks: the gathered launch returns every rank's heads,
        # bit for bit what each rank's own launch computes (all ranks' inputs come from seeds, so this rank can
        # compute the others' heads itself)
        from bqq_b200.decoder_stack import attention_decode
        hd, max_seq, lh, lkv = 128, 96, 4, 1
        ang = torch.arange(max_seq).float()[:, None] * (1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd)))[None, :]
        cos, sin = ang.cos().to(torch.bfloat16).to(dev), ang.sin().to(torch.bfloat16).to(dev)

        def inputs(q, B):
            g = torch.Generator().manual_seed(900 + q)
            return (torch.randn(B, 1, lh + 2 * lkv, hd, generator=g).to(torch.bfloat16).to(dev),
                    torch.randn(B, max_seq, lkv, hd, generator=g).to(torch.bfloat16).to(dev),
                    torch.randn(B, max_seq, lkv, hd, generator=g).to(torch.bfloat16).to(dev))
        for B, pos in ((1, 0), (2, 70), (1, 95)):
            lens = torch.full((B,), pos, dtype=torch.int32, device=dev)
            want = []
            for q in range(world):
                qkv, kc, vc = inputs(q, B)
                want.append(attention_decode(qkv, kc, vc, cos, sin, lens, lh, lkv))
            want = torch.cat(want, dim=2)
            for _ in range(2):
                qkv, kc, vc = inputs(rank, B)
                got = attention_decode(qkv, kc, vc, cos, sin, lens, lh, lkv, peer=grp)
                torch.cuda.synchronize()
                assert got.shape == (B, 1, world * lh, hd) and torch.equal(got, want), (rank, 'attention', B, pos)
        grp.status()
        grp.close()
        with open(os.path.join(result_dir, f'ok{rank}'), 'w') as f:
            f.write('ok')
    finally:
        dist.destroy_process_group()


def _run(world, tmp_path):
    mp.start_processes(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True,
                       start_method='spawn')
    assert all((tmp_path / f'ok{r}').exists() for r in range(world))


def test_peer_gather_single_rank(tmp_path):
    _run(1, tmp_path)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_peer_gather_two_ranks(tmp_path):
    _run(2, tmp_path)


def test_wait_on_a_silent_peer_runs_out_and_is_reported():
    """Failure detection without a fault: a two-rank group whose second region is a local buffer that no
    rank ever writes.  The gather's polls on that rank's slots run out after the group's clock budget
    (a few milliseconds here), the kernel ends normally, bqq_peer_status reports BQQ_ERR_TIMEOUT, and a
    fresh group on the same GPU works afterwards."""
    import ctypes as C

    from bqq_b200 import _cabi
    lib = _cabi.lib
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    gather_bytes = 2 * 256 * 4
    regions = []
    for _ in range(2):
        ptr, handle = C.c_void_p(), C.create_string_buffer(_cabi.PEER_HANDLE_BYTES)
        _cabi.check(lib.bqq_peer_alloc(gather_bytes, C.byref(ptr), handle), 'bqq_peer_alloc')
        regions.append(ptr.value)
    try:
        silent = _cabi.BqqPeerGroup(0, 2, (C.c_void_p * _cabi.MAX_PEERS)(*regions), gather_bytes, 5_000_000)
        y = torch.arange(256, dtype=torch.float32, device=dev).reshape(1, 256)
        out = torch.full((1, 512), -1.0, device=dev)
        _cabi.check(lib.bqq_peer_gather(C.byref(silent), y.data_ptr(), _cabi.F32, 1, 256, 256, out.data_ptr(), 512, stream),
                    'bqq_peer_gather')
        torch.cuda.synchronize()                                  # the kernel returns by itself
        assert lib.bqq_peer_status(C.byref(silent), stream) == -8     # BQQ_ERR_TIMEOUT
        assert _cabi.strerror(-8) == 'a bounded device-side wait gave up'
        assert torch.equal(out[:, :256], y)                       # the own slice still arrived
        # the context is intact: a one-rank group on a fresh region gathers correctly, twice
        alone = _cabi.BqqPeerGroup(0, 1, (C.c_void_p * _cabi.MAX_PEERS)(regions[1]), gather_bytes, 0)
        for rep in range(2):
            out1 = torch.empty(1, 256, device=dev)
            _cabi.check(lib.bqq_peer_gather(C.byref(alone), (y + rep).data_ptr(), _cabi.F32, 1, 256, 256, out1.data_ptr(),
                                            256, stream), 'bqq_peer_gather')
            assert lib.bqq_peer_status(C.byref(alone), stream) == 0
            assert torch.equal(out1, y + rep)
    finally:
        torch.cuda.synchronize()
        for p in regions:
            lib.bqq_peer_free(p)
