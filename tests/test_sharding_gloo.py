"""CPU, world_size 2 (gloo): the host-side logic of the column-parallel path - row-patch
ranges, shard construction, and the all-gather layout - with the oracle standing in for the
per-rank compute (the CUDA forward itself cannot run here)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import bqq_oracle as O
from tests.helpers import synth_layer


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, result_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from bqq_b200.bqq_modules import BinaryQuadratic
        from bqq_b200.sharded import ColumnParallelBinaryQuadratic, gather_columns, row_patch_range
        Y, Z, A, bias, X = synth_layer(2, 8, 6, 32, 32, 32, 3, seed=21, bias=True)
        full = BinaryQuadratic(Y.float(), Z.float(), A, bias=bias)
        cp = ColumnParallelBinaryQuadratic(full, rank, world)
        lo, hi = row_patch_range(8, rank, world)
        sh = cp.shard
        assert sh.row_width == hi - lo and sh.Y.shape[1] == hi - lo
        assert torch.equal(sh.Y, full.Y[:, lo:hi]) and torch.equal(sh.d.data, full.d.data[lo:hi])
        assert torch.equal(sh.bias.data, full.bias.data[lo * 32:hi * 32])
        # per-rank compute by the oracle on the shard's tensors, then the real gather code
        a, b, c, d = (getattr(sh, n).detach().numpy() for n in 'abcd')
        y_local = O.forward(sh.Y.numpy(), sh.Z.numpy(), a, b, c, d, X.numpy(), sh.bias.detach().numpy())
        y_local = torch.from_numpy(y_local).reshape(1, 3, -1)         # leading dims survive the gather
        y = gather_columns(y_local)
        a, b, c, d = O.split_coefficients(A.numpy())
        ref = O.forward(Y.numpy(), Z.numpy(), a, b, c, d, X.numpy(), bias.numpy()).reshape(1, 3, -1)
        assert tuple(y.shape) == (1, 3, 256)
        np.testing.assert_array_equal(y.numpy(), ref)                  # exact: no reduction is involved
        with open(os.path.join(result_dir, f'ok{rank}'), 'w') as f:
            f.write('ok')
    finally:
        dist.destroy_process_group()


def test_column_parallel_host_logic_world2(tmp_path):
    world = 2
    mp.start_processes(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True,
                       start_method='spawn')
    assert all((tmp_path / f'ok{r}').exists() for r in range(world))


def test_row_patch_range_errors():
    from bqq_b200.sharded import row_patch_range
    assert row_patch_range(32, 3, 8) == (12, 16)
    with pytest.raises(ValueError):
        row_patch_range(30, 0, 8)
