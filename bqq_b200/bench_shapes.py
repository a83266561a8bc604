"""Per-shape decode timings: one layer shape at a time, enough distinct copies of the layer to exceed the L2,
all forwards of the copies captured in one CUDA graph, CUDA-event time per forward.

    python -m bqq_b200.bench_shapes              # batch 1, 4 and 16 over the BASELINE decode shapes
    python -m bqq_b200.bench_shapes 1            # batch 1 only
"""
from __future__ import annotations

import sys

import torch

from . import _cabi
from .profile_layer import synthetic_layer

SHAPES = [(2048, 2048, 2), (2048, 2048, 4), (2048, 6144, 2), (6144, 2048, 2), (4096, 4096, 2), (4096, 14336, 2),
          (4096, 14336, 4)]


def time_shape(out_f, in_f, bits, batches, device, peak_gbs=None):
    dims = _cabi.dims(bits, out_f // 32, in_f // 32, 32, 32, 32)
    nbytes = _cabi.lib.bqq_algorithmic_bytes(dims)
    ncopies = max(2, int(300e6 // nbytes) + 1)
    layers = [synthetic_layer(out_f, in_f, bits, device, seed=s) for s in range(ncopies)]
    for L in layers:
        L._ensure_packed()
    stream = torch.cuda.Stream(device)
    rows = []
    for M in batches:
        x = torch.randn(M, in_f, device=device, dtype=torch.bfloat16)
        with torch.cuda.stream(stream), torch.no_grad():
            for L in layers:
                L(x)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for L in layers:
                    L(x)
            for _ in range(3):
                graph.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(10):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            graph.reset()
        us = e0.elapsed_time(e1) * 1e3 / (10 * ncopies)
        total = nbytes + M * (in_f + out_f) * 2
        rows.append((M, us, total / us / 1e3))
    return rows


def main():
    batches = [int(a) for a in sys.argv[1:]] or [1, 4, 16]
    device = torch.device('cuda', 0)
    for (o, i, b) in SHAPES:
        for (M, us, gbs) in time_shape(o, i, b, batches, device):
            print(f'{o}x{i}, {b} bit layers, batch {M}: {us:8.2f} us/forward  {gbs:8.1f} GB/s', flush=True)
        torch.cuda.empty_cache()


if __name__ == '__main__':
    main()
