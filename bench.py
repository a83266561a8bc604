"""Benchmark of the BinaryQuadratic forward on B200.

Headline workload ("decode_sweep_b1"): the decode GEMV sweep of synthetic BinaryQuadratic layers
  shapes 2048x2048, 2048x6144, 6144x2048, 4096x14336 (out x in), 2/3/4 bit layers,
  P=Q=r=32, Bernoulli(0.5) bits, N(0,0.02) fp32 coefficients, bf16 activations, batch 1.
A step is one forward through all 12 layers, replayed from a CUDA graph.  The 12 layers hold
208.5 MB of packed bits + coefficients, more than the 126 MB L2, so every step streams them from
HBM again.  The `--steps` block is repeated until about half a second has been timed; the median
block gives `ms_per_step`, the spread is reported beside it.

value  = algorithmic bytes (packed bits + fp32 coefficients + x + y) per second, summed over
         all ranks, inputs resident in HBM, timed with CUDA events on the launching stream.
e2e    = the same with HOST activations and outputs every layer, every step: pinned x is read,
         the forward runs, y lands in pinned host memory (one GPU: module.bind_host, i.e. the C
         entry point bqq_forward_host; several GPUs: the gathered forward on device-visible
         aliases of the pinned buffers).  The step is captured once and replayed, one stream
         synchronisation per step to read the outputs.
With N > 1 ranks (weak scaling) each rank owns one row-patch shard of layers N times as tall
(its shard has the base shape) and every layer's outputs are gathered on all ranks by the
library's peer-to-peer stores (NCCL only carries the set-up, the value check and the timing
reduction).  Before timing, every gathered output is compared with the ranks' own slices
(all-gathered once over NCCL): `gather_check` must be "exact".

The same JSON line carries, beside the headline: the sweep at batch 4 and 16, the prefill
configuration (2048 tokens on 4096x4096, 2 bit layers), the bit-depth-extended large layers
(8192x28672 and 28672x8192, 2+1 bit layers, r=64, batch 1 and 32, sharded over the ranks) and
the decoder stack (tokens/s, strong scaling).  `--no-extras` skips them.

Other workloads (each prints its own lines, no JSON contract):
  --workload layer --out O --in I --bits B --batch M [--group G --rank R]   one layer, a few forwards
                                                                             (the program to put under a profiler)
  --workload shapes [--batches 1 4 16]                                       per-shape decode table

`--impl reference` times the CPU port of the reference algorithm (oracle/bqq_oracle.c,
dense-weight rebuild + matmul, all host threads) on the same 12 layers.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(2048, 2048), (2048, 6144), (6144, 2048), (4096, 14336)]   # (out, in)
BITS = [2, 3, 4]
P = Q = R = 32
PEER_TIMEOUT = False   # set when a bounded wait of the peer gather gave up (reported in the JSON line)
# DRAM bytes / algorithmic bytes of the decode kernel: a constant taken from one ncu capture of the largest
# layer (dram read + write 62.09 MB for 61.72 MB algorithmic), not a measurement of this run
TRAFFIC_RATIO = 62.09 / 61.72
MIN_TIMED_SECONDS = 0.5
DTYPE_NOTE = 'fixed16 x fixed23 on int8 tensor-core MMAs (exact s32), fp32 across patches'


def sweep():
    return [(o, i, bw) for (o, i) in SHAPES for bw in BITS]


def alg_bytes(out_f, in_f, bw, M=1, act_bytes=2, group=32, rank=None):
    rank = group if rank is None else rank
    rw, cw = out_f // group, in_f // group
    bits = bw * rw * cw * (group * rank + rank * group)
    return bits // 8 + 4 * rw * cw * (3 * bw + 1) + M * (in_f + out_f) * act_bytes


def peaks():
    try:
        with open(os.path.join(ROOT, 'MEASURED_PEAKS.json')) as f:
            d = json.load(f)
            return float(d['hbm_gbs']), float(d.get('bf16_tflops', 1590.0)), 'measured'
    except Exception:
        return 6650.0, 1590.0, 'fallback'


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index=0):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--id={self.index}', f'--query-gpu={q}',
                                          '--format=csv,noheader,nounits', '-lms', '100'],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ['hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap']
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(',')]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith('active'):
                    reasons.add(n)
        sm.sort()
        return {'sm_mhz': sm[len(sm) // 2] if sm else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': sorted(reasons), 'samples': len(sm)}


def make_layer(out_f, in_f, bw, device, seed, group=32, rank=None, last_bit_scale=None):
    """Seeded synthetic layer built directly on the device (bits Bernoulli(0.5), coefficients N(0,0.02));
    `last_bit_scale`: standard deviation of the last bit layer's coefficients (a depth extension)."""
    import torch
    from bqq_b200.bqq_modules import BinaryQuadratic
    rank = group if rank is None else rank
    g = torch.Generator(device=device).manual_seed(seed)
    rw, cw = out_f // group, in_f // group
    Y = torch.rand(bw, rw, cw, group, rank, generator=g, device=device) > 0.5
    Z = torch.rand(bw, rw, cw, rank, group, generator=g, device=device) > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=g, device=device) * 0.02
    if last_bit_scale is not None:
        A[-1] *= last_bit_scale / 0.02
    layer = BinaryQuadratic(Y, Z, A)
    layer._ensure_packed()
    return layer


def drop_bool_factors(layer):
    """Free the dense bool Y / Z of a packed synthetic layer (32 times the planes' size); the planes stay."""
    import torch
    from bqq_b200.bqq_modules import _tensor_key
    dev = layer.Y.device
    layer.Y = torch.empty(0, dtype=torch.bool, device=dev)
    layer.Z = torch.empty(0, dtype=torch.bool, device=dev)
    layer._state().plane_key = (_tensor_key(layer.Y), _tensor_key(layer.Z))


def timed_blocks(replay, stream, min_seconds=MIN_TIMED_SECONDS, min_blocks=5, max_blocks=400, sync=None):
    """Time `replay()` (one block of steps) repeatedly with CUDA events on `stream` until `min_seconds`
    have been timed; returns the list of block times in ms.  `sync()` (optional) runs after each block
    inside the timed region (the end-to-end arm synchronises the stream there)."""
    import torch
    times = []
    total = 0.0
    while len(times) < min_blocks or (total < min_seconds * 1e3 and len(times) < max_blocks):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        replay()
        if sync is not None:
            sync()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1)
        times.append(ms)
        total += ms
    return times


def median(v):
    s = sorted(v)
    return s[len(s) // 2]


def cpu_port_time(layers_np, repeats=1, nthreads=0):
    """Seconds for one pass of the CPU port over the given layers (all host threads)."""
    from oracle import c_oracle
    t0 = time.perf_counter()
    for _ in range(repeats):
        for (Y, Z, a, b, c, d, X) in layers_np:
            c_oracle.forward(Y, Z, a, b, c, d, X, nthreads=nthreads)
    return (time.perf_counter() - t0) / repeats


def make_layer_np(out_f, in_f, bw, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    rw, cw = out_f // P, in_f // Q
    Y = rng.integers(0, 2, (bw, rw, cw, P, R), dtype=np.uint8)
    Z = rng.integers(0, 2, (bw, rw, cw, R, Q), dtype=np.uint8)
    A = (rng.standard_normal((bw, rw, cw, 4)) * 0.02).astype(np.float32)
    a, b, c = (A[..., k][..., None, None] for k in range(3))
    d = A[..., 3].sum(0)[..., None, None]
    X = rng.standard_normal((1, in_f)).astype(np.float32)
    return Y, Z, a, b, c, d, X


def run_reference(args):
    """CPU port of the reference algorithm on the same sweep; rank 0 only."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    from oracle import c_oracle
    cores = c_oracle.max_threads()
    layers = [make_layer_np(o, i, bw, 100 + n) for n, (o, i, bw) in enumerate(sweep())]
    total = sum(alg_bytes(o, i, bw) for (o, i, bw) in sweep())
    for _ in range(args.warmup):
        cpu_port_time(layers[:3])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_port_time(layers)
    dt = (time.perf_counter() - t0) / args.steps
    val = total / dt / 1e9
    line = {
        'impl': 'reference', 'metric': 'packed-weight HBM GB/s at batch 1', 'value': val, 'unit': 'GB/s',
        'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3,
        'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'decode_sweep_b1', 'layers': len(layers), 'P': P, 'Q': Q, 'r': R,
                   'activations': 'fp32 on this arm (the CPU port), bf16 on the GPU arm', 'batch': 1},
        'cpu_baseline': {'value': val, 'unit': 'GB/s', 'cores': cores, 'kind': 'port',
                         'sample': 'all 12 layers of the sweep per step',
                         'note': 'C port of the reference forward (dense W rebuild + matmul, pthreads); the '
                                 "reference's own Python forward is slower (see reference_python_forward)"},
        'e2e': {'value': val, 'unit': 'GB/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def reference_python_seconds():
    """Seconds of one forward of the reference's own Python module on a 2048x2048 layer with 2 bit layers
    (all host threads), when a checkout of the reference is available ($BQQ_REFERENCE_ROOT); else None."""
    ref = os.environ.get('BQQ_REFERENCE_ROOT')
    src = os.path.join(ref, 'neural_network_compression', 'src', 'bqq_modules.py') if ref else None
    if not src or not os.path.exists(src):
        return None
    import importlib.util
    import torch
    spec = importlib.util.spec_from_file_location('_ref_bqq_modules_bench', src)
    rm = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rm)
    g = torch.Generator().manual_seed(0)
    Y = (torch.rand(2, 64, 64, 32, 32, generator=g) > 0.5).float()
    Z = (torch.rand(2, 64, 64, 32, 32, generator=g) > 0.5).float()
    A = torch.randn(2, 64, 64, 4, generator=g) * 0.02
    layer = rm.BinaryQuadratic(Y, Z, A)
    x = torch.randn(1, 2048, generator=g)
    with torch.no_grad():
        layer(x)
        t0 = time.perf_counter()
        for _ in range(3):
            layer(x)
    return (time.perf_counter() - t0) / 3


def shutdown(world, graphs, peer=None):
    """Release captured graphs and the peer gather buffers before the communicator goes away, and
    never let teardown hang the job."""
    import torch
    import torch.distributed as dist
    for g in graphs:
        g.reset()
    torch.cuda.synchronize()
    if world > 1:
        timer = threading.Timer(30.0, lambda: os._exit(0))
        timer.daemon = True
        timer.start()
        if peer is not None:
            try:
                peer.status()          # raises if a bounded wait on a peer gave up during the run
            except RuntimeError as exc:
                print(f'bench: {exc}: the gathered outputs of this run are not valid', file=sys.stderr)
                global PEER_TIMEOUT
                PEER_TIMEOUT = True
            peer.close()
        dist.barrier()
        dist.destroy_process_group()
        timer.cancel()


def host_alias(t):
    """CUDA tensor that aliases a pinned host tensor (unified addressing: the device sees pinned host
    memory at its host address); kernels that get it read or write host memory directly."""
    import torch

    class _Iface:
        pass

    obj = _Iface()
    flat = t.view(torch.int16) if t.element_size() == 2 else t.view(torch.int32)
    obj.__cuda_array_interface__ = {'shape': tuple(flat.shape), 'typestr': '<i2' if t.element_size() == 2 else '<i4',
                                    'data': (flat.data_ptr(), False), 'version': 2}
    alias = torch.as_tensor(obj, device='cuda')
    alias._host_keepalive = t
    return alias.view(t.dtype)


# ---------------------------------------------------------------------------------------------------
# other workloads
# ---------------------------------------------------------------------------------------------------

def run_layer(args):
    """A few forwards of one synthetic layer: the program to put under a profiler."""
    import torch
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    layer = make_layer(args.out, args.inp, args.bits, dev, seed=1, group=args.group, rank=args.rank)
    x = torch.randn(args.batch, args.inp, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        for _ in range(args.reps):
            y = layer(x)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.no_grad():
        e0.record()
        for _ in range(args.reps):
            y = layer(x)
        e1.record()
    torch.cuda.synchronize()
    print(f'{args.out}x{args.inp}, {args.bits} bit layers, group {args.group}, batch {args.batch}: '
          f'{e0.elapsed_time(e1) * 1e3 / args.reps:.1f} us per forward (same layer repeated, warm L2); '
          f'max |y| {float(y.float().abs().max()):.3f}')


def time_copies(out_f, in_f, bits, batches, device, group=32, rank=None, last_bit_scale=None, reps=10):
    """CUDA-event microseconds per forward of one layer shape: enough distinct copies of the layer to exceed
    the L2, all their forwards captured in one graph.  Returns {M: (us, GB/s)}."""
    import torch
    nbytes = alg_bytes(out_f, in_f, bits, M=0, group=group, rank=rank)
    ncopies = max(2, int(300e6 // nbytes) + 1)
    layers = [make_layer(out_f, in_f, bits, device, seed=s, group=group, rank=rank, last_bit_scale=last_bit_scale)
              for s in range(ncopies)]
    for L in layers:
        drop_bool_factors(L)
    stream = torch.cuda.Stream(device)
    res = {}
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
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            graph.reset()
        us = e0.elapsed_time(e1) * 1e3 / (reps * ncopies)
        res[M] = (us, (nbytes + M * (in_f + out_f) * 2) / us / 1e3)
    del layers
    torch.cuda.empty_cache()
    return res


def run_shapes(args):
    import torch
    dev = torch.device('cuda', 0)
    torch.cuda.set_device(dev)
    peak = peaks()[0]
    shapes = [(2048, 2048, 2), (2048, 2048, 4), (2048, 6144, 2), (6144, 2048, 2), (2048, 6144, 4), (6144, 2048, 4),
              (4096, 4096, 2), (4096, 14336, 2), (4096, 14336, 4), (28672, 4096, 2)]
    for (o, i, b) in shapes:
        for M, (us, gbs) in time_copies(o, i, b, args.batches, dev).items():
            print(f'{o}x{i}, {b} bit layers, batch {M}: {us:8.2f} us/forward  {gbs:8.1f} GB/s  {100 * gbs / peak:5.1f} % of peak',
                  flush=True)


# ---------------------------------------------------------------------------------------------------
# extras of the headline run
# ---------------------------------------------------------------------------------------------------

def fp8_dense_peak(device):
    """Dense fp8 (e4m3) GEMM throughput measured the way the bf16 peak was: 8192^3, best of 10, CUDA events.
    Returns TFLOP/s or None when this torch build has no scaled fp8 matmul."""
    import torch
    try:
        n = 8192
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()      # column-major second operand
        one = torch.ones((), device=device)
        for _ in range(3):
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        return 2 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def extra_prefill(device, bf16_peak):
    """Prefill configuration: x [2048, 4096] bf16 on a 4096x4096 layer with 2 bit layers, P=Q=r=32."""
    import torch
    layer = make_layer(4096, 4096, 2, device, seed=33)
    x = torch.randn(2048, 4096, device=device, dtype=torch.bfloat16)
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=device)
    with torch.no_grad():
        for _ in range(3):
            layer(x)
        torch.cuda.synchronize()
        times = []
        for _ in range(15):
            flush.zero_()                                   # L2 flush between timed forwards
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            layer(x)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    us = median(times) * 1e3
    tflops = 2 * 2048 * 4096 * 4096 / (us * 1e-6) / 1e12
    fp8 = fp8_dense_peak(device)
    out = {'workload': '2048 tokens x 4096 -> 4096, 2 bit layers, P=Q=r=32, bf16 in and out', 'us': us,
           'tflops_dense_equiv': tflops, 'frac_bf16': tflops / bf16_peak, 'bf16_peak_tflops': bf16_peak,
           'fp8_peak_tflops': fp8, 'fp8_peak_kind': 'measured in this run (torch._scaled_mm e4m3 8192^3, best of 10)'
           if fp8 else 'nominal 2 x bf16 peak (no fp8 matmul in this torch build)',
           'frac_fp8': tflops / (fp8 if fp8 else 2 * bf16_peak), 'l2': 'flushed between timed forwards'}
    del layer, x, flush
    torch.cuda.empty_cache()
    return out


def extra_sweep_batched(layers, cfgs, device, stream, steps):
    """The same 12 layers at batch 4 and 16 (GB/s on algorithmic bytes of this rank)."""
    import torch
    out = {}
    for M in (4, 16):
        xs = [torch.randn(M, i, device=device, dtype=torch.bfloat16) for (o, i, bw) in cfgs]
        with torch.cuda.stream(stream), torch.no_grad():
            for L, x in zip(layers, xs):
                L(x)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for L, x in zip(layers, xs):
                    L(x)
            for _ in range(3):
                graph.replay()
            stream.synchronize()
            times = timed_blocks(lambda: [graph.replay() for _ in range(steps)], stream, min_seconds=0.1)
            graph.reset()
        ms = median(times) / steps
        nbytes = sum(alg_bytes(o, i, bw, M=M) for (o, i, bw) in cfgs)
        out[f'm{M}'] = {'value': nbytes / (ms * 1e-3) / 1e9, 'unit': 'GB/s', 'ms_per_step': ms}
    return out


def extra_large_layer(device, rank, world, peer_factory, stream):
    """Bit-depth-extended large layers: 2+1 bit layers (the added one with N(0,0.005) coefficients), P=Q=r=64,
    bf16 activations, batch 1 and 32, row patches sharded over the ranks, outputs gathered on every rank."""
    import torch
    import torch.distributed as dist
    out = {}
    peer = None
    if world > 1:
        try:
            peer = peer_factory(28672 * 2)              # one gathered row of the widest output
        except RuntimeError:
            peer = None
    checks = []
    for (o, i) in ((8192, 28672), (28672, 8192)):
        # enough distinct copies of the rank's shard to exceed the L2 between two uses of one copy
        shard_bytes = alg_bytes(o // world, i, 3, group=64)
        ncopies = max(2, int(300e6 // shard_bytes) + 1)
        layers = []
        for c in range(ncopies):
            layer = make_layer(o // world, i, 3, device, seed=50 + rank + 16 * c, group=64, rank=64, last_bit_scale=0.005)
            drop_bool_factors(layer)
            layers.append(layer)
        torch.cuda.empty_cache()
        for M in (1, 32):
            x = torch.randn(M, i, device=device, dtype=torch.bfloat16)
            gathered = torch.empty(M, o, device=device, dtype=torch.bfloat16)
            by_peer = peer is not None and M <= 16

            def fwd(layer):
                with torch.no_grad():
                    if world == 1:
                        return layer(x)
                    if by_peer:
                        return layer.forward_gathered(x, peer, out=gathered)
                    from bqq_b200.sharded import gather_columns
                    return gather_columns(layer(x))

            with torch.cuda.stream(stream):
                for layer in layers:
                    fwd(layer)
                stream.synchronize()
                if by_peer:
                    # the rows gathered by peer stores against a library all-gather of the shards' own outputs
                    from bqq_b200.sharded import gather_columns
                    with torch.no_grad():
                        want = gather_columns(layers[0](x))
                        got = layers[0].forward_gathered(x, peer, out=gathered)
                    stream.synchronize()
                    checks.append(bool(torch.equal(want, got)))
                if world == 1 or by_peer:
                    # one graph over all copies, replayed: the ranks stay in step through the gathers themselves
                    if world > 1:
                        dist.barrier()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream):
                        for layer in layers:
                            fwd(layer)
                    for _ in range(3):
                        graph.replay()
                    stream.synchronize()
                    reps = 10
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    for _ in range(reps):
                        graph.replay()
                    e1.record(stream)
                    stream.synchronize()
                    us = e0.elapsed_time(e1) * 1e3 / (reps * ncopies)
                    graph.reset()
                    how = f'graph replay over {ncopies} copies of the shard (> L2)'
                else:
                    times = []
                    for n in range(10):
                        dist.barrier()
                        torch.cuda.synchronize()
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        fwd(layers[n % ncopies])
                        e1.record(stream)
                        stream.synchronize()
                        times.append(e0.elapsed_time(e1))
                    us = median(times) * 1e3
                    how = f'eager launches after a barrier, copies of the shard in rotation ({ncopies}, > L2)'
            if world > 1:
                t = torch.tensor([us], device=device, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                us = float(t.item())
            nbytes = alg_bytes(o, i, 3, M=M, group=64)
            out[f'{o}x{i}_m{M}'] = {'us': us, 'GB/s': nbytes / us / 1e3,
                                    'gather': 'none' if world == 1 else ('peer stores' if by_peer else 'nccl'),
                                    'timing': how}
        del layers, layer
        torch.cuda.empty_cache()
    if peer is not None:
        peer.status()
        peer.close()
    out['note'] = 'whole-layer algorithmic bytes / max-over-ranks time of one forward incl. the gather'
    if checks:
        out['gather_check'] = 'exact' if all(checks) else 'MISMATCH'
    return out


def extra_stack(device, rank, world, peer_factory, new_tokens=128, prompt=512, batches=(1, 8)):
    """Decoder stack (32 layers, hidden 4096, intermediate 14336, 32/8 heads, vocabulary 128256, 2 bit layers,
    P=Q=r=32): 512-token prompts, 128 greedy tokens at batch 1 (the headline of this object) and batch 8, decode step
    replayed from a CUDA graph; layers sharded over the ranks (strong scaling)."""
    import torch
    import torch.distributed as dist
    from bqq_b200.decoder_stack import DecoderStack, StackConfig
    cfg = StackConfig(max_seq=prompt + new_tokens)
    peer = peer_factory(max(batches) * max(cfg.intermediate, cfg.hidden, cfg.vocab) * 2) if world > 1 else None
    model = DecoderStack(cfg, device, seed=0, rank=rank, world=world, peer=peer)
    stream = torch.cuda.Stream(device)
    steps = new_tokens - 1
    runs = {}
    for batch in batches:
        gen = torch.Generator(device=device).manual_seed(1)
        ids0 = torch.randint(0, cfg.vocab, (batch, prompt), generator=gen, device=device)
        cache = model.new_cache(batch)
        with torch.cuda.stream(stream):
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            ids = model.prefill(ids0, cache)
            pos = torch.full((1,), prompt, device=device, dtype=torch.int64)
            static_ids = ids.clone()
            model.decode_step(static_ids, cache, pos)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                nxt = model.decode_step(static_ids, cache, pos)
                static_ids.copy_(nxt)
                pos.add_(1)
            best_decode = best_prefill = None
            for _ in range(3 if batch == 1 else 2):
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                e0.record(stream)
                ids = model.prefill(ids0, cache)
                e1.record(stream)
                static_ids.copy_(ids)
                pos.fill_(prompt)
                for _ in range(steps):
                    graph.replay()
                e2.record(stream)
                stream.synchronize()
                pre, dec = e0.elapsed_time(e1), e1.elapsed_time(e2)
                best_prefill = pre if best_prefill is None else min(best_prefill, pre)
                best_decode = dec if best_decode is None else min(best_decode, dec)
            graph.reset()
        if world > 1:
            t = torch.tensor([best_decode, best_prefill], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            best_decode, best_prefill = t.tolist()
        runs[batch] = {'tokens_per_s': batch * steps / (best_decode * 1e-3), 'ms_per_step': best_decode / steps,
                       'prefill_ms': best_prefill}
        del cache, graph
        torch.cuda.empty_cache()
    first = batches[0]
    res = {'tokens_per_s': runs[first]['tokens_per_s'], 'ms_per_step': runs[first]['ms_per_step'], 'batch': first,
           'layers': cfg.layers, 'scaling': 'strong', 'prompt': prompt, 'new_tokens': new_tokens,
           'prefill_ms': runs[first]['prefill_ms'], 'bqq_bytes_per_token_per_gpu': model.bqq_bytes_per_token(),
           'gathers': 'none' if world == 1 else 'peer stores', 'lm_head': 'dense bf16, included',
           'attention': 'decode steps: bqq_attention_decode of this library (rotary embedding, cache append, attention '
                        'and, with several ranks, the gather of its outputs in one launch); prefill: flash_attn '
                        'library call',
           'coefficients': 'N(0, 0.02/sqrt(in/4096)) for a, 0.05 of that for b, c, d (keeps activations finite '
                           'through 32 random layers; speed does not depend on the values)'}
    for batch in batches[1:]:
        res[f'batch{batch}'] = runs[batch]
    torch.cuda.synchronize()
    if peer is not None:
        peer.status()
        peer.close()
    del model
    torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------------------------------
# headline
# ---------------------------------------------------------------------------------------------------

def run_rates(args):
    """Issue rates of the candidate instructions (bqq_instruction_rate), one JSON line."""
    import ctypes
    import torch
    from bqq_b200 import _cabi
    torch.cuda.set_device(0)
    names = ['mma.sync m16n8k32 u8*s8', 'mma.sync m16n8k16 f16', 'mma.sync m16n8k32 e4m3', 'mma.sync m16n8k64 u4*s4',
             'mma.sync m16n8k256 b1 and.popc', 'lop3', 'add.f32', 'mad.lo.u32', 'popc', 'shfl']
    out = {}
    for kind, name in enumerate(names):
        v = ctypes.c_double()
        rc = _cabi.lib.bqq_instruction_rate(kind, 4096, ctypes.byref(v), None)
        out[name] = round(v.value, 3) if rc == 0 else _cabi.strerror(rc)
        print(f'{name:34s} {out[name]}', file=sys.stderr, flush=True)
    print(json.dumps({'workload': 'rates', 'unit': 'warp-instructions per SM and clock (nominal SM clock)', 'rates': out}),
          flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=10)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-extras', action='store_true', help='headline sweep only')
    ap.add_argument('--workload', default='decode_sweep_b1', choices=['decode_sweep_b1', 'layer', 'shapes', 'rates'])
    ap.add_argument('--out', type=int, default=4096)
    ap.add_argument('--in', dest='inp', type=int, default=14336)
    ap.add_argument('--bits', type=int, default=4)
    ap.add_argument('--batch', type=int, default=1)
    ap.add_argument('--group', type=int, default=32, help='P = Q')
    ap.add_argument('--rank', type=int, default=None, help='r (default: the group size)')
    ap.add_argument('--reps', type=int, default=3)
    ap.add_argument('--batches', type=int, nargs='*', default=[1, 4, 16])
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == 'reference':
        return run_reference(args)
    if args.workload == 'layer':
        return run_layer(args)
    if args.workload == 'shapes':
        return run_shapes(args)
    if args.workload == 'rates':
        return run_rates(args)

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)

    # ---- layers: every rank owns one row-patch shard with the base shape (weak scaling) ----
    cfgs = sweep()
    layers = [make_layer(o, i, bw, device, 1000 * rank + n) for n, (o, i, bw) in enumerate(cfgs)]
    xs = [torch.randn(1, i, device=device, dtype=torch.bfloat16) for (o, i, bw) in cfgs]
    with torch.no_grad():
        for L, x in zip(layers, xs):
            L(x)
    torch.cuda.synchronize()
    step_bytes = sum(alg_bytes(o, i, bw) for (o, i, bw) in cfgs)
    from bqq_b200 import _cabi
    launches_per_step = sum(_cabi.lib.bqq_decode_launches(L._dims(), 1) for L in layers)
    gathers = [torch.empty(1, world * o, device=device, dtype=torch.bfloat16) for (o, i, bw) in cfgs] if world > 1 else None
    peer = None

    def peer_factory(nbytes):
        from bqq_b200.peer import PeerGatherGroup
        return PeerGatherGroup(nbytes, device)

    if world > 1:
        try:
            peer = peer_factory(max(world * o * 2 for (o, i, bw) in cfgs))
        except RuntimeError as exc:          # raised on every rank alike: fall back to the process group's all-gather
            if rank == 0:
                print(f'bench: {exc}; gathering with NCCL instead', file=sys.stderr)

    def gathered_forward(L, x, out):
        if peer is not None:
            return L.forward_gathered(x, peer, out=out)        # decode kernel stores its row patches to the peers
        dist.all_gather_into_tensor(out.view(world, -1), L(x).view(-1))
        return out

    def step():
        with torch.no_grad():
            for n, (L, x) in enumerate(zip(layers, xs)):
                if world > 1:
                    gathered_forward(L, x, gathers[n])
                else:
                    L(x)

    stream = torch.cuda.Stream(device)
    gather_check = None
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
        stream.synchronize()
        if world > 1:
            # every gathered output against the ranks' own slices, exchanged once over NCCL (outside the timed region)
            ok = True
            with torch.no_grad():
                for n, (L, x) in enumerate(zip(layers, xs)):
                    mine = L(x).contiguous()
                    every = torch.empty(world, mine.numel(), device=device, dtype=mine.dtype)
                    dist.all_gather_into_tensor(every, mine.view(-1))
                    stream.synchronize()
                    ok = ok and torch.equal(every.view(1, -1), gathers[n])
            flag = torch.tensor([0 if ok else 1], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            gather_check = 'exact' if int(flag.item()) == 0 else 'MISMATCH'
        # several steps per captured graph (a decoder model replays hundreds of layers per graph launch; one
        # step here has 12): the steps run back to back without a host round trip in between
        group = next(g for g in (10, 5, 4, 2, 1) if args.steps % g == 0)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(group):
                step()
        for _ in range((args.warmup + group - 1) // group):
            graph.replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        # with several ranks every rank must replay the same number of blocks: the count is fixed from a first block
        probe = timed_blocks(lambda: [graph.replay() for _ in range(args.steps // group)], stream, min_seconds=0.0,
                             min_blocks=1, max_blocks=1)[0]
        nblocks = max(5, min(400, int(math.ceil(MIN_TIMED_SECONDS * 1e3 / max(probe, 1e-3)))))
        if world > 1:
            nb = torch.tensor([nblocks], device=device)
            dist.all_reduce(nb, op=dist.ReduceOp.MAX)
            nblocks = int(nb.item())
            dist.barrier()
        torch.cuda.synchronize()
        blocks = timed_blocks(lambda: [graph.replay() for _ in range(args.steps // group)], stream, min_seconds=0.0,
                              min_blocks=nblocks, max_blocks=nblocks)
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        clocks = sampler.stop() if rank == 0 else None
        ms = median(blocks)

        # ---- end to end: host activations in, host outputs back, every layer, every step ----
        xh = [x.cpu().pin_memory() for x in xs]
        yh = [torch.empty(1, world * o, dtype=torch.bfloat16).pin_memory() for (o, i, bw) in cfgs]
        with torch.no_grad():
            if world == 1:
                bound = [L.bind_host(xh[n], yh[n])[0] for n, L in enumerate(layers)]
            else:
                try:
                    x_alias = [host_alias(t) for t in xh]
                    y_alias = [host_alias(t) for t in yh]
                    e2e_route = 'forward_gathered on device-visible aliases of the pinned host buffers'
                except Exception:                            # no aliasing in this torch build: copy-engine transfers
                    x_alias = y_alias = None
                    e2e_route = 'tensor.to(device) + forward_gathered + copy_ to pinned host memory'
                # layers whose CTAs each read all of x get it staged on the device by one small copy kernel
                staged = [_cabi.lib.bqq_decode_launches(L._dims(), 1) == 1 for L in layers]

        def e2e_body():
            with torch.no_grad():
                for n, L in enumerate(layers):
                    if world > 1 and x_alias is None:
                        y = gathered_forward(L, xh[n].to(device, non_blocking=True), gathers[n])
                        yh[n].copy_(y, non_blocking=True)
                    elif world > 1:
                        xin = x_alias[n]
                        if staged[n]:
                            xs[n].copy_(xin)                  # a kernel reading pinned host memory, no copy engine
                            xin = xs[n]
                        gathered_forward(L, xin, y_alias[n])  # the receiving kernel writes the rows to host memory
                    else:
                        bound[n]()                            # one C call: copy in, kernels, copy out

        for _ in range(3):
            e2e_body()
        stream.synchronize()
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph, stream=stream):
            e2e_body()
        for _ in range(3):
            e2e_graph.replay()
            stream.synchronize()
        e2e_steps = max(10, min(args.steps, 100))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

        def e2e_block():
            for _ in range(e2e_steps):
                e2e_graph.replay()
                stream.synchronize()          # the host reads the outputs of every step

        e2e_blocks = timed_blocks(e2e_block, stream, min_seconds=0.0, min_blocks=max(5, nblocks // 4),
                                  max_blocks=max(5, nblocks // 4))
        e2e_ms = median(e2e_blocks)

        extras = {}
        if not args.no_extras:
            extras['sweep_batched'] = extra_sweep_batched(layers, cfgs, device, stream, group)

    if world > 1:
        t = torch.tensor([ms, e2e_ms, max(blocks), min(blocks)], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, blk_max, blk_min = t.tolist()
    else:
        blk_max, blk_min = max(blocks), min(blocks)

    for g in (graph, e2e_graph):
        g.reset()
    del layers, xs
    torch.cuda.empty_cache()
    hbm_peak, bf16_peak, peak_kind = peaks()
    if not args.no_extras:
        with torch.cuda.stream(stream):
            extras['large_layer'] = extra_large_layer(device, rank, world, peer_factory, stream)
        if rank == 0:
            extras['prefill'] = extra_prefill(device, bf16_peak)
        if world > 1:
            dist.barrier()
        try:
            extras['stack'] = extra_stack(device, rank, world, peer_factory)
        except Exception as exc:                                # never lose the headline to an extra
            extras['stack'] = {'error': f'{type(exc).__name__}: {exc}'}

    shutdown(world, [], peer)          # communicator torn down before rank 0 spends time on the CPU baseline
    if gather_check == 'MISMATCH' or PEER_TIMEOUT:
        if rank == 0:
            print('bench: gathered outputs differ from the shards\' outputs' if gather_check == 'MISMATCH'
                  else 'bench: a peer wait timed out', file=sys.stderr)
        sys.exit(3)
    if rank == 0:
        total_bytes = step_bytes * world
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        e2e_val = total_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
        per_gpu = step_bytes * args.steps / (ms * 1e-3) / 1e9
        line = {
            'metric': 'packed-weight HBM GB/s at batch 1', 'value': value, 'unit': 'GB/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms / args.steps,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': DTYPE_NOTE,
            'data': 'synthetic',
            'config': {'workload': 'decode_sweep_b1', 'layers': len(cfgs), 'P': P, 'Q': Q, 'r': R,
                       'activations': 'bf16', 'batch': 1, 'bytes_per_step_per_gpu': step_bytes,
                       'steps_per_graph_launch': group,
                       'l2': 'working set per step (208.5 MB of packed planes) exceeds the 126 MB L2',
                       'parallelism': 'single GPU' if world == 1 else (
                           f'row-patch shards x{world}, outputs stored to the peers from the epilogue of the decode kernel and '
                           'received by a few more CTAs of the same launch (bqq_forward_decode_gathered)' if peer is not None else
                           f'row-patch shards x{world}, NCCL all-gather of outputs (peer gather set-up failed)')},
            'timing': {'blocks': len(blocks), 'block_steps': args.steps, 'median_block_ms': ms,
                       'min_block_ms': blk_min, 'max_block_ms': blk_max,
                       'timed_seconds': sum(blocks) * 1e-3},
            'e2e': {'value': e2e_val, 'unit': 'GB/s',
                    'h2d_bytes_per_step': sum(i * 2 for (o, i, bw) in cfgs),
                    'd2h_bytes_per_step': sum(world * o * 2 for (o, i, bw) in cfgs),
                    'steps': e2e_steps, 'ms_per_step': e2e_ms / e2e_steps,
                    'route': 'bqq_forward_host (module.bind_host)' if world == 1 else e2e_route},
            # decode kernel (+ activation preparation kernel) per layer; the gather runs inside the decode launch
            'gpu_launches': launches_per_step * args.steps,
            'roofline': {'bound': 'hbm', 'achieved': per_gpu, 'peak': hbm_peak, 'unit': 'GB/s',
                         'frac': per_gpu / hbm_peak, 'traffic': TRAFFIC_RATIO * step_bytes / len(cfgs),
                         'traffic_note': 'constant from profiles: dram read+write bytes of one ncu capture (4096x14336, '
                                         '4 bit layers: 62.09 MB for 61.72 MB algorithmic) scaled by algorithmic bytes',
                         'peak_kind': peak_kind,
                         'kernel': 'bqq_decode_kernel',
                         'avg_launch_us': ms * 1e3 / (args.steps * len(cfgs)),
                         'bytes_per_launch': step_bytes / len(cfgs)},
            'clocks': clocks,
        }
        if gather_check is not None:
            line['gather_check'] = gather_check
        line.update(extras)
        if not args.no_cpu_baseline:
            sample = [(2048, 2048, 2), (2048, 6144, 2), (4096, 14336, 2)]
            lnp = [make_layer_np(o, i, bw, 7 + n) for n, (o, i, bw) in enumerate(sample)]
            cpu_port_time(lnp[:1])
            reps = 3
            dt = cpu_port_time(lnp, repeats=reps)
            from oracle import c_oracle
            line['cpu_baseline'] = {
                'value': sum(alg_bytes(o, i, bw) for (o, i, bw) in sample) / dt / 1e9, 'unit': 'GB/s',
                'cores': c_oracle.max_threads(), 'kind': 'port',
                'sample': '2048x2048, 2048x6144 and 4096x14336 at 2 bit layers, fp32, batch 1, 3 passes',
                'note': 'C port of the reference forward (dense W rebuild + matmul, pthreads, all cores): a stronger '
                        "baseline than the reference's own Python forward"}
            ref_s = reference_python_seconds()
            if ref_s is not None:
                port_s = cpu_port_time(lnp[:1], repeats=3)
                line['cpu_baseline']['reference_python_forward'] = {
                    'layer': '2048x2048, 2 bit layers, fp32, batch 1', 'seconds': ref_s, 'port_seconds': port_s,
                    'port_speedup': ref_s / port_s}
        print(json.dumps(line), flush=True)


if __name__ == '__main__':
    main()
