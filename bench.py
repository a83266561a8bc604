"""Benchmark of the BinaryQuadratic decode forward (batch 1) on B200.

Workload ("decode_sweep_b1"): the decode GEMV sweep of synthetic BinaryQuadratic layers
  shapes 2048x2048, 2048x6144, 6144x2048, 4096x14336 (out x in), 2/3/4 bit layers,
  P=Q=r=32, Bernoulli(0.5) bits, N(0,0.02) fp32 coefficients, bf16 activations, batch 1.
A step is one forward through all 12 layers (12 launches of the decode kernel), replayed
from a CUDA graph.  The 12 layers hold 208.5 MB of packed bits + coefficients, more than
the 126 MB L2, so every step streams them from HBM again.

value  = algorithmic bytes (packed bits + fp32 coefficients + x + y) per second, summed over
         all ranks, inputs resident in HBM, timed with CUDA events on the launching stream.
e2e    = the same through module.bind_host (the C entry point bqq_forward_host) with HOST
         activations: pinned x -> device copy, forward, device -> pinned host copy of y, every
         layer, every step (the step is captured once and replayed), one stream synchronisation
         per step to read the outputs.
With N > 1 ranks (weak scaling) each rank owns one row-patch shard of layers N times as
tall (its shard has the base shape) and every layer's outputs are gathered on all ranks by the
library's peer-to-peer store kernel (bqq_peer_gather; NCCL only carries the set-up and the timing
reduction).

`--impl reference` times the CPU port of the reference algorithm (oracle/bqq_oracle.c,
dense-weight rebuild + matmul, all host threads) on the same 12 layers.
"""
from __future__ import annotations

import argparse
import json
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
L2_BYTES = 126e6
PEER_TIMEOUT = False   # set when a bounded wait of the peer gather gave up (reported in the JSON line)
TRAFFIC_RATIO = 62.09 / 61.72   # measured DRAM bytes / algorithmic bytes (profiles/decode_kernel_4096x14336_bw4_m1.md)


def sweep():
    return [(o, i, bw) for (o, i) in SHAPES for bw in BITS]


def alg_bytes(out_f, in_f, bw, M=1, act_bytes=2):
    rw, cw = out_f // P, in_f // Q
    bits = bw * rw * cw * (P * R + R * Q)
    return bits // 8 + 4 * rw * cw * (3 * bw + 1) + M * (in_f + out_f) * act_bytes


def peaks():
    try:
        with open(os.path.join(ROOT, 'MEASURED_PEAKS.json')) as f:
            return float(json.load(f)['hbm_gbs']), 'measured'
    except Exception:
        return 6650.0, 'fallback'


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


def make_layer(out_f, in_f, bw, device, seed):
    """Seeded synthetic layer built directly on the device (bits Bernoulli(0.5), coefficients N(0,0.02))."""
    import torch
    from bqq_b200.bqq_modules import BinaryQuadratic
    g = torch.Generator(device=device).manual_seed(seed)
    rw, cw = out_f // P, in_f // Q
    Y = torch.rand(bw, rw, cw, P, R, generator=g, device=device) > 0.5
    Z = torch.rand(bw, rw, cw, R, Q, generator=g, device=device) > 0.5
    A = torch.randn(bw, rw, cw, 4, generator=g, device=device) * 0.02
    return BinaryQuadratic(Y, Z, A)


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
                   'note': 'CPU port of the reference forward (dense W rebuild + matmul), every layer of the sweep'},
        'cpu_baseline': {'value': val, 'unit': 'GB/s', 'cores': cores, 'kind': 'port',
                         'sample': 'all 12 layers of the sweep per step'},
        'e2e': {'value': val, 'unit': 'GB/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=200)
    ap.add_argument('--warmup', type=int, default=10)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--no-cpu-baseline', action='store_true')
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == 'reference':
        return run_reference(args)

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
            L(x)                       # packs planes and coefficients
    for L in layers:                   # the bool factors are not needed on the device any more
        L._ensure_packed()
    torch.cuda.synchronize()
    step_bytes = sum(alg_bytes(o, i, bw) for (o, i, bw) in cfgs)
    from bqq_b200 import _cabi
    launches_per_step = sum(_cabi.lib.bqq_decode_launches(L._dims(), 1) for L in layers)
    gathers = [torch.empty(1, world * o, device=device, dtype=torch.bfloat16) for (o, i, bw) in cfgs] if world > 1 else None
    peer = None
    if world > 1:
        from bqq_b200.peer import PeerGatherGroup
        try:
            peer = PeerGatherGroup(max(world * o * 2 for (o, i, bw) in cfgs), device)
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
    with torch.cuda.stream(stream):
        for _ in range(3):
            step()
        stream.synchronize()
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps // group):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop() if rank == 0 else None

        # ---- end to end: host activations in, host outputs back, through module.forward ----
        xh = [x.cpu().pin_memory() for x in xs]
        yh = [torch.empty(1, o, dtype=torch.bfloat16).pin_memory() for (o, i, bw) in cfgs]

        with torch.no_grad():
            bound = [L.bind_host(xh[n], yh[n])[0] for n, L in enumerate(layers)] if world == 1 else None

        def e2e_body():
            with torch.no_grad():
                for n, L in enumerate(layers):
                    if world > 1:
                        y = gathered_forward(L, xh[n].to(device, non_blocking=True), gathers[n])
                        yh[n].copy_(y[:, :yh[n].shape[1]], non_blocking=True)
                    else:
                        bound[n]()                        # one C call: copy in, kernels, copy out

        for _ in range(3):
            e2e_body()
        stream.synchronize()
        # a serving loop replays the whole step (copies in, kernels, copies out) as one captured graph and
        # synchronises once per step to read the outputs
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph, stream=stream):
            e2e_body()

        def e2e_step():
            e2e_graph.replay()
            stream.synchronize()

        for _ in range(3):
            e2e_step()
        e2e_steps = max(10, min(args.steps, 100))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        f1.record(stream)
        stream.synchronize()
        e2e_ms = f0.elapsed_time(f1)

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()

    shutdown(world, [graph, e2e_graph], peer)          # communicator torn down before rank 0 spends time on the CPU baseline
    if rank == 0:
        peak, peak_kind = peaks()
        total_bytes = step_bytes * world
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        e2e_val = total_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
        per_gpu = step_bytes * args.steps / (ms * 1e-3) / 1e9
        line = {
            'metric': 'packed-weight HBM GB/s at batch 1', 'value': value, 'unit': 'GB/s', 'n_gpus': world,
            'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': ms / args.steps,
            'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'int8',
            'data': 'synthetic',
            'config': {'workload': 'decode_sweep_b1', 'layers': len(cfgs), 'P': P, 'Q': Q, 'r': R,
                       'activations': 'bf16', 'batch': 1, 'bytes_per_step_per_gpu': step_bytes,
                       'steps_per_graph_launch': group,
                       'l2': 'working set per step (208.5 MB of packed planes) exceeds the 126 MB L2',
                       'parallelism': 'single GPU' if world == 1 else (
                           f'row-patch shards x{world}, outputs stored to the peers from the epilogue of the decode kernel '
                           '(bqq_forward_decode_gathered)' + (' -- A PEER WAIT TIMED OUT, RESULT INVALID' if PEER_TIMEOUT else '')
                           if peer is not None else
                           f'row-patch shards x{world}, NCCL all-gather of outputs (peer gather set-up failed)')},
            'e2e': {'value': e2e_val, 'unit': 'GB/s',
                    'h2d_bytes_per_step': sum(i * 2 for (o, i, bw) in cfgs),
                    'd2h_bytes_per_step': sum(o * 2 for (o, i, bw) in cfgs),
                    'steps': e2e_steps, 'ms_per_step': e2e_ms / e2e_steps},
            # decode kernel (+ activation preparation kernel) per layer, + the gather kernel when sharded
            'gpu_launches': (launches_per_step + (len(cfgs) if peer is not None else 0)) * args.steps,
            'roofline': {'bound': 'hbm', 'achieved': per_gpu, 'peak': peak, 'unit': 'GB/s',
                         'frac': per_gpu / peak, 'traffic': TRAFFIC_RATIO * step_bytes / len(cfgs),
                         'traffic_note': 'dram read+write bytes of one ncu capture (4096x14336, 4 bit layers: '
                                         '62.09 MB for 61.72 MB algorithmic) scaled by algorithmic bytes',
                         'peak_kind': peak_kind,
                         'kernel': 'bqq_decode_kernel',
                         'avg_launch_us': ms * 1e3 / (args.steps * len(cfgs)),
                         'bytes_per_launch': step_bytes / len(cfgs)},
            'clocks': clocks,
        }
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
                'sample': '2048x2048, 2048x6144 and 4096x14336 at 2 bit layers, fp32, batch 1, 3 passes'}
        print(json.dumps(line), flush=True)


if __name__ == '__main__':
    main()
