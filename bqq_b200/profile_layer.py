"""Run the forward of one synthetic BinaryQuadratic layer a few times: the program to put under a profiler.

    python -m bqq_b200.profile_layer --out 4096 --in 14336 --bits 4 --batch 1
    ncu --set full --clock-control none -k regex:bqq_decode -s 1 -c 1 -o prof \\
        python -m bqq_b200.profile_layer --out 4096 --in 14336 --bits 4 --batch 1

Bits are Bernoulli(0.5), coefficients N(0, 0.02), activations N(0, 1) in bf16 (seeded); batch <= 16 takes the
decode kernel, larger batches the reconstruction + tensor-core GEMM.
"""
from __future__ import annotations

import argparse

import torch

from .bqq_modules import BinaryQuadratic


def synthetic_layer(out_f: int, in_f: int, bits: int, device, seed: int = 1, group: int = 32, rank: int | None = None):
    """Seeded synthetic layer built directly on the device."""
    rank = group if rank is None else rank
    g = torch.Generator(device=device).manual_seed(seed)
    rw, cw = out_f // group, in_f // group
    Y = torch.rand(bits, rw, cw, group, rank, generator=g, device=device) > 0.5
    Z = torch.rand(bits, rw, cw, rank, group, generator=g, device=device) > 0.5
    A = torch.randn(bits, rw, cw, 4, generator=g, device=device) * 0.02
    return BinaryQuadratic(Y, Z, A)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument('--out', type=int, default=4096)
    ap.add_argument('--in', dest='inp', type=int, default=14336)
    ap.add_argument('--bits', type=int, default=4)
    ap.add_argument('--batch', type=int, default=1)
    ap.add_argument('--group', type=int, default=32, help='P = Q')
    ap.add_argument('--rank', type=int, default=None, help='r (default: the group size)')
    ap.add_argument('--reps', type=int, default=3)
    args = ap.parse_args()
    dev = torch.device('cuda', 0)
    layer = synthetic_layer(args.out, args.inp, args.bits, dev, group=args.group, rank=args.rank)
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
    print(f'{args.out}x{args.inp}, {args.bits} bit layers, batch {args.batch}: '
          f'{e0.elapsed_time(e1) * 1e3 / args.reps:.1f} us per forward (same layer repeated, warm L2); '
          f'max |y| {float(y.float().abs().max()):.3f}')


if __name__ == '__main__':
    main()
