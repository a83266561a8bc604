"""Decode benchmark of the random-init Llama-style BinaryQuadratic decoder stack.

Counterpart of the reference's lm/benchmark_inference.py (random BQQ model, greedy decode with
a KV cache, 3 warm-up + timed runs): prompts of `--prompt` random token ids, `--new` decoded
tokens, batch `--batch`; the decode step is captured once in a CUDA graph and replayed.  Run
under torchrun for several GPUs (row-patch shards, NCCL all-gathers).  Prints one JSON line with
tokens/s and the packed bytes streamed per token.

    python -m bqq_b200.bench_stack --layers 32 --batch 1
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m bqq_b200.bench_stack
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .decoder_stack import DecoderStack, StackConfig


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--layers', type=int, default=32)
    ap.add_argument('--hidden', type=int, default=4096)
    ap.add_argument('--intermediate', type=int, default=14336)
    ap.add_argument('--heads', type=int, default=32)
    ap.add_argument('--kv-heads', type=int, default=8)
    ap.add_argument('--vocab', type=int, default=128256)
    ap.add_argument('--bits', type=int, default=2)
    ap.add_argument('--group', type=int, default=32)
    ap.add_argument('--batch', type=int, default=1)
    ap.add_argument('--prompt', type=int, default=512)
    ap.add_argument('--new', type=int, default=128)
    ap.add_argument('--repeats', type=int, default=3)
    ap.add_argument('--nccl-gathers', action='store_true', help='gather with the process group instead of peer stores')
    ap.add_argument('--library-attention', action='store_true',
                    help='decode steps use flash_attn (or torch ops) instead of the attention kernel of this package')
    ap.add_argument('--mark-one-step', action='store_true',
                    help='after the timed runs, replay one decode step between cudaProfilerStart/Stop (for a profiler '
                         'started with capture off: the launch list of exactly one step)')
    args = ap.parse_args()

    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)

    cfg = StackConfig(layers=args.layers, hidden=args.hidden, intermediate=args.intermediate, heads=args.heads,
                      kv_heads=args.kv_heads, vocab=args.vocab, bit_width=args.bits, group=args.group,
                      max_seq=args.prompt + args.new, own_attention=not args.library_attention)
    peer = None
    if world > 1 and not args.nccl_gathers:
        from .peer import PeerGatherGroup
        # decode-sized gathers (one row per sequence) go peer to peer; the prefill's stay on the process group
        peer = PeerGatherGroup(args.batch * max(cfg.intermediate, cfg.hidden, cfg.vocab) * 2, device)
    model = DecoderStack(cfg, device, seed=0, rank=rank, world=world, peer=peer)
    gen = torch.Generator(device=device).manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (args.batch, args.prompt), generator=gen, device=device)
    cache = model.new_cache(args.batch)

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        ids = model.prefill(prompt, cache)                      # also warms up every layer
        pos = torch.full((1,), args.prompt, device=device, dtype=torch.int64)
        static_ids = ids.clone()
        model.decode_step(static_ids, cache, pos)               # warm-up outside the graph
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            nxt = model.decode_step(static_ids, cache, pos)
            static_ids.copy_(nxt)
            pos.add_(1)
        best_decode, best_prefill = None, None
        for _ in range(args.repeats):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0.record(stream)
            ids = model.prefill(prompt, cache)
            e1.record(stream)
            static_ids.copy_(ids)
            pos.fill_(args.prompt)
            for _ in range(args.new - 1):
                graph.replay()
            e2.record(stream)
            stream.synchronize()
            pre, dec = e0.elapsed_time(e1), e1.elapsed_time(e2)
            best_prefill = pre if best_prefill is None else min(best_prefill, pre)
            best_decode = dec if best_decode is None else min(best_decode, dec)
    if args.mark_one_step:
        with torch.cuda.stream(stream):
            stream.synchronize()
            torch.cuda.profiler.start()
            graph.replay()
            stream.synchronize()
            torch.cuda.profiler.stop()
    if world > 1:
        t = torch.tensor([best_decode, best_prefill], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best_decode, best_prefill = t.tolist()
    if rank == 0:
        steps = args.new - 1
        print(json.dumps({
            'workload': 'llama_style_decoder_stack', 'layers': cfg.layers, 'hidden': cfg.hidden,
            'intermediate': cfg.intermediate, 'bits': cfg.bit_width, 'group': cfg.group, 'batch': args.batch,
            'prompt': args.prompt, 'new_tokens': args.new, 'n_gpus': world,
            'decode_tokens_per_s': args.batch * steps / (best_decode * 1e-3),
            'decode_ms_per_step': best_decode / steps,
            'prefill_ms': best_prefill, 'prefill_tokens_per_s': args.batch * args.prompt / (best_prefill * 1e-3),
            'bqq_bytes_per_token_per_gpu': model.bqq_bytes_per_token(),
            'gathers': 'none' if world == 1 else ('nccl' if peer is None else 'peer stores'),
            'lm_head': 'dense bf16, included', 'data': 'synthetic (random init, random prompt ids)'}),
            flush=True)
    graph.reset()
    torch.cuda.synchronize()
    if world > 1:
        import threading
        timer = threading.Timer(30.0, lambda: os._exit(0))     # teardown must never hang the job
        timer.daemon = True
        timer.start()
        if peer is not None:
            peer.status()
            peer.close()
        dist.barrier()
        dist.destroy_process_group()
        timer.cancel()


if __name__ == '__main__':
    main()
