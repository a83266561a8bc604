"""GPU: the decoder-stack harness (bqq_b200/decoder_stack.py) on a tiny configuration: its hidden states against
a dense re-computation with the layers' reconstructed weights, and the graph-replayed decode loop against the eager one."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _dense_layer(layer, x, k_cache, v_cache, pos, rot, cfg):
    """One decoder block with dense weights (get_weight) and plain torch ops: what the harness' fused calls must equal."""
    from bqq_b200.decoder_stack import _rope
    B, T, _ = x.shape
    hd = cfg.head_dim
    lh, lkv = layer.local_heads, layer.local_kv
    W = {n: getattr(layer, n).get_weight(torch.float32) for n in ('qkv_proj', 'o_proj', 'gate_up_proj', 'down_proj')}
    xf = x.float()
    hx = F.rms_norm(xf, (cfg.hidden,), layer.norm1.float(), 1e-5)
    qkv = (hx @ W['qkv_proj'].T).view(B, T, lh + 2 * lkv, hd)
    qk = _rope(qkv[:, :, :lh + lkv], rot)
    q = qk[:, :, :lh].transpose(1, 2)
    k_cache[:, pos:pos + T] = qk[:, :, lh:]
    v_cache[:, pos:pos + T] = qkv[:, :, lh + lkv:]
    att = F.scaled_dot_product_attention(q, k_cache[:, :pos + T].transpose(1, 2), v_cache[:, :pos + T].transpose(1, 2),
                                         is_causal=(T > 1 and pos == 0), enable_gqa=True)
    att = att.transpose(1, 2).reshape(B, T, lh * hd)
    xf = xf + att @ W['o_proj'].T
    gu = F.rms_norm(xf, (cfg.hidden,), layer.norm2.float(), 1e-5) @ W['gate_up_proj'].T
    n = gu.shape[-1] // 2
    return xf + (F.silu(gu[..., :n]) * gu[..., n:]) @ W['down_proj'].T


def test_tiny_stack_matches_dense_recomputation_and_graph_replay():
    from bqq_b200.decoder_stack import DecoderStack, StackConfig
    dev = torch.device('cuda', 0)
    cfg = StackConfig(layers=2, hidden=256, intermediate=512, heads=4, kv_heads=2, vocab=512, bit_width=2, group=32,
                      max_seq=24)
    model = DecoderStack(cfg, dev, seed=3)
    from bqq_b200.bqq_modules import BinaryQuadratic
    with torch.no_grad():                           # narrow layers get large random weights: keep the activations O(1)
        for m in model.modules():
            if isinstance(m, BinaryQuadratic):
                for name in 'abcd':
                    getattr(m, name).mul_(0.05)
    g = torch.Generator(device=dev).manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (2, 9), generator=g, device=dev)
    cache = model.new_cache(2)
    with torch.no_grad():
        # hidden states of the prefill (9 tokens: decode-sized rows -> fused kernels) against dense fp32 blocks
        x = model.embed[prompt]
        xd = x.float()
        dcache = torch.zeros_like(cache, dtype=torch.float32)
        rot = model.rot[:9]
        fa = (model.cos, model.sin, torch.zeros(2, dtype=torch.int32, device=dev)) if model.use_flash else None
        for li, layer in enumerate(model.layers):
            x = layer(x, cache[li, 0], cache[li, 1], 0, rot, fa=fa)
            xd = _dense_layer(layer, xd, dcache[li, 0], dcache[li, 1], 0, rot, cfg)
        err = (x.float() - xd).abs().max() / xd.abs().max()
        assert err < 3e-2, err                      # bf16 hidden states through two blocks

        # one more token per sequence (2 rows: the fused normalisation / SwiGLU / residual kernels) against dense blocks
        x = model.embed[prompt[:, :1]]
        xd = x.float()
        rot1 = model.rot[9:10]
        fa = (model.cos, model.sin, torch.full((2,), 9, dtype=torch.int32, device=dev)) if model.use_flash else None
        for li, layer in enumerate(model.layers):
            x = layer(x, cache[li, 0], cache[li, 1], 9, rot1, fa=fa)
            xd = _dense_layer(layer, xd, dcache[li, 0], dcache[li, 1], 9, rot1, cfg)
        err = (x.float() - xd).abs().max() / xd.abs().max()
        assert err < 3e-2, err

        # greedy decode: eager steps and one captured graph give the same tokens
        ids0 = model.prefill(prompt, cache)
        ref_cache = cache.clone()
        pos = torch.full((1,), 9, device=dev, dtype=torch.int64)
        ids = ids0.clone()
        eager = []
        for _ in range(6):
            ids = model.decode_step(ids, cache, pos)
            pos.add_(1)
            eager.append(ids.clone())
        cache.copy_(ref_cache)
        pos.fill_(9)
        static = ids0.clone()
        st = torch.cuda.Stream(dev)
        with torch.cuda.stream(st):
            model.decode_step(static, cache.clone(), pos)         # warm-up outside the graph
            st.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                nxt = model.decode_step(static, cache, pos)
                static.copy_(nxt)
                pos.add_(1)
            # the capture itself did not execute: state is still that of the prefill
            replayed = []
            for _ in range(6):
                graph.replay()
                st.synchronize()
                replayed.append(static.clone())
            graph.reset()
        assert all(torch.equal(a, b) for a, b in zip(eager, replayed))
