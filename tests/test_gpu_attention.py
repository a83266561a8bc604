"""GPU: the single-token attention kernel of the decoder-stack harness (bqq_attention_decode) against plain torch
ops in fp32: rotary embedding of the new q and k, cache append, attention over the cached rows with grouped heads."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(qkv, kc, vc, cos, sin, lens, heads, kv):
    B, _, H, hd = qkv.shape
    out = torch.empty(B, 1, heads, hd, dtype=torch.float32, device=qkv.device)
    kc, vc = kc.clone(), vc.clone()
    for b in range(B):
        pos = int(lens[b])
        c, s = cos[pos].float(), sin[pos].float()

        def rot(x):                                             # x [n, hd]: pairs (x[2i], x[2i+1])
            x0, x1 = x[:, 0::2].float(), x[:, 1::2].float()
            return torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1).flatten(-2).to(torch.bfloat16)
        q = rot(qkv[b, 0, :heads]).float()
        kc[b, pos] = rot(qkv[b, 0, heads:heads + kv])
        vc[b, pos] = qkv[b, 0, heads + kv:]
        K, V = kc[b, :pos + 1].float(), vc[b, :pos + 1].float()   # [L, kv, hd]
        for h in range(heads):
            g = h // (heads // kv)
            w = torch.softmax(K[:, g] @ q[h] / math.sqrt(hd), dim=0)
            out[b, 0, h] = w @ V[:, g]
    return out, kc, vc


@pytest.mark.parametrize('B,heads,kv,positions,max_seq', [
    (1, 32, 8, [0, 5, 63, 64, 200, 639], 640),   # the stack on one GPU: 20 splits of at most 32 keys
    (2, 4, 1, [0, 31, 300], 640),                 # a shard of it (heads / 8), two sequences
    (1, 8, 8, [7, 130], 640),                     # one query head per kv head
    (3, 64, 4, [1, 100], 640),                    # 16 query heads per kv head (four per warp)
    (2, 8, 2, [0, 17, 31], 32),                   # short cache: one split, outputs written without the combination
    (1, 32, 8, [70, 2047, 4000, 4095], 4096),     # long cache: 32 splits of up to 128 keys, several tiles per CTA
])
def test_attention_decode_matches_torch(B, heads, kv, positions, max_seq):
    from bqq_b200.decoder_stack import attention_decode
    dev = torch.device('cuda')
    hd = 128
    g = torch.Generator(device=dev).manual_seed(5)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device=dev).float() / hd))
    ang = torch.arange(max_seq, device=dev).float()[:, None] * inv[None, :]
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    for pos in positions:
        kc = torch.randn(B, max_seq, kv, hd, generator=g, device=dev).to(torch.bfloat16)
        vc = torch.randn(B, max_seq, kv, hd, generator=g, device=dev).to(torch.bfloat16)
        qkv = torch.randn(B, 1, heads + 2 * kv, hd, generator=g, device=dev).to(torch.bfloat16)
        lens = torch.tensor([max(0, pos - 3 * b) for b in range(B)], dtype=torch.int32, device=dev)
        want, kc_want, vc_want = _reference(qkv, kc, vc, cos, sin, lens.tolist(), heads, kv)
        for _ in range(2):                                      # twice: the tickets must be back at zero
            kc_got, vc_got = kc.clone(), vc.clone()
            got = attention_decode(qkv, kc_got, vc_got, cos, sin, lens, heads, kv)
            torch.cuda.synchronize()
            assert got is not None and got.shape == (B, 1, heads, hd)
            assert torch.equal(vc_got, vc_want)
            assert (kc_got.float() - kc_want.float()).abs().max().item() <= 2 ** -6     # one bf16 rounding of the rotation
            err = (got.float() - want).abs().max().item()
            assert err <= 2e-2 * max(1.0, want.abs().max().item()), (pos, err)


def test_attention_decode_refuses_what_it_cannot_do():
    import ctypes
    from bqq_b200 import _cabi
    from bqq_b200.decoder_stack import attention_decode
    dev = torch.device('cuda')
    qkv = torch.zeros(1, 1, 6, 64, device=dev, dtype=torch.bfloat16)           # head_dim 64: not this kernel's
    kc = torch.zeros(1, 8, 1, 64, device=dev, dtype=torch.bfloat16)
    cs = torch.zeros(8, 32, device=dev, dtype=torch.bfloat16)
    lens = torch.zeros(1, dtype=torch.int32, device=dev)
    assert attention_decode(qkv, kc, kc.clone(), cs, cs, lens, 4, 1) is None
    p = kc.data_ptr()
    lib = _cabi.lib
    assert lib.bqq_attention_decode(p, 768, p, p, 512, 8, p, p, p, 1, 4, 1, 64, _cabi.BF16, p, 256, p, 1 << 20, None) == -3
    assert lib.bqq_attention_decode(p, 768, p, p, 512, 8, p, p, p, 1, 4, 1, 128, _cabi.F16, p, 256, p, 1 << 20, None) == -6
    assert lib.bqq_attention_decode(p, 768, p, p, 512, 8, p, p, p, 1, 4, 3, 128, _cabi.BF16, p, 256, p, 1 << 20, None) == -2
    assert lib.bqq_attention_decode(p, 768, p, p, 512, 8, p, p, p, 1, 4, 1, 128, _cabi.BF16, p, 256, p, 16, None) == -5
    # a position outside the cache is skipped by the kernel: nothing is written
    kc2 = torch.zeros(1, 8, 1, 128, device=dev, dtype=torch.bfloat16)
    q2 = torch.ones(1, 1, 6, 128, device=dev, dtype=torch.bfloat16)
    cs2 = torch.ones(8, 64, device=dev, dtype=torch.bfloat16)
    bad = torch.tensor([8], dtype=torch.int32, device=dev)
    out = attention_decode(q2, kc2, kc2.clone(), cs2, cs2, bad, 4, 1)
    torch.cuda.synchronize()
    assert out is not None and float(kc2.abs().max()) == 0.0
