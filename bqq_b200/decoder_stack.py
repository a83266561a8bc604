"""Random-init Llama-style decoder stack whose Linear layers are BinaryQuadratic.

This is the harness for the full-model decode configuration: 32 layers, hidden 4096,
intermediate 14336, 32 query / 8 KV heads, vocabulary 128256, every q/k/v/o/gate/up/down
projection replaced by a BinaryQuadratic layer (2 bit layers, P=Q=r=32), embeddings and
lm_head kept dense because the reference's replacement skips names containing 'head'
(lm/build_bqq_model.py:89-91) and the reference benchmark also skips 'embed'
(lm/benchmark_inference.py:47-49).  It follows the recipe of the reference's only end-to-end
decode loop (lm/benchmark_inference.py:24-85): random binary factors, greedy decode with a
KV cache.

Only the BinaryQuadratic layers are the product here.  In a decode step rotary embedding, cache append and
attention are one kernel of this library between two projections (bqq_attention_decode, part of the same chain of
programmatic dependent launches); the prefill uses one flash_attn library call where that package is present
(plain torch ops otherwise); the dense lm_head is a torch matmul (plumbing).  With world > 1 the layers are
column-parallel (bqq_b200/sharded.py): q/k/v (one stacked layer) are sharded by heads so attention
runs on local heads, gate/up (one stacked layer) share one sharding so SwiGLU is local, o_proj and down_proj are row-patch
sharded; four gathers per layer, all without reductions.  With a PeerGatherGroup the gathers are the
library's peer-to-peer stores (o_proj and down_proj send their row patches from the decode kernel's
epilogue, the attention output and the SwiGLU product go through the gather kernel); results too large
for the group's buffers (prefill) fall back to the process group's all-gather.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .bqq_modules import BinaryQuadratic
from .sharded import gather_columns

_ATT_WS: dict = {}


def attention_decode(qkv, k_cache, v_cache, cos, sin, lens, heads, kv_heads, peer=None):
    """Attention of one new token per sequence with this library's kernel (bqq_attention_decode): rotary embedding
    of q and k at position lens[b], append of k and v to the caches, softmax(q K^T / sqrt(d)) V over the cached
    rows.  qkv [B, 1, heads + 2 kv_heads, 128] bf16, caches [B, max_seq, kv_heads, 128]; returns [B, 1, heads, 128].
    With `peer` (a PeerGatherGroup; heads and kv_heads are this rank's) the outputs of all ranks are gathered in the
    same launch and [B, 1, world * heads, 128] is returned, the ranks' heads in rank order.
    Returns None where the kernel does not apply (other types or head sizes), so the caller can take another route."""
    from . import _cabi
    B, T, H, hd = qkv.shape
    if (T != 1 or hd != 128 or qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or heads // kv_heads > 16
            or not qkv.is_contiguous() or k_cache.stride(1) != kv_heads * hd or k_cache.stride(2) != hd
            or v_cache.stride() != k_cache.stride() or not cos.is_contiguous() or not sin.is_contiguous()
            or cos.dtype != torch.bfloat16 or lens.dtype != torch.int32):
        return None
    need = _cabi.lib.bqq_attention_decode_workspace_bytes(B, heads, kv_heads)
    stream = torch.cuda.current_stream(qkv.device)
    key = (qkv.device, stream.cuda_stream, B, heads, kv_heads)
    ws = _ATT_WS.get(key)
    if ws is None:
        ws = _ATT_WS[key] = torch.zeros(need, dtype=torch.uint8, device=qkv.device)
    out = torch.empty((B, 1, heads, hd), dtype=qkv.dtype, device=qkv.device)
    if peer is not None:
        gathered = torch.empty((B, 1, peer.world * heads, hd), dtype=qkv.dtype, device=qkv.device)
        _cabi.check(_cabi.lib.bqq_attention_decode_gathered(
            peer.descriptor(), qkv.data_ptr(), qkv.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), k_cache.stride(0),
            k_cache.shape[1], cos.data_ptr(), sin.data_ptr(), lens.data_ptr(), B, heads, kv_heads, hd, _cabi.BF16,
            out.data_ptr(), out.stride(0), gathered.data_ptr(), gathered.stride(0), ws.data_ptr(), ws.numel(),
            stream.cuda_stream), 'bqq_attention_decode_gathered')
        return gathered
    _cabi.check(_cabi.lib.bqq_attention_decode(qkv.data_ptr(), qkv.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
                                               k_cache.stride(0), k_cache.shape[1], cos.data_ptr(), sin.data_ptr(),
                                               lens.data_ptr(), B, heads, kv_heads, hd, _cabi.BF16, out.data_ptr(),
                                               out.stride(0), ws.data_ptr(), ws.numel(), stream.cuda_stream),
                'bqq_attention_decode')
    return out


try:        # library kernel for the attention part of the harness: rotary embedding, cache append and attention in one launch
    from flash_attn import flash_attn_with_kvcache as _flash_kvcache
except Exception:                                   # not installed: the plain torch ops below do the same
    _flash_kvcache = None


@dataclass
class StackConfig:
    layers: int = 32
    hidden: int = 4096
    intermediate: int = 14336
    heads: int = 32
    kv_heads: int = 8
    vocab: int = 128256
    bit_width: int = 2
    group: int = 32            # P = Q = r
    max_seq: int = 1024
    rope_theta: float = 500000.0
    own_attention: bool = True     # decode steps: this library's attention kernel (else flash_attn / torch ops)

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


def random_bq(out_f: int, in_f: int, cfg: StackConfig, device, gen) -> BinaryQuadratic:
    """Random BinaryQuadratic of the given shape, built on the device (bits Bernoulli(0.5),
    coefficients N(0, 0.02)); same construction as make_random_bqq in the reference benchmark."""
    gs, bw = cfg.group, cfg.bit_width
    rw, cw = out_f // gs, in_f // gs
    Y = torch.rand(bw, rw, cw, gs, gs, generator=gen, device=device) > 0.5
    Z = torch.rand(bw, rw, cw, gs, gs, generator=gen, device=device) > 0.5
    # coefficients scaled so activations keep a sane magnitude through 32 layers
    A = torch.randn(bw, rw, cw, 4, generator=gen, device=device) * (0.02 / math.sqrt(in_f / 4096))
    A[..., 1:] *= 0.05        # b, c, d act on sums of many entries
    bq = BinaryQuadratic(Y, Z, A)
    bq._ensure_packed()
    return bq


class DecoderLayer(nn.Module):
    def __init__(self, cfg: StackConfig, device, gen, rank: int, world: int, peer=None):
        super().__init__()
        self.cfg, self.rank, self.world, self.peer = cfg, rank, world, peer
        hd = cfg.head_dim
        self.local_heads = cfg.heads // world
        self.local_kv = max(1, cfg.kv_heads // world)
        if cfg.heads % world or (cfg.kv_heads % world and world % cfg.kv_heads):
            raise ValueError('heads must divide evenly over the ranks')
        h = cfg.hidden
        # each rank builds only its own row-patch shard (a shard is a layer with fewer row patches).
        # q, k and v share their input, so their row patches are stacked into one layer (one launch
        # instead of three); likewise gate and up.  Row patches are independent, so this is the same math.
        self.qkv_proj = random_bq((self.local_heads + 2 * self.local_kv) * hd, h, cfg, device, gen)
        self.o_proj = random_bq(h // world, h, cfg, device, gen)
        self.gate_up_proj = random_bq(2 * (cfg.intermediate // world), h, cfg, device, gen)
        self.down_proj = random_bq(h // world, cfg.intermediate, cfg, device, gen)
        self.norm1 = nn.Parameter(torch.ones(h, device=device, dtype=torch.bfloat16))
        self.norm2 = nn.Parameter(torch.ones(h, device=device, dtype=torch.bfloat16))

    def _fits(self, rows, cols, esize):
        return self.peer is not None and rows * cols * self.world * esize <= self.peer.max_bytes

    def _gather(self, y):
        if self.world == 1:
            return y
        if self._fits(y.numel() // y.shape[-1], y.shape[-1], y.element_size()):
            return self.peer.gather(y)
        return gather_columns(y)

    def _proj_gathered(self, proj, x, residual):
        """residual + row-patch sharded projection, outputs gathered on every rank."""
        rows = x.numel() // x.shape[-1]
        if rows <= 16 and self._fits(rows, proj.row_width * proj.y_row, x.element_size()):
            return proj.forward_gathered(x, self.peer, residual=residual)    # residual added before the rows are sent
        return residual + self._gather(proj(x))

    def forward(self, x, k_cache, v_cache, pos, rot, mask=None, fa=None):
        """x [B, T, hidden]; caches [B, max_seq, local_kv, head_dim].

        Prefill: `pos` is a Python int, positions pos..pos+T are written and attention is causal over
        the prefix.  Decode (T = 1, graph-capturable): `pos` is a 1-element device tensor, the cache
        row is written with index_copy_ and `mask` [1,1,1,max_seq] hides the unwritten tail.
        `fa` = (cos, sin, lens): with flash_attn present, rotary embedding, cache append and attention
        are one library kernel (lens int32 [B] = tokens already in the cache)."""
        cfg = self.cfg
        B, T, _ = x.shape
        hd = cfg.head_dim
        lh, lkv = self.local_heads, self.local_kv
        # normalisation, SwiGLU and residual adds are folded into the layers' kernels (forward_fused)
        qkv = self.qkv_proj.forward_fused(x, rms_weight=self.norm1, eps=1e-5).view(B, T, lh + 2 * lkv, hd)
        att, gathered = None, False
        if fa is not None and T == 1 and cfg.own_attention:
            # with several ranks the kernel also gathers its outputs (no separate gather launch)
            by_peer = self.world > 1 and self._fits(B, lh * hd, x.element_size())
            att = attention_decode(qkv, k_cache, v_cache, fa[0], fa[1], fa[2], lh, lkv, peer=self.peer if by_peer else None)
            gathered = att is not None and by_peer
        if att is not None:
            pass
        elif fa is not None and _flash_kvcache is not None and x.dtype in (torch.bfloat16, torch.float16):
            cos, sin, lens = fa
            att = _flash_kvcache(qkv[:, :, :lh], k_cache, v_cache, k=qkv[:, :, lh:lh + lkv], v=qkv[:, :, lh + lkv:],
                                 rotary_cos=cos, rotary_sin=sin, cache_seqlens=lens, causal=True,
                                 rotary_interleaved=True)                                 # [B, T, lh, hd]
        else:
            qk = _rope(qkv[:, :, :lh + lkv], rot)                    # rotary embedding on q and k heads at once
            q = qk[:, :, :lh].transpose(1, 2)
            k, v = qk[:, :, lh:], qkv[:, :, lh + lkv:]
            if mask is None:
                k_cache[:, pos:pos + T] = k
                v_cache[:, pos:pos + T] = v
                att = F.scaled_dot_product_attention(q, k_cache[:, :pos + T].transpose(1, 2),
                                                     v_cache[:, :pos + T].transpose(1, 2),
                                                     is_causal=(T > 1 and pos == 0), enable_gqa=True)
            else:
                k_cache.index_copy_(1, pos, k)
                v_cache.index_copy_(1, pos, v)
                att = F.scaled_dot_product_attention(q, k_cache.transpose(1, 2), v_cache.transpose(1, 2),
                                                     attn_mask=mask, enable_gqa=True)
            att = att.transpose(1, 2)
        if gathered:
            att = att.reshape(B, T, self.world * self.local_heads * hd)                   # gather 1: inside the attention launch
        else:
            att = self._gather(att.reshape(B, T, self.local_heads * hd))                  # gather 1
        if self.world == 1:
            x = self.o_proj.forward_fused(att, residual=x)
            gu = self.gate_up_proj.forward_fused(x, rms_weight=self.norm2, eps=1e-5)
            return self.down_proj.forward_fused(gu, swiglu=True, residual=x)
        x = self._proj_gathered(self.o_proj, att, x)                                        # gather 2
        rows = x.numel() // x.shape[-1]
        if rows <= 16 and self._fits(rows, 2 * (self.cfg.intermediate // self.world), x.element_size()):
            # the [gate | up] rows of all ranks are gathered by the layer's own launch, SwiGLU is applied by
            # down_proj as it reads them: no element-wise kernel, no separate gather
            gu = self.gate_up_proj.forward_gathered(x, self.peer, rms_weight=self.norm2, eps=1e-5, out_segments=2)
            return self.down_proj.forward_gathered(gu, self.peer, swiglu=True, residual=x)  # gathers 3 and 4
        gu = self.gate_up_proj.forward_fused(x, rms_weight=self.norm2, eps=1e-5)
        n = gu.shape[-1] // 2
        act = F.silu(gu[..., :n]) * gu[..., n:]
        act = self._gather(act)                                                             # gather 3
        return self._proj_gathered(self.down_proj, act, x)                                  # gather 4


def _rope(x, rot):
    """x [B, T, heads, head_dim], rot complex [T, head_dim/2]: rotate the pairs (x[2i], x[2i+1])."""
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    return torch.view_as_real(xc * rot[None, :, None, :]).flatten(-2).to(x.dtype)


class DecoderStack(nn.Module):
    def __init__(self, cfg: StackConfig, device, seed: int = 0, rank: int = 0, world: int = 1, peer=None):
        super().__init__()
        self.cfg, self.rank, self.world, self.device, self.peer = cfg, rank, world, device, peer
        gen = torch.Generator(device=device).manual_seed(seed + 7919 * rank)
        shared = torch.Generator(device=device).manual_seed(seed)            # identical on every rank
        self.embed = (torch.randn(cfg.vocab, cfg.hidden, generator=shared, device=device) * 0.5).to(torch.bfloat16)
        self.layers = nn.ModuleList(DecoderLayer(cfg, device, gen, rank, world, peer) for _ in range(cfg.layers))
        self.norm = torch.ones(cfg.hidden, device=device, dtype=torch.bfloat16)
        # dense bf16 lm_head, vocabulary sharded over the ranks
        self.lm_head = (torch.randn(cfg.vocab // world, cfg.hidden, generator=gen, device=device)
                        * (1.0 / math.sqrt(cfg.hidden))).to(torch.bfloat16)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=device).float() / cfg.head_dim))
        ang = torch.arange(cfg.max_seq, device=device).float()[:, None] * inv[None, :]
        self.rot = torch.polar(torch.ones_like(ang), ang)           # e^{i * position * frequency}, [max_seq, head_dim/2]
        self.cos, self.sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        self.use_flash = _flash_kvcache is not None

    def bqq_bytes_per_token(self) -> int:
        """Packed bits + fp32 coefficients streamed per decoded token on this rank."""
        from . import _cabi
        total = 0
        for layer in self.layers:
            for m in layer.children():
                if isinstance(m, BinaryQuadratic):
                    total += _cabi.lib.bqq_algorithmic_bytes(m._dims())
        return total

    def new_cache(self, batch: int):
        cfg = self.cfg
        kv = max(1, cfg.kv_heads // self.world)
        shape = (cfg.layers, 2, batch, cfg.max_seq, kv, cfg.head_dim)
        return torch.zeros(shape, device=self.device, dtype=torch.bfloat16)

    def _head(self, x_last):
        h = F.rms_norm(x_last, (self.cfg.hidden,), self.norm, 1e-5)
        logits = h @ self.lm_head.T                               # [B, vocab/world]
        if self.world > 1:
            rows = logits.numel() // logits.shape[-1]
            if self.peer is not None and rows * logits.shape[-1] * self.world * logits.element_size() <= self.peer.max_bytes:
                logits = self.peer.gather(logits)
            else:
                logits = gather_columns(logits)
        # argmax in two stages (a single reduction over 128256 columns runs in one CTA): per chunk, then over the chunks
        V = logits.shape[-1]
        c = next((c for c in range(min(V, 1024), 63, -1) if V % c == 0), 0)
        if c == 0:
            return logits.argmax(dim=-1)
        vals, idx = logits.reshape(-1, V // c, c).max(dim=2)
        best = vals.argmax(dim=1, keepdim=True)
        return (best * c + idx.gather(1, best)).squeeze(1)

    @torch.no_grad()
    def prefill(self, ids, cache):
        """ids [B, T] prompt -> first generated token ids [B]; fills cache positions 0..T."""
        x = self.embed[ids]
        T = ids.shape[1]
        rot = self.rot[:T]
        fa = (self.cos, self.sin, torch.zeros(ids.shape[0], dtype=torch.int32, device=self.device)) if self.use_flash else None
        for li, layer in enumerate(self.layers):
            x = layer(x, cache[li, 0], cache[li, 1], 0, rot, fa=fa)
        return self._head(x[:, -1])

    @torch.no_grad()
    def decode_step(self, ids, cache, pos):
        """One greedy decode step with static shapes (CUDA-graph capturable).
        ids [B] int64, pos 1-element int64 device tensor; returns next ids [B]."""
        x = self.embed[ids].unsqueeze(1)
        fa = ((self.cos, self.sin, pos.to(torch.int32).expand(ids.shape[0]).contiguous())
              if (self.use_flash or self.cfg.own_attention) else None)
        needs_torch_route = fa is None or (not self.use_flash and (
            x.dtype != torch.bfloat16 or self.cfg.head_dim != 128 or self.cfg.heads // self.cfg.kv_heads > 16))
        rot = self.rot.index_select(0, pos) if needs_torch_route else None
        mask = ((torch.arange(self.cfg.max_seq, device=self.device) <= pos).view(1, 1, 1, -1)
                if needs_torch_route else None)
        for li, layer in enumerate(self.layers):
            x = layer(x, cache[li, 0], cache[li, 1], pos, rot, mask, fa=fa)
        return self._head(x[:, -1])
