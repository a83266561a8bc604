// Decode kernel (M <= 16 rows of X): the packed planes are streamed once and both
// contractions run on the int8 tensor cores (mma.sync m16n8k32, u8 x s8 -> s32).
//
// Per (row patch i, col patch j, bit b) with coefficients (a,b,c,d):
//   xsum = sum_q x[j,q];  t_k = sum_q Z[k,q] x[j,q];  u_k = a t_k + b xsum
//   y[i,p] += sum_k Y[p,k] u_k + c sum_k t_k (+ d xsum once per patch)
// which is BinaryQuadratic.forward without materialising W
// (neural_network_compression/src/bqq_modules.py:34-46; the identity of
// src/bqq_cuda.cu:82-84,134-156).
//
// Binary operand: a lane's 32-bit plane word holds a 4-row x 8-column fragment;
// `word & (0x01010101 << rr)` is directly an A-operand register whose bytes are
// 0 or 2^rr, so a bit costs 1/4 of a logic instruction to expand.  The power of
// two is removed again when the s32 results are converted.
// Real operand: x is quantised per col patch to 16-bit block fixed point (two s8
// digits) by a small preparation kernel, u per warp to 24-bit fixed point (three s8
// digits); digits occupy
// separate B-operand columns, so the integer products are exact and the only
// errors are the two roundings (about 2^-16 of the patch maximum of |x|).
//
// Work split: CTA = (row patch i, bit layer b, chunk of col-patch groups, M tile);
// warp w owns super-groups w, w+4, ... of the chunk.  The split never depends on
// the number of row patches, so a row shard of a layer produces bit-identical
// outputs.  CTA partial sums go to scratch; the last CTA of a row patch adds
// them in a fixed order, adds bias and converts to the output type.
#pragma once
#include "bqq_async.cuh"
#include "bqq_common.cuh"

namespace bqq {

constexpr int kDW = 4;                   // warps per CTA
constexpr int kDT = kDW * 32;
constexpr int kMaxCounters = 65536;      // fixed-size counter region at the start of the workspace
constexpr size_t kCounterBytes = (size_t)kMaxCounters * 4;

struct DecodePlan {
  int variant;     // geometry variant: 0 (PT,QT,RT)=(1,1,1), 1 (2,2,1), 2 (2,2,2), 3 (4,4,2)
  int NB;          // rows of X per CTA: 1 or 4
  int mtiles;      // ceil(M / NB)
  int sgw;         // super-groups per warp
  int nchunks;     // chunks per bit layer
  int nparts;      // partial sums per output = bw * nchunks
  size_t smem;
  size_t partial_floats;
  size_t xdig_bytes, xmeta_bytes;   // workspace regions written by the activation preparation kernel
};

struct DecodeParams {
  const uint4* zp;
  const uint4* yp;
  const void *a, *b, *c, *d;
  const void* x;
  void* y;
  const void* bias;
  float* partial;
  unsigned* counters;
  const uint8_t* xdig;       // s8 digits of x, [Mp][JG][digit][QT][half][t][sub] words (preparation kernel)
  const float* xscale;       // [Mp][cwp] block scale of x
  const float* xsum;         // [Mp][cwp] sum_q x
  const float* xl1;          // [Mp][cwp] sum_q |x|
  int Mp, cwp;               // M and cw rounded up to the kernel's tiles (rows per CTA, 4 col patches)
  int64_t ldx, ldy;
  int coef_dtype, x_dtype, y_dtype, bias_dtype;
  int M, bw, rw, cw, P, Q;
  int PTg, QTg, RTg;       // 32-blocks of the planes as packed
  int JG, NS;
  int sgw, nchunks, mtiles;
  int coef_vec;            // 1: fp32 coefficients, cw % 4 == 0, 16-byte aligned -> 128-bit loads
};

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// same with a zero accumulator input (first k-step of a contraction)
__device__ __forceinline__ void mma_u8s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ uint32_t pick(const uint4& v, int sub) {
  return sub == 0 ? v.x : (sub == 1 ? v.y : (sub == 2 ? v.z : v.w));
}

// Shared-memory carve-up (bytes), shared by host plan and kernel.  Everything a CTA reads from
// global memory is staged here by bulk copies issued at kernel start: the plane words of its chunk
// (one mbarrier per step of 4 super-groups), coefficients, x digits and x statistics.
struct DecodeSmem {
  int bars, zs, ys, xd, coef, meta, udig, red, total;
  __host__ __device__ DecodeSmem(int sgw, int NB, int PT, int QT, int RT) {
    const int nsg = kDW * sgw;                        // super-groups per chunk
    int o = 0;
    bars = o;  o += 128;                              // up to 9 mbarriers (8 steps + misc)
    zs = o;    o += nsg * RT * QT * 512;              // uint4 [nsg][RT][QT][32]
    ys = o;    o += nsg * PT * RT * 512;              // uint4 [nsg][PT][RT][32]
    xd = o;    o += NB * nsg * 2 * QT * 128;          // uint4 [NB][nsg][digit][QT][8]
    coef = o;  o += 4 * nsg * 16;                     // float [a|b|c|d][nsg*4]
    meta = o;  o += NB * 3 * nsg * 16;                // float [NB][scale|sum|l1][nsg*4]
    udig = o;  o += kDW * kGroup * NB * 4 * RT * 32;  // u8 [warps][4 sub][NB][4 slots][RP]
    red = o;   o += kDW * NB * PT * 32 * 4;           // f32 [warps][NB][PP]
    total = o;
  }
};
constexpr int kMaxSgw = 8;

// ---- activation preparation ------------------------------------------------------------------
// One pass over x [M, cw*Q]: per (row m, col patch j) the 16-bit block fixed point digits
//   xdig (s8 digits: x_int = lo + 256*hi, x ~ x_int * scale), 2*32*QT bytes per pair,
// and xscale / xsum / xl1 [Mp][cwp] = scale, sum_q x, sum_q |x|.  Rows m >= M and col patches
// j >= cw (Mp, cwp: M and cw rounded up to the kernel's tiles) are written as zeros so that the
// decode kernel needs no edge tests.  8 lanes share one (m, j) pair.
template <int QT>
__global__ void __launch_bounds__(128)
bqq_xprep_kernel(const void* __restrict__ x, int x_dtype, int64_t ldx, int M, int cw, int Q, int Mp, int cwp,
                 uint8_t* __restrict__ xdig, float* __restrict__ xscale, float* __restrict__ xsum,
                 float* __restrict__ xl1) {
  constexpr int QP = QT * 32;
  // the decode kernel of this layer may start now: it first streams its weight planes and only
  // then waits (griddepcontrol.wait) for this grid to finish
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int sub8 = threadIdx.x & 7;
  const int pairs = Mp * cwp;
  const int pair = (blockIdx.x * 128 + threadIdx.x) >> 3;
  const bool inside = pair < pairs;
  const int m = inside ? pair / cwp : 0, j = inside ? pair % cwp : 0;
  const bool live = inside && m < M && j < cw;
  float v[4 * QT];
  float amax = 0.f, sum = 0.f, l1 = 0.f;
#pragma unroll
  for (int e = 0; e < 4 * QT; ++e) {
    const int q = sub8 * 4 * QT + e;
    v[e] = (live && q < Q) ? load_as_float(x, (size_t)m * ldx + (size_t)j * Q + q, x_dtype) : 0.f;
    amax = fmaxf(amax, fabsf(v[e]));
    sum += v[e];
    l1 += fabsf(v[e]);
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  if (!inside) return;
  const float inv = amax > 0.f ? 32512.f / amax : 0.f;
  // digit layout [Mp][JG][digit][QT][half][t][sub] words (4 consecutive q each): the 4 col patches of a
  // super-group are adjacent, so a lane of the decode kernel fetches its B-operand words of a whole
  // super-group with one 128-bit load per (digit, half)
  const int JG = cwp / kGroup;
  uint32_t* words = reinterpret_cast<uint32_t*>(xdig);
#pragma unroll
  for (int w4 = 0; w4 < QT; ++w4) {
    uint32_t D[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) D[e] = (uint32_t)(__float2int_rn(v[w4 * 4 + e] * inv) + 0x8080) ^ 0x8080u;
    const int q4 = sub8 * QT + w4;                 // index of this group of 4 consecutive q
    const int qt = q4 >> 3, half = (q4 >> 2) & 1, tt = q4 & 3;
    const size_t base = ((size_t)m * JG + (j >> 2)) * 2;
    // x_int = lo + 256*hi with both digits signed bytes
    words[((((base + 0) * QT + qt) * 2 + half) * 4 + tt) * kGroup + (j & 3)] =
        __byte_perm(__byte_perm(D[0], D[1], 0x0040), __byte_perm(D[2], D[3], 0x0040), 0x5410);
    words[((((base + 1) * QT + qt) * 2 + half) * 4 + tt) * kGroup + (j & 3)] =
        __byte_perm(__byte_perm(D[0], D[1], 0x0051), __byte_perm(D[2], D[3], 0x0051), 0x5410);
  }
  if (sub8 == 0) {
    xscale[pair] = amax * (1.f / 32512.f);
    xsum[pair] = sum;
    xl1[pair] = l1;
  }
}

template <int PT, int QT, int RT, int NB>
__global__ void __launch_bounds__(kDT)
bqq_decode_kernel(const DecodeParams p) {
  constexpr int RP = RT * 32;
  constexpr int PP = PT * 32;
  constexpr int NT2 = NB == 1 ? 1 : 2;              // n-tiles of the second contraction
  extern __shared__ __align__(128) uint8_t sm[];
  const int nsg = kDW * p.sgw;                      // super-groups per chunk (smem row pitch)
  const DecodeSmem L(p.sgw, NB, PT, QT, RT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L.bars);      // [0..sgw) steps, [kMaxSgw] misc
  const uint4* zs = reinterpret_cast<const uint4*>(sm + L.zs);
  const uint4* ys = reinterpret_cast<const uint4*>(sm + L.ys);
  const uint4* xd = reinterpret_cast<const uint4*>(sm + L.xd);
  const float* scoef = reinterpret_cast<const float*>(sm + L.coef);
  const float* smeta = reinterpret_cast<const float*>(sm + L.meta);
  uint8_t* udig = sm + L.udig;
  float* red = reinterpret_cast<float*>(sm + L.red);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;

  int bid = blockIdx.x;
  const int chunk = bid % p.nchunks; bid /= p.nchunks;
  const int bit = bid % p.bw;
  const int i = bid / p.bw;
  const int m0 = blockIdx.y * NB;
  const int jg0 = chunk * nsg;                      // first col-patch group of the chunk
  const int nvalid = min(nsg, p.JG - jg0);          // super-groups that exist in this chunk
  const uint32_t crow = (uint32_t)(((size_t)bit * p.rw + i) * p.cw);   // coefficient row of (bit, i)
  const uint32_t drow = (uint32_t)((size_t)i * p.cw);

  // ---- one thread issues every copy of the CTA; consumers wait on the mbarriers -----------------
  if (tid == 0) {
    for (int b = 0; b <= kMaxSgw; ++b) mbar_init(bars + b, 1);
    mbar_init_fence();
    const uint32_t n16 = (uint32_t)nvalid * 16u;                    // bytes of nvalid*4 floats
    uint32_t misc = NB * (3 * n16 + (uint32_t)nvalid * 2 * QT * 128);
    if (p.coef_vec) misc += 3 * n16 + (bit == 0 ? n16 : 0u);
    mbar_expect_tx(bars + kMaxSgw, misc);
    // weights first: they do not depend on the activation preparation kernel
    const uint32_t zb = (uint32_t)p.RTg * p.QTg * 512, yb = (uint32_t)p.PTg * p.RTg * 512;   // bytes per super-group
    const size_t sg0 = (size_t)i * p.NS + (size_t)bit * p.JG + jg0;
    for (int it = 0; it < p.sgw; ++it) {
      const int nv = min(kDW, nvalid - kDW * it);
      if (nv <= 0) break;
      mbar_expect_tx(bars + it, (uint32_t)nv * (zb + yb));
      bulk_load(const_cast<uint4*>(zs) + (size_t)it * kDW * (zb / 16), p.zp + (sg0 + kDW * it) * (zb / 16),
                (uint32_t)nv * zb, bars + it);
      bulk_load(const_cast<uint4*>(ys) + (size_t)it * kDW * (yb / 16), p.yp + (sg0 + kDW * it) * (yb / 16),
                (uint32_t)nv * yb, bars + it);
    }
    if (p.coef_vec) {
      float* sc = const_cast<float*>(scoef);
      bulk_load(sc, reinterpret_cast<const float*>(p.a) + crow + jg0 * kGroup, n16, bars + kMaxSgw);
      bulk_load(sc + nsg * 4, reinterpret_cast<const float*>(p.b) + crow + jg0 * kGroup, n16, bars + kMaxSgw);
      bulk_load(sc + nsg * 8, reinterpret_cast<const float*>(p.c) + crow + jg0 * kGroup, n16, bars + kMaxSgw);
      if (bit == 0)
        bulk_load(sc + nsg * 12, reinterpret_cast<const float*>(p.d) + drow + jg0 * kGroup, n16, bars + kMaxSgw);
    }
    // the x digits and statistics come from the preparation kernel launched just before this one
    // (programmatic dependent launch): wait for it to complete before copying its output
    asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
    for (int beta = 0; beta < NB; ++beta) {
      const size_t row = (size_t)(m0 + beta) * p.cwp + (size_t)jg0 * kGroup;
      float* sm_meta = const_cast<float*>(smeta) + beta * 3 * nsg * 4;
      bulk_load(sm_meta, p.xscale + row, n16, bars + kMaxSgw);
      bulk_load(sm_meta + nsg * 4, p.xsum + row, n16, bars + kMaxSgw);
      bulk_load(sm_meta + nsg * 8, p.xl1 + row, n16, bars + kMaxSgw);
      bulk_load(const_cast<uint4*>(xd) + (size_t)beta * nsg * 2 * QT * 8,
                reinterpret_cast<const uint4*>(p.xdig) + ((size_t)(m0 + beta) * p.JG + jg0) * 2 * QT * 8,
                (uint32_t)nvalid * 2 * QT * 128, bars + kMaxSgw);
    }
  }

  // ---- zero the digit exchange buffer (slot 3 of every row must stay zero) --------------------
  constexpr int kUSub = NB * 4 * RP;                 // bytes of one col patch's u digits
  uint8_t* my_udig = udig + (size_t)warp * kGroup * kUSub;
  for (int e = lane; e < kGroup * kUSub / 4; e += 32) reinterpret_cast<uint32_t*>(my_udig)[e] = 0u;
  __syncthreads();                                   // barriers are initialised for every waiter
  bool ok = mbar_wait(bars + kMaxSgw, 0);

  // ---- fixed-point scale of u for this warp: bound |a| sum|x| + |b| |sum x| over its patch-bits
  const int my_beta = NB == 1 ? 0 : t;
  float ub = 0.f;
  {
    const int it = lane >> 2, sub = lane & 3;
    const int sgi = kDW * it + warp;                 // super-group index inside the chunk
    const int j = (jg0 + sgi) * kGroup + sub;
    if (it < p.sgw && sgi < nvalid && j < p.cw) {
      float ca, cb;
      if (p.coef_vec) {
        ca = fabsf(scoef[sgi * 4 + sub]);
        cb = fabsf(scoef[nsg * 4 + sgi * 4 + sub]);
      } else {
        ca = fabsf(load_as_float(p.a, crow + j, p.coef_dtype));
        cb = fabsf(load_as_float(p.b, crow + j, p.coef_dtype));
      }
#pragma unroll
      for (int beta = 0; beta < NB; ++beta) {
        const float* mrow = smeta + beta * 3 * nsg * 4;
        ub = fmaxf(ub, fmaf(ca, mrow[nsg * 8 + sgi * 4 + sub], cb * fabsf(mrow[nsg * 4 + sgi * 4 + sub])));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ub = fmaxf(ub, __shfl_xor_sync(0xffffffffu, ub, o));
  }
  const float inv_us = ub > 0.f ? 4128768.f / ub : 0.f;      // |u| * inv_us < 2^22
  __syncwarp();

  int acc[PT][2][NT2][4];
#pragma unroll
  for (int pt = 0; pt < PT; ++pt)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[pt][mt][nt][e] = 0;
  float cacc = 0.f, dacc = 0.f;
  const float rs_t = 1.f / (float)(1 << t);
  const int e0 = t == 0, e1 = t == 1, e2 = t == 2, e3 = t == 3;
  const int f0 = e0 << 8, f1 = e1 << 8, f2 = e2 << 8, f3 = e3 << 8;
  // lane constants: where this lane's B-operand column (n = g) finds its x digits, where the
  // lane's row of X keeps scale and sum, where its u digits go and come from
  const uint4* xlane = xd + ((size_t)(NB == 1 ? 0 : (g >> 1)) * nsg * 2 + (g & 1)) * (QT * 8) + t;
  const float* mrow = smeta + my_beta * 3 * nsg * 4;   // [scale | sum | l1] of this lane's row of X
  uint8_t* ust = my_udig + (NB == 1 ? g + 8 * t : t * 4 * RP + g);
  const uint8_t* uld[NT2];
#pragma unroll
  for (int nt = 0; nt < NT2; ++nt) {
    const int beta = NB == 1 ? 0 : 2 * nt + (g >> 2);
    const int slot = NB == 1 ? min(g, 3) : (g & 3);      // slot 3 stays zero
    uld[nt] = my_udig + (beta * 4 + slot) * RP + 4 * t;
  }
  constexpr float kMagic = 12582912.f;                // 1.5 * 2^23: float -> int by mantissa alignment
  constexpr uint32_t kUnbias = 0x808080u - 0x4B400000u;

  for (int it = 0; it < p.sgw; ++it) {
    const int sgi = kDW * it + warp;                  // super-group index inside the chunk
    if (sgi >= nvalid) break;
    ok = mbar_wait(bars + it, 0) && ok;
    // plane words of this super-group
    uint4 zw[RT][QT], yw[PT][RT];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int qt = 0; qt < QT; ++qt)
        zw[rt][qt] = (rt < p.RTg && qt < p.QTg) ? zs[((size_t)(sgi * p.RTg + rt) * p.QTg + qt) * 32 + lane]
                                                  : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int pt = 0; pt < PT; ++pt)
#pragma unroll
      for (int rt = 0; rt < RT; ++rt)
        yw[pt][rt] = (pt < p.PTg && rt < p.RTg) ? ys[((size_t)(sgi * p.PTg + pt) * p.RTg + rt) * 32 + lane]
                                                  : make_uint4(0u, 0u, 0u, 0u);
    // per super-group: coefficients, x scale / sum and the x digit registers of its 4 col patches
    float ca4[4], cb4[4], cc4[4], cd4[4];
    if (p.coef_vec) {
      const float4 va = *reinterpret_cast<const float4*>(scoef + sgi * 4);
      const float4 vb = *reinterpret_cast<const float4*>(scoef + nsg * 4 + sgi * 4);
      const float4 vc = *reinterpret_cast<const float4*>(scoef + nsg * 8 + sgi * 4);
      ca4[0] = va.x; ca4[1] = va.y; ca4[2] = va.z; ca4[3] = va.w;
      cb4[0] = vb.x; cb4[1] = vb.y; cb4[2] = vb.z; cb4[3] = vb.w;
      cc4[0] = vc.x; cc4[1] = vc.y; cc4[2] = vc.z; cc4[3] = vc.w;
      if (bit == 0) {
        const float4 vd = *reinterpret_cast<const float4*>(scoef + nsg * 12 + sgi * 4);
        cd4[0] = vd.x; cd4[1] = vd.y; cd4[2] = vd.z; cd4[3] = vd.w;
      } else {
        cd4[0] = cd4[1] = cd4[2] = cd4[3] = 0.f;
      }
    } else {
      const uint32_t jb = (uint32_t)(jg0 + sgi) * kGroup;
#pragma unroll
      for (int sub = 0; sub < kGroup; ++sub) {
        const bool in = (int)(jb + sub) < p.cw;          // ragged last group: zero coefficients
        ca4[sub] = in ? load_as_float(p.a, crow + jb + sub, p.coef_dtype) : 0.f;
        cb4[sub] = in ? load_as_float(p.b, crow + jb + sub, p.coef_dtype) : 0.f;
        cc4[sub] = in ? load_as_float(p.c, crow + jb + sub, p.coef_dtype) : 0.f;
        cd4[sub] = (in && bit == 0) ? load_as_float(p.d, drow + jb + sub, p.coef_dtype) : 0.f;
      }
    }
    const float4 xsc4 = *reinterpret_cast<const float4*>(mrow + sgi * 4);
    const float4 xs4 = *reinterpret_cast<const float4*>(mrow + nsg * 4 + sgi * 4);
    const float xscv[4] = {xsc4.x, xsc4.y, xsc4.z, xsc4.w};
    const float xsv[4] = {xs4.x, xs4.y, xs4.z, xs4.w};
    uint32_t bx0[kGroup][QT], bx1[kGroup][QT];
#pragma unroll
    for (int qt = 0; qt < QT; ++qt) {
      const uint4 h0 = xlane[(size_t)sgi * (2 * QT * 8) + qt * 8];
      const uint4 h1 = xlane[(size_t)sgi * (2 * QT * 8) + qt * 8 + 4];
      bx0[0][qt] = h0.x; bx0[1][qt] = h0.y; bx0[2][qt] = h0.z; bx0[3][qt] = h0.w;
      bx1[0][qt] = h1.x; bx1[1][qt] = h1.y; bx1[2][qt] = h1.z; bx1[3][qt] = h1.w;
    }

#pragma unroll
    for (int sub = 0; sub < kGroup; ++sub) {
      const float ca = ca4[sub], cc = cc4[sub];
      const float xs = xsv[sub];
      const float bxs = cb4[sub] * xs;
      dacc = fmaf(cd4[sub], xs, dacc);

      // ---- first contraction: T[k][digit] = sum_q Z[k][q] xdigit[q] --------------------
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        int c1[2][4];
#pragma unroll
        for (int qt = 0; qt < QT; ++qt) {
          const uint32_t w = pick(zw[rt][qt], sub);
          const uint32_t w4 = w >> 4;
          if (qt == 0) {
            mma_u8s8_first(c1[0], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u,
                           bx0[sub][qt], bx1[sub][qt]);
            mma_u8s8_first(c1[1], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u,
                           bx0[sub][qt], bx1[sub][qt]);
          } else {
            mma_u8s8(c1[0], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u,
                     bx0[sub][qt], bx1[sub][qt]);
            mma_u8s8(c1[1], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u,
                     bx0[sub][qt], bx1[sub][qt]);
          }
        }
        if (NB == 1) {
          // every lane sees (lo, hi) in its two columns; lane (g,t) finishes row k = 32rt + g + 8t
          // (branch-free: lane constants e_r = [t == r], f_r = 256 e_r pick the row and join the digits)
          const int I = c1[0][0] * e0 + c1[0][1] * f0 + c1[0][2] * e1 + c1[0][3] * f1 +
                        c1[1][0] * e2 + c1[1][1] * f2 + c1[1][2] * e3 + c1[1][3] * f3;
          const float tf = (float)I * (xscv[sub] * rs_t);
          cacc = fmaf(cc, tf, cacc);
          const uint32_t D = ((uint32_t)__float_as_int(fmaf(fmaf(ca, tf, bxs), inv_us, kMagic)) + kUnbias) ^ 0x808080u;
          uint8_t* dst = ust + sub * kUSub + rt * 32;
          dst[0] = (uint8_t)D;
          dst[RP] = (uint8_t)(D >> 8);
          dst[2 * RP] = (uint8_t)(D >> 16);
        } else {
          // lane (g,t) owns row t of X: finishes rows k = 32rt + g + 8rr, rr = 0..3
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int lo = c1[rr >> 1][2 * (rr & 1)];
            const int hi = c1[rr >> 1][2 * (rr & 1) + 1];
            const float tf = (float)(lo + (hi << 8)) * (xscv[sub] * (1.f / (float)(1 << rr)));
            cacc = fmaf(cc, tf, cacc);
            const uint32_t D = ((uint32_t)__float_as_int(fmaf(fmaf(ca, tf, bxs), inv_us, kMagic)) + kUnbias) ^ 0x808080u;
            uint8_t* dst = ust + sub * kUSub + rt * 32 + 8 * rr;
            dst[0] = (uint8_t)D;
            dst[RP] = (uint8_t)(D >> 8);
            dst[2 * RP] = (uint8_t)(D >> 16);
          }
        }
      }
    }
    __syncwarp();

    // ---- second contraction: V[p][digit] += sum_k Y[p][k] udigit[k] --------------------
#pragma unroll
    for (int sub = 0; sub < kGroup; ++sub) {
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        uint32_t bu[NT2][2];
#pragma unroll
        for (int nt = 0; nt < NT2; ++nt) {
          bu[nt][0] = *reinterpret_cast<const uint32_t*>(uld[nt] + sub * kUSub + rt * 32);
          bu[nt][1] = *reinterpret_cast<const uint32_t*>(uld[nt] + sub * kUSub + rt * 32 + 16);
        }
#pragma unroll
        for (int pt = 0; pt < PT; ++pt) {
          const uint32_t w = pick(yw[pt][rt], sub);
          const uint32_t w4 = w >> 4;
#pragma unroll
          for (int nt = 0; nt < NT2; ++nt) {
            mma_u8s8(acc[pt][0][nt], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u,
                     bu[nt][0], bu[nt][1]);
            mma_u8s8(acc[pt][1][nt], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u,
                     bu[nt][0], bu[nt][1]);
          }
        }
      }
    }
    __syncwarp();
  }

  if (!ok && lane == 0) atomicExch(p.counters + (kMaxCounters - 1), 1u);   // a bounded wait gave up

  // ---- warp epilogue: digits -> float, undo the 2^rr row scales, add c and d terms -----------
  // cacc holds the lane's share of c * sum_k t_k for row my_beta of X; dacc the d term.
  float cterm = cacc;
  if (NB == 1) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cterm += __shfl_xor_sync(0xffffffffu, cterm, o);
  } else {
#pragma unroll
    for (int o = 16; o >= 4; o >>= 1) cterm += __shfl_xor_sync(0xffffffffu, cterm, o);   // lanes with equal t
  }
  cterm += dacc;
  const float us = ub * (1.f / 4128768.f);
#pragma unroll
  for (int nt = 0; nt < NT2; ++nt) {
    // which row of X and which digits this lane's two columns carry
    const int beta = NB == 1 ? 0 : 2 * nt + (t >> 1);
    const int tt = NB == 1 ? t : (t & 1);
    const float w_even = tt == 0 ? 1.f : (tt == 1 ? 65536.f : 0.f);
    const float w_odd = tt == 0 ? 256.f : 0.f;
    const float ct_b = NB == 1 ? cterm : __shfl_sync(0xffffffffu, cterm, (lane & ~3) | beta);
#pragma unroll
    for (int pt = 0; pt < PT; ++pt)
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int rr = 2 * mt + half;
          float v = w_even * (float)acc[pt][mt][nt][2 * half] + w_odd * (float)acc[pt][mt][nt][2 * half + 1];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          if (NB == 1) v += __shfl_xor_sync(0xffffffffu, v, 2);
          const float out = fmaf(v, us * (1.f / (float)(1 << rr)), ct_b);
          const bool writer = NB == 1 ? (t == 0) : ((t & 1) == 0);
          if (writer) red[(size_t)(warp * NB + beta) * PP + pt * 32 + g + 8 * rr] = out;
        }
  }
  __syncthreads();

  // ---- CTA result, then the cross-CTA reduction in a fixed order ----------------------------
  const int nparts = p.bw * p.nchunks;
  const int part = bit * p.nchunks + chunk;
  const int mrows = p.mtiles * NB;
  const size_t out_stride = (size_t)p.rw * PP;
  if (nparts == 1) {
    for (int idx = tid; idx < NB * PP; idx += kDT) {
      const int beta = idx / PP, pp = idx % PP;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kDW; ++w) v += red[(size_t)(w * NB + beta) * PP + pp];
      if (pp < p.P && m0 + beta < p.M) {
        const int o = i * p.P + pp;
        if (p.bias) v += load_as_float(p.bias, o, p.bias_dtype);
        store_from_float(p.y, (size_t)(m0 + beta) * p.ldy + o, p.y_dtype, v);
      }
    }
    return;
  }
  for (int idx = tid; idx < NB * PP; idx += kDT) {
    const int beta = idx / PP, pp = idx % PP;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kDW; ++w) v += red[(size_t)(w * NB + beta) * PP + pp];
    p.partial[((size_t)part * mrows + m0 + beta) * out_stride + (size_t)i * PP + pp] = v;
  }
  __threadfence();
  __syncthreads();
  __shared__ unsigned ticket;
  if (tid == 0) ticket = atomicAdd(p.counters + i * p.mtiles + blockIdx.y, 1u);
  __syncthreads();
  if (ticket != (unsigned)(nparts - 1)) return;
  __threadfence();
  for (int idx = tid; idx < NB * PP; idx += kDT) {
    const int beta = idx / PP, pp = idx % PP;
    if (pp < p.P && m0 + beta < p.M) {
      float v = 0.f;
      for (int sp = 0; sp < nparts; ++sp)
        v += __ldcg(p.partial + ((size_t)sp * mrows + m0 + beta) * out_stride + (size_t)i * PP + pp);
      const int o = i * p.P + pp;
      if (p.bias) v += load_as_float(p.bias, o, p.bias_dtype);
      store_from_float(p.y, (size_t)(m0 + beta) * p.ldy + o, p.y_dtype, v);
    }
  }
  if (tid == 0) p.counters[i * p.mtiles + blockIdx.y] = 0u;   // ready for the next call
}

template <int PT, int QT, int RT, int NB>
static int launch_decode_variant(const DecodeParams& p, const DecodePlan& pl, cudaStream_t st) {
  auto kern = bqq_decode_kernel<PT, QT, RT, NB>;
  if (pl.smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess)
      return BQQ_ERR_CUDA;
  }
  const int pairs = p.Mp * p.cwp;
  bqq_xprep_kernel<QT><<<(pairs * 8 + 127) / 128, 128, 0, st>>>(
      p.x, p.x_dtype, p.ldx, p.M, p.cw, p.Q, p.Mp, p.cwp, const_cast<uint8_t*>(p.xdig),
      const_cast<float*>(p.xscale), const_cast<float*>(p.xsum), const_cast<float*>(p.xl1));
  // decode kernel: programmatic dependent launch after the preparation kernel, so that its weight
  // copies overlap the preparation; the kernel itself waits before it touches the prepared x
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.rw * p.bw * p.nchunks, pl.mtiles);
  cfg.blockDim = dim3(kDT);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return launch_status();
}

// One translation unit per geometry variant (compiled in parallel).
template <int VARIANT>
int decode_launch_variant(const DecodeParams& p, const DecodePlan& pl, cudaStream_t st);

#define BQQ_DECODE_VARIANT(VARIANT, PT, QT, RT)                                                    \
  template <>                                                                                      \
  int decode_launch_variant<VARIANT>(const DecodeParams& p, const DecodePlan& pl, cudaStream_t st) { \
    return pl.NB == 1 ? launch_decode_variant<PT, QT, RT, 1>(p, pl, st)                            \
                      : launch_decode_variant<PT, QT, RT, 4>(p, pl, st);                           \
  }

}  // namespace bqq
