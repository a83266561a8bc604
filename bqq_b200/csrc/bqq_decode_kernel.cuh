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
// digits), u per CTA to 24-bit fixed point (three s8 digits); digits occupy
// separate B-operand columns, so the integer products are exact and the only
// errors are the two roundings (about 2^-16 of the patch maximum of |x|).
//
// Work split: CTA = (row patch i, bit layer b, chunk of col-patch groups, M tile);
// warp w owns super-groups w, w+4, ... of the chunk.  The split never depends on
// the number of row patches, so a row shard of a layer produces bit-identical
// outputs.  CTA partial sums go to scratch; the last CTA of a row patch adds
// them in a fixed order, adds bias and converts to the output type.
#pragma once
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
  int64_t ldx, ldy;
  int coef_dtype, x_dtype, y_dtype, bias_dtype;
  int M, bw, rw, cw, P, Q;
  int PTg, QTg, RTg;       // 32-blocks of the planes as packed
  int JG, NS;
  int sgw, nchunks, mtiles;
#ifdef BQQ_BOUNDS_CHECK
  unsigned long long lim_z, lim_y, lim_coef, lim_d, lim_x, lim_y_out, lim_partial, lim_smem;
  volatile unsigned long long* dbg;   // host-mapped report: [0]=count, then {code, index, limit, where}
#endif
};

#ifdef BQQ_BOUNDS_CHECK
// Self-check build: every global access and the main shared-memory accesses compare their
// index with the extent; a violation is recorded and the access skipped.
__device__ inline bool bqq_chk(volatile unsigned long long* dbg, int code, unsigned long long idx,
                               unsigned long long lim) {
  if (idx < lim) return true;
  if (dbg) {
    unsigned long long n = atomicAdd((unsigned long long*)dbg, 1ull);
    if (n < 15) {
      dbg[1 + 4 * n] = (unsigned long long)code;
      dbg[2 + 4 * n] = idx;
      dbg[3 + 4 * n] = lim;
      dbg[4 + 4 * n] = ((unsigned long long)blockIdx.x << 32) | ((unsigned long long)blockIdx.y << 16) | threadIdx.x;
      __threadfence_system();
    }
  }
  return false;
}
#define BQQ_CHK(code, idx, lim) bqq_chk(p.dbg, code, (unsigned long long)(idx), (unsigned long long)(lim))
#else
#define BQQ_CHK(code, idx, lim) true
#endif

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pick(const uint4& v, int sub) {
  return sub == 0 ? v.x : (sub == 1 ? v.y : (sub == 2 ? v.z : v.w));
}

// Shared-memory carve-up (bytes), shared by host plan and kernel.
struct DecodeSmem {
  int xdig, xscale, xsum, xl1, ubound, udig, red, total;
  __host__ __device__ DecodeSmem(int JC, int NB, int QT, int RT, int PT) {
    int o = 0;
    xdig = o;   o += JC * NB * 2 * QT * 32;          // u8 [JC][NB][2][QP]
    xscale = o; o += JC * NB * 4;
    xsum = o;   o += JC * NB * 4;
    xl1 = o;    o += JC * NB * 4;
    ubound = o; o += 16;
    o = (o + 15) & ~15;
    udig = o;   o += kDW * NB * 4 * RT * 32;          // u8 [warps][NB][4 slots][RP]
    red = o;    o += kDW * NB * PT * 32 * 4;          // f32 [warps][NB][PP]
    total = o;
  }
};

template <int PT, int QT, int RT, int NB>
__global__ void __launch_bounds__(kDT)
bqq_decode_kernel(const DecodeParams p) {
  constexpr int QP = QT * 32;
  constexpr int RP = RT * 32;
  constexpr int PP = PT * 32;
  constexpr int NT2 = NB == 1 ? 1 : 2;              // n-tiles of the second contraction
  extern __shared__ __align__(16) uint8_t sm[];
  const int JC = kGroup * kDW * p.sgw;              // col patches staged per CTA
  const DecodeSmem L(JC, NB, QT, RT, PT);
  uint8_t* xdig = sm + L.xdig;
  float* xscale = reinterpret_cast<float*>(sm + L.xscale);
  float* xsum = reinterpret_cast<float*>(sm + L.xsum);
  float* xl1 = reinterpret_cast<float*>(sm + L.xl1);
  int* ubound = reinterpret_cast<int*>(sm + L.ubound);
  uint8_t* udig = sm + L.udig;
  float* red = reinterpret_cast<float*>(sm + L.red);

#ifdef BQQ_BOUNDS_CHECK
  if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) BQQ_CHK(30, L.total - 1, p.lim_smem);
#endif
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
  const int jg0 = chunk * kDW * p.sgw;              // first col-patch group of the chunk
  const int j0 = jg0 * kGroup;

  // ---- plane loads of the warp's first super-group go out before the prologue ----
  uint4 zw[RT][QT], yw[PT][RT];
  auto load_planes = [&](int jg) {
    const size_t sg = (size_t)i * p.NS + (size_t)bit * p.JG + jg;
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int qt = 0; qt < QT; ++qt)
        zw[rt][qt] = (rt < p.RTg && qt < p.QTg && jg < p.JG &&
                      BQQ_CHK(1, ((sg * p.RTg + rt) * p.QTg + qt) * 32 + lane, p.lim_z))
                         ? load_plane_u4(p.zp + ((sg * p.RTg + rt) * p.QTg + qt) * 32 + lane)
                         : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int pt = 0; pt < PT; ++pt)
#pragma unroll
      for (int rt = 0; rt < RT; ++rt)
        yw[pt][rt] = (pt < p.PTg && rt < p.RTg && jg < p.JG &&
                      BQQ_CHK(2, ((sg * p.PTg + pt) * p.RTg + rt) * 32 + lane, p.lim_y))
                         ? load_plane_u4(p.yp + ((sg * p.PTg + pt) * p.RTg + rt) * 32 + lane)
                         : make_uint4(0u, 0u, 0u, 0u);
  };
  load_planes(jg0 + warp);

  // ---- prologue 1: x statistics and s8 digits per (col patch, row of X) ----------
  if (tid < 4) ubound[tid] = 0;
  for (int e = tid; e < kDW * NB * 4 * RP / 4; e += kDT) reinterpret_cast<uint32_t*>(udig)[e] = 0u;
  {
    const int sub8 = lane & 7;                      // 8 lanes share one (col patch, row) pair
    const int pairs = JC * NB;
    for (int base = warp * 4; base < pairs; base += kDW * 4) {
      const int pair = base + (lane >> 3);
      const int jl = pair / NB, beta = pair % NB;
      const int j = j0 + jl, m = m0 + beta;
      const bool live = pair < pairs && j < p.cw && m < p.M;
      float v[4 * QT];
      float amax = 0.f, sum = 0.f, l1 = 0.f;
#pragma unroll
      for (int e = 0; e < 4 * QT; ++e) {
        const int q = sub8 * 4 * QT + e;
        v[e] = (live && q < p.Q && BQQ_CHK(3, (size_t)m * p.ldx + (size_t)j * p.Q + q, p.lim_x)) ? load_as_float(p.x, (size_t)m * p.ldx + (size_t)j * p.Q + q, p.x_dtype) : 0.f;
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
      if (pair < pairs) {
        const float inv = amax > 0.f ? 32512.f / amax : 0.f;
        uint32_t lo[QT], hi[QT];
#pragma unroll
        for (int w4 = 0; w4 < QT; ++w4) {
          uint32_t D[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) D[e] = (uint32_t)(__float2int_rn(v[w4 * 4 + e] * inv) + 0x8080) ^ 0x8080u;
          // x_int = lo + 256*hi with both digits signed bytes
          lo[w4] = __byte_perm(__byte_perm(D[0], D[1], 0x0040), __byte_perm(D[2], D[3], 0x0040), 0x5410);
          hi[w4] = __byte_perm(__byte_perm(D[0], D[1], 0x0051), __byte_perm(D[2], D[3], 0x0051), 0x5410);
        }
        uint8_t* row = xdig + (size_t)(pair * 2) * QP + sub8 * 4 * QT;
        if (!BQQ_CHK(20, L.xdig + (size_t)(pair * 2 + 1) * QP + sub8 * 4 * QT + 4 * QT - 1, L.xscale)) continue;
#pragma unroll
        for (int w4 = 0; w4 < QT; ++w4) {
          *reinterpret_cast<uint32_t*>(row + w4 * 4) = lo[w4];
          *reinterpret_cast<uint32_t*>(row + QP + w4 * 4) = hi[w4];
        }
        if (sub8 == 0 && BQQ_CHK(27, pair, JC * NB)) {
          xscale[pair] = amax * (1.f / 32512.f);
          xsum[pair] = sum;
          xl1[pair] = l1;
        }
      }
    }
  }
  __syncthreads();
  // ---- prologue 2: bound on |u| over the CTA's patch-bits, per row of X ---------------
  for (int jl = tid; jl < JC; jl += kDT) {
    const int j = j0 + jl;
    if (j < p.cw && BQQ_CHK(4, ((size_t)bit * p.rw + i) * p.cw + j, p.lim_coef)) {
      const size_t ci = ((size_t)bit * p.rw + i) * p.cw + j;
      const float ca = fabsf(load_as_float(p.a, ci, p.coef_dtype));
      const float cb = fabsf(load_as_float(p.b, ci, p.coef_dtype));
#pragma unroll
      for (int beta = 0; beta < NB; ++beta) {
        const float bound = ca * xl1[jl * NB + beta] + cb * fabsf(xsum[jl * NB + beta]);
        atomicMax(ubound + beta, __float_as_int(bound));     // non-negative floats order like ints
      }
    }
  }
  __syncthreads();
  // lane-private view of the fixed-point scale of u
  const int my_beta = NB == 1 ? 0 : t;
  const float ub = __int_as_float(ubound[my_beta]);
  const float inv_us = ub > 0.f ? 4128768.f / ub : 0.f;      // |u| * inv_us < 2^22

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
  uint8_t* my_udig = udig + (size_t)warp * NB * 4 * RP;
  const float rs_t = 1.f / (float)(1 << t);

  for (int it = 0; it < p.sgw; ++it) {
    const int jg = jg0 + warp + kDW * it;
    if (it > 0) load_planes(jg);
    if (jg >= p.JG) break;
#pragma unroll
    for (int sub = 0; sub < kGroup; ++sub) {
      const int j = jg * kGroup + sub;
      if (j >= p.cw) break;
      const int jl = j - j0;
      const size_t ci = ((size_t)bit * p.rw + i) * p.cw + j;
      if (!BQQ_CHK(5, ci, p.lim_coef) || !BQQ_CHK(6, (size_t)i * p.cw + j, p.lim_d)) break;
      if (!BQQ_CHK(21, jl * NB + my_beta, JC * NB)) break;
      const float ca = load_as_float(p.a, ci, p.coef_dtype);
      const float cb = load_as_float(p.b, ci, p.coef_dtype);
      const float cc = load_as_float(p.c, ci, p.coef_dtype);
      const float xs = xsum[jl * NB + my_beta];
      const float xsc = xscale[jl * NB + my_beta];
      if (bit == 0) dacc = fmaf(load_as_float(p.d, (size_t)i * p.cw + j, p.coef_dtype), xs, dacc);
      const float bx = cb * xs;
      // B-operand source rows of x: column n = g of the fragment
      const uint8_t* xrow = xdig + (size_t)((jl * NB + (NB == 1 ? 0 : (g >> 1))) * 2 + (g & 1)) * QP + 4 * t;
      if (!BQQ_CHK(22, L.xdig + (size_t)((jl * NB + (NB == 1 ? 0 : (g >> 1))) * 2 + (g & 1)) * QP + 4 * t + (QT - 1) * 32 + 19, L.xscale)) break;

      // ---- first contraction: T[k][digit] = sum_q Z[k][q] xdigit[q] --------------------
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        int c1[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int e = 0; e < 4; ++e) c1[mt][e] = 0;
#pragma unroll
        for (int qt = 0; qt < QT; ++qt) {
          const uint32_t w = pick(zw[rt][qt], sub);
          const uint32_t w4 = w >> 4;
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xrow + qt * 32);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xrow + qt * 32 + 16);
          mma_u8s8(c1[0], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u, b0, b1);
          mma_u8s8(c1[1], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u, b0, b1);
        }
        if (NB == 1) {
          // every lane sees (lo, hi) in its two columns; lane (g,t) finishes row k = 32rt + g + 8t
          const int lo = t == 0 ? c1[0][0] : (t == 1 ? c1[0][2] : (t == 2 ? c1[1][0] : c1[1][2]));
          const int hi = t == 0 ? c1[0][1] : (t == 1 ? c1[0][3] : (t == 2 ? c1[1][1] : c1[1][3]));
          const float tf = (float)(lo + (hi << 8)) * (xsc * rs_t);
          cacc = fmaf(cc, tf, cacc);
          const uint32_t D = (uint32_t)(__float2int_rn(fmaf(ca, tf, bx) * inv_us) + 0x808080) ^ 0x808080u;
          uint8_t* dst = my_udig + rt * 32 + g + 8 * t;
          dst[0] = (uint8_t)D;
          dst[RP] = (uint8_t)(D >> 8);
          dst[2 * RP] = (uint8_t)(D >> 16);
        } else {
          // lane (g,t) owns row t of X: finishes rows k = 32rt + g + 8rr, rr = 0..3
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int lo = c1[rr >> 1][2 * (rr & 1)];
            const int hi = c1[rr >> 1][2 * (rr & 1) + 1];
            const float tf = (float)(lo + (hi << 8)) * (xsc * (1.f / (float)(1 << rr)));
            cacc = fmaf(cc, tf, cacc);
            const uint32_t D = (uint32_t)(__float2int_rn(fmaf(ca, tf, bx) * inv_us) + 0x808080) ^ 0x808080u;
            uint8_t* dst = my_udig + (size_t)t * 4 * RP + rt * 32 + g + 8 * rr;
            if (!BQQ_CHK(24, (size_t)(dst + 2 * RP - sm), L.red) || !BQQ_CHK(25, L.udig, (size_t)(dst - sm) + 1)) continue;
            dst[0] = (uint8_t)D;
            dst[RP] = (uint8_t)(D >> 8);
            dst[2 * RP] = (uint8_t)(D >> 16);
          }
        }
      }
      __syncwarp();

      // ---- second contraction: V[p][digit] += sum_k Y[p][k] udigit[k] ------------------
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        uint32_t bu[NT2][2];
#pragma unroll
        for (int nt = 0; nt < NT2; ++nt) {
          const int beta = NB == 1 ? 0 : 2 * nt + (g >> 2);
          const int slot = NB == 1 ? min(g, 3) : (g & 3);      // slot 3 stays zero
          const uint8_t* urow = my_udig + (size_t)(beta * 4 + slot) * RP + rt * 32 + 4 * t;
          if (!BQQ_CHK(26, (size_t)(urow + 19 - sm), L.red)) continue;
          bu[nt][0] = *reinterpret_cast<const uint32_t*>(urow);
          bu[nt][1] = *reinterpret_cast<const uint32_t*>(urow + 16);
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
      __syncwarp();
    }
  }

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
  const float us_mine = ub * (1.f / 4128768.f);
#pragma unroll
  for (int nt = 0; nt < NT2; ++nt) {
    // which row of X and which digits this lane's two columns carry
    const int beta = NB == 1 ? 0 : 2 * nt + (t >> 1);
    const int tt = NB == 1 ? t : (t & 1);
    const float w_even = tt == 0 ? 1.f : (tt == 1 ? 65536.f : 0.f);
    const float w_odd = tt == 0 ? 256.f : 0.f;
    const float us_b = NB == 1 ? us_mine : __shfl_sync(0xffffffffu, us_mine, (lane & ~3) | beta);
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
          const float out = fmaf(v, us_b * (1.f / (float)(1 << rr)), ct_b);
          const bool writer = NB == 1 ? (t == 0) : ((t & 1) == 0);
          if (writer && BQQ_CHK(23, L.red + ((size_t)(warp * NB + beta) * PP + pt * 32 + g + 8 * rr) * 4 + 3, L.total))
            red[(size_t)(warp * NB + beta) * PP + pt * 32 + g + 8 * rr] = out;
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
      if (pp < p.P && m0 + beta < p.M && BQQ_CHK(7, (size_t)(m0 + beta) * p.ldy + i * p.P + pp, p.lim_y_out)) {
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
    if (BQQ_CHK(8, ((size_t)part * mrows + m0 + beta) * out_stride + (size_t)i * PP + pp, p.lim_partial))
      p.partial[((size_t)part * mrows + m0 + beta) * out_stride + (size_t)i * PP + pp] = v;
  }
  __threadfence();
  __syncthreads();
  __shared__ unsigned ticket;
  if (tid == 0) ticket = BQQ_CHK(9, i * p.mtiles + blockIdx.y, kMaxCounters) ? atomicAdd(p.counters + i * p.mtiles + blockIdx.y, 1u) : 0u;
  __syncthreads();
  if (ticket != (unsigned)(nparts - 1)) return;
  __threadfence();
  for (int idx = tid; idx < NB * PP; idx += kDT) {
    const int beta = idx / PP, pp = idx % PP;
    if (pp < p.P && m0 + beta < p.M && BQQ_CHK(10, (size_t)(m0 + beta) * p.ldy + i * p.P + pp, p.lim_y_out) &&
        BQQ_CHK(11, ((size_t)(nparts - 1) * mrows + m0 + beta) * out_stride + (size_t)i * PP + pp, p.lim_partial)) {
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
  dim3 grid(p.rw * p.bw * p.nchunks, pl.mtiles);
  kern<<<grid, kDT, pl.smem, st>>>(p);
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
