// Decode kernel (M <= 16 rows of X): the packed planes are streamed once and both
// contractions run on the int8 tensor cores (mma.sync m16n8k32, u8 x s8 and u8 x u8 -> s32).
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
// digits) by a small preparation kernel or by the decode CTA itself, u per warp to
// 23-bit fixed point (three unsigned base-256 digits of round(u / scale) + offset,
// read off the bit pattern of one fused multiply-add; a fourth B column of ones
// accumulates the row sums of Y that remove the offset again).  Digits occupy
// separate B-operand columns, so the integer products are exact and the only
// errors are the two roundings (about 2^-16 of the patch maximum of |x|).
//
// How the two contractions meet (M = 1): the four col patches of a super-group put their x
// digits into four different column pairs of the first contraction's B operand (the other
// columns are zero) and accumulate into ONE accumulator tile, so lane (g,t) ends up with the
// sums of col patch t for the four ranks 4g .. 4g+3 of every 32-rank block - no selection
// between registers.  It turns them into digits, transposes the 4 x 3 bytes in registers and
// stores one word per digit; a lane of the second contraction reads the words of all four col
// patches with two 128-bit loads.  With several rows of X the column pairs carry the rows
// instead and the col patches are handled one after the other.
//
// Work split: CTA = (row patch i, bit layer b, chunk of col-patch groups, M tile);
// warp w owns a contiguous run of super-groups of the chunk and streams its plane
// words and x digits through a private ring of shared-memory slots filled by 16-byte
// asynchronous copies (cp.async groups), so warps never wait for one another in the
// main loop; coefficients and x statistics of the chunk arrive by bulk copies on one
// mbarrier.  The split never depends on the number of row patches, so a row shard of a
// layer produces bit-identical outputs.  CTA partial sums go to scratch; the last
// CTA of a row patch adds them in a fixed order, adds bias (and an optional residual)
// and converts to the output type.  Short single-chunk layers at M = 1 instead give
// one CTA all bit layers of a row patch (template flag MB): it prepares x itself and
// its sums never leave shared memory.
#pragma once
#include "bqq_async.cuh"
#include "bqq_common.cuh"

namespace bqq {

// tunables (measured on B200): ring slots for slot sizes of 1.3 .. 4 KB, register cap of the 32x32x32 variant
// with 4 rows of X (the batch-1 variant is capped at 72 registers = 7 CTAs per SM, 80 when one CTA takes all bit layers)
#ifndef BQQ_MID_STAGES
#define BQQ_MID_STAGES 3
#endif
#ifndef BQQ_NB4_REGS
#define BQQ_NB4_REGS 80
#endif
#ifndef BQQ_NB1_REGS
#define BQQ_NB1_REGS 72
#endif
constexpr int kDW = 4;                   // warps per CTA
constexpr int kDT = kDW * 32;
constexpr int kMaxCounters = 65536;      // fixed-size counter region at the start of the workspace
constexpr size_t kCounterBytes = (size_t)kMaxCounters * 4;

struct DecodePlan {
  int variant;     // geometry variant: 0 (PT,QT,RT)=(1,1,1), 1 (2,2,1), 2 (2,2,2), 3 (4,4,2)
  int NB;          // rows of X per CTA: 1 or 4
  int mtiles;      // ceil(M / NB)
  int sgw;         // super-groups per warp
  int bpc;         // bit layers per CTA (kDW warps each): 1, or all of them for short single-chunk layers
  int self_prep;   // 1: the decode CTAs prepare x themselves (one launch); 0: a preparation kernel runs first
  int nrecv;       // receiving CTAs appended to the grid (peer gather in the same launch), else 0
  int nchunks;     // chunks per bit layer
  int nparts;      // partial sums per output = (bw / bpc) * nchunks
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
  const uint8_t* xdig;       // s8 digits of x, [Mp/NB][JG][NB][digit][QT][half][t][sub] words (preparation kernel)
  const float* xscale;       // [Mp][cwp] block scale of x
  const float* xsum;         // [Mp][cwp] sum_q x
  const float* xl1;          // [Mp][cwp] sum_q |x|
  int Mp, cwp;               // M and cw rounded up to the kernel's tiles (rows per CTA, 4 col patches)
  int64_t ldx, ldy;
  int coef_dtype, x_dtype, y_dtype, bias_dtype;
  int M, bw, rw, cw, P, Q;
  int PTg, QTg, RTg;       // 32-blocks of the planes as packed
  int JG, NS;
  int sgw, nchunks, mtiles, bpc;
  // optional fused prologue (what is applied to x on the way in) and residual added to the outputs
  const void* norm_w;
  const void* res;
  int64_t ld_res;
  int pro_mode, norm_dtype, res_dtype;
  float eps;
  // optional peer-to-peer send of the outputs (row-patch shards; all zero when unused): the regions of
  // every rank as mapped here, this rank, words of one local output row, bytes of one slot half
  uint8_t* peer_regions[BQQ_MAX_PEERS];
  int peer_world, peer_rank, peer_row_words;
  unsigned long long peer_half;
  // ... and the receiving side in the same launch: the CTAs blockIdx.x >= ncompute only wait for every rank's
  // words in this rank's region and write the gathered rows [M][world * row words] to peer_out
  uint32_t* peer_out;
  long long peer_ld_out;     // row pitch of peer_out in 32-bit words
  long long peer_wait;       // clock budget of one wait on a peer
  int ncompute;              // CTAs along x that compute (the rest receive)
  int peer_seg_words;        // > 0: the local row is two halves of this many words, gathered as [half 0 of every rank |
                             // half 1 of every rank] (a stacked gate / up layer whose consumer wants [gate | up])
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

// unsigned x unsigned (second contraction: the u digits are unsigned bytes)
__device__ __forceinline__ void mma_u8u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pick(const uint4& v, int sub) {
  return sub == 0 ? v.x : (sub == 1 ? v.y : (sub == 2 ? v.z : v.w));
}

constexpr int kMaxSgw = 32;              // upper bound of super-groups per warp (resident coefficients: 64 B each)
// u digit exchange at M = 1, per 32-rank block: 128 words.  The word of digit d, lane group G (ranks 4G .. 4G+3,
// produced by the lanes with g = G) and col patch sub sits at
//   32 d + 4 ((2 (G & 3) + (sub >> 1) + (d & 1)) & 7) + 2 (sub & 1) + (G >> 2),
// so that a 128-bit load gives a consumer (b0, b1) of two col patches in operand order (b0: G = t, b1: G = t + 4)
// and both the producers' stores (fixed d) and the consumers' loads (two neighbouring digits) touch every bank once.
constexpr int kUBlock = 128;

// Shared-memory carve-up (bytes), shared by host plan and kernel.  Per warp a ring of `stages`
// slots, each holding one super-group: its Z words, Y words and the x digits of the CTA's rows.
// Resident for the whole chunk: coefficients and x statistics (one mbarrier).
struct DecodeSmem {
  int bars, ring, slot, stages, yoff, xoff, coef, meta, udig, red, xres, xstat, total;
  // xp: the CTA prepares x itself (digits and statistics of its chunk live in shared memory)
  __host__ __device__ constexpr DecodeSmem(int sgw, int NB, int PT, int QT, int RT, int bpc = 1, bool xp = false)
      : bars(0), ring(0), slot(0), stages(0), yoff(0), xoff(0), coef(0), meta(0), udig(0), red(0), xres(0), xstat(0),
        total(0) {
    const int nsg = kDW * sgw;                        // super-groups per chunk
    const int nwarps = kDW * bpc;
    int o = 0;
    bars = o;  o += 128;                              // one mbarrier per bit layer of the CTA
    yoff = RT * QT * 512;                             // slot: uint4 Z[RT][QT][32] | Y[PT][RT][32] | X[NB][digit][QT][8]
    xoff = yoff + PT * RT * 512;
    slot = xoff + NB * 2 * QT * 128;
    stages = slot <= 1280 ? 4 : (slot <= 4096 ? BQQ_MID_STAGES : 2);
    ring = o;  o += nwarps * stages * slot;
    coef = o;  o += bpc * 4 * nsg * 16;               // float [bit][a|b|c|d][nsg*4]
    meta = o;  o += bpc * NB * 3 * nsg * 16;          // float [bit][NB][scale|sum|l1][nsg*4]
    // u digits: M = 1: words [warps][RT][4 digits][8 lane groups][4 sub];
    // more rows: bytes [warps][4 sub][NB][4 digits][RP] (+ 16 bytes of padding per row of X)
    udig = o;  o += nwarps * (NB == 1 ? RT * kUBlock * 4 : kGroup * NB * (4 * RT * 32 + 16));
    red = o;   o += nwarps * NB * PT * 32 * 4;        // f32 [warps][NB][PP]
    // CTAs that prepare x themselves: digits and statistics of the whole chunk
    xres = o;  o += xp ? nsg * NB * 2 * QT * 128 : 0;        // uint4 [nsg][NB][digit][QT][8]
    xstat = o; o += xp ? 3 * nsg * 16 : 0;                   // float [scale|sum|l1][nsg*4]
    total = o;
  }
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- activation preparation ------------------------------------------------------------------
// One pass over x [M, cw*Q]: per (row m, col patch j) the 16-bit block fixed point digits
//   xdig (s8 digits: x_int = lo + 256*hi, x ~ x_int * scale), 2*32*QT bytes per pair,
// and xscale / xsum / xl1 [Mp][cwp] = scale, sum_q x, sum_q |x|.  Rows m >= M and col patches
// j >= cw (Mp, cwp: M and cw rounded up to the kernel's tiles) are written as zeros so that the
// decode kernel needs no edge tests.  8 lanes share one (m, j) pair.
// Body shared by the preparation kernel and the decode kernel that prepares x itself: one
// (row, col patch) pair per 8 lanes.  `live` pairs read x[m, j*Q ...]; the others write zeros.
// Digits go to words[] at the pair's place (M tile `mtile`, row `beta` inside it), statistics to
// index `stat` of xscale / xsum / xl1.  Every lane of the warp must call it (shuffles).
// Where the activation comes from, and what is applied to it on the way in (BqqFusion::prologue):
// nothing, RMS normalisation (x * inv_rms * w[n]; inv_rms of the row is computed by the caller of
// xprep_pair), or SwiGLU (silu(x[n]) * x[n + n_in], x holding [gate | up] rows of 2 * n_in elements).
struct XSource {
  const void* x;
  const void* w;
  int64_t ld;
  int dtype, w_dtype, mode, n_in;
  float eps;
};
__device__ __forceinline__ float load_x(const XSource& s, int m, int n, float inv_rms) {
  float v = load_as_float(s.x, (size_t)m * s.ld + n, s.dtype);
  if (s.mode == BQQ_PRO_RMSNORM) {
    v = v * inv_rms * load_as_float(s.w, n, s.w_dtype);
  } else if (s.mode == BQQ_PRO_SWIGLU) {
    const float u = load_as_float(s.x, (size_t)m * s.ld + s.n_in + n, s.dtype);
    v = v / (1.f + __expf(-v)) * u;
  }
  return v;
}
// Four consecutive elements n0 .. n0+3 of a tensor of type `dt` as floats; one 8- or 16-byte load when the
// address allows it, four element loads otherwise.
__device__ __forceinline__ void load_quad(const void* base, size_t idx, int dt, float (&v)[4]) {
  if (dt == BQQ_F32) {
    const float* p = reinterpret_cast<const float*>(base) + idx;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
      const float4 q = *reinterpret_cast<const float4*>(p);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] = p[e];
    }
    return;
  }
  const uint16_t* p = reinterpret_cast<const uint16_t*>(base) + idx;
  uint32_t w0, w1;
  if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    w0 = q.x; w1 = q.y;
  } else {
    w0 = (uint32_t)p[0] | ((uint32_t)p[1] << 16);
    w1 = (uint32_t)p[2] | ((uint32_t)p[3] << 16);
  }
  if (dt == BQQ_BF16) {
    v[0] = __uint_as_float(w0 << 16); v[1] = __uint_as_float(w0 & 0xFFFF0000u);
    v[2] = __uint_as_float(w1 << 16); v[3] = __uint_as_float(w1 & 0xFFFF0000u);
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w0));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&w1));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
}
// x[m, n0 .. n0+3] after the prologue (all four columns exist)
__device__ __forceinline__ void load_x_quad(const XSource& s, int m, int n0, float inv_rms, float (&v)[4]) {
  load_quad(s.x, (size_t)m * s.ld + n0, s.dtype, v);
  if (s.mode == BQQ_PRO_RMSNORM) {
    float w[4];
    load_quad(s.w, n0, s.w_dtype, w);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = v[e] * inv_rms * w[e];
  } else if (s.mode == BQQ_PRO_SWIGLU) {
    float u[4];
    load_quad(s.x, (size_t)m * s.ld + s.n_in + n0, s.dtype, u);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = v[e] / (1.f + __expf(-v[e])) * u[e];
  }
}
// Sum of squares of row m over this thread's share of the columns (threads tid, tid + n, ...).
__device__ __forceinline__ float row_sumsq_share(const XSource& s, int m, int tid, int nthreads) {
  float acc = 0.f;
  if ((s.n_in & 3) == 0) {
    for (int n = 4 * tid; n < s.n_in; n += 4 * nthreads) {
      float v[4];
      load_quad(s.x, (size_t)m * s.ld + n, s.dtype, v);
      acc = fmaf(v[0], v[0], acc); acc = fmaf(v[1], v[1], acc);
      acc = fmaf(v[2], v[2], acc); acc = fmaf(v[3], v[3], acc);
    }
  } else {
    for (int n = tid; n < s.n_in; n += nthreads) {
      const float v = load_as_float(s.x, (size_t)m * s.ld + n, s.dtype);
      acc = fmaf(v, v, acc);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  return acc;                                       // the warp's share, in every lane
}

// `jsrc` is the col patch whose x is read, `j` its place in the output (they differ when a CTA prepares only
// its own chunk: j counts from the chunk's first col patch, a multiple of 4).
template <int QT>
__device__ __forceinline__ void xprep_pair(const XSource& xs, float inv_rms, int Q, int NB, int JG,
                                           bool write, bool live, int m, int jsrc, int j, int mtile, int beta, int sub8,
                                           uint32_t* __restrict__ words, float* __restrict__ xscale,
                                           float* __restrict__ xsum, float* __restrict__ xl1, int stat) {
  float v[4 * QT];
  float amax = 0.f, sum = 0.f, l1 = 0.f;
#pragma unroll
  for (int w4 = 0; w4 < QT; ++w4) {
    const int q0 = sub8 * 4 * QT + 4 * w4;
    float quad[4] = {0.f, 0.f, 0.f, 0.f};
    if (live && q0 + 4 <= Q) {
      load_x_quad(xs, m, jsrc * Q + q0, inv_rms, quad);
    } else if (live) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (q0 + e < Q) quad[e] = load_x(xs, m, jsrc * Q + q0 + e, inv_rms);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      v[4 * w4 + e] = quad[e];
      amax = fmaxf(amax, fabsf(quad[e]));
      sum += quad[e];
      l1 += fabsf(quad[e]);
    }
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
  }
  if (!write) return;
  const float inv = amax > 0.f ? 32512.f / amax : 0.f;
  // digit layout [M tile][JG][NB][digit][QT][half][t][sub] words (4 consecutive q each): the rows of an M tile
  // and the 4 col patches of a super-group are adjacent, so one run of copies brings a super-group's digits and
  // a lane of the decode kernel fetches its B-operand words with one 128-bit load per (digit, half)
#pragma unroll
  for (int w4 = 0; w4 < QT; ++w4) {
    uint32_t D[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) D[e] = (uint32_t)(__float2int_rn(v[w4 * 4 + e] * inv) + 0x8080) ^ 0x8080u;
    const int q4 = sub8 * QT + w4;                 // index of this group of 4 consecutive q
    const int qt = q4 >> 3, half = (q4 >> 2) & 1, tt = q4 & 3;
    const size_t base = (((size_t)mtile * JG + (j >> 2)) * NB + beta) * 2;
    // x_int = lo + 256*hi with both digits signed bytes
    words[((((base + 0) * QT + qt) * 2 + half) * 4 + tt) * kGroup + (j & 3)] =
        __byte_perm(__byte_perm(D[0], D[1], 0x0040), __byte_perm(D[2], D[3], 0x0040), 0x5410);
    words[((((base + 1) * QT + qt) * 2 + half) * 4 + tt) * kGroup + (j & 3)] =
        __byte_perm(__byte_perm(D[0], D[1], 0x0051), __byte_perm(D[2], D[3], 0x0051), 0x5410);
  }
  if (sub8 == 0) {
    xscale[stat] = amax * (1.f / 32512.f);
    xsum[stat] = sum;
    xl1[stat] = l1;
  }
}

template <int QT>
__global__ void __launch_bounds__(128)
bqq_xprep_kernel(const XSource xs, int M, int cw, int Q, int cwp, int NB,
                 uint8_t* __restrict__ xdig, float* __restrict__ xscale, float* __restrict__ xsum,
                 float* __restrict__ xl1) {
  // the decode kernel of this layer may start now: it first streams its weight planes and only
  // then waits (griddepcontrol.wait) for this grid to finish.  This grid itself may have been
  // started before the preceding kernel of the stream finished: wait for it before reading x or
  // writing the workspace.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int m = blockIdx.y;                         // row of X (rows >= M are written as zeros)
  float inv_rms = 1.f;
  if (xs.mode == BQQ_PRO_RMSNORM) {                 // every block sums its row's squares itself (a few KB from L2)
    __shared__ float part[4];
    const float w = m < M ? row_sumsq_share(xs, m, threadIdx.x, 128) : 0.f;
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = w;
    __syncthreads();
    inv_rms = rsqrtf((part[0] + part[1] + part[2] + part[3]) / (float)xs.n_in + xs.eps);
  }
  const int j = (blockIdx.x * 128 + threadIdx.x) >> 3;
  const bool inside = j < cwp;
  xprep_pair<QT>(xs, inv_rms, Q, NB, cwp / kGroup, inside, inside && m < M && j < cw, m, inside ? j : 0, inside ? j : 0, m / NB, m % NB,
                 threadIdx.x & 7, reinterpret_cast<uint32_t*>(xdig), xscale, xsum, xl1, m * cwp + j);
}

// Final output of one lane (row `row` of X, local output column `o`) also travels to every rank of a
// peer gather group: the 32-bit word that holds it goes with the gather's sequence number as one
// scalar 64-bit store into slot [row][rank-major column] of every region (see bqq_peer.cu).  16-bit outputs
// are paired with the neighbouring lane's (o is even on even lanes).  Every lane of the warp calls it.
__device__ __forceinline__ void peer_send(const DecodeParams& p, bool valid, int row, int o, float v, int lane) {
  uint32_t word;
  bool sender = valid;
  if (p.y_dtype == BQQ_F32) {
    word = __float_as_uint(v);
  } else {
    const uint32_t h = p.y_dtype == BQQ_BF16 ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v))
                                              : (uint32_t)__half_as_ushort(__float2half_rn(v));
    const uint32_t up = __shfl_down_sync(0xffffffffu, h, 1);
    word = h | (up << 16);
    sender = valid && !(lane & 1);
  }
  if (!sender) return;
  const unsigned* mine = reinterpret_cast<const unsigned*>(p.peer_regions[p.peer_rank]);
  const unsigned count = *reinterpret_cast<const volatile unsigned*>(mine) + 1u;
  const unsigned seq = count | 0x80000000u;
  const size_t wcol = p.y_dtype == BQQ_F32 ? (size_t)o : (size_t)o >> 1;
  size_t col = (size_t)p.peer_rank * p.peer_row_words + wcol;            // rank-major columns
  if (p.peer_seg_words) {
    const size_t sw = (size_t)p.peer_seg_words, seg = wcol >= sw ? 1 : 0;
    col = seg * p.peer_world * sw + p.peer_rank * sw + (wcol - seg * sw);
  }
  const size_t slot = (size_t)row * p.peer_world * p.peer_row_words + col;
  const size_t off = kPeerCtrlBytes + (count & 1u) * p.peer_half + slot * 8;
  for (int q = 0; q < p.peer_world; ++q)
    peer_slot_store(p.peer_regions[q] + off, word, seq);
}

// Receiving CTAs of a gathered decode launch (blockIdx.x >= ncompute): poll every slot of this rank's region until
// it carries the gather's sequence number (bounded), write the data words to the caller's tensor.  They run beside
// the computing CTAs of the same launch, which never wait for them.
__device__ __forceinline__ void peer_receive(const DecodeParams& p) {
  __shared__ int s_giveup;
  // the output tensor may still be read by earlier kernels of the stream; later kernels need not wait for the polling
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x;
  if (tid == 0) s_giveup = 0;
  __syncthreads();
  unsigned* mine = reinterpret_cast<unsigned*>(p.peer_regions[p.peer_rank]);
  if (blockIdx.y == 0) {
    const unsigned count = *reinterpret_cast<volatile unsigned*>(mine) + 1u;
    const unsigned e = count | 0x80000000u;
    const uint8_t* slots = reinterpret_cast<const uint8_t*>(mine) + kPeerCtrlBytes + (count & 1u) * p.peer_half;
    const long long grow = (long long)p.peer_row_words * p.peer_world;
    const long long n = (long long)p.M * grow;
    const long long step = (long long)(gridDim.x - p.ncompute) * blockDim.x;
    // four slots per round: their loads are in flight together, so a thread that owns many words does not pay one
    // L2 round trip per word; a slot that has not arrived yet is polled (bounded) on its own
    for (long long w0 = (long long)(blockIdx.x - p.ncompute) * blockDim.x + tid; w0 < n; w0 += 4 * step) {
      uint2 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const long long w = w0 + k * step;
        v[k] = w < n ? peer_slot_load(slots + 8 * w) : make_uint2(0u, e);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const long long w = w0 + k * step;
        if (w >= n) break;
        if (v[k].y != e) {
          const long long t0 = clock64();
          while (v[k].y != e && !*reinterpret_cast<volatile int*>(&s_giveup)) {
            if (clock64() - t0 > p.peer_wait) { s_giveup = 1; break; }
            v[k] = peer_slot_load(slots + 8 * w);
          }
        }
        const long long r = w / grow, c = w - r * grow;
        p.peer_out[r * p.peer_ld_out + c] = v[k].x;
      }
    }
  }
  __syncthreads();
  if (tid == 0 && blockIdx.y == 0) {
    if (s_giveup) atomicExch(mine + 1, 1u);
    // Every word of this gather has arrived, so every sender of this rank has read the gather count (a sender reads
    // it before its first store): the last receiving CTA may advance it.  Computing CTAs take no part in this.
    __threadfence();
    if (atomicAdd(mine + 2, 1u) == gridDim.x - p.ncompute - 1u) {
      mine[2] = 0u;
      *reinterpret_cast<volatile unsigned*>(mine) = *reinterpret_cast<volatile unsigned*>(mine) + 1u;
    }
  }
}

// MB: the CTA prepares x itself (no preparation kernel ran) and takes p.bpc bit layers of its row patch (4 warps
// each): all of them for short single-chunk layers, else one.
template <int PT, int QT, int RT, int NB, bool MB>
__global__ void __maxnreg__(PT == 1 ? (NB == 1 ? (MB ? 80 : BQQ_NB1_REGS) : BQQ_NB4_REGS) : 255)
bqq_decode_kernel(const DecodeParams p) {
  if (p.peer_world && (int)blockIdx.x >= p.ncompute) {
    peer_receive(p);
    return;
  }
  const int bpc = MB ? p.bpc : 1;
  constexpr int RP = RT * 32;
  constexpr int PP = PT * 32;
  constexpr int NT2 = NB == 1 ? 1 : 2;              // n-tiles of the second contraction
  extern __shared__ __align__(128) uint8_t sm[];
  const int nsg = kDW * p.sgw;                      // super-groups per chunk (pitch of the resident arrays)
  const DecodeSmem L(p.sgw, NB, PT, QT, RT, bpc, MB);
  constexpr int S = DecodeSmem(1, NB, PT, QT, RT).stages;
  constexpr int kSlot = DecodeSmem(1, NB, PT, QT, RT).slot;
  constexpr int kYoff = DecodeSmem(1, NB, PT, QT, RT).yoff / 16, kXoff = DecodeSmem(1, NB, PT, QT, RT).xoff / 16;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;                        // CTA-wide: ring, digit buffer, sums
  const int wq = MB ? warp % kDW : warp;            // position inside the chunk
  const int bq = MB ? warp / kDW : 0;               // bit layer inside the CTA's group
  const int g = lane >> 2;
  const int t = lane & 3;
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + L.bars) + bq;
  const float* scoef = reinterpret_cast<const float*>(sm + L.coef) + bq * 4 * nsg * 4;
  const float* smeta = reinterpret_cast<const float*>(sm + L.meta) + bq * NB * 3 * nsg * 4;
  float* red = reinterpret_cast<float*>(sm + L.red);

  int bid = blockIdx.x;
  const int nbg = p.bw / bpc;                       // bit groups
  const int chunk = bid % p.nchunks; bid /= p.nchunks;
  const int bitgroup = bid % nbg;
  const int bit = bitgroup * bpc + bq;
  const int i = bid / nbg;
  const int m0 = blockIdx.y * NB;
  const int jg0 = chunk * nsg;                      // first col-patch group of the chunk
  const int nvalid = min(nsg, p.JG - jg0);          // super-groups that exist in this chunk
  const int li0 = wq * p.sgw;                       // this warp's first super-group inside the chunk
  const int nw = max(0, min(p.sgw, nvalid - li0));  // and how many it owns
  const uint32_t crow = (uint32_t)(((size_t)bit * p.rw + i) * p.cw);   // coefficient row of (bit, i)
  const uint32_t drow = (uint32_t)((size_t)i * p.cw);

  // ---- ring of this warp: every lane copies 16-byte pieces; a lane's Z and Y pieces are the very
  // words it will use as tensor core operands, the x digits are shared by the warp ----------------
  uint4* wring = reinterpret_cast<uint4*>(sm + L.ring + (size_t)warp * S * kSlot);
  // uint4 per super-group; the 32x32x32 variant is only ever used with one block per plane
  const int zq = RT * QT == 1 ? 32 : p.RTg * p.QTg * 32, yq = PT * RT == 1 ? 32 : p.PTg * p.RTg * 32;
  const int RTg = RT == 1 ? 1 : p.RTg, QTg = QT == 1 ? 1 : p.QTg, PTg = PT == 1 ? 1 : p.PTg;
  constexpr int xq = NB * 2 * QT * 8;
  const size_t sg0 = (size_t)i * p.NS + (size_t)bit * p.JG + jg0 + li0;
  const uint4* zsrc = p.zp + sg0 * zq + lane;
  const uint4* ysrc = p.yp + sg0 * yq + lane;
  const uint4* xsrc = reinterpret_cast<const uint4*>(p.xdig) + ((size_t)blockIdx.y * p.JG + jg0 + li0) * xq + lane;
  auto issue_planes = [&](int n) {
    uint4* dst = wring + (n % S) * (kSlot / 16) + lane;
#pragma unroll
    for (int b = 0; b < RT * QT; ++b)
      if (b * 32 < zq) cp_async16(dst + b * 32, zsrc + (size_t)n * zq + b * 32);
#pragma unroll
    for (int b = 0; b < PT * RT; ++b)
      if (b * 32 < yq) cp_async16(dst + kYoff + b * 32, ysrc + (size_t)n * yq + b * 32);
  };
  auto issue_x = [&](int n) {
    uint4* dst = wring + (n % S) * (kSlot / 16) + kXoff + lane;
#pragma unroll
    for (int b = 0; b < (xq + 31) / 32; ++b)
      if (b * 32 + lane < xq) cp_async16(dst + b * 32, xsrc + (size_t)n * xq + b * 32);
  };

  if (tid == 0) {
    for (int b = 0; b < bpc; ++b) mbar_init(bar + b, MB ? 1 : 2);
    mbar_init_fence();
  }
  // weights first: they do not depend on the activation preparation kernel
#pragma unroll
  for (int s = 0; s < S - 1; ++s)
    if (s < nw) issue_planes(s);
  __syncthreads();                                   // the barrier is initialised for every waiter

  // ---- coefficients and x statistics of the chunk: bulk copies on the mbarrier ------------------
  if (lane == 0 && wq == 1) {
    const uint32_t n16 = (uint32_t)nvalid * 16u;                    // bytes of nvalid*4 floats
    if (p.coef_vec) {
      mbar_expect_tx(bar, 3 * n16 + (bit == 0 ? n16 : 0u));
      float* sc = const_cast<float*>(scoef);
      bulk_load(sc, reinterpret_cast<const float*>(p.a) + crow + jg0 * kGroup, n16, bar);
      bulk_load(sc + nsg * 4, reinterpret_cast<const float*>(p.b) + crow + jg0 * kGroup, n16, bar);
      bulk_load(sc + nsg * 8, reinterpret_cast<const float*>(p.c) + crow + jg0 * kGroup, n16, bar);
      if (bit == 0)
        bulk_load(sc + nsg * 12, reinterpret_cast<const float*>(p.d) + drow + jg0 * kGroup, n16, bar);
    } else {
      mbar_expect_tx(bar, 0u);
    }
  }
  const uint4* xres = reinterpret_cast<const uint4*>(sm + L.xres);      // MB only
  const float* xstat = reinterpret_cast<const float*>(sm + L.xstat);    // MB only
  if (MB) {
    // this CTA prepares x itself (no preparation kernel was launched): every 8 lanes take one col patch.
    // x and the workspace belong to earlier kernels of the stream until they have finished.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float* st = const_cast<float*>(xstat);
    const XSource xs = {p.x, p.norm_w, p.ldx, p.x_dtype, p.norm_dtype, p.pro_mode, p.cw * p.Q, p.eps};
    float inv_rms = 1.f;
    if (p.pro_mode == BQQ_PRO_RMSNORM) {              // the CTA reads its row of x anyway: sum the squares first
      const float w = m0 < p.M ? row_sumsq_share(xs, m0, tid, kDT * bpc) : 0.f;
      if (lane == 0) red[warp] = w;
      __syncthreads();
      float tot = 0.f;
      for (int w2 = 0; w2 < kDW * bpc; ++w2) tot += red[w2];
      inv_rms = rsqrtf(tot / (float)xs.n_in + p.eps);
      __syncthreads();                               // red is reused for the warps' sums at the end
    }
    for (int pair = tid >> 3; pair < nsg * kGroup; pair += (kDT * bpc) >> 3) {
      const int j = jg0 * kGroup + pair;             // col patch of the layer; `pair` counts inside the chunk
      xprep_pair<QT>(xs, inv_rms, p.Q, NB, nsg, true, j < p.cw && m0 < p.M, m0, j, pair, 0, 0, tid & 7,
                     reinterpret_cast<uint32_t*>(sm + L.xres), st, st + nsg * 4, st + nsg * 8, pair);
    }
    __syncthreads();
  } else {
    // the x digits and statistics come from the preparation kernel launched just before this one
    // (programmatic dependent launch): wait for it to complete before reading its output
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  if (!MB && lane == 0 && wq == 2) {
    const uint32_t n16 = (uint32_t)nvalid * 16u;
    mbar_expect_tx(bar, NB * 3 * n16);
#pragma unroll
    for (int beta = 0; beta < NB; ++beta) {
      const size_t row = (size_t)(m0 + beta) * p.cwp + (size_t)jg0 * kGroup;
      float* sm_meta = const_cast<float*>(smeta) + beta * 3 * nsg * 4;
      bulk_load(sm_meta, p.xscale + row, n16, bar);
      bulk_load(sm_meta + nsg * 4, p.xsum + row, n16, bar);
      bulk_load(sm_meta + nsg * 8, p.xl1 + row, n16, bar);
    }
  }
  // one copy group per super-group: group k complete means super-group k has arrived
#pragma unroll
  for (int s = 0; s < S - 1; ++s) {
    if (!MB && s < nw) issue_x(s);
    cp_async_commit();
  }

  // ---- digit exchange buffer: digits 0..2 are rewritten for every super-group (col patch), digit 3 is a
  // column of ones whose products count the Y bits of each row (removes the offset of the unsigned digits)
  // M > 1: bytes [sub][row of X][digit][rank]; rows of X are 16 bytes further apart than their 4 digits need, so
  // that the word loads of the two rows an n-tile covers fall into different banks
  constexpr int kURow = 4 * RP + 16;
  constexpr int kUSub = NB * kURow;                  // bytes of one col patch's u digits
  uint8_t* my_udig = sm + L.udig + (size_t)warp * (NB == 1 ? RT * kUBlock * 4 : kGroup * kUSub);
  // only the ones need writing: digits 0..2 are fully rewritten before every use
  if (NB == 1) {
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
      reinterpret_cast<uint32_t*>(my_udig)[rt * kUBlock + 96 + lane] = 0x01010101u;
  } else {
    for (int e = lane; e < kGroup * NB * (RP / 4); e += 32) {
      const int sub = e / (NB * (RP / 4)), rem = e % (NB * (RP / 4));
      reinterpret_cast<uint32_t*>(my_udig + sub * kUSub + (rem / (RP / 4)) * kURow + 3 * RP)[rem % (RP / 4)] = 0x01010101u;
    }
  }
  bool ok = mbar_wait(bar, 0);

  // ---- fold the x statistics into the coefficients of this warp's patch-bits (in place of the
  // statistics):  alpha = a * scale,  beta = b * sum,  gamma = c * scale;  d * sum is summed right
  // here.  The fixed-point scale of u for this warp comes from the bound |a| sum|x| + |b| |sum x|.
  constexpr float kUOff = 4128768.f;                 // 63 * 65536: the offset touches the top digit only
  // u is scaled so that the bound maps to kUScale, 0.8 % inside the offset: t is computed from the rounded
  // x digits and can exceed the bound taken from the unrounded x by up to Q / 65024 of it (and does, for
  // narrow patches whose Z row is all ones and whose x share one sign); without the slack such a rank fell
  // below 2^23 and its digits were garbage
  constexpr float kUScale = 4096000.f;
  // float -> integer by mantissa alignment: 2^23 + kUOff + round(u * inv_us); the low three bytes of
  // the float's bit pattern are then the unsigned base-256 digits of round(u * inv_us) + kUOff
  constexpr float kMagic = 8388608.f + kUOff;
  const int my_beta = NB == 1 ? 0 : t;
  float* wmeta = const_cast<float*>(smeta);
  float ub = 0.f;
  float dsum[NB];
#pragma unroll
  for (int beta = 0; beta < NB; ++beta) dsum[beta] = 0.f;
  for (int e = lane; e < nw * kGroup; e += 32) {
    const int idx = li0 * kGroup + e;                // (super-group, col patch) inside the chunk
    const int j = jg0 * kGroup + idx;
    float ca = 0.f, cb = 0.f, cc = 0.f, cd = 0.f;    // ragged last group: zero coefficients
    if (j < p.cw) {
      if (p.coef_vec) {
        ca = scoef[idx];
        cb = scoef[nsg * 4 + idx];
        cc = scoef[nsg * 8 + idx];
        if (bit == 0) cd = scoef[nsg * 12 + idx];
      } else {
        ca = load_as_float(p.a, crow + j, p.coef_dtype);
        cb = load_as_float(p.b, crow + j, p.coef_dtype);
        cc = load_as_float(p.c, crow + j, p.coef_dtype);
        if (bit == 0) cd = load_as_float(p.d, drow + j, p.coef_dtype);
      }
    }
#pragma unroll
    for (int beta = 0; beta < NB; ++beta) {
      float* mr = wmeta + beta * 3 * nsg * 4;
      const float* raw = MB ? xstat : mr;              // MB: statistics shared by the CTA's bit layers
      const float sc = raw[idx], sx = raw[nsg * 4 + idx], l1 = raw[nsg * 8 + idx];
      ub = fmaxf(ub, fmaf(fabsf(ca), l1, fabsf(cb * sx)));
      dsum[beta] = fmaf(cd, sx, dsum[beta]);
      mr[idx] = ca * sc;
      mr[nsg * 4 + idx] = cb * sx;
      mr[nsg * 8 + idx] = cc * sc;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ub = fmaxf(ub, __shfl_xor_sync(0xffffffffu, ub, o));
  // u * inv_us lies in [-kUScale, kUScale] (a little beyond at most); adding kUOff makes it a non-negative
  // 23-bit integer
  const float inv_us = ub > 0.f ? kUScale / ub : 0.f;
  // second pass over the lane's own entries: alpha *= inv_us, beta = beta * inv_us + magic, so that one
  // fused multiply-add per rank yields the digits of u
  for (int e = lane; e < nw * kGroup; e += 32) {
    const int idx = li0 * kGroup + e;
#pragma unroll
    for (int beta = 0; beta < NB; ++beta) {
      float* mr = wmeta + beta * 3 * nsg * 4;
      mr[idx] *= inv_us;
      mr[nsg * 4 + idx] = fmaf(mr[nsg * 4 + idx], inv_us, kMagic);
    }
  }
  float dacc = 0.f;
#pragma unroll
  for (int beta = 0; beta < NB; ++beta) {
    float v = dsum[beta];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (beta == my_beta) dacc = v;
  }
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
  float cacc = 0.f;
  // lane constants.  M = 1: column n = g of the first contraction's B operand carries digit g & 1 of col patch
  // g >> 1 (zero for the other col patches); the lane finishes col patch t.  M > 1: column pair t carries row t of
  // X; the lane finishes that row for every col patch.
  const int my_sub = g >> 1;
  const int xword = NB == 1 ? kXoff * 4 + (g & 1) * (QT * 32) + t * 4 + my_sub : 0;   // 32-bit words inside a slot
  const int xlane = kXoff + g * (QT * 8) + t;                                          // uint4 index (M > 1)
  const float* mrow = smeta + my_beta * 3 * nsg * 4;   // [alpha | beta | gamma] of this lane's row of X
  // where the lane's u digits go ...
  // M = 1: word of digit 0 (digit 2: + 64 words; digit 1: the 16-byte group index is one higher, modulo 8)
  uint8_t* ust = NB == 1 ? my_udig + 4 * (8 * (g & 3) + 2 * t + (g >> 2)) : my_udig + t * kURow + 4 * g;
  const int ust1 = 32 + 4 * ((2 * (g & 3) + (t >> 1) + 1) & 7) + 2 * (t & 1) + (g >> 2) - (8 * (g & 3) + 2 * t + (g >> 2));
  // ... and where its B operand of the second contraction comes from
  const uint8_t* uld[NT2];
#pragma unroll
  for (int nt = 0; nt < NT2; ++nt) {
    const int beta = 2 * nt + (g >> 2);                  // M > 1: row of X and digit of column n = g
    uld[nt] = NB == 1 ? my_udig + 4 * (32 * (g & 3)) : my_udig + beta * kURow + (g & 3) * RP + 4 * t;
  }
  // M = 1: byte offsets from uld[0] of the two 128-bit groups of digit g & 3: col patches 0, 1 and 2, 3
  const int u01 = 16 * ((2 * t + (g & 1)) & 7), u23 = 16 * ((2 * t + 1 + (g & 1)) & 7);
#pragma unroll(NB == 1 ? 4 : 1)
  for (int n = 0; n < nw; ++n) {
    // refill the slot consumed in the previous iteration with the super-group S - 1 ahead
    if (n + S - 1 < nw) {
      issue_planes(n + S - 1);
      if (!MB) issue_x(n + S - 1);
    }
    cp_async_commit();
    cp_async_wait<S - 1>();                           // this lane's pieces of super-group n have landed
    __syncwarp();                                     // ... and every other lane's (x digits, u digit buffer reuse)
    const uint4* zs = wring + (n % S) * (kSlot / 16);
    const uint4* ys = zs + kYoff;
    const int li = li0 + n;                           // super-group index inside the chunk
    // plane words of this super-group
    uint4 zw[RT][QT], yw[PT][RT];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int qt = 0; qt < QT; ++qt)
        zw[rt][qt] = (rt < RTg && qt < QTg) ? zs[(rt * QTg + qt) * 32 + lane] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int pt = 0; pt < PT; ++pt)
#pragma unroll
      for (int rt = 0; rt < RT; ++rt)
        yw[pt][rt] = (pt < PTg && rt < RTg) ? ys[(pt * RTg + rt) * 32 + lane] : make_uint4(0u, 0u, 0u, 0u);
    if (NB == 1) {
      // ---- M = 1 --------------------------------------------------------------------------------------
      // x digits of this lane's B column: digit g & 1 of col patch g >> 1 (one word per half of q)
      const uint32_t* xw = reinterpret_cast<const uint32_t*>(MB ? xres + li * xq - kXoff : zs) + xword;
      uint32_t bx0[QT], bx1[QT];
#pragma unroll
      for (int qt = 0; qt < QT; ++qt) {
        bx0[qt] = xw[qt * 32];
        bx1[qt] = xw[qt * 32 + 16];
      }
      // folded coefficients of col patch t
      const float ca = mrow[li * 4 + t], cb = mrow[nsg * 4 + li * 4 + t], cc = mrow[nsg * 8 + li * 4 + t];
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        // first contraction, all four col patches into one tile: T[k][2 sub + digit] = sum_q Z_sub[k][q] xdigit_sub[q]
        int c1[2][4];
#pragma unroll
        for (int sub = 0; sub < kGroup; ++sub) {
#pragma unroll
          for (int qt = 0; qt < QT; ++qt) {
            const uint32_t w = pick(zw[rt][qt], sub);
            const uint32_t w4 = w >> 4;
            const uint32_t b0 = my_sub == sub ? bx0[qt] : 0u, b1 = my_sub == sub ? bx1[qt] : 0u;
            if (sub == 0 && qt == 0) {
              mma_u8s8_first(c1[0], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u, b0, b1);
              mma_u8s8_first(c1[1], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u, b0, b1);
            } else {
              mma_u8s8(c1[0], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u, b0, b1);
              mma_u8s8(c1[1], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u, b0, b1);
            }
          }
        }
        // the lane's columns 2t, 2t+1 are (lo, hi) of col patch t; its rows are the ranks 32rt + 4g + rr
        uint32_t D[4];
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          const int lo = c1[rr >> 1][2 * (rr & 1)];
          const int hi = c1[rr >> 1][2 * (rr & 1) + 1];
          const float tf = (float)(lo + (hi << 8)) * (1.f / (float)(1 << rr));
          cacc = fmaf(cc, tf, cacc);
          D[rr] = (uint32_t)__float_as_int(fmaf(ca, tf, cb));
        }
        // 4 ranks x 3 digits -> one word per digit (byte e = rank 4g + e): the B operand words of the second contraction
        const uint32_t p01a = __byte_perm(D[0], D[1], 0x5140), p01b = __byte_perm(D[0], D[1], 0x6262);
        const uint32_t p23a = __byte_perm(D[2], D[3], 0x5140), p23b = __byte_perm(D[2], D[3], 0x6262);
        uint32_t* dst = reinterpret_cast<uint32_t*>(ust) + rt * kUBlock;
        dst[0] = __byte_perm(p01a, p23a, 0x5410);
        dst[ust1] = __byte_perm(p01a, p23a, 0x7632);
        dst[64] = __byte_perm(p01b, p23b, 0x5410);
      }
      __syncwarp();

      // ---- second contraction: V[p][digit] += sum_k Y[p][k] udigit[k] --------------------
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        // (b0, b1) of col patches 0, 1 and of col patches 2, 3: already in operand order
        const uint4 bu01 = *reinterpret_cast<const uint4*>(uld[0] + rt * 4 * kUBlock + u01);
        const uint4 bu23 = *reinterpret_cast<const uint4*>(uld[0] + rt * 4 * kUBlock + u23);
        const uint32_t bu[kGroup][2] = {{bu01.x, bu01.y}, {bu01.z, bu01.w}, {bu23.x, bu23.y}, {bu23.z, bu23.w}};
#pragma unroll
        for (int sub = 0; sub < kGroup; ++sub) {
#pragma unroll
          for (int pt = 0; pt < PT; ++pt) {
            const uint32_t w = pick(yw[pt][rt], sub);
            const uint32_t w4 = w >> 4;
            mma_u8u8(acc[pt][0][0], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u,
                     bu[sub][0], bu[sub][1]);
            mma_u8u8(acc[pt][1][0], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u,
                     bu[sub][0], bu[sub][1]);
          }
        }
      }
    } else {
      // ---- several rows of X: column pair t of the first contraction carries row t ---------------------
      // per super-group: folded coefficients and the x digit registers of its 4 col patches
      const float4 va = *reinterpret_cast<const float4*>(mrow + li * 4);
      const float4 vb = *reinterpret_cast<const float4*>(mrow + nsg * 4 + li * 4);
      const float4 vc = *reinterpret_cast<const float4*>(mrow + nsg * 8 + li * 4);
      const float ca4[4] = {va.x, va.y, va.z, va.w};
      const float cb4[4] = {vb.x, vb.y, vb.z, vb.w};
      const float cc4[4] = {vc.x, vc.y, vc.z, vc.w};
      uint32_t bx0[kGroup][QT], bx1[kGroup][QT];
#pragma unroll
      for (int qt = 0; qt < QT; ++qt) {
        const uint4 h0 = zs[xlane + qt * 8];
        const uint4 h1 = zs[xlane + qt * 8 + 4];
        bx0[0][qt] = h0.x; bx0[1][qt] = h0.y; bx0[2][qt] = h0.z; bx0[3][qt] = h0.w;
        bx1[0][qt] = h1.x; bx1[1][qt] = h1.y; bx1[2][qt] = h1.z; bx1[3][qt] = h1.w;
      }
#pragma unroll
      for (int sub = 0; sub < kGroup; ++sub) {
        const float ca = ca4[sub], cb = cb4[sub], cc = cc4[sub];
        // ---- first contraction: T[k][2 row + digit] = sum_q Z[k][q] xdigit_row[q] --------------------
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
          // lane (g,t) owns row t of X: finishes the ranks k = 32rt + 4g + rr, rr = 0..3
          uint32_t D[4];
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) {
            const int lo = c1[rr >> 1][2 * (rr & 1)];
            const int hi = c1[rr >> 1][2 * (rr & 1) + 1];
            const float tf = (float)(lo + (hi << 8)) * (1.f / (float)(1 << rr));
            cacc = fmaf(cc, tf, cacc);
            D[rr] = (uint32_t)__float_as_int(fmaf(ca, tf, cb));
          }
          // the four ranks are neighbours in the digit rows: one word per digit
          const uint32_t p01a = __byte_perm(D[0], D[1], 0x5140), p01b = __byte_perm(D[0], D[1], 0x6262);
          const uint32_t p23a = __byte_perm(D[2], D[3], 0x5140), p23b = __byte_perm(D[2], D[3], 0x6262);
          uint32_t* dst = reinterpret_cast<uint32_t*>(ust + sub * kUSub + rt * 32);
          dst[0] = __byte_perm(p01a, p23a, 0x5410);
          dst[RP / 4] = __byte_perm(p01a, p23a, 0x7632);
          dst[2 * RP / 4] = __byte_perm(p01b, p23b, 0x5410);
        }
      }
      __syncwarp();

      // ---- second contraction: V[p][2 row' + digit'] += sum_k Y[p][k] udigit[k] --------------------
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
              mma_u8u8(acc[pt][0][nt], w & 0x01010101u, w & 0x02020202u, w4 & 0x01010101u, w4 & 0x02020202u,
                       bu[nt][0], bu[nt][1]);
              mma_u8u8(acc[pt][1][nt], w & 0x04040404u, w & 0x08080808u, w4 & 0x04040404u, w4 & 0x08080808u,
                       bu[nt][0], bu[nt][1]);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  if (!ok && lane == 0) atomicExch(p.counters + (kMaxCounters - 1), 1u);   // a bounded wait gave up
  // The weights are consumed: the next kernel of the stream may become resident now (programmatic
  // dependent launch; it starts once every CTA of this grid has got here).  A following kernel of this
  // library prefetches its weights meanwhile and waits for this grid to finish before it touches
  // anything else.  Triggering earlier would park the whole next grid on the SMs while this one runs.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

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
  const float us = ub * (1.f / kUScale);
#pragma unroll
  for (int nt = 0; nt < NT2; ++nt) {
    // which row of X and which digits this lane's two columns carry: (digit 0, digit 1) or
    // (digit 2, ones); the ones column times 63 removes the offset from the top digit exactly
    const int beta = NB == 1 ? 0 : 2 * nt + (t >> 1);
    const int tt = NB == 1 ? t : (t & 1);
    const float w_even = tt == 0 ? 1.f : (tt == 1 ? 65536.f : 0.f);
    const float w_odd = tt == 0 ? 256.f : 0.f;
    const int k63 = tt == 1 ? 63 : 0;
    const float ct_b = NB == 1 ? cterm : __shfl_sync(0xffffffffu, cterm, (lane & ~3) | beta);
#pragma unroll
    for (int pt = 0; pt < PT; ++pt)
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int rr = 2 * mt + half;
          const int a_even = acc[pt][mt][nt][2 * half], a_odd = acc[pt][mt][nt][2 * half + 1];
          float v = w_even * (float)(a_even - k63 * a_odd) + w_odd * (float)a_odd;
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          if (NB == 1) v += __shfl_xor_sync(0xffffffffu, v, 2);
          const float out = fmaf(v, us * (1.f / (float)(1 << rr)), ct_b);
          const bool writer = NB == 1 ? (t == 0) : ((t & 1) == 0);
          if (writer) red[(size_t)(warp * NB + beta) * PP + pt * 32 + g + 8 * rr] = out;
        }
  }

  // ---- the other warps hand their sums to warp 0 and retire ----------------------------------
  __threadfence_block();
  const int nthreads = kDT * bpc;
  if (warp != 0) {
    asm volatile("bar.arrive 1, %0;" ::"r"(nthreads) : "memory");
    return;
  }
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");

  // ---- CTA result, then the cross-CTA reduction in a fixed order (warp 0) ---------------------
  const int nparts = nbg * p.nchunks;
  const int part = bitgroup * p.nchunks + chunk;
  const int mrows = p.mtiles * NB;
  const size_t out_stride = (size_t)p.rw * PP;
  if (nparts == 1) {
    for (int idx = lane; idx < NB * PP; idx += 32) {
      const int beta = idx / PP, pp = idx % PP;
      float v = 0.f;
      // same association as the scratch route (the 4 warps of a bit layer first, then the bit layers in
      // order), so that both routes give identical bits
      for (int b = 0; b < bpc; ++b) {
        float sb = 0.f;
#pragma unroll
        for (int w = 0; w < kDW; ++w) sb += red[(size_t)((b * kDW + w) * NB + beta) * PP + pp];
        v += sb;
      }
      const bool valid = pp < p.P && m0 + beta < p.M;
      const int o = i * p.P + pp;
      if (valid) {
        if (p.bias) v += load_as_float(p.bias, o, p.bias_dtype);
        if (p.res) v += load_as_float(p.res, (size_t)(m0 + beta) * p.ld_res + o, p.res_dtype);
        store_from_float(p.y, (size_t)(m0 + beta) * p.ldy + o, p.y_dtype, v);
      }
      if (p.peer_world) peer_send(p, valid, m0 + beta, o, v, lane);
    }
    return;
  }
  for (int idx = lane; idx < NB * PP; idx += 32) {
    const int beta = idx / PP, pp = idx % PP;
    float v = 0.f;
    for (int b = 0; b < bpc; ++b) {
      float sb = 0.f;
#pragma unroll
      for (int w = 0; w < kDW; ++w) sb += red[(size_t)((b * kDW + w) * NB + beta) * PP + pp];
      v += sb;
    }
    p.partial[((size_t)part * mrows + m0 + beta) * out_stride + (size_t)i * PP + pp] = v;
  }
  // the lanes' partial sums are ordered before lane 0's ticket by the warp barrier, and the ticket is one
  // acquire-release atomic at GPU scope: the CTA that draws the last ticket sees every other CTA's sums
  __syncwarp();
  unsigned ticket = 0;
  if (lane == 0)
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                 : "=r"(ticket) : "l"(p.counters + i * p.mtiles + blockIdx.y) : "memory");
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  if (ticket != (unsigned)(nparts - 1)) return;
  for (int idx = lane; idx < NB * PP; idx += 32) {
    const int beta = idx / PP, pp = idx % PP;
    const bool valid = pp < p.P && m0 + beta < p.M;
    const int o = i * p.P + pp;
    float v = 0.f;
    if (valid) {
      for (int sp = 0; sp < nparts; ++sp)
        v += __ldcg(p.partial + ((size_t)sp * mrows + m0 + beta) * out_stride + (size_t)i * PP + pp);
      if (p.bias) v += load_as_float(p.bias, o, p.bias_dtype);
      if (p.res) v += load_as_float(p.res, (size_t)(m0 + beta) * p.ld_res + o, p.res_dtype);
      store_from_float(p.y, (size_t)(m0 + beta) * p.ldy + o, p.y_dtype, v);
    }
    if (p.peer_world) peer_send(p, valid, m0 + beta, o, v, lane);
  }
  if (lane == 0) p.counters[i * p.mtiles + blockIdx.y] = 0u;   // ready for the next call
}

template <int PT, int QT, int RT, int NB>
static int launch_decode_variant(const DecodeParams& p, const DecodePlan& pl, cudaStream_t st) {
  auto kern = (PT == 1 && NB == 1 && pl.self_prep) ? bqq_decode_kernel<PT, QT, RT, NB, (PT == 1 && NB == 1)>
                                                   : bqq_decode_kernel<PT, QT, RT, NB, false>;
  if (pl.smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess)
      return BQQ_ERR_CUDA;
  }
  const bool merged = PT == 1 && NB == 1 && pl.self_prep;   // such CTAs prepare x themselves
  // Every kernel is launched as a programmatic dependent of whatever precedes it in the stream: it may
  // become resident while that kernel still runs, prefetches weights, and executes griddepcontrol.wait
  // before it reads activations or touches the workspace.  After a kernel that never triggers early
  // (any kernel outside this library) this is an ordinary launch.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (!merged) {
    const XSource xs = {p.x, p.norm_w, p.ldx, p.x_dtype, p.norm_dtype, p.pro_mode, p.cw * p.Q, p.eps};
    cudaLaunchConfig_t xc = {};
    xc.gridDim = dim3((p.cwp * 8 + 127) / 128, p.Mp);
    xc.blockDim = dim3(128);
    xc.stream = st;
    xc.attrs = attr;
    xc.numAttrs = 1;
    if (cudaLaunchKernelEx(&xc, bqq_xprep_kernel<QT>, xs, p.M, p.cw, p.Q, p.cwp, (int)NB,
                           const_cast<uint8_t*>(p.xdig), const_cast<float*>(p.xscale), const_cast<float*>(p.xsum),
                           const_cast<float*>(p.xl1)) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  }
  cudaLaunchConfig_t cfg = {};
  // p.ncompute computing CTAs along x; with a peer gather a few more that only receive
  cfg.gridDim = dim3(p.ncompute + pl.nrecv, pl.mtiles);
  cfg.blockDim = dim3(kDT * p.bpc);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = st;
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
