// Decode forward (M <= 16 rows of X): streams the packed planes exactly once.
//
// Per (row patch i, col patch j, bit b) with coefficients (a,b,c,d):
//   xsum = sum_q x[j,q];  t_k = sum_q Z[k,q] x[j,q];  u_k = a t_k + b xsum
//   y[i,p] += sum_k Y[p,k] u_k + c sum_k t_k (+ d xsum once per patch)
// which is BinaryQuadratic.forward without materialising W
// (neural_network_compression/src/bqq_modules.py:34-46; the same identity as
// src/bqq_cuda.cu:82-84,134-156).  All sums are fp32.
//
// Work split: CTA = (row patch i, split of the patch-bit sequence, M tile);
// a warp owns whole super-groups (4 patch-bits): lane k holds Z row k for the
// first contraction, lane p holds Y row p for the second; 128-bit loads fetch
// one word of 4 consecutive patch-bits per lane.  Partial sums of the splits
// go to a scratch buffer; the last CTA to finish a row patch adds them in
// split order (deterministic), adds bias and converts to the output type.
#include "bqq_decode_kernel.cuh"

namespace bqq {

template <int MT>
int decode_launch_mt(const DecodeParams& p, const DecodePlan& pl, int RW, int PC, cudaStream_t st);
extern template int decode_launch_mt<1>(const DecodeParams&, const DecodePlan&, int, int, cudaStream_t);
extern template int decode_launch_mt<4>(const DecodeParams&, const DecodePlan&, int, int, cudaStream_t);
extern template int decode_launch_mt<8>(const DecodeParams&, const DecodePlan&, int, int, cudaStream_t);

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static DecodePlan make_decode_plan(const Geom& g, int M) {
  DecodePlan pl;
  pl.MT = M <= 1 ? 1 : (M <= 4 ? 4 : 8);
  pl.mtiles = (M + pl.MT - 1) / pl.MT;
  const int target_ctas = kNumSM * 8;
  int splits = (target_ctas + g.rw * pl.mtiles - 1) / (g.rw * pl.mtiles);
  if (splits < 1) splits = 1;
  int sgps = (g.NS + splits - 1) / splits;
  if (sgps > kDecodeWarps) sgps = (sgps + kDecodeWarps - 1) / kDecodeWarps * kDecodeWarps;
  // staged x must fit in shared memory: JC * MT * QW*32 floats <= 64 KiB
  const int QP = g.QW * 32;
  int max_jc = (64 * 1024) / (pl.MT * QP * 4);
  int max_sgps = ((max_jc - 2) * g.bw) / kGroup;
  if (max_sgps < 1) max_sgps = 1;
  if (sgps > max_sgps) sgps = max_sgps;
  if (sgps < 1) sgps = 1;
  pl.sgps = sgps;
  pl.splits = (g.NS + sgps - 1) / sgps;
  int jc = (sgps * kGroup - 1) / g.bw + 2;
  if (jc > g.cw) jc = g.cw;
  pl.JC = jc;
  const int pc = g.PP / 32;
  pl.PCK = pc <= 1 ? 1 : (pc <= 2 ? 2 : 4);
  const int PPK = pl.PCK * 32;                  // Y rows as the kernel variant sees them
  size_t floats = (size_t)jc * pl.MT * QP      // x
                + (((size_t)jc * pl.MT + 3) & ~(size_t)3)   // xsum
                + (size_t)kDecodeWarps * pl.MT * g.RP    // u exchange
                + (size_t)kDecodeWarps * pl.MT * PPK;    // cross-warp reduction
  pl.smem = floats * 4;
  pl.partial_floats = pl.splits > 1 ? (size_t)pl.splits * pl.mtiles * pl.MT * g.rw * PPK : 0;
  pl.counter_words = pl.splits > 1 ? (size_t)g.rw * pl.mtiles : 0;
  return pl;
}

size_t decode_workspace_bytes(const BqqDims* dims, int M) {
  Geom g(*dims);
  DecodePlan pl = make_decode_plan(g, M);
  return align_up(pl.counter_words * 4, 256) + align_up(pl.partial_floats * 4, 256);
}

int decode_launch(const BqqLayer* L, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                  int y_dtype, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t st) {
  Geom g(L->dims);
  DecodePlan pl = make_decode_plan(g, M);
  DecodeParams p;
  p.zp = reinterpret_cast<const uint4*>(L->zplanes);
  p.yp = reinterpret_cast<const uint4*>(L->yplanes);
  p.coef = reinterpret_cast<const float4*>(L->coef);
  p.x = x; p.y = y; p.bias = L->bias;
  p.ldx = ldx; p.ldy = ldy;
  p.x_dtype = x_dtype; p.y_dtype = y_dtype; p.bias_dtype = L->bias_dtype;
  p.M = M; p.bw = g.bw; p.rw = g.rw; p.cw = g.cw; p.P = g.P; p.Q = g.Q; p.QW = g.QW; p.NPB = g.NPB; p.NS = g.NS;
  p.PPg = g.PP;
  p.splits = pl.splits; p.sgps = pl.sgps; p.JC = pl.JC; p.mtiles = pl.mtiles;
  p.partial = nullptr; p.counters = nullptr;
  if (pl.splits > 1) {
    size_t need = decode_workspace_bytes(&L->dims, M);
    if (!ws || ws_bytes < need) return BQQ_ERR_WORKSPACE;
    if (((uintptr_t)ws & 255) != 0) return BQQ_ERR_MISALIGNED;
    p.counters = reinterpret_cast<unsigned*>(ws);
    p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + align_up(pl.counter_words * 4, 256));
  }
  switch (pl.MT) {
    case 1: return decode_launch_mt<1>(p, pl, g.RW, pl.PCK, st);
    case 4: return decode_launch_mt<4>(p, pl, g.RW, pl.PCK, st);
    case 8: return decode_launch_mt<8>(p, pl, g.RW, pl.PCK, st);
  }
  return BQQ_ERR_UNSUPPORTED;
}

}  // namespace bqq
