// Host side of the decode forward: launch plan and dispatch to the kernel variants
// (algorithm and kernel in bqq_decode_kernel.cuh).
#include <cstdlib>

#include "bqq_decode_kernel.cuh"

namespace bqq {

template <> int decode_launch_variant<0>(const DecodeParams&, const DecodePlan&, cudaStream_t);
template <> int decode_launch_variant<1>(const DecodeParams&, const DecodePlan&, cudaStream_t);
template <> int decode_launch_variant<2>(const DecodeParams&, const DecodePlan&, cudaStream_t);
template <> int decode_launch_variant<3>(const DecodeParams&, const DecodePlan&, cudaStream_t);

static const int kVariantPT[4] = {1, 2, 2, 4};
static const int kVariantQT[4] = {1, 2, 2, 4};
static const int kVariantRT[4] = {1, 1, 2, 2};
static const int kVariantMaxSgw[4] = {4, 2, 1, 1};

#ifdef BQQ_BOUNDS_CHECK
static volatile unsigned long long* g_decode_dbg = nullptr;
#endif

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// The plan depends on the patch geometry, the number of col patches and M only
// (never on the number of row patches), so row shards reduce in the same order.
static DecodePlan make_decode_plan(const Geom& g, int M) {
  DecodePlan pl;
  pl.variant = -1;
  for (int v = 0; v < 4; ++v)
    if (g.PT <= kVariantPT[v] && g.QT <= kVariantQT[v] && g.RT <= kVariantRT[v]) { pl.variant = v; break; }
  if (pl.variant < 0) { pl.smem = 0; return pl; }
  pl.NB = M <= 1 ? 1 : 4;
  pl.mtiles = (M + pl.NB - 1) / pl.NB;
  int sgw = g.JG <= 16 ? 1 : (g.JG <= 64 ? 2 : 4);
  if (sgw > kVariantMaxSgw[pl.variant]) sgw = kVariantMaxSgw[pl.variant];
  pl.sgw = sgw;
  pl.nchunks = (g.JG + kDW * sgw - 1) / (kDW * sgw);
  pl.nparts = g.bw * pl.nchunks;
  const int PTv = kVariantPT[pl.variant], QTv = kVariantQT[pl.variant], RTv = kVariantRT[pl.variant];
  pl.smem = (size_t)DecodeSmem(kGroup * kDW * sgw, pl.NB, QTv, RTv, PTv).total;
  pl.partial_floats = pl.nparts > 1 ? (size_t)pl.nparts * pl.mtiles * pl.NB * g.rw * PTv * 32 : 0;
  return pl;
}

size_t decode_workspace_bytes(const BqqDims* dims, int M) {
  Geom g(*dims);
  DecodePlan pl = make_decode_plan(g, M);
  if (pl.variant < 0) return 0;
  return kCounterBytes + align_up(pl.partial_floats * 4, 256);
}

int decode_launch(const BqqLayer* L, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                  int y_dtype, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t st) {
  Geom g(L->dims);
  DecodePlan pl = make_decode_plan(g, M);
  if (pl.variant < 0) return BQQ_ERR_UNSUPPORTED;
  if ((size_t)g.rw * pl.mtiles > (size_t)kMaxCounters) return BQQ_ERR_UNSUPPORTED;
  DecodeParams p;
  p.zp = reinterpret_cast<const uint4*>(L->zplanes);
  p.yp = reinterpret_cast<const uint4*>(L->yplanes);
  p.a = L->a; p.b = L->b; p.c = L->c; p.d = L->d; p.coef_dtype = L->coef_dtype;
  p.x = x; p.y = y; p.bias = L->bias;
  p.ldx = ldx; p.ldy = ldy;
  p.x_dtype = x_dtype; p.y_dtype = y_dtype; p.bias_dtype = L->bias_dtype;
  p.M = M; p.bw = g.bw; p.rw = g.rw; p.cw = g.cw; p.P = g.P; p.Q = g.Q;
  p.PTg = g.PT; p.QTg = g.QT; p.RTg = g.RT; p.JG = g.JG; p.NS = g.NS;
  p.sgw = pl.sgw; p.nchunks = pl.nchunks; p.mtiles = pl.mtiles;
  p.partial = nullptr; p.counters = nullptr;
  if (pl.nparts > 1) {
    const size_t need = decode_workspace_bytes(&L->dims, M);
    if (!ws || ws_bytes < need) return BQQ_ERR_WORKSPACE;
    if (((uintptr_t)ws & 255) != 0) return BQQ_ERR_MISALIGNED;
    p.counters = reinterpret_cast<unsigned*>(ws);
    p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kCounterBytes);
  }
#ifdef BQQ_BOUNDS_CHECK
  p.lim_z = g.z_words() / 4; p.lim_y = g.y_words() / 4;
  p.lim_coef = (unsigned long long)g.bw * g.rw * g.cw; p.lim_d = (unsigned long long)g.rw * g.cw;
  p.lim_x = (unsigned long long)(M - 1) * ldx + g.in_features();
  p.lim_y_out = (unsigned long long)(M - 1) * ldy + g.out_features();
  p.lim_partial = pl.partial_floats; p.lim_smem = pl.smem;
  if (getenv("BQQ_DBG_EXTRA_SMEM")) pl.smem += 65536;
  p.dbg = g_decode_dbg;
#endif
  switch (pl.variant) {
    case 0: return decode_launch_variant<0>(p, pl, st);
    case 1: return decode_launch_variant<1>(p, pl, st);
    case 2: return decode_launch_variant<2>(p, pl, st);
    case 3: return decode_launch_variant<3>(p, pl, st);
  }
  return BQQ_ERR_UNSUPPORTED;
}

}  // namespace bqq

#ifdef BQQ_BOUNDS_CHECK
// Self-check builds only: where the decode kernel reports out-of-range indices (host-mapped memory).
extern "C" void bqq_debug_set_decode_report(volatile unsigned long long* host_mapped) { bqq::g_decode_dbg = host_mapped; }
#endif
