// Host side of the decode forward: launch plan and dispatch to the kernel variants
// (algorithm and kernel in bqq_decode_kernel.cuh).
#include "bqq_decode_kernel.cuh"

namespace bqq {

template <> int decode_launch_variant<0>(const DecodeParams&, const DecodePlan&, cudaStream_t);
template <> int decode_launch_variant<1>(const DecodeParams&, const DecodePlan&, cudaStream_t);
template <> int decode_launch_variant<2>(const DecodeParams&, const DecodePlan&, cudaStream_t);
template <> int decode_launch_variant<3>(const DecodeParams&, const DecodePlan&, cudaStream_t);

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static const int kVariantPT[4] = {1, 2, 2, 4};
static const int kVariantQT[4] = {1, 2, 2, 4};
static const int kVariantRT[4] = {1, 1, 2, 2};

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
  // chunks per (row patch, bit layer), from measured sweeps on 2048..14336 input features: one chunk up to
  // 32 col-patch groups (and then one CTA for all bit layers at M = 1), two up to 64; wider layers want about
  // 8 CTAs per row patch over all bit layers (4 chunks at 2 bit layers, 2 at 4), chunks of at least 16 groups
  int nchunks = g.JG <= 32 ? 1 : 2;
  if (g.JG > 64) {
    const int k = (g.JG + 127) / 128;
    nchunks = std::max(k, std::min(g.JG / 16, (8 * k + g.bw / 2) / g.bw));
  }
  if (pl.NB > 1 && g.JG > 64) nchunks = std::max(nchunks, (g.JG + 31) / 32);   // batched rows: shorter chunks balance better
  int sgw = (g.JG + kDW * nchunks - 1) / (kDW * nchunks);
  if (sgw > kMaxSgw) sgw = kMaxSgw;
  pl.sgw = sgw;
  pl.nchunks = (g.JG + kDW * sgw - 1) / (kDW * sgw);
  // short single-chunk layers at batch 1: one CTA takes all bit layers of a row patch, so the sums never
  // leave the CTA (no scratch round trip); 4 warps per bit layer, at most 16 warps.  Tall layers (many row
  // patches) fill the machine better with one CTA per bit layer (measured: 6144x4096 prefers the former,
  // 28672x4096 the latter).  Both routes add in the same order and give identical bits, so this one choice
  // may depend on the number of row patches.
  pl.bpc = (pl.variant == 0 && pl.NB == 1 && pl.nchunks == 1 && g.bw <= 4 && g.rw * g.bw * kDW <= 3072) ? g.bw : 1;
  // a CTA of 16 warps is alone on its SM: with more row patches than SMs a second, mostly empty wave would follow
  // (6144x2048 with 4 bit layers: 11.8 us); two CTAs of 8 warps per row patch fit three to an SM (9.3 us)
  if (pl.bpc == 4 && g.rw > 148) pl.bpc = 2;
  pl.nparts = (g.bw / pl.bpc) * pl.nchunks;
  // CTAs that take all bit layers of a short layer also prepare the x digits themselves (one launch).  Measured:
  // letting the CTAs of chunked layers prepare their own chunk as well (no preparation kernel at all) is slower,
  // 2048x6144 7.1 -> 9.4 us, 4096x14336 with 4 bit layers 23 -> 38 us: every CTA then starts with the read and
  // quantisation of x before it can use its first plane words.
  pl.self_prep = pl.bpc > 1 ? 1 : 0;
  const int PTv = kVariantPT[pl.variant], QTv = kVariantQT[pl.variant], RTv = kVariantRT[pl.variant];
  pl.smem = (size_t)DecodeSmem(sgw, pl.NB, PTv, QTv, RTv, pl.bpc, pl.self_prep != 0).total;
  const size_t Mp = (size_t)pl.mtiles * pl.NB, cwp = (size_t)g.JG * kGroup;
  pl.xdig_bytes = align_up(Mp * cwp * 2 * QTv * 32, 256);
  pl.xmeta_bytes = 3 * align_up(Mp * cwp * 4, 256);     // scale, sum, l1
  pl.partial_floats = pl.nparts > 1 ? (size_t)pl.nparts * pl.mtiles * pl.NB * g.rw * PTv * 32 : 0;
  return pl;
}

size_t decode_counter_bytes() { return kCounterBytes; }

int decode_launches(const BqqDims* dims, int M) {
  Geom g(*dims);
  DecodePlan pl = make_decode_plan(g, M);
  if (pl.variant < 0) return BQQ_ERR_UNSUPPORTED;
  return pl.self_prep ? 1 : 2;
}

size_t decode_workspace_bytes(const BqqDims* dims, int M) {
  Geom g(*dims);
  DecodePlan pl = make_decode_plan(g, M);
  if (pl.variant < 0) return 0;
  return kCounterBytes + pl.xdig_bytes + pl.xmeta_bytes + align_up(pl.partial_floats * 4, 256);
}

int decode_launch(const BqqLayer* L, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                  int y_dtype, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t st, const BqqPeerGroup* peer,
                  const BqqFusion* fusion, void* gathered, int64_t ld_gathered) {
  Geom g(L->dims);
  DecodePlan pl = make_decode_plan(g, M);
  pl.nrecv = 0;
  if (pl.variant < 0) return BQQ_ERR_UNSUPPORTED;
  if ((size_t)g.rw * pl.mtiles > (size_t)kMaxCounters - 1) return BQQ_ERR_UNSUPPORTED;   // last word: status
  if ((size_t)g.bw * g.rw * g.cw >= (1ull << 31)) return BQQ_ERR_UNSUPPORTED;           // 32-bit coefficient offsets
  DecodeParams p;
  p.zp = reinterpret_cast<const uint4*>(L->zplanes);
  p.yp = reinterpret_cast<const uint4*>(L->yplanes);
  p.a = L->a; p.b = L->b; p.c = L->c; p.d = L->d; p.coef_dtype = L->coef_dtype;
  p.x = x; p.y = y; p.bias = L->bias;
  p.ldx = ldx; p.ldy = ldy;
  p.x_dtype = x_dtype; p.y_dtype = y_dtype; p.bias_dtype = L->bias_dtype;
  p.M = M; p.bw = g.bw; p.rw = g.rw; p.cw = g.cw; p.P = g.P; p.Q = g.Q;
  p.PTg = g.PT; p.QTg = g.QT; p.RTg = g.RT; p.JG = g.JG; p.NS = g.NS;
  p.sgw = pl.sgw; p.bpc = pl.bpc; p.nchunks = pl.nchunks; p.mtiles = pl.mtiles;
  const size_t need = decode_workspace_bytes(&L->dims, M);
  if (!ws || ws_bytes < need) return BQQ_ERR_WORKSPACE;
  if (((uintptr_t)ws & 255) != 0) return BQQ_ERR_MISALIGNED;
  char* wsb = reinterpret_cast<char*>(ws);
  p.counters = reinterpret_cast<unsigned*>(wsb);
  p.xdig = reinterpret_cast<const uint8_t*>(wsb + kCounterBytes);
  p.Mp = pl.mtiles * pl.NB; p.cwp = g.JG * kGroup;
  {
    const size_t one = pl.xmeta_bytes / 3;
    char* meta = wsb + kCounterBytes + pl.xdig_bytes;
    p.xscale = reinterpret_cast<const float*>(meta);
    p.xsum = reinterpret_cast<const float*>(meta + one);
    p.xl1 = reinterpret_cast<const float*>(meta + 2 * one);
  }
  p.partial = reinterpret_cast<float*>(wsb + kCounterBytes + pl.xdig_bytes + pl.xmeta_bytes);
  p.coef_vec = (L->coef_dtype == BQQ_F32 && g.cw % 4 == 0 && (((uintptr_t)L->a | (uintptr_t)L->b |
                                                                 (uintptr_t)L->c | (uintptr_t)L->d) & 15) == 0)
                   ? 1 : 0;
  p.norm_w = p.res = nullptr;
  p.ld_res = 0;
  p.pro_mode = BQQ_PRO_NONE;
  p.norm_dtype = p.res_dtype = 0;
  p.eps = 0.f;
  if (fusion) {
    p.pro_mode = fusion->prologue;
    p.norm_w = fusion->norm_weight; p.norm_dtype = fusion->norm_dtype; p.eps = fusion->eps;
    p.res = fusion->residual; p.ld_res = fusion->ld_residual; p.res_dtype = fusion->residual_dtype;
  }
  for (int q = 0; q < BQQ_MAX_PEERS; ++q) p.peer_regions[q] = nullptr;
  p.peer_world = p.peer_rank = p.peer_row_words = 0;
  p.peer_half = 0;
  p.peer_out = nullptr;
  p.peer_ld_out = p.peer_wait = 0;
  p.ncompute = g.rw * (g.bw / pl.bpc) * pl.nchunks;
  p.peer_seg_words = 0;
  if (peer) {
    const size_t es = dtype_size(y_dtype);
    if (((size_t)g.out_features() * es) % 4 || (es == 2 && (g.P & 1))) return BQQ_ERR_MISALIGNED;   // outputs travel as 32-bit words
    for (int q = 0; q < peer->world; ++q) p.peer_regions[q] = reinterpret_cast<uint8_t*>(peer->regions[q]);
    p.peer_world = peer->world;
    p.peer_rank = peer->rank;
    p.peer_row_words = (int)((size_t)g.out_features() * es / 4);
    p.peer_half = peer_half_bytes(peer->gather_bytes);
    if (fusion && fusion->out_segments == 2) {
      if (p.peer_row_words % 2) return BQQ_ERR_MISALIGNED;
      p.peer_seg_words = p.peer_row_words / 2;
    } else if (fusion && fusion->out_segments > 2) {
      return BQQ_ERR_UNSUPPORTED;
    }
    // the receiving side runs in the same launch: a few CTAs that poll this rank's region and write the rows
    if (!gathered) return BQQ_ERR_NULL;
    if ((((size_t)ld_gathered * es) % 4) || ((uintptr_t)gathered & 3)) return BQQ_ERR_MISALIGNED;
    p.peer_out = reinterpret_cast<uint32_t*>(gathered);
    p.peer_ld_out = (long long)((size_t)ld_gathered * es / 4);
    p.peer_wait = peer->wait_cycles ? (long long)peer->wait_cycles : 2000000000LL;
    const long long words = (long long)M * p.peer_row_words * peer->world;
    const int threads = kDT * pl.bpc;
    // receiving CTAs: about two words per thread, at most 32 CTAs
    pl.nrecv = (int)std::min<long long>(32, std::max<long long>(1, (words + 2 * threads - 1) / (2 * threads)));
  }
  switch (pl.variant) {
    case 0: return decode_launch_variant<0>(p, pl, st);
    case 1: return decode_launch_variant<1>(p, pl, st);
    case 2: return decode_launch_variant<2>(p, pl, st);
    case 3: return decode_launch_variant<3>(p, pl, st);
  }
  return BQQ_ERR_UNSUPPORTED;
}

}  // namespace bqq

