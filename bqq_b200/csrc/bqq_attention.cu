// Single-token attention of the decoder-stack harness (one launch per layer): rotary embedding of the new q and k
// heads, append of k and v to the cache, and attention of every query head over the cached keys, split over the key
// range ("flash decoding") with a fixed-order combination by the last CTA of each (sequence, kv head).
// Glue between the BinaryQuadratic projections of a decoder block; the reference's host models call torch's
// scaled_dot_product_attention here and have no kernel of their own.
//
// Grid (splits, kv heads, sequences), 128 threads.  A CTA owns one kv head and a contiguous range of keys; its four
// warps take the query heads of the group in turn (warp w: heads w, w + 4, ...).  K and V rows of a tile of 64 keys
// are copied to shared memory with cp.async (issued before the wait for the preceding kernel: cached rows are old);
// a lane owns a key for q.K and four output dimensions for P.V; running maximum and sum per head live in the
// warp.  The CTA whose range ends at the new position computes the rotated k itself, writes k and v into the cache
// and into its tile.  Partial results (m, l, 128 numerators) go to scratch; the CTA that draws the last ticket of its
// (sequence, kv head) adds them in split order and writes bf16 outputs.
// With a peer gather group (heads sharded over the ranks of one node) the finished output words also go, with the
// gather's sequence number, into every rank's slot region (the protocol of bqq_peer.cu), and a few more CTAs of the
// same grid (blockIdx.x >= splits) wait, bounded, for all ranks' words and write the gathered rows.
#include <cuda_bf16.h>
#include <string.h>

#include <algorithm>

#include "bqq_common.cuh"

namespace bqq {

constexpr int kAttDim = 128;                 // head dimension
constexpr int kAttTile = 64;                 // keys per shared-memory tile
constexpr int kAttRow = kAttDim * 2 + 16;    // bytes per tile row: 256 of data + 16 of padding (conflict-free 16-byte row reads)
constexpr int kAttThreads = 128;
constexpr int kAttMaxGroup = 16;             // query heads per kv head
constexpr int kAttMaxSplits = 32;
constexpr int kAttPart = 4 + kAttDim;       // floats of one partial result: m, l, two unused, 128 numerators (16-byte aligned)

struct AttParams {
  const __nv_bfloat16* qkv;      // [B][heads + 2 kv_heads][128]
  long long ld_qkv;              // elements between sequences
  __nv_bfloat16* kc;             // [B][max_seq][kv_heads][128]
  __nv_bfloat16* vc;
  long long ld_cache;            // elements between sequences of a cache
  const __nv_bfloat16* cosv;     // [max_seq][64]
  const __nv_bfloat16* sinv;
  const int* lens;               // [B] tokens already cached = position of the new token
  __nv_bfloat16* out;            // [B][heads][128]
  long long ld_out;
  float* partial;                // [B][heads][splits][4 + 128]
  unsigned* tickets;             // [B][kv_heads], zero between launches
  int heads, kv_heads, max_seq, splits;
  float scale;
  // optional gather of the outputs over the ranks of a peer group (all zero when unused)
  uint8_t* peer_regions[BQQ_MAX_PEERS];
  int peer_world, peer_rank;
  unsigned long long peer_half;  // bytes of one half of a region's slot area
  long long peer_wait;           // clock budget of one wait on a peer
  uint32_t* peer_out;            // gathered rows [B][world * heads * 64] words
  long long peer_ld_out;         // its row pitch in words
};

// Words w0 (dimensions 4 lane, 4 lane + 1) and w1 (the next two) of query head `head` of sequence b: into slot
// [b][rank-major column] of every rank's region, each with the sequence number of this gather.
__device__ __forceinline__ void att_peer_send(const AttParams& p, int b, int head, int lane, uint32_t w0, uint32_t w1) {
  const unsigned* mine = reinterpret_cast<const unsigned*>(p.peer_regions[p.peer_rank]);
  const unsigned count = *reinterpret_cast<const volatile unsigned*>(mine) + 1u;
  const unsigned seq = count | 0x80000000u;
  const size_t row_words = (size_t)p.heads * (kAttDim / 2);
  const size_t slot = ((size_t)b * p.peer_world + p.peer_rank) * row_words + (size_t)head * (kAttDim / 2) + 2 * lane;
  const size_t off = kPeerCtrlBytes + (count & 1u) * p.peer_half + slot * 8;
  for (int q = 0; q < p.peer_world; ++q) {
    peer_slot_store(p.peer_regions[q] + off, w0, seq);
    peer_slot_store(p.peer_regions[q] + off + 8, w1, seq);
  }
}

// Receiving CTAs (blockIdx.x >= splits): poll every slot of this rank's region until it carries the gather's sequence
// number (bounded), write the data words to the gathered rows; the last one to finish advances the gather count.
__device__ __forceinline__ void att_peer_receive(const AttParams& p) {
  __shared__ int s_giveup;
  // the gathered tensor may still be read by earlier kernels of the stream
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int tid = threadIdx.x;
  if (tid == 0) s_giveup = 0;
  __syncthreads();
  unsigned* mine = reinterpret_cast<unsigned*>(p.peer_regions[p.peer_rank]);
  const unsigned count = *reinterpret_cast<volatile unsigned*>(mine) + 1u;
  const unsigned e = count | 0x80000000u;
  const uint8_t* slots = reinterpret_cast<const uint8_t*>(mine) + kPeerCtrlBytes + (count & 1u) * p.peer_half;
  const long long grow = (long long)p.heads * (kAttDim / 2) * p.peer_world;     // words of one gathered row
  const long long n = (long long)gridDim.z * grow;
  const int per_x = (int)gridDim.x - p.splits;
  const long long receivers = (long long)per_x * gridDim.y * gridDim.z;
  const long long me = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * per_x + ((int)blockIdx.x - p.splits);
  // four slots per round, their loads in flight together; a slot that has not arrived yet is polled on its own
  const long long step = receivers * blockDim.x;
  for (long long w0 = me * blockDim.x + tid; w0 < n; w0 += 4 * step) {
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
  __syncthreads();
  if (tid == 0) {
    if (s_giveup) atomicExch(mine + 1, 1u);
    // every word has arrived, so every sender of this rank has read the gather count: the last receiver advances it
    __threadfence();
    if (atomicAdd(mine + 2, 1u) == (unsigned)(receivers - 1)) {
      mine[2] = 0u;
      *reinterpret_cast<volatile unsigned*>(mine) = count;
    }
  }
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// four finished outputs of a lane (dimensions 4 lane .. 4 lane + 3 of one query head): to the local tensor and, with a
// peer group, to every rank
__device__ __forceinline__ void att_write(const AttParams& p, int b, int head, int lane, float v0, float v1, float v2, float v3) {
  const __nv_bfloat162 h0 = __floats2bfloat162_rn(v0, v1), h1 = __floats2bfloat162_rn(v2, v3);
  __nv_bfloat16* o = p.out + (size_t)b * p.ld_out + (size_t)head * kAttDim + 4 * lane;
  *reinterpret_cast<__nv_bfloat162*>(o) = h0;
  *reinterpret_cast<__nv_bfloat162*>(o + 2) = h1;
  if (p.peer_world)
    att_peer_send(p, b, head, lane, *reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
}

__global__ void __launch_bounds__(kAttThreads)
bqq_attention_decode_kernel(const AttParams p) {
  extern __shared__ __align__(16) uint8_t asm_[];
  uint8_t* sk = asm_;                                        // [64][272]
  uint8_t* sv = sk + kAttTile * kAttRow;                     // [64][272]
  float* sq = reinterpret_cast<float*>(sv + kAttTile * kAttRow);   // [group][128] rotated, scaled q
  __shared__ int s_last;

  if (p.peer_world && (int)blockIdx.x >= p.splits) {
    att_peer_receive(p);
    return;
  }
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = p.heads / p.kv_heads;
  const int pos = p.lens[b];                                 // written long before the preceding kernel started
  if (pos < 0 || pos >= p.max_seq) return;                   // no room in the cache: every CTA of the sequence leaves
  const int L = pos + 1;                                     // keys after the append
  int chunk = (L + p.splits - 1) / p.splits;
  chunk = (chunk + 7) & ~7;
  const int k0 = split * chunk, k1 = min(L, k0 + chunk);
  const __nv_bfloat16* kbase = p.kc + (size_t)b * p.ld_cache + (size_t)hk * kAttDim;
  const __nv_bfloat16* vbase = p.vc + (size_t)b * p.ld_cache + (size_t)hk * kAttDim;
  const size_t krow = (size_t)p.kv_heads * kAttDim;          // elements between keys

  // rows [t0, t0 + n) of K and V -> shared memory, 16 bytes per copy (row pos of the cache is stale: replaced below)
  auto load_tile = [&](int t0, int n) {
    for (int c = tid; c < n * 32; c += kAttThreads) {
      const int r = c >> 5, part = c & 31;                   // 16 x 16 bytes of K, then 16 of V
      const size_t off = (size_t)(t0 + r) * krow + (size_t)(part & 15) * 8;
      if (part < 16) cp_async16(sk + r * kAttRow + part * 16, kbase + off);
      else cp_async16(sv + r * kAttRow + (part - 16) * 16, vbase + off);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (k0 < k1) load_tile(k0, min(kAttTile, k1 - k0));

  // q, k, v of the new token come from the preceding kernel
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const __nv_bfloat16* row = p.qkv + (size_t)b * p.ld_qkv;
  const __nv_bfloat16* cs = p.cosv + (size_t)pos * (kAttDim / 2);
  const __nv_bfloat16* sn = p.sinv + (size_t)pos * (kAttDim / 2);
  for (int e = tid; e < group * (kAttDim / 2); e += kAttThreads) {       // one rotated pair per step
    const int g = e / (kAttDim / 2), i = e % (kAttDim / 2);
    const __nv_bfloat16* q = row + (size_t)(hk * group + g) * kAttDim;
    const float x0 = __bfloat162float(q[2 * i]), x1 = __bfloat162float(q[2 * i + 1]);
    const float c = __bfloat162float(cs[i]), s = __bfloat162float(sn[i]);
    // the library kernel this replaces rounds the rotated q to bf16 before the product; so does this one
    sq[g * kAttDim + 2 * i] = __bfloat162float(__float2bfloat16_rn(x0 * c - x1 * s)) * p.scale;
    sq[g * kAttDim + 2 * i + 1] = __bfloat162float(__float2bfloat16_rn(x0 * s + x1 * c)) * p.scale;
  }
  const bool owns_new = pos >= k0 && pos < k1;               // exactly one split holds the new position

  // per head (warp): running maximum, sum, and the lane's four numerators
  float m_run[kAttMaxGroup / 4], l_run[kAttMaxGroup / 4], acc[kAttMaxGroup / 4][4];
#pragma unroll
  for (int s = 0; s < kAttMaxGroup / 4; ++s) {
    m_run[s] = -INFINITY; l_run[s] = 0.f;
    acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.f;
  }

  for (int t0 = k0; t0 < k1; t0 += kAttTile) {
    const int n = min(kAttTile, k1 - t0);
    if (t0 != k0) {
      __syncthreads();                                       // everyone is done with the previous tile
      load_tile(t0, n);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (owns_new && pos >= t0 && pos < t0 + n) {
      // the new token's row: rotated k and v, into the tile and into the cache
      const int r = pos - t0;
      if (tid < kAttDim / 2) {
        const __nv_bfloat16* k = row + (size_t)(p.heads + hk) * kAttDim;
        const float x0 = __bfloat162float(k[2 * tid]), x1 = __bfloat162float(k[2 * tid + 1]);
        const float c = __bfloat162float(cs[tid]), s = __bfloat162float(sn[tid]);
        const __nv_bfloat162 kr = __floats2bfloat162_rn(x0 * c - x1 * s, x0 * s + x1 * c);
        *reinterpret_cast<__nv_bfloat162*>(sk + r * kAttRow + tid * 4) = kr;
        *reinterpret_cast<__nv_bfloat162*>(p.kc + (size_t)b * p.ld_cache + (size_t)pos * krow + (size_t)hk * kAttDim + 2 * tid) = kr;
      } else {
        const int i = tid - kAttDim / 2;
        const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(row + (size_t)(p.heads + p.kv_heads + hk) * kAttDim + 2 * i);
        *reinterpret_cast<__nv_bfloat162*>(sv + r * kAttRow + i * 4) = v2;
        *reinterpret_cast<__nv_bfloat162*>(p.vc + (size_t)b * p.ld_cache + (size_t)pos * krow + (size_t)hk * kAttDim + 2 * i) = v2;
      }
    }
    __syncthreads();                                         // q, the tile and the new row are in place

#pragma unroll
    for (int s = 0; s < kAttMaxGroup / 4; ++s) {
      const int g = warp + 4 * s;
      if (g >= group) break;
      const float4* q4 = reinterpret_cast<const float4*>(sq + g * kAttDim);
      // scores of keys lane and lane + 32 of the tile
      float sc[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int r = lane + 32 * h;
        float dot = -INFINITY;
        if (r < n) {
          const uint4* kr = reinterpret_cast<const uint4*>(sk + r * kAttRow);
          float d0 = 0.f, d1 = 0.f;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            const uint4 kw = kr[c];
            const float4 qa = q4[2 * c], qb = q4[2 * c + 1];
            d0 = fmaf(bf_lo(kw.x), qa.x, d0); d1 = fmaf(bf_hi(kw.x), qa.y, d1);
            d0 = fmaf(bf_lo(kw.y), qa.z, d0); d1 = fmaf(bf_hi(kw.y), qa.w, d1);
            d0 = fmaf(bf_lo(kw.z), qb.x, d0); d1 = fmaf(bf_hi(kw.z), qb.y, d1);
            d0 = fmaf(bf_lo(kw.w), qb.z, d0); d1 = fmaf(bf_hi(kw.w), qb.w, d1);
          }
          dot = d0 + d1;
        }
        sc[h] = dot;
      }
      float mx = fmaxf(sc[0], sc[1]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m_run[s], mx);               // finite: the tile has at least one key
      const float fix = __expf(m_run[s] - m_new);            // 0 on the first tile
      const float p0 = __expf(sc[0] - m_new), p1 = __expf(sc[1] - m_new);   // exp(-inf) = 0 for absent keys
      float ps = p0 + p1;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      l_run[s] = l_run[s] * fix + ps;
      m_run[s] = m_new;
      float a0 = acc[s][0] * fix, a1 = acc[s][1] * fix, a2 = acc[s][2] * fix, a3 = acc[s][3] * fix;
      // numerators of dimensions 4 lane .. 4 lane + 3
      for (int r = 0; r < n; ++r) {
        const float pr = __shfl_sync(0xffffffffu, r < 32 ? p0 : p1, r & 31);
        const uint2 vw = *reinterpret_cast<const uint2*>(sv + r * kAttRow + lane * 8);
        a0 = fmaf(pr, bf_lo(vw.x), a0); a1 = fmaf(pr, bf_hi(vw.x), a1);
        a2 = fmaf(pr, bf_lo(vw.y), a2); a3 = fmaf(pr, bf_hi(vw.y), a3);
      }
      acc[s][0] = a0; acc[s][1] = a1; acc[s][2] = a2; acc[s][3] = a3;
    }
  }

  // ---- results ----
  if (p.splits == 1) {
#pragma unroll
    for (int s = 0; s < kAttMaxGroup / 4; ++s) {
      const int g = warp + 4 * s;
      if (g >= group) break;
      const float inv = 1.f / l_run[s];
      att_write(p, b, hk * group + g, lane, acc[s][0] * inv, acc[s][1] * inv, acc[s][2] * inv, acc[s][3] * inv);
    }
    return;
  }
#pragma unroll
  for (int s = 0; s < kAttMaxGroup / 4; ++s) {
    const int g = warp + 4 * s;
    if (g >= group) break;
    float* dst = p.partial + (((size_t)b * p.heads + hk * group + g) * p.splits + split) * kAttPart;
    if (lane == 0) { dst[0] = m_run[s]; dst[1] = l_run[s]; }            // (-inf, 0) for an empty range
    *reinterpret_cast<float4*>(dst + 4 + 4 * lane) = make_float4(acc[s][0], acc[s][1], acc[s][2], acc[s][3]);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned* ticket = p.tickets + (size_t)b * p.kv_heads + hk;
    const unsigned t = atomicAdd(ticket, 1u);
    s_last = t == (unsigned)p.splits - 1u;
    if (s_last) *ticket = 0u;                                 // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int g = warp; g < group; g += 4) {
    const float* src = p.partial + (((size_t)b * p.heads + hk * group + g) * p.splits) * kAttPart;
    // lane s holds split s: maximum over the splits, then the weight of each split and the common denominator
    float2 ml = make_float2(-INFINITY, 0.f);
    if (lane < p.splits) ml = __ldcg(reinterpret_cast<const float2*>(src + (size_t)lane * kAttPart));
    float mx = ml.x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float w_own = __expf(ml.x - mx);                    // 0 for empty ranges and for lanes without a split
    float l = w_own * ml.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);   // butterfly: the same sum in every lane, every launch
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
    for (int s = 0; s < p.splits; ++s) {                      // split order: the same sum on every launch
      const float w = __shfl_sync(0xffffffffu, w_own, s);
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)s * kAttPart + 4 + 4 * lane));
      a0 = fmaf(w, v.x, a0); a1 = fmaf(w, v.y, a1); a2 = fmaf(w, v.z, a2); a3 = fmaf(w, v.w, a3);
    }
    const float inv = 1.f / l;
    att_write(p, b, hk * group + g, lane, a0 * inv, a1 * inv, a2 * inv, a3 * inv);
  }
}

// Splits of the key range: ranges of at most 32 keys when the cache is full (one pass of a warp over the tile), but
// no more CTAs than about two per SM and no more than 32 splits (one lane per split in the combination).
static int att_splits(int B, int kv_heads, int max_seq) {
  const int by_len = (max_seq + 31) / 32, by_sm = (2 * 148 + B * kv_heads - 1) / (B * kv_heads);
  const int s = by_len < by_sm ? by_len : by_sm;
  return s < 1 ? 1 : (s > kAttMaxSplits ? kAttMaxSplits : s);
}
static size_t att_partial_bytes(int B, int heads) {
  return ((size_t)B * heads * kAttMaxSplits * kAttPart * sizeof(float) + 255) / 256 * 256;
}

}  // namespace bqq

extern "C" size_t bqq_attention_decode_workspace_bytes(int B, int heads, int kv_heads) {
  using namespace bqq;
  if (B < 1 || heads < 1 || kv_heads < 1) return 0;
  return 256 * (((size_t)B * kv_heads * sizeof(unsigned) + 255) / 256) + att_partial_bytes(B, heads);
}

static int attention_launch(const void* qkv, int64_t ld_qkv, void* k_cache, void* v_cache, int64_t ld_cache,
                            int max_seq, const void* cos_table, const void* sin_table, const int32_t* lens,
                            int B, int heads, int kv_heads, int head_dim, int dtype, void* out, int64_t ld_out,
                            void* workspace, size_t workspace_bytes, void* stream, const BqqPeerGroup* peer,
                            void* gathered, int64_t ld_gathered) {
  using namespace bqq;
  if (!qkv || !k_cache || !v_cache || !cos_table || !sin_table || !lens || !out || !workspace) return BQQ_ERR_NULL;
  if (B < 1 || heads < 1 || kv_heads < 1 || max_seq < 1 || heads % kv_heads != 0) return BQQ_ERR_BAD_SHAPE;
  if (head_dim != kAttDim || heads / kv_heads > kAttMaxGroup || B > 65535 || kv_heads > 65535) return BQQ_ERR_UNSUPPORTED;
  if (dtype != BQQ_BF16) return BQQ_ERR_DTYPE;
  if (workspace_bytes < bqq_attention_decode_workspace_bytes(B, heads, kv_heads)) return BQQ_ERR_WORKSPACE;
  if (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out | (uintptr_t)workspace) & 15) return BQQ_ERR_MISALIGNED;
  if ((ld_qkv | ld_cache | ld_out) & 7) return BQQ_ERR_MISALIGNED;
  AttParams p;
  memset(&p, 0, sizeof(p));
  p.qkv = reinterpret_cast<const __nv_bfloat16*>(qkv);
  p.ld_qkv = ld_qkv;
  p.kc = reinterpret_cast<__nv_bfloat16*>(k_cache);
  p.vc = reinterpret_cast<__nv_bfloat16*>(v_cache);
  p.ld_cache = ld_cache;
  p.cosv = reinterpret_cast<const __nv_bfloat16*>(cos_table);
  p.sinv = reinterpret_cast<const __nv_bfloat16*>(sin_table);
  p.lens = lens;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  p.tickets = reinterpret_cast<unsigned*>(workspace);
  p.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256 * (((size_t)B * kv_heads * sizeof(unsigned) + 255) / 256));
  p.heads = heads; p.kv_heads = kv_heads; p.max_seq = max_seq;
  p.splits = att_splits(B, kv_heads, max_seq);
  p.scale = 1.f / sqrtf((float)head_dim);
  int recv_x = 0;
  if (peer) {
    if (!gathered) return BQQ_ERR_NULL;
    if (peer->world < 1 || peer->world > BQQ_MAX_PEERS || peer->rank < 0 || peer->rank >= peer->world) return BQQ_ERR_BAD_SHAPE;
    const size_t row_bytes = (size_t)heads * kAttDim * 2;
    if ((size_t)B * row_bytes * peer->world > peer->gather_bytes) return BQQ_ERR_WORKSPACE;
    if (ld_gathered < (int64_t)heads * kAttDim * peer->world) return BQQ_ERR_BAD_SHAPE;
    if (((uintptr_t)gathered & 3) || (ld_gathered & 1)) return BQQ_ERR_MISALIGNED;
    for (int q = 0; q < peer->world; ++q) {
      if (!peer->regions[q]) return BQQ_ERR_NULL;
      p.peer_regions[q] = reinterpret_cast<uint8_t*>(peer->regions[q]);
    }
    p.peer_world = peer->world;
    p.peer_rank = peer->rank;
    p.peer_half = peer_half_bytes(peer->gather_bytes);
    p.peer_wait = peer->wait_cycles ? (long long)peer->wait_cycles : 2000000000LL;
    p.peer_out = reinterpret_cast<uint32_t*>(gathered);
    p.peer_ld_out = ld_gathered / 2;
    // receiving CTAs: about one thread per two words of the gathered rows, spread over the (kv head, sequence) columns
    const long long words = (long long)B * heads * (kAttDim / 2) * peer->world;
    const long long cols = (long long)kv_heads * B;
    recv_x = (int)std::min<long long>(8, std::max<long long>(1, (words / 2 + kAttThreads * cols - 1) / (kAttThreads * cols)));
  }
  const size_t smem = (size_t)2 * kAttTile * kAttRow + (size_t)(heads / kv_heads) * kAttDim * sizeof(float);
  if (cudaFuncSetAttribute(bqq_attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return BQQ_ERR_CUDA;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.splits + recv_x, kv_heads, B);
  cfg.blockDim = dim3(kAttThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, bqq_attention_decode_kernel, p) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return launch_status();
}

extern "C" int bqq_attention_decode(const void* qkv, int64_t ld_qkv, void* k_cache, void* v_cache, int64_t ld_cache,
                                    int max_seq, const void* cos_table, const void* sin_table, const int32_t* lens,
                                    int B, int heads, int kv_heads, int head_dim, int dtype, void* out, int64_t ld_out,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  return attention_launch(qkv, ld_qkv, k_cache, v_cache, ld_cache, max_seq, cos_table, sin_table, lens, B, heads, kv_heads,
                          head_dim, dtype, out, ld_out, workspace, workspace_bytes, stream, nullptr, nullptr, 0);
}

extern "C" int bqq_attention_decode_gathered(const BqqPeerGroup* group, const void* qkv, int64_t ld_qkv, void* k_cache,
                                             void* v_cache, int64_t ld_cache, int max_seq, const void* cos_table,
                                             const void* sin_table, const int32_t* lens, int B, int heads, int kv_heads,
                                             int head_dim, int dtype, void* out_local, int64_t ld_out, void* gathered,
                                             int64_t ld_gathered, void* workspace, size_t workspace_bytes, void* stream) {
  if (!group) return BQQ_ERR_NULL;
  return attention_launch(qkv, ld_qkv, k_cache, v_cache, ld_cache, max_seq, cos_table, sin_table, lens, B, heads, kv_heads,
                          head_dim, dtype, out_local, ld_out, workspace, workspace_bytes, stream, group, gathered, ld_gathered);
}
