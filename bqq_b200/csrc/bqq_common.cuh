// Shared geometry, plane-layout arithmetic, element-type helpers and launch
// checks for the bqq_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bqq_b200.h"

namespace bqq {

constexpr int kGroup = 4;  // col patches interleaved in one 128-bit lane load

// Derived sizes of the packed planes of one layer.
//
// Patches are padded to PT x QT x RT blocks of 32 (rows of Y, columns of Z,
// rank).  For a row patch i the super-group s = b*JG + jg holds col patches
// j = 4*jg + sub of bit layer b.  Word order:
//   Z [rw][NS][RT][QT][32 lanes][4 sub]     Y [rw][NS][PT][RT][32 lanes][4 sub]
// Lane = 4*g + t.  Bits inside a word (fragment order of the int8 tensor-core
// operand the decode kernel expands with byte masks):
//   Z bit 8e + 4qh + rr = Z[k = 32rt + 4g + rr][q = 32qt + 16qh + 4t + e]
//   Y bit 8e + 4kh + rr = Y[p = 32pt + g + 8rr][k = 32rt + 16kh + 4t + e]
// (the four rows of a Z word are four consecutive ranks: the lane that finishes them in the decode kernel
// owns exactly one B-operand word of the second contraction, whose k order is that of the Y word's bytes)
struct Geom {
  int bw, rw, cw, P, Q, r;
  int PT, QT, RT;      // 32-blocks of P, Q, r
  int JG, NS;          // col-patch groups per bit layer, super-groups per row patch
  __host__ __device__ Geom() {}
  __host__ __device__ explicit Geom(const BqqDims& d)
      : bw(d.bw), rw(d.rw), cw(d.cw), P(d.P), Q(d.Q), r(d.r) {
    PT = (P + 31) / 32;
    QT = (Q + 31) / 32;
    RT = (r + 31) / 32;
    JG = (cw + kGroup - 1) / kGroup;
    NS = bw * JG;
  }
  __host__ __device__ size_t z_words() const { return (size_t)rw * NS * RT * QT * 32 * kGroup; }
  __host__ __device__ size_t y_words() const { return (size_t)rw * NS * PT * RT * 32 * kGroup; }
  __host__ __device__ int out_features() const { return rw * P; }
  __host__ __device__ int in_features() const { return cw * Q; }

  // word offset and bit position of Z[b,i,j][k][q]
  __host__ __device__ size_t z_word(int b, int i, int j, int k, int q, int* bit) const {
    const int rt = k >> 5, g = (k >> 2) & 7, rr = k & 3;
    const int qt = q >> 5, qh = (q >> 4) & 1, t = (q >> 2) & 3, e = q & 3;
    *bit = 8 * e + 4 * qh + rr;
    const size_t s = (size_t)b * JG + j / kGroup;
    return (((((size_t)i * NS + s) * RT + rt) * QT + qt) * 32 + (4 * g + t)) * kGroup + (j % kGroup);
  }
  // word offset and bit position of Y[b,i,j][p][k]
  __host__ __device__ size_t y_word(int b, int i, int j, int p, int k, int* bit) const {
    const int pt = p >> 5, rr = (p >> 3) & 3, g = p & 7;
    const int rt = k >> 5, kh = (k >> 4) & 1, t = (k >> 2) & 3, e = k & 3;
    *bit = 8 * e + 4 * kh + rr;
    const size_t s = (size_t)b * JG + j / kGroup;
    return (((((size_t)i * NS + s) * PT + pt) * RT + rt) * 32 + (4 * g + t)) * kGroup + (j % kGroup);
  }
};

inline int check_dims(const BqqDims* d) {
  if (!d) return BQQ_ERR_NULL;
  if (d->bw <= 0 || d->rw <= 0 || d->cw <= 0 || d->P <= 0 || d->Q <= 0 || d->r <= 0)
    return BQQ_ERR_BAD_SHAPE;
  if (d->P > BQQ_MAX_P || d->Q > BQQ_MAX_Q || d->r > BQQ_MAX_R) return BQQ_ERR_UNSUPPORTED;
  if ((int64_t)d->rw * d->P > (1 << 30) || (int64_t)d->cw * d->Q > (1 << 30)) return BQQ_ERR_UNSUPPORTED;
  return BQQ_OK;
}

inline int dtype_size(int dt) {
  switch (dt) {
    case BQQ_F32: return 4;
    case BQQ_BF16: return 2;
    case BQQ_F16: return 2;
    default: return 0;
  }
}

// Load one element of type code `dt` as float.  Plain loads on purpose: a read-only
// (__ldg) load may be hoisted above the guard that protects it, and callers guard
// optional (possibly NULL) pointers and ragged edges with ordinary branches.
__device__ __forceinline__ float load_as_float(const void* p, size_t idx, int dt) {
  if (dt == BQQ_F32) return reinterpret_cast<const float*>(p)[idx];
  if (dt == BQQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  return __half2float(reinterpret_cast<const __half*>(p)[idx]);
}

// 128-bit streaming load of plane words (read once, keep out of L1).  Volatile asm so
// that it stays behind the bounds test of its caller.
__device__ __forceinline__ uint4 load_plane_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ void store_from_float(void* p, size_t idx, int dt, float v) {
  if (dt == BQQ_F32) reinterpret_cast<float*>(p)[idx] = v;
  else if (dt == BQQ_BF16) reinterpret_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[idx] = __float2half_rn(v);
}

// Round a value to the 16-bit type `dt` and back (used to split a weight into hi + lo parts).
__device__ __forceinline__ float round_to(float v, int dt) {
  if (dt == BQQ_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  if (dt == BQQ_F16) return __half2float(__float2half_rn(v));
  return v;
}

// Power-of-two scale that maps a bound on |W| to at most 2^14 (fp16-safe range).
// bound_parts = {max(|a|+|b|+|c|), max|d|}; |W| <= mult * parts[0] + parts[1], mult = bw * r.
__device__ __forceinline__ float w_scale_from_bound(const float* bound_parts, float mult) {
  const float bound = fmaf(mult, bound_parts[0], bound_parts[1]);
  if (!(bound > 0.f) || !isfinite(bound)) return 1.f;
  int e;
  frexpf(bound, &e);                 // bound = f * 2^e, f in [0.5, 1)
  int s = 14 - e;
  s = max(-100, min(100, s));
  return exp2f((float)s);
}

// One slot of a peer gather region: (data word, sequence number) as ONE scalar 64-bit access at
// system scope.  A naturally aligned scalar 64-bit access is single-copy atomic; a two-element
// vector access is not promised to be, so the pair never travels as .v2.u32.
__device__ __forceinline__ void peer_slot_store(void* p, uint32_t data, uint32_t seq) {
  const unsigned long long v = (unsigned long long)data | ((unsigned long long)seq << 32);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint2 peer_slot_load(const void* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return make_uint2((uint32_t)v, (uint32_t)(v >> 32));
}

// Roles of a kernel in a chain of programmatic dependent launches (every kernel of such a chain is launched with
// the programmatic stream serialisation attribute; without the attribute the instructions do nothing).
//   kPdlWaitFirst  needs what its predecessors wrote: waits for them to complete, then lets its successor start
//   kPdlOverlap    independent of its predecessor: lets its successor start at once and runs beside its
//                  predecessor; one CTA waits for the predecessor at the very end, so that "this grid has
//                  completed" still implies "everything before it has completed" for whoever waits on it
constexpr int kPdlNone = 0, kPdlWaitFirst = 1, kPdlOverlap = 2;
__device__ __forceinline__ void pdl_enter(int mode) {
  if (mode == kPdlWaitFirst) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (mode != kPdlNone) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_exit(int mode) {
  if (mode == kPdlOverlap && blockIdx.x == 0 && blockIdx.y == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? BQQ_OK : BQQ_ERR_CUDA;
}

// Entry points implemented in the other translation units.
// `peer` (may be NULL): the decode kernel also stores its outputs into the peers' gather regions
int decode_launch(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                  int y_dtype, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t stream,
                  const BqqPeerGroup* peer = nullptr, const BqqFusion* fusion = nullptr,
                  void* gathered = nullptr, int64_t ld_gathered = 0);   // with `peer`: the gathered rows [M, world * out]
size_t peer_half_bytes(size_t gather_bytes);   // bytes of one half of a peer region's slot area
size_t decode_workspace_bytes(const BqqDims* dims, int M);
constexpr size_t kPeerCtrlBytes = 512;   // control words at the start of a peer gather region (bqq_peer.cu)

int decode_launches(const BqqDims* dims, int M);   // kernels per decode call: 1 or 2
size_t decode_counter_bytes();   // leading part of the decode workspace that must start zeroed
// row patches [i0, i1) only (i1 < 0: all); pdl: role in a chain of programmatic dependent launches
int reconstruct_launch(const BqqLayer* layer, void* W, void* W_lo, int w_dtype, float scale,
                       const float* bound_parts, cudaStream_t stream, int i0 = 0, int i1 = -1, int pdl = kPdlNone);
int coef_bound_launch(const BqqLayer* layer, float* bound_parts, cudaStream_t stream);   // bound_parts zero on entry
int prefill_launch(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                   int y_dtype, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t stream);
size_t prefill_workspace_bytes(const BqqDims* dims, int M);

}  // namespace bqq
