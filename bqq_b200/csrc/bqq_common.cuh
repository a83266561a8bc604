// Shared geometry, element-type helpers and launch checks for the bqq_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "bqq_b200.h"

namespace bqq {

constexpr int kGroup = 4;  // patch-bits interleaved in one 128-bit lane load

// Derived sizes of the packed planes of one layer.
struct Geom {
  int bw, rw, cw, P, Q, r;
  int QW, RW, RP, PP;  // words per Z row / Y row, padded Z rows / Y rows
  int NPB, NS;         // patch-bits per row patch, super-groups per row patch
  __host__ __device__ Geom() {}
  __host__ __device__ explicit Geom(const BqqDims& d)
      : bw(d.bw), rw(d.rw), cw(d.cw), P(d.P), Q(d.Q), r(d.r) {
    QW = (Q + 31) / 32;
    RW = (r + 31) / 32;
    RP = RW * 32;
    PP = ((P + 31) / 32) * 32;
    NPB = cw * bw;
    NS = (NPB + kGroup - 1) / kGroup;
  }
  __host__ __device__ size_t z_words_per_sg() const { return (size_t)QW * RP * kGroup; }
  __host__ __device__ size_t y_words_per_sg() const { return (size_t)RW * PP * kGroup; }
  __host__ __device__ size_t z_words() const { return (size_t)rw * NS * z_words_per_sg(); }
  __host__ __device__ size_t y_words() const { return (size_t)rw * NS * y_words_per_sg(); }
  // per patch-bit records (a,b,c,d) followed by a 4-float trailer:
  // [0] = max(|a|+|b|+|c|), [1] = max|d| over the layer (bound on |W| = bw*r*[0] + [1])
  __host__ __device__ size_t coef_records() const { return (size_t)rw * NS * kGroup; }
  __host__ __device__ size_t coef_floats() const { return coef_records() * 4 + 4; }
  __host__ __device__ int out_features() const { return rw * P; }
  __host__ __device__ int in_features() const { return cw * Q; }
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

// Load one element of type code `dt` as float.
__device__ __forceinline__ float load_as_float(const void* p, size_t idx, int dt) {
  if (dt == BQQ_F32) return reinterpret_cast<const float*>(p)[idx];
  if (dt == BQQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
  return __half2float(reinterpret_cast<const __half*>(p)[idx]);
}

__device__ __forceinline__ void store_from_float(void* p, size_t idx, int dt, float v) {
  if (dt == BQQ_F32) reinterpret_cast<float*>(p)[idx] = v;
  else if (dt == BQQ_BF16) reinterpret_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[idx] = __float2half_rn(v);
}

// Power-of-two scale that maps a bound on |W| to at most 2^14 (fp16-safe range).
// `trailer` is the 4-float tail of the coefficient buffer, mult = bw * r.
__device__ __forceinline__ float w_scale_from_trailer(const float* trailer, float mult) {
  const float bound = fmaf(mult, __ldg(trailer), __ldg(trailer + 1));
  if (!(bound > 0.f) || !isfinite(bound)) return 1.f;
  int e;
  frexpf(bound, &e);                 // bound = f * 2^e, f in [0.5, 1)
  int s = 14 - e;
  s = max(-100, min(100, s));
  return exp2f((float)s);
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? BQQ_OK : BQQ_ERR_CUDA;
}

// Entry points implemented in the other translation units.
int decode_launch(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                  int y_dtype, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t stream);
size_t decode_workspace_bytes(const BqqDims* dims, int M);
int reconstruct_launch(const BqqLayer* layer, void* W, int w_dtype, float scale, cudaStream_t stream);
int prefill_launch(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                   int y_dtype, int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t stream);
size_t prefill_workspace_bytes(const BqqDims* dims, int M);

}  // namespace bqq
