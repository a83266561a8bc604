// Decode kernel template and its per-batch-tile launcher (see bqq_decode.cu for
// the algorithm).  Instantiated once per batch tile MT in bqq_decode_mt*.cu so
// the translation units compile in parallel.
#pragma once
#include "bqq_common.cuh"

namespace bqq {

constexpr int kNumSM = 148;
constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;

struct DecodePlan {
  int MT;        // rows of X per CTA
  int mtiles;    // ceil(M / MT)
  int splits;    // CTAs per (row patch, M tile)
  int sgps;      // super-groups per split
  int JC;        // col patches staged per CTA
  int PCK;       // 32-row chunks of Y the kernel variant covers (1, 2 or 4)
  size_t smem;   // dynamic shared memory bytes
  size_t partial_floats;
  size_t counter_words;
};

struct DecodeParams {
  const uint4* zp;
  const uint4* yp;
  const float4* coef;
  const void* x;
  void* y;
  const void* bias;
  float* partial;
  unsigned* counters;
  int64_t ldx, ldy;
  int x_dtype, y_dtype, bias_dtype;
  int M, bw, rw, cw, P, Q, QW, NPB, NS;
  int PPg;                   // padded Y rows of the planes (row pitch of a Y word block)
  int splits, sgps, JC, mtiles;
};

__device__ __forceinline__ uint32_t pick(const uint4& v, int sub) {
  return sub == 0 ? v.x : (sub == 1 ? v.y : (sub == 2 ? v.z : v.w));
}

template <int MT, int RW, int PC>
__global__ void __launch_bounds__(kDecodeThreads)
bqq_decode_kernel(const DecodeParams p) {
  const int QW = p.QW;
  const int QP = QW * 32;
  constexpr int RP = RW * 32;
  constexpr int PP = PC * 32;
  extern __shared__ __align__(16) float smem[];
  float* xs = smem;                                   // [JC][MT][QP]
  float* xsum = xs + (size_t)p.JC * MT * QP;          // [JC][MT]
  float* us = xsum + (((size_t)p.JC * MT + 3) & ~(size_t)3);   // [warps][MT][RP], 16-byte aligned
  float* red = us + kDecodeWarps * MT * RP;           // [warps][MT][PP]

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int i = blockIdx.x / p.splits;
  const int split = blockIdx.x % p.splits;
  const int m0 = blockIdx.y * MT;

  const int s0 = split * p.sgps;
  const int s1 = min(p.NS, s0 + p.sgps);
  const int j0 = (s0 * kGroup) / p.bw;

  // ---- stage x (as fp32) and per-col-patch sums -----------------------------
  for (int idx = tid; idx < p.JC * MT * QP; idx += kDecodeThreads) {
    int q = idx % QP;
    int m = (idx / QP) % MT;
    int j = j0 + idx / (QP * MT);
    float v = 0.f;
    if (j < p.cw && q < p.Q && m0 + m < p.M)
      v = load_as_float(p.x, (size_t)(m0 + m) * p.ldx + (size_t)j * p.Q + q, p.x_dtype);
    xs[idx] = v;
  }
  __syncthreads();
  for (int pair = warp; pair < p.JC * MT; pair += kDecodeWarps) {
    float s = 0.f;
    for (int w = 0; w < QW; ++w) s += xs[(size_t)pair * QP + w * 32 + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) xsum[pair] = s;
  }
  __syncthreads();

  float acc[PC][MT];
  float cacc[MT];
  float dacc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    cacc[m] = 0.f;
    dacc[m] = 0.f;
#pragma unroll
    for (int pc = 0; pc < PC; ++pc) acc[pc][m] = 0.f;
  }
  float* my_us = us + warp * MT * RP;

  for (int s = s0 + warp; s < s1; s += kDecodeWarps) {
    const size_t sg = (size_t)i * p.NS + s;
    uint4 zw[RW];      // word qw = 0 of each Z row chunk; further words are fetched in the q loop
    uint4 yw[PC][RW];
#pragma unroll
    for (int rc = 0; rc < RW; ++rc) zw[rc] = __ldg(p.zp + (sg * QW) * RP + rc * 32 + lane);
#pragma unroll
    for (int pc = 0; pc < PC; ++pc)
#pragma unroll
      for (int kw = 0; kw < RW; ++kw)
        yw[pc][kw] = pc * 32 < p.PPg ? __ldg(p.yp + (sg * RW + kw) * p.PPg + pc * 32 + lane)
                                     : make_uint4(0u, 0u, 0u, 0u);
    float4 cf[kGroup];
#pragma unroll
    for (int sub = 0; sub < kGroup; ++sub) cf[sub] = __ldg(p.coef + sg * kGroup + sub);

#pragma unroll
    for (int sub = 0; sub < kGroup; ++sub) {
      int n = s * kGroup + sub;
      int j = min(n / p.bw, p.cw - 1);   // padding patch-bits have zero planes and coefficients
      const float* xj = xs + (size_t)(j - j0) * MT * QP;
      const float* xsj = xsum + (size_t)(j - j0) * MT;
      const float4 co = cf[sub];

      // ---- first contraction: lane k, t_k = sum_q Z[k,q] x[q] ---------------
#pragma unroll
      for (int rc = 0; rc < RW; ++rc) {
        float t[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) t[m] = 0.f;
        for (int qw = 0; qw < QW; ++qw) {
          const uint32_t w = pick(qw == 0 ? zw[rc] : __ldg(p.zp + (sg * QW + qw) * RP + rc * 32 + lane), sub);
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              const float4 xv = *reinterpret_cast<const float4*>(xj + m * QP + qw * 32 + q4 * 4);
              if (w & (1u << (q4 * 4 + 0))) t[m] += xv.x;
              if (w & (1u << (q4 * 4 + 1))) t[m] += xv.y;
              if (w & (1u << (q4 * 4 + 2))) t[m] += xv.z;
              if (w & (1u << (q4 * 4 + 3))) t[m] += xv.w;
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float xs_m = xsj[m];
          cacc[m] = fmaf(co.z, t[m], cacc[m]);
          my_us[m * RP + rc * 32 + lane] = fmaf(co.x, t[m], co.y * xs_m);
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) dacc[m] = fmaf(co.w, xsj[m], dacc[m]);
      __syncwarp();

      // ---- second contraction: lane p, y_p += sum_k Y[p,k] u_k -------------
#pragma unroll
      for (int kw = 0; kw < RW; ++kw) {
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const float4 uv = *reinterpret_cast<const float4*>(my_us + m * RP + kw * 32 + k4 * 4);
#pragma unroll
            for (int pc = 0; pc < PC; ++pc) {
              const uint32_t w = pick(yw[pc][kw], sub);
              if (w & (1u << (k4 * 4 + 0))) acc[pc][m] += uv.x;
              if (w & (1u << (k4 * 4 + 1))) acc[pc][m] += uv.y;
              if (w & (1u << (k4 * 4 + 2))) acc[pc][m] += uv.z;
              if (w & (1u << (k4 * 4 + 3))) acc[pc][m] += uv.w;
            }
          }
        }
      }
      __syncwarp();
    }
  }

  // ---- fold the c and d terms, reduce across the CTA's warps ---------------
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float cs = cacc[m];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cs += __shfl_xor_sync(0xffffffffu, cs, o);
    cs += dacc[m];
#pragma unroll
    for (int pc = 0; pc < PC; ++pc) red[(warp * MT + m) * PP + pc * 32 + lane] = acc[pc][m] + cs;
  }
  __syncthreads();

  const int out_stride = p.rw * PP;   // floats per (split, m) row in the partial buffer
  if (p.splits == 1) {
    for (int idx = tid; idx < MT * PP; idx += kDecodeThreads) {
      int m = idx / PP, pp = idx % PP;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kDecodeWarps; ++w) v += red[(w * MT + m) * PP + pp];
      if (pp < p.P && m0 + m < p.M) {
        int o = i * p.P + pp;
        if (p.bias) v += load_as_float(p.bias, o, p.bias_dtype);
        store_from_float(p.y, (size_t)(m0 + m) * p.ldy + o, p.y_dtype, v);
      }
    }
    return;
  }

  const int mrows = p.mtiles * MT;
  for (int idx = tid; idx < MT * PP; idx += kDecodeThreads) {
    int m = idx / PP, pp = idx % PP;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) v += red[(w * MT + m) * PP + pp];
    p.partial[((size_t)split * mrows + m0 + m) * out_stride + i * PP + pp] = v;
  }
  __threadfence();
  __syncthreads();
  __shared__ unsigned ticket;
  if (tid == 0) ticket = atomicAdd(p.counters + i * p.mtiles + blockIdx.y, 1u);
  __syncthreads();
  if (ticket != (unsigned)(p.splits - 1)) return;
  __threadfence();
  for (int idx = tid; idx < MT * PP; idx += kDecodeThreads) {
    int m = idx / PP, pp = idx % PP;
    if (pp < p.P && m0 + m < p.M) {
      float v = 0.f;
      for (int sp = 0; sp < p.splits; ++sp)
        v += __ldcg(p.partial + ((size_t)sp * mrows + m0 + m) * out_stride + i * PP + pp);
      int o = i * p.P + pp;
      if (p.bias) v += load_as_float(p.bias, o, p.bias_dtype);
      store_from_float(p.y, (size_t)(m0 + m) * p.ldy + o, p.y_dtype, v);
    }
  }
  if (tid == 0) p.counters[i * p.mtiles + blockIdx.y] = 0u;   // ready for the next call
}

template <int MT, int RW, int PC>
static int launch_one(const DecodeParams& p, const DecodePlan& pl, cudaStream_t st) {
  auto kern = bqq_decode_kernel<MT, RW, PC>;
  if (pl.smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess)
      return BQQ_ERR_CUDA;
  }
  dim3 grid(p.rw * p.splits, pl.mtiles);
  kern<<<grid, kDecodeThreads, pl.smem, st>>>(p);
  return launch_status();
}

template <int MT>
int decode_launch_mt(const DecodeParams& p, const DecodePlan& pl, int RW, int PC, cudaStream_t st) {
  if (RW == 1) {
    if (PC == 1) return launch_one<MT, 1, 1>(p, pl, st);
    if (PC == 2) return launch_one<MT, 1, 2>(p, pl, st);
    if (PC <= 4) return launch_one<MT, 1, 4>(p, pl, st);
  } else if (RW == 2) {
    if (PC == 1) return launch_one<MT, 2, 1>(p, pl, st);
    if (PC == 2) return launch_one<MT, 2, 2>(p, pl, st);
    if (PC <= 4) return launch_one<MT, 2, 4>(p, pl, st);
  }
  return BQQ_ERR_UNSUPPORTED;
}

}  // namespace bqq
