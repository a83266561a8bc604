// Dense weight from packed planes:
//   W[i*P+p, j*Q+q] = sum_b ( a_b popc(Yrow_b[p] & Zcol_b[q]) + b_b popc(Yrow_b[p])
//                             + c_b popc(Zcol_b[q]) ) + d
// i.e. BinaryQuadratic.get_weight (neural_network_compression/src/bqq_modules.py:48-55),
// with the AND+popcount idea of reconstruct_W_kernel (src/bqq_cuda.cu:198-246).
// A warp owns one 32x32 block of one patch: lane l first gathers row l of Y and
// column l of Z (bits over the rank) out of the fragment-ordered plane words with
// nibble/byte multiply tricks, then the block is produced row by row (row words
// broadcast by shuffle, accumulators in registers) so every store is a contiguous
// 32-element run.
#include "bqq_common.cuh"

namespace bqq {

constexpr int kReconWarps = 4;

struct ReconParams {
  const uint32_t* zp;
  const uint32_t* yp;
  const void *a, *b, *c, *d;
  void* W;
  void* W_lo;                  // optional second part: W - round(W), same type and layout
  const float* bound_parts;    // optional: entries are also scaled by w_scale_from_bound
  float scale;
  int coef_dtype, w_dtype;
  Geom g;
  long long total_tasks;       // rw * cw * PT * QT
};

// Spread the 4 low bits of n to the least significant bits of 4 bytes.
__device__ __forceinline__ uint32_t nibble_to_bytes(uint32_t n) { return (n * 0x00204081u) & 0x01010101u; }
// Collect the least significant bits of 4 bytes into a nibble (byte e -> bit e).
__device__ __forceinline__ uint32_t bytes_to_nibble(uint32_t y) { return ((y & 0x01010101u) * 0x01020408u) >> 24; }

// element type of W as a compile-time choice: the store loop is the bulk of the kernel
template <int DT> struct WType;
template <> struct WType<BQQ_F32> {
  using T = float;
  static __device__ __forceinline__ T cvt(float v) { return v; }
  static __device__ __forceinline__ float back(T v) { return v; }
};
template <> struct WType<BQQ_BF16> {
  using T = __nv_bfloat16;
  static __device__ __forceinline__ T cvt(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float back(T v) { return __bfloat162float(v); }
};
template <> struct WType<BQQ_F16> {
  using T = __half;
  static __device__ __forceinline__ T cvt(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float back(T v) { return __half2float(v); }
};

template <int RT, int DT, bool LO>
__global__ void __launch_bounds__(kReconWarps * 32)
bqq_reconstruct_kernel(const ReconParams p) {
  using WT = typename WType<DT>::T;
  const Geom& g = p.g;
  const int lane = threadIdx.x & 31;
  const float scale = p.bound_parts ? p.scale * w_scale_from_bound(p.bound_parts, (float)(g.bw * g.r)) : p.scale;
  const size_t ldw = (size_t)g.cw * g.Q;
  // this lane as a row of Y (p = 32pt + lane = 32pt + gp + 8rp) and as a column of Z
  // (q = 32qt + lane = 32qt + 16qh + 4tq + eq)
  const int gp = lane & 7, rp = lane >> 3;
  const int qh = (lane >> 4) & 1, tq = (lane >> 2) & 3, eq = lane & 3;
  const int zbase = 8 * eq + 4 * qh;

  for (long long task = (long long)blockIdx.x * kReconWarps + (threadIdx.x >> 5); task < p.total_tasks;
       task += (long long)gridDim.x * kReconWarps) {
    long long u = task;
    const int qt = (int)(u % g.QT); u /= g.QT;
    const int pt = (int)(u % g.PT); u /= g.PT;
    const int j = (int)(u % g.cw);
    const int i = (int)(u / g.cw);
    const int sub = j % kGroup;

    float acc[32];
#pragma unroll
    for (int pp = 0; pp < 32; ++pp) acc[pp] = 0.f;
    float colterm = load_as_float(p.d, (size_t)i * g.cw + j, p.coef_dtype);   // d + sum_b c_b popc(Zcol_b)
    float rowterm = 0.f;                                                      // sum_b b_b popc(Yrow_b), lane = row
    for (int b = 0; b < g.bw; ++b) {
      const size_t ci = ((size_t)b * g.rw + i) * g.cw + j;
      const float ca = load_as_float(p.a, ci, p.coef_dtype);
      const float cb = load_as_float(p.b, ci, p.coef_dtype);
      const float cc = load_as_float(p.c, ci, p.coef_dtype);
      const size_t sg = (size_t)i * g.NS + (size_t)b * g.JG + j / kGroup;
      uint32_t yr[RT], zc[RT];
      int ys = 0, zs = 0;
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        yr[rt] = 0u;
        zc[rt] = 0u;
        if (rt < g.RT) {
          // row of Y: ranks 16kh + 4t + e sit in the words of lanes 4*gp + t at bits 8e + 4kh + rp
          const uint32_t* yb = p.yp + (((sg * g.PT + pt) * g.RT + rt) * 32) * kGroup + sub;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const uint32_t w = yb[(4 * gp + t) * kGroup] >> rp;
            yr[rt] |= bytes_to_nibble(w) << (4 * t);
            yr[rt] |= bytes_to_nibble(w >> 4) << (16 + 4 * t);
          }
          // column of Z: ranks gg + 8rr sit in the words of lanes 4*gg + tq at bits 8eq + 4qh + rr
          const uint32_t* zb = p.zp + (((sg * g.RT + rt) * g.QT + qt) * 32) * kGroup + sub;
#pragma unroll
          for (int gg = 0; gg < 8; ++gg) {
            const uint32_t w = zb[(4 * gg + tq) * kGroup] >> zbase;
            zc[rt] |= nibble_to_bytes(w & 0xFu) << gg;
          }
          ys += __popc(yr[rt]);
          zs += __popc(zc[rt]);
        }
      }
      rowterm = fmaf(cb, (float)ys, rowterm);
      colterm = fmaf(cc, (float)zs, colterm);
#pragma unroll
      for (int pp = 0; pp < 32; ++pp) {
        int core = 0;
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) core += __popc(__shfl_sync(0xffffffffu, yr[rt], pp) & zc[rt]);
        // int -> float on the FP32 pipe (core <= 64): 2^23 + core as a bit pattern, minus 2^23
        acc[pp] = fmaf(ca, __int_as_float(0x4B000000 | core) - 8388608.f, acc[pp]);
      }
    }
    const int prow_max = min(32, g.P - 32 * pt);
    const int ql = 32 * qt + lane;
    const size_t at0 = (size_t)(i * g.P + 32 * pt) * ldw + (size_t)j * g.Q + ql;
    WT* wrow = reinterpret_cast<WT*>(p.W) + at0;
    WT* lrow = LO ? reinterpret_cast<WT*>(p.W_lo) + at0 : nullptr;
    const bool col_ok = ql < g.Q;
#pragma unroll
    for (int pp = 0; pp < 32; ++pp) {
      const float rterm = __shfl_sync(0xffffffffu, rowterm, pp);
      if (pp < prow_max && col_ok) {
        const float w = (acc[pp] + colterm + rterm) * scale;
        const WT wv = WType<DT>::cvt(w);
        wrow[(size_t)pp * ldw] = wv;
        if (LO) lrow[(size_t)pp * ldw] = WType<DT>::cvt(w - WType<DT>::back(wv));
      }
    }
  }
}

template <int RT>
static void reconstruct_dispatch(const ReconParams& p, int blocks, cudaStream_t st) {
  const int threads = kReconWarps * 32;
  const bool lo = p.W_lo != nullptr;
  if (p.w_dtype == BQQ_F32) bqq_reconstruct_kernel<RT, BQQ_F32, false><<<blocks, threads, 0, st>>>(p);
  else if (p.w_dtype == BQQ_BF16) {
    if (lo) bqq_reconstruct_kernel<RT, BQQ_BF16, true><<<blocks, threads, 0, st>>>(p);
    else bqq_reconstruct_kernel<RT, BQQ_BF16, false><<<blocks, threads, 0, st>>>(p);
  } else {
    if (lo) bqq_reconstruct_kernel<RT, BQQ_F16, true><<<blocks, threads, 0, st>>>(p);
    else bqq_reconstruct_kernel<RT, BQQ_F16, false><<<blocks, threads, 0, st>>>(p);
  }
}

int reconstruct_launch(const BqqLayer* L, void* W, void* W_lo, int w_dtype, float scale, const float* bound_parts,
                       cudaStream_t st) {
  ReconParams p;
  p.g = Geom(L->dims);
  p.zp = L->zplanes; p.yp = L->yplanes;
  p.a = L->a; p.b = L->b; p.c = L->c; p.d = L->d; p.coef_dtype = L->coef_dtype;
  p.W = W; p.W_lo = W_lo; p.scale = scale; p.bound_parts = bound_parts; p.w_dtype = w_dtype;
  p.total_tasks = (long long)p.g.rw * p.g.cw * p.g.PT * p.g.QT;
  long long blocks = (p.total_tasks + kReconWarps - 1) / kReconWarps;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  if (w_dtype == BQQ_F32 && W_lo) return BQQ_ERR_UNSUPPORTED;     // a second part only exists for 16-bit types
  if (p.g.RT == 1) reconstruct_dispatch<1>(p, (int)blocks, st);
  else reconstruct_dispatch<2>(p, (int)blocks, st);
  return launch_status();
}

// bound_parts[0] = max(|a|+|b|+|c|), bound_parts[1] = max|d| (both must be zero on entry)
__global__ void coef_bound_kernel(const void* a, const void* b, const void* c, const void* d, int dt, size_t nabc,
                                  size_t nd, float* bound_parts) {
  float m0 = 0.f, m1 = 0.f;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < nabc; t += (size_t)gridDim.x * blockDim.x)
    m0 = fmaxf(m0, fabsf(load_as_float(a, t, dt)) + fabsf(load_as_float(b, t, dt)) + fabsf(load_as_float(c, t, dt)));
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < nd; t += (size_t)gridDim.x * blockDim.x)
    m1 = fmaxf(m1, fabsf(load_as_float(d, t, dt)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
  }
  if ((threadIdx.x & 31) == 0) {      // non-negative floats order like ints
    atomicMax(reinterpret_cast<int*>(bound_parts), __float_as_int(m0));
    atomicMax(reinterpret_cast<int*>(bound_parts) + 1, __float_as_int(m1));
  }
}

int coef_bound_launch(const BqqLayer* L, float* bound_parts, cudaStream_t st) {
  Geom g(L->dims);
  if (cudaMemsetAsync(bound_parts, 0, 8, st) != cudaSuccess) return BQQ_ERR_CUDA;
  const size_t nabc = (size_t)g.bw * g.rw * g.cw, nd = (size_t)g.rw * g.cw;
  int blocks = (int)((nabc + 255) / 256 < 592 ? (nabc + 255) / 256 : 592);
  coef_bound_kernel<<<blocks, 256, 0, st>>>(L->a, L->b, L->c, L->d, L->coef_dtype, nabc, nd, bound_parts);
  return launch_status();
}

}  // namespace bqq
