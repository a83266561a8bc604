// Dense weight from packed planes:
//   W[i*P+p, j*Q+q] = sum_b ( a_b popc(Yrow_b[p] & Zcol_b[q]) + b_b popc(Yrow_b[p])
//                             + c_b popc(Zcol_b[q]) ) + d
// i.e. BinaryQuadratic.get_weight (neural_network_compression/src/bqq_modules.py:48-55),
// with the AND+popcount idea of reconstruct_W_kernel (src/bqq_cuda.cu:198-246).
// A warp owns one 32x32 block of one patch: lane l first gathers row l of Y and
// column l of Z (bits over the rank) out of the fragment-ordered plane words, then
// the block is produced row by row so every store is a contiguous 32-element run.
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

__global__ void __launch_bounds__(kReconWarps * 32)
bqq_reconstruct_kernel(const ReconParams p) {
  extern __shared__ uint32_t rsm[];          // [warps][2][bw][RT][32]: row words of Y, column words of Z
  const Geom& g = p.g;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  uint32_t* yrow = rsm + (size_t)warp * 2 * g.bw * g.RT * 32;
  uint32_t* zcol = yrow + (size_t)g.bw * g.RT * 32;
  const float scale = p.bound_parts ? p.scale * w_scale_from_bound(p.bound_parts, (float)(g.bw * g.r)) : p.scale;
  const size_t ldw = (size_t)g.cw * g.Q;

  for (long long task = (long long)blockIdx.x * kReconWarps + warp; task < p.total_tasks;
       task += (long long)gridDim.x * kReconWarps) {
    long long u = task;
    const int qt = (int)(u % g.QT); u /= g.QT;
    const int pt = (int)(u % g.PT); u /= g.PT;
    const int j = (int)(u % g.cw);
    const int i = (int)(u / g.cw);
    const int pl = 32 * pt + lane;           // this lane's row of Y
    const int ql = 32 * qt + lane;           // this lane's column of Z

    float colterm = load_as_float(p.d, (size_t)i * g.cw + j, p.coef_dtype);   // d + sum_b c_b popc(Zcol_b)
    float rowterm = 0.f;                                                      // sum_b b_b popc(Yrow_b), lane = row
    for (int b = 0; b < g.bw; ++b) {
      const size_t ci = ((size_t)b * g.rw + i) * g.cw + j;
      const float cb = load_as_float(p.b, ci, p.coef_dtype);
      const float cc = load_as_float(p.c, ci, p.coef_dtype);
      int ys = 0, zs = 0;
      for (int rt = 0; rt < g.RT; ++rt) {
        uint32_t yr = 0, zc = 0;
        // row pl of Y: ranks 32rt + 16kh + 4t + e live in the words of lanes 4*(pl&7) + t
        for (int t = 0; t < 4; ++t) {
          int bit;
          const uint32_t w = p.yp[g.y_word(b, i, j, pl, 32 * rt + 4 * t, &bit)];
          const int rr = (pl >> 3) & 3;
#pragma unroll
          for (int kh = 0; kh < 2; ++kh)
#pragma unroll
            for (int e = 0; e < 4; ++e) yr |= ((w >> (8 * e + 4 * kh + rr)) & 1u) << (16 * kh + 4 * t + e);
        }
        // column ql of Z: ranks 32rt + gg + 8rr live in the words of lanes 4*gg + t(ql)
        for (int gg = 0; gg < 8; ++gg) {
          int bit;
          const uint32_t w = p.zp[g.z_word(b, i, j, 32 * rt + gg, ql, &bit)];
          const int base = bit & ~3;          // 8e + 4qh
#pragma unroll
          for (int rr = 0; rr < 4; ++rr) zc |= ((w >> (base + rr)) & 1u) << (gg + 8 * rr);
        }
        yrow[(b * g.RT + rt) * 32 + lane] = yr;
        zcol[(b * g.RT + rt) * 32 + lane] = zc;
        ys += __popc(yr);
        zs += __popc(zc);
      }
      rowterm = fmaf(cb, (float)ys, rowterm);
      colterm = fmaf(cc, (float)zs, colterm);
    }
    __syncwarp();

    const int prow_max = min(32, g.P - 32 * pt);
    for (int pp = 0; pp < prow_max; ++pp) {
      float acc = colterm + __shfl_sync(0xffffffffu, rowterm, pp);
      for (int b = 0; b < g.bw; ++b) {
        const float ca = load_as_float(p.a, ((size_t)b * g.rw + i) * g.cw + j, p.coef_dtype);
        int core = 0;
        for (int rt = 0; rt < g.RT; ++rt)
          core += __popc(yrow[(b * g.RT + rt) * 32 + pp] & zcol[(b * g.RT + rt) * 32 + lane]);
        acc = fmaf(ca, (float)core, acc);
      }
      if (ql < g.Q) {
        const size_t at = (size_t)(i * g.P + 32 * pt + pp) * ldw + (size_t)j * g.Q + ql;
        const float w = acc * scale;
        store_from_float(p.W, at, p.w_dtype, w);
        if (p.W_lo) store_from_float(p.W_lo, at, p.w_dtype, w - round_to(w, p.w_dtype));
      }
    }
    __syncwarp();
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
  const size_t smem = (size_t)kReconWarps * 2 * p.g.bw * p.g.RT * 32 * sizeof(uint32_t);
  if (smem > 48 * 1024) return BQQ_ERR_UNSUPPORTED;
  long long blocks = (p.total_tasks + kReconWarps - 1) / kReconWarps;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  bqq_reconstruct_kernel<<<(int)blocks, kReconWarps * 32, smem, st>>>(p);
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
