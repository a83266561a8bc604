// Dense weight from packed planes:
//   W[i*P+p, j*Q+q] = sum_b ( a_b popc(Yrow_b[p] & Zcol_b[q]) + b_b popc(Yrow_b[p])
//                             + c_b popc(Zcol_b[q]) ) + d
// i.e. BinaryQuadratic.get_weight (neural_network_compression/src/bqq_modules.py:48-55).
// Same AND+popcount idea as reconstruct_W_kernel (src/bqq_cuda.cu:198-246), but a
// warp owns 32 consecutive columns of one patch so every store is a contiguous
// row segment.  The Z planes keep bits over q, so the warp first transposes
// its 32 columns to bits-over-k words with ballots.
#include "bqq_common.cuh"

namespace bqq {

constexpr int kReconWarps = 4;

struct ReconParams {
  const uint32_t* zp;
  const uint32_t* yp;
  const float4* coef;
  void* W;
  void* W_lo;               // optional second part: W - round(W), same type and layout
  const float* trailer;     // optional coefficient trailer: entries are also scaled by w_scale_from_trailer
  float scale;
  int w_dtype;
  int bw, rw, cw, P, Q, r, QW, RW, RP, PP, NS;
  long long total_tasks;    // rw * cw * QW
};

__global__ void __launch_bounds__(kReconWarps * 32)
bqq_reconstruct_kernel(const ReconParams p) {
  extern __shared__ uint32_t zcol_s[];   // [warps][bw][RW][32]
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  uint32_t* zcol = zcol_s + (size_t)warp * p.bw * p.RW * 32;
  const float scale = p.trailer ? p.scale * w_scale_from_trailer(p.trailer, (float)(p.bw * p.r)) : p.scale;
  const size_t ldw = (size_t)p.cw * p.Q;

  for (long long task = (long long)blockIdx.x * kReconWarps + warp; task < p.total_tasks;
       task += (long long)gridDim.x * kReconWarps) {
    const int qw = (int)(task % p.QW);
    const int j = (int)((task / p.QW) % p.cw);
    const int i = (int)(task / ((long long)p.QW * p.cw));
    const int q = qw * 32 + lane;

    // ---- transpose: zcol[b][kw][lane q] = bits over k of column q -------------
    float colterm = 0.f;   // sum_b c_b popc(Zcol_b[q]) + d
    for (int b = 0; b < p.bw; ++b) {
      const int n = j * p.bw + b;
      const size_t sg = (size_t)i * p.NS + n / kGroup;
      const int sub = n % kGroup;
      const float4 co = __ldg(p.coef + sg * kGroup + sub);
      int zs = 0;
      for (int kw = 0; kw < p.RW; ++kw) {
        // lane k holds Z row (kw*32+k), word qw
        const uint32_t zrow = __ldg(p.zp + (((sg * p.QW + qw) * p.RP + kw * 32 + lane) * kGroup + sub));
        uint32_t mine = 0;
#pragma unroll
        for (int qq = 0; qq < 32; ++qq) {
          const uint32_t bal = __ballot_sync(0xffffffffu, (zrow >> qq) & 1u);
          if (lane == qq) mine = bal;
        }
        zcol[(b * p.RW + kw) * 32 + lane] = mine;
        zs += __popc(mine);
      }
      colterm = fmaf(co.z, (float)zs, colterm);
      colterm += co.w;
    }
    __syncwarp();

    // ---- rows of the patch ---------------------------------------------------
    for (int pp = 0; pp < p.P; ++pp) {
      float acc = colterm;
      for (int b = 0; b < p.bw; ++b) {
        const int n = j * p.bw + b;
        const size_t sg = (size_t)i * p.NS + n / kGroup;
        const int sub = n % kGroup;
        const float4 co = __ldg(p.coef + sg * kGroup + sub);
        int core = 0, ys = 0;
        for (int kw = 0; kw < p.RW; ++kw) {
          const uint32_t yrow = __ldg(p.yp + (((sg * p.RW + kw) * p.PP + pp) * kGroup + sub));
          core += __popc(yrow & zcol[(b * p.RW + kw) * 32 + lane]);
          ys += __popc(yrow);
        }
        acc = fmaf(co.x, (float)core, acc);
        acc = fmaf(co.y, (float)ys, acc);
      }
      if (q < p.Q) {
        const size_t at = (size_t)(i * p.P + pp) * ldw + (size_t)j * p.Q + q;
        const float w = acc * scale;
        store_from_float(p.W, at, p.w_dtype, w);
        if (p.W_lo) store_from_float(p.W_lo, at, p.w_dtype, w - load_as_float(p.W, at, p.w_dtype));
      }
    }
    __syncwarp();
  }
}

int reconstruct_launch_dev(const BqqLayer* L, void* W, void* W_lo, int w_dtype, float scale, const float* trailer,
                           cudaStream_t st) {
  Geom g(L->dims);
  ReconParams p;
  p.zp = L->zplanes; p.yp = L->yplanes; p.coef = reinterpret_cast<const float4*>(L->coef);
  p.W = W; p.W_lo = W_lo; p.scale = scale; p.trailer = trailer; p.w_dtype = w_dtype;
  p.bw = g.bw; p.rw = g.rw; p.cw = g.cw; p.P = g.P; p.Q = g.Q; p.r = g.r;
  p.QW = g.QW; p.RW = g.RW; p.RP = g.RP; p.PP = g.PP; p.NS = g.NS;
  p.total_tasks = (long long)g.rw * g.cw * g.QW;
  size_t smem = (size_t)kReconWarps * g.bw * g.RW * 32 * sizeof(uint32_t);
  if (smem > 48 * 1024) return BQQ_ERR_UNSUPPORTED;
  long long blocks = (p.total_tasks + kReconWarps - 1) / kReconWarps;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  bqq_reconstruct_kernel<<<(int)blocks, kReconWarps * 32, smem, st>>>(p);
  return launch_status();
}

int reconstruct_launch(const BqqLayer* L, void* W, int w_dtype, float scale, cudaStream_t st) {
  return reconstruct_launch_dev(L, W, nullptr, w_dtype, scale, nullptr, st);
}

}  // namespace bqq
