// Dense weight from packed planes:
//   W[i*P+p, j*Q+q] = sum_b ( a_b popc(Yrow_b[p] & Zcol_b[q]) + b_b popc(Yrow_b[p])
//                             + c_b popc(Zcol_b[q]) ) + d
// i.e. BinaryQuadratic.get_weight (neural_network_compression/src/bqq_modules.py:48-55); replaces
// reconstruct_W_kernel (src/bqq_cuda.cu:198-246).
// A warp owns one 32x32 block of one patch and forms the counts Y Z on the tensor cores
// (mma.sync m16n8k16, fp16 operands that are 2.0 or zero, fp32 accumulators: the sums are exact).  The Y plane word of a lane is already an A fragment (rows of Y over the rank);
// the Z plane word is a fragment over q whose four rows are four consecutive ranks, exactly the four
// ranks a lane of the B fragment needs for one column: the lane fetches the words of four plane lanes
// (four shuffles) and expands one nibble per rank half and 8-column tile.
// Row and column sums come from two more products with an all-ones operand, so one bit layer costs
// 28 MMAs, 44 FMAs and about 90 integer instructions per warp.
#include <algorithm>

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
  int pairs;                   // 1: two neighbouring entries of a row may be stored as one aligned word
  Geom g;
  int tasks_per_row;           // cw * PT * QT: 32x32 blocks of one row patch
  int i0, i1;                  // row patches [i0, i1) are rebuilt
  // How the launch takes part in a chain of programmatic dependent launches (kPdl* in bqq_common.cuh)
  int pdl;
};

// element type of W as a compile-time choice
template <int DT> struct WType;
template <> struct WType<BQQ_F32> {
  using T = float;
  using T2 = float2;
  static __device__ __forceinline__ T cvt(float v) { return v; }
  static __device__ __forceinline__ T2 cvt2(float v0, float v1) { return make_float2(v0, v1); }
  static __device__ __forceinline__ float back(T v) { return v; }
};
template <> struct WType<BQQ_BF16> {
  using T = __nv_bfloat16;
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ T cvt(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ T2 cvt2(float v0, float v1) { return __floats2bfloat162_rn(v0, v1); }
  static __device__ __forceinline__ float back(T v) { return __bfloat162float(v); }
};
template <> struct WType<BQQ_F16> {
  using T = __half;
  using T2 = __half2;
  static __device__ __forceinline__ T cvt(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ T2 cvt2(float v0, float v1) { return __floats2half2_rn(v0, v1); }
  static __device__ __forceinline__ float back(T v) { return __half2float(v); }
};

// Bits POS + 8 ODD and POS + 8 ODD + 16 of w as two fp16 numbers, each 2.0 (0x4000) or zero: entries ODD and
// ODD + 2 of the four consecutive ranks a plane word holds for one row (column) at in-byte position POS.
template <int POS, int ODD>
__device__ __forceinline__ uint32_t bits_as_half2(uint32_t w) {
  constexpr int src = POS + 8 * ODD;
  return (src <= 14 ? w << (14 - src) : w >> (src - 14)) & 0x40004000u;
}
constexpr uint32_t kOnesHalf2 = 0x3C003C00u;     // 1.0 twice
constexpr float kBitValue = 2.0f;                // value of a set entry

// D = A B (+ D): A 16x16 (rows g and g+8 of a lane), B 16x8 (column g), fp16 operands, fp32 accumulators.
// The order of the 16 entries of k is the same in A and B, so any order serves.
__device__ __forceinline__ void mma_f16_first(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Fragments of rank half KH: rows g + 8 R0 and g + 8 (R0 + 1) of Y, entries {0, 2} and {1, 3} of the lane's ranks
template <int KH, int R0>
__device__ __forceinline__ void y_frag(uint32_t (&a)[4], uint32_t yw) {
  a[0] = bits_as_half2<4 * KH + R0, 0>(yw);
  a[1] = bits_as_half2<4 * KH + R0 + 1, 0>(yw);
  a[2] = bits_as_half2<4 * KH + R0, 1>(yw);
  a[3] = bits_as_half2<4 * KH + R0 + 1, 1>(yw);
}
// B fragment from a nibble m of a Z plane word: bits rr = 0..3 are Z[k0 + rr][q] for the four ranks of one lane of
// the A fragment, whose k order is (0, 2 | 1, 3).  One multiplication moves bit 0 (1) to bit 14 and bit 2 (3) to
// bit 30, the places where an fp16 pair reads 2.0; the other partial products fall outside the mask.
__device__ __forceinline__ void z_frag(uint32_t (&b)[2], uint32_t m) {
  b[0] = (m * 0x10004000u) & 0x40004000u;
  b[1] = (m * 0x08002000u) & 0x40004000u;
}

// First word of Y and of Z (for the lane that reads plane lane `zsrc`) and first coefficient of one 32x32 block.
struct ReconTask {
  const uint32_t* y;
  const uint32_t* z;
  size_t ci;                   // i * cw + j
  int i, j, pt, qt;
};

template <int RT>
__device__ __forceinline__ ReconTask recon_locate(const ReconParams& p, int i, unsigned tj, int lane, int zsrc) {
  const Geom& g = p.g;
  ReconTask t;
  t.i = i;
  t.qt = 0; t.pt = 0; t.j = (int)tj;
  if (g.PT * g.QT != 1) {
    unsigned u = tj;
    t.qt = (int)(u % (unsigned)g.QT); u /= (unsigned)g.QT;
    t.pt = (int)(u % (unsigned)g.PT);
    t.j = (int)(u / (unsigned)g.PT);
  }
  const int sub = t.j % kGroup;
  const size_t sg0 = (size_t)i * g.NS + t.j / kGroup;
  t.y = p.yp + ((sg0 * g.PT + t.pt) * RT * 32 + lane) * kGroup + sub;
  t.z = p.zp + ((sg0 * RT * g.QT + t.qt) * 32 + zsrc) * kGroup + sub;
  t.ci = (size_t)i * g.cw + t.j;
  return t;
}

template <int RT, int DT, bool LO>
__global__ void __launch_bounds__(kReconWarps * 32, 4)
bqq_reconstruct_kernel(const ReconParams p) {
  using WT = typename WType<DT>::T;
  using WT2 = typename WType<DT>::T2;
  const Geom& g = p.g;
  const int lane = threadIdx.x & 31;
  const int g8 = lane >> 2, t4 = lane & 3;
  pdl_enter(p.pdl);
  const float scale = p.bound_parts ? p.scale * w_scale_from_bound(p.bound_parts, (float)(g.bw * g.r)) : p.scale;
  const float s_core = scale / (kBitValue * kBitValue), s_sum = scale / kBitValue;
  const size_t ldw = (size_t)g.cw * g.Q;
  // Z word -> B fragments.  Plane lane 4 gz + tz holds, at bit 8e + 4qh + rr, Z[k = 4 gz + rr][q = 16 qh + 4 tz + e].
  // Lane (n = g8, t = t4) of a B fragment needs, for rank half kh and 8-column tile nt = 2 qh + x, the ranks
  // 16 kh + 4 t + rr of column q = 8 nt + n: the nibble at byte n & 3, half qh, of plane lane
  // 16 kh + 4 t + 2 x + (n >> 2).  It reads the plane word of lane `lane` itself as its own Z word (zsrc = lane).
  const int zsrc = lane;
  const int zfrom = 4 * t4 + (g8 >> 2);               // + 16 kh + 2 x
  const uint32_t zbyte = 0x4440u | (uint32_t)(g8 & 3);   // byte n & 3 into the low byte, zeros above
  const size_t ystep = (size_t)g.JG * g.PT * RT * 32 * kGroup, zstep = (size_t)g.JG * RT * g.QT * 32 * kGroup;
  const size_t cstep = (size_t)g.rw * g.cw;

  // A warp walks blocks first, first + stride, ... of the layer (row patch i, block tj of the row patch); the
  // plane words and coefficients of the next step, and at the end those of the next block, are fetched one step ahead.
  const unsigned tpr = (unsigned)p.tasks_per_row;
  const unsigned stride = gridDim.x * kReconWarps;
  unsigned tj = blockIdx.x * kReconWarps + (threadIdx.x >> 5);
  int i = (int)(tj / tpr);
  tj -= (unsigned)i * tpr;
  i += p.i0;
  bool have = i < p.i1;
  ReconTask cur = recon_locate<RT>(p, have ? i : 0, have ? tj : 0u, lane, zsrc);
  uint32_t yw_n = 0u, zw_n = 0u;
  float ca_n = 0.f, cb_n = 0.f, cc_n = 0.f, d_n = 0.f;
  if (have) {
    yw_n = cur.y[0];
    zw_n = cur.z[0];
    ca_n = load_as_float(p.a, cur.ci, p.coef_dtype);
    cb_n = load_as_float(p.b, cur.ci, p.coef_dtype);
    cc_n = load_as_float(p.c, cur.ci, p.coef_dtype);
    d_n = load_as_float(p.d, cur.ci, p.coef_dtype);
  }

  while (have) {
    unsigned ntj = tj + stride;
    int ni = i;
    if (ntj >= tpr) {
      const unsigned k = ntj / tpr;
      ni += (int)k;
      ntj -= k * tpr;
    }
    const bool have_next = ni < p.i1;
    const ReconTask nxt = have_next ? recon_locate<RT>(p, ni, ntj, lane, zsrc) : cur;

    float acc[2][4][4];          // [16-row tile][8-column tile][fragment entry]
    float rowt[2][2];            // sum_b b_b popc(Yrow_b) of rows g8 (+8) of each 16-row tile
    float colt[4][2];            // d + sum_b c_b popc(Zcol_b) of columns 2 t4 (+1) of each 8-column tile
    const float dterm = d_n * scale;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      rowt[mt][0] = rowt[mt][1] = 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.f;
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) colt[nt][0] = colt[nt][1] = dterm;

    for (int b = 0; b < g.bw; ++b) {
      const float ca = ca_n * s_core, cb = cb_n * s_sum, cc = cc_n * s_sum;
      const bool more = b + 1 < g.bw;
      if (more || have_next) {
        const size_t ci = more ? cur.ci + (size_t)(b + 1) * cstep : nxt.ci;
        ca_n = load_as_float(p.a, ci, p.coef_dtype);
        cb_n = load_as_float(p.b, ci, p.coef_dtype);
        cc_n = load_as_float(p.c, ci, p.coef_dtype);
        if (!more) d_n = load_as_float(p.d, ci, p.coef_dtype);
      }
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        const uint32_t yw = yw_n;
        uint32_t zw = zw_n;
        if (rt + 1 < RT) {
          yw_n = cur.y[(size_t)b * ystep + (size_t)(rt + 1) * 32 * kGroup];
          zw_n = cur.z[(size_t)b * zstep + (size_t)(rt + 1) * g.QT * 32 * kGroup];
        } else if (more) {
          yw_n = cur.y[(size_t)(b + 1) * ystep];
          zw_n = cur.z[(size_t)(b + 1) * zstep];
        } else if (have_next) {
          yw_n = nxt.y[0];
          zw_n = nxt.z[0];
        }
        // fragments of both rank halves: 16-row tile mt holds rows g8 + 8 (2 mt + h), 8-column tile nt columns 8 nt + n
        uint32_t a[2][2][4], bz[4][2][2];
        y_frag<0, 0>(a[0][0], yw); y_frag<1, 0>(a[0][1], yw);
        y_frag<0, 2>(a[1][0], yw); y_frag<1, 2>(a[1][1], yw);
#pragma unroll
        for (int kh = 0; kh < 2; ++kh)
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const uint32_t byte = __byte_perm(__shfl_sync(0xffffffffu, zw, zfrom + 16 * kh + 2 * x), 0u, zbyte);
            z_frag(bz[x][kh], byte & 0xFu);          // qh = 0: tile x
            z_frag(bz[2 + x][kh], byte >> 4);        // qh = 1: tile 2 + x
          }
        // independent accumulation chains are interleaved: the second MMA of a chain waits for the first
        float d0[4], d1[4], dz[4];
        mma_f16_first(d0, a[0][0], kOnesHalf2, kOnesHalf2);                   // row sums
        mma_f16_first(d1, a[1][0], kOnesHalf2, kOnesHalf2);
        mma_f16(d0, a[0][1], kOnesHalf2, kOnesHalf2);
        mma_f16(d1, a[1][1], kOnesHalf2, kOnesHalf2);
        rowt[0][0] = fmaf(cb, d0[0], rowt[0][0]);
        rowt[0][1] = fmaf(cb, d0[2], rowt[0][1]);
        rowt[1][0] = fmaf(cb, d1[0], rowt[1][0]);
        rowt[1][1] = fmaf(cb, d1[2], rowt[1][1]);
        const uint32_t ones[4] = {kOnesHalf2, kOnesHalf2, kOnesHalf2, kOnesHalf2};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          mma_f16_first(dz, ones, bz[nt][0][0], bz[nt][0][1]);                // column sums
          mma_f16_first(d0, a[0][0], bz[nt][0][0], bz[nt][0][1]);
          mma_f16_first(d1, a[1][0], bz[nt][0][0], bz[nt][0][1]);
          mma_f16(dz, ones, bz[nt][1][0], bz[nt][1][1]);
          mma_f16(d0, a[0][1], bz[nt][1][0], bz[nt][1][1]);
          mma_f16(d1, a[1][1], bz[nt][1][0], bz[nt][1][1]);
          colt[nt][0] = fmaf(cc, dz[0], colt[nt][0]);
          colt[nt][1] = fmaf(cc, dz[1], colt[nt][1]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[0][nt][e] = fmaf(ca, d0[e], acc[0][nt][e]);
            acc[1][nt][e] = fmaf(ca, d1[e], acc[1][nt][e]);
          }
        }
      }
    }

    // 32 x 32 entries: a lane holds two neighbouring columns of rows g8 + 8 (2 mt + h) in every 8-column tile
    const int row0 = 32 * cur.pt + g8, col0 = 32 * cur.qt + 2 * t4;
    const size_t at0 = ((size_t)cur.i * g.P + row0) * ldw + (size_t)cur.j * g.Q + col0;
    WT* wp = reinterpret_cast<WT*>(p.W) + at0;
    WT* lp = LO ? reinterpret_cast<WT*>(p.W_lo) + at0 : nullptr;
    const bool whole = p.pairs && 32 * cur.pt + 32 <= g.P && 32 * cur.qt + 32 <= g.Q;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const size_t roff = (size_t)(16 * mt + 8 * h) * ldw;
        const bool row_ok = whole || row0 + 16 * mt + 8 * h < g.P;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const float v0 = acc[mt][nt][2 * h] + rowt[mt][h] + colt[nt][0];
          const float v1 = acc[mt][nt][2 * h + 1] + rowt[mt][h] + colt[nt][1];
          WT* w = wp + roff + 8 * nt;
          if (whole) {
            const WT2 wv = WType<DT>::cvt2(v0, v1);
            *reinterpret_cast<WT2*>(w) = wv;
            if (LO)
              *reinterpret_cast<WT2*>(lp + roff + 8 * nt) =
                  WType<DT>::cvt2(v0 - WType<DT>::back(wv.x), v1 - WType<DT>::back(wv.y));
          } else if (row_ok) {
            const int col = col0 + 8 * nt;
            if (col < g.Q) {
              const WT w0 = WType<DT>::cvt(v0);
              w[0] = w0;
              if (LO) lp[roff + 8 * nt] = WType<DT>::cvt(v0 - WType<DT>::back(w0));
            }
            if (col + 1 < g.Q) {
              const WT w1 = WType<DT>::cvt(v1);
              w[1] = w1;
              if (LO) lp[roff + 8 * nt + 1] = WType<DT>::cvt(v1 - WType<DT>::back(w1));
            }
          }
        }
      }

    cur = nxt;
    i = ni;
    tj = ntj;
    have = have_next;
  }
  pdl_exit(p.pdl);
}

template <typename K>
static int recon_launch_one(K kern, const ReconParams& p, dim3 blocks, cudaStream_t st) {
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = blocks;
  cfg.blockDim = dim3(kReconWarps * 32);
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl != kPdlNone ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return launch_status();
}

template <int RT>
static int reconstruct_dispatch(const ReconParams& p, dim3 blocks, cudaStream_t st) {
  const bool lo = p.W_lo != nullptr;
  if (p.w_dtype == BQQ_F32) return recon_launch_one(bqq_reconstruct_kernel<RT, BQQ_F32, false>, p, blocks, st);
  if (p.w_dtype == BQQ_BF16)
    return lo ? recon_launch_one(bqq_reconstruct_kernel<RT, BQQ_BF16, true>, p, blocks, st)
              : recon_launch_one(bqq_reconstruct_kernel<RT, BQQ_BF16, false>, p, blocks, st);
  return lo ? recon_launch_one(bqq_reconstruct_kernel<RT, BQQ_F16, true>, p, blocks, st)
            : recon_launch_one(bqq_reconstruct_kernel<RT, BQQ_F16, false>, p, blocks, st);
}

int reconstruct_launch(const BqqLayer* L, void* W, void* W_lo, int w_dtype, float scale, const float* bound_parts,
                       cudaStream_t st, int i0, int i1, int pdl) {
  ReconParams p;
  p.g = Geom(L->dims);
  p.i0 = i0;
  p.i1 = i1 < 0 ? p.g.rw : i1;
  p.pdl = pdl;
  p.zp = L->zplanes; p.yp = L->yplanes;
  p.a = L->a; p.b = L->b; p.c = L->c; p.d = L->d; p.coef_dtype = L->coef_dtype;
  p.W = W; p.W_lo = W_lo; p.scale = scale; p.bound_parts = bound_parts; p.w_dtype = w_dtype;
  p.tasks_per_row = p.g.cw * p.g.PT * p.g.QT;      // in_features <= 2^30 keeps this far below 2^31
  const uintptr_t pair_mask = 2 * (uintptr_t)dtype_size(w_dtype) - 1;
  p.pairs = (p.g.Q % 2 == 0 && ((uintptr_t)W & pair_mask) == 0 && ((uintptr_t)W_lo & pair_mask) == 0) ? 1 : 0;
  // resident warps walk the blocks: 4 CTAs per SM on 148 SMs
  const long long tasks = (long long)p.tasks_per_row * (p.i1 - p.i0);
  if (tasks <= 0) return BQQ_OK;
  const dim3 blocks((unsigned)std::min<long long>((tasks + kReconWarps - 1) / kReconWarps, 148LL * 4));
  if (w_dtype == BQQ_F32 && W_lo) return BQQ_ERR_UNSUPPORTED;     // a second part only exists for 16-bit types
  if (p.g.RT == 1) return reconstruct_dispatch<1>(p, blocks, st);
  return reconstruct_dispatch<2>(p, blocks, st);
}

// bound_parts[0] = max(|a|+|b|+|c|), bound_parts[1] = max|d| (both must be zero on entry: the caller clears them)
__global__ void coef_bound_kernel(const void* a, const void* b, const void* c, const void* d, int dt, size_t nabc,
                                  size_t nd, float* bound_parts) {
  pdl_enter(kPdlWaitFirst);          // the bound words were cleared by a memset node: nothing to overlap with
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
  // one pair of atomics per block: the warps' maxima meet in shared memory first
  __shared__ float part[2][8];
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) { part[0][warp] = m0; part[1][warp] = m1; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) { m0 = fmaxf(m0, part[0][w]); m1 = fmaxf(m1, part[1][w]); }
    // non-negative floats order like ints
    atomicMax(reinterpret_cast<int*>(bound_parts), __float_as_int(m0));
    atomicMax(reinterpret_cast<int*>(bound_parts) + 1, __float_as_int(m1));
  }
}

int coef_bound_launch(const BqqLayer* L, float* bound_parts, cudaStream_t st) {
  Geom g(L->dims);
  const size_t nabc = (size_t)g.bw * g.rw * g.cw, nd = (size_t)g.rw * g.cw;
  int blocks = (int)((nabc + 255) / 256 < 296 ? (nabc + 255) / 256 : 296);
  coef_bound_kernel<<<blocks, 256, 0, st>>>(L->a, L->b, L->c, L->d, L->coef_dtype, nabc, nd, bound_parts);
  return launch_status();
}

}  // namespace bqq
