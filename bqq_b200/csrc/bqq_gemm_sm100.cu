// Prefill forward: y[M,N] = x[M,K] @ W[N,K]^T with W rebuilt once from the packed
// planes into scratch memory, then a TMA + tcgen05 tensor-core GEMM with the fp32
// accumulator in tensor memory.  W is stored in the 16-bit format of the
// activations: fp16 (scaled by a power of two so that the bound on |W| maps to
// 2^14) for fp16 x, or as a bf16 pair hi + lo for bf16 x, in which case the K
// loop runs once per (x part, W part) pass into the same accumulator; fp32 x is
// split into bf16 hi + lo the same way (passes hi*hi, hi*lo, lo*hi).  Replaces reconstruct_W_kernel + torch::mm of
// the reference (neural_network_compression/src/bqq_cuda.cu:198-246, 367-383).
//
// GEMM kernel, one (128 MT) x BN output tile per CTA (BN = 256, 128, 64 or 32; MT = 1 or 2 row
// halves that share the B tile: with MT = 2 a k-block moves 64 KB for 256 x 256 outputs instead of
// 48 KB for 128 x 256, a third less traffic from the L2 per product), 6 warps:
//   warp 0   TMA producer: ring of {A (128 MT)x64, B BNx64} 16-bit tiles (4 stages, 3 for the
//            256 x 256 tile), 128-byte swizzle, completion on mbarriers
//   warp 1   allocates tensor memory (MT accumulators of BN columns); one lane issues tcgen05.mma
//            (M=128, N=BN, K=16 per instruction) and commits stage releases to mbarriers
//   warps 2-5 epilogue: tcgen05.ld 32 lanes x 32 columns, scale, bias, convert, store
// Every mbarrier wait is bounded by a clock budget; on expiry the kernel records
// a status code in global memory, drains its copies and returns.
//
// The call is a chain of programmatic dependent launches over column panels of W (about one wave of
// GEMM tiles each): bound, rebuild panel 0, stage x, then alternately multiply panel p and rebuild
// panel p+1.  A GEMM waits for everything before it and then lets the next rebuild start at once, so the
// rebuild of a panel (ALU work) runs beside the GEMM of the previous one (TMA and tensor pipe).
#include <cuda.h>

#include "bqq_async.cuh"
#include "bqq_common.cuh"

namespace bqq {

constexpr int kBM = 128;
constexpr int kBK = 64;          // 64 x 2 bytes = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
__host__ __device__ constexpr int gemm_stages(int BN, int MT) { return (BN == 256 && MT == 2) ? 3 : 4; }
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes,
// 128-byte swizzled, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address, 16-byte units
  d |= (uint64_t)1 << 16;                              // leading byte offset (one 16-byte unit; unused by swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                              // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                              // 128-byte swizzle
  return d;
}

struct GemmParams {
  void* y;
  const void* bias;
  const float* bound_parts;  // device {max(|a|+|b|+|c|), max|d|} when W was scaled (fp16), else NULL
  float bound_mult;          // bw * r
  const float* row_unscale;  // optional per-row factor of y (activation rows were scaled on staging)
  unsigned* status;          // device word, set nonzero when a wait timed out
  int64_t ldy;
  int y_dtype, bias_dtype;
  int M, N, K;
  int passes;                // K sweeps accumulated into one tile (1..3)
  int a_sel[3];              // per pass: 0 = first activation map, 1 = second (low half of fp32 x)
  int b_row[3];              // per pass: row offset into the stacked W map (0 = hi / only part, N = lo part)
  uint32_t idesc;
  int n_tile0;               // first BN-column tile of this launch (column panels of W are multiplied one after the other)
};

template <int BN, int MT>
__global__ void __launch_bounds__(kGemmThreads, 1)
bqq_gemm_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t gsm[];
  constexpr int kStages = gemm_stages(BN, MT);
  constexpr uint32_t kAHalf = kBM * kBK * 2;              // one 128-row half of the A tile
  constexpr uint32_t kABytes = MT * kAHalf;
  constexpr uint32_t kBBytes = BN * kBK * 2;
  constexpr uint32_t kCols = BN * MT;                     // tensor-memory columns: MT accumulators side by side
  // 1024-byte aligned tiles (required by the 128-byte swizzle)
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gsm) + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = base;
  uint8_t* sB = base + kStages * kABytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sB + kStages * kBBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* acc_bar = empty_bar + kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile uint32_t* failed = tmem_slot + 1;

  // everything before this launch (the rebuilt panel of W, the staged x) has to be complete; the next kernel of the
  // stream (the rebuild of the following panel) may start now and run beside this one
  pdl_enter(kPdlWaitFirst);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x + p.n_tile0) * BN;
  const int m0 = blockIdx.y * (kBM * MT);
  const int kblocks = (p.K + kBK - 1) / kBK;
  const int iters = kblocks * p.passes;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
    mbar_init(acc_bar, 1);
    *failed = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < iters; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1u;
        if (*failed || !mbar_wait(empty_bar + s, ph ^ 1u)) { *failed = 1; break; }
        mbar_expect_tx(full_bar + s, kABytes + kBBytes);
        const int kb = it % kblocks;
        const int pass = it / kblocks;
        const CUtensorMap* ma = p.a_sel[pass] == 0 ? &map_a0 : &map_a1;
        tma_load_2d(sA + s * kABytes, ma, full_bar + s, kb * kBK, m0);
        tma_load_2d(sB + s * kBBytes, &map_b, full_bar + s, kb * kBK, p.b_row[pass] + n0);
        issued = it + 1;
      }
      if (*failed) {
        // drain: copies already issued must land before the CTA exits
        int first = issued > kStages ? issued - kStages : 0;
        for (int it = first; it < issued; ++it)
          mbar_wait(full_bar + it % kStages, (uint32_t)(it / kStages) & 1u);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (uint32_t)(it / kStages) & 1u;
        if (*failed || !mbar_wait(full_bar + s, ph)) { *failed = 1; ok = false; break; }
        tc_fence_after();
        const uint64_t bdesc = make_smem_desc(smem_u32(sB + s * kBBytes));
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t adesc = make_smem_desc(smem_u32(sA + s * kABytes + mt * kAHalf));
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)   // 16 elements = 32 bytes = 2 descriptor units per step
            tc_mma_f16(tmem_base + (uint32_t)(mt * BN), adesc + 2 * k, bdesc + 2 * k, p.idesc, (it | k) != 0 ? 1u : 0u);
        }
        tc_commit(empty_bar + s);            // frees the stage when these MMAs have read it
      }
      tc_commit(acc_bar);                    // accumulator complete (or abandoned)
    }
  } else {
    // epilogue warps 2..5 own tensor-memory lanes 32*(warp%4) .. +31
    const int quarter = warp & 3;
    const bool ok = mbar_wait(acc_bar, 0) && !*failed;
    if (!ok) *failed = 1;
    tc_fence_after();
    if (ok) {
      const float w_unscale = p.bound_parts ? 1.f / w_scale_from_bound(p.bound_parts, p.bound_mult) : 1.f;
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
      const int m = m0 + mt * kBM + quarter * 32 + lane;
      const float row_f = (p.row_unscale && m < p.M) ? p.row_unscale[m] : 1.f;
      const float inv_scale = w_unscale * row_f;
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BN + c * 32), v);
        tc_wait_ld();
        const int nb = n0 + c * 32;
        if (m < p.M && nb < p.N) {
          const size_t row = (size_t)m * p.ldy;
          const bool full = nb + 32 <= p.N;
          if (full && p.y_dtype != BQQ_F32 && (((row + nb) * 2 + (uintptr_t)p.y) & 15) == 0) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.y) + row + nb);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float f0 = __uint_as_float(v[g * 8 + 2 * e]) * inv_scale;
                float f1 = __uint_as_float(v[g * 8 + 2 * e + 1]) * inv_scale;
                if (p.bias) {
                  f0 += load_as_float(p.bias, nb + g * 8 + 2 * e, p.bias_dtype);
                  f1 += load_as_float(p.bias, nb + g * 8 + 2 * e + 1, p.bias_dtype);
                }
                if (p.y_dtype == BQQ_BF16) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(f0, f1);
                  w[e] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                  __half2 h = __floats2half2_rn(f0, f1);
                  w[e] = *reinterpret_cast<uint32_t*>(&h);
                }
              }
              dst[g] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              if (nb + e < p.N) {
                float f = __uint_as_float(v[e]) * inv_scale;
                if (p.bias) f += load_as_float(p.bias, nb + e, p.bias_dtype);
                store_from_float(p.y, row + nb + e, p.y_dtype, f);
              }
            }
          }
        }
      }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
  if (threadIdx.x == 0 && *failed) atomicExch(p.status, 1u);
}

// ---- x staging: any dtype / stride -> dense 16-bit rows (hi, lo for fp32) ----
__global__ void stage_x_kernel(const void* __restrict__ x, int x_dtype, int64_t ldx, int M, int K, int Kp,
                               uint16_t* __restrict__ hi, uint16_t* __restrict__ lo) {
  pdl_enter(kPdlOverlap);
  const size_t n = (size_t)M * Kp;
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    const int k = (int)(t % Kp);
    const size_t m = t / Kp;
    if (x_dtype == BQQ_F32) {
      float v = k < K ? reinterpret_cast<const float*>(x)[m * ldx + k] : 0.f;
      __nv_bfloat16 h = __float2bfloat16_rn(v);
      __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
      hi[t] = *reinterpret_cast<uint16_t*>(&h);
      lo[t] = *reinterpret_cast<uint16_t*>(&l);
    } else {
      hi[t] = k < K ? reinterpret_cast<const uint16_t*>(x)[m * ldx + k] : (uint16_t)0;
    }
  }
  pdl_exit(kPdlOverlap);
}

// bf16 rows -> fp16 rows scaled by a per-row power of two (max |x| of the row maps to at most 2^14,
// so nothing overflows and every bf16 value in range converts exactly); row_unscale[m] = 1 / scale.
// One block per row; with `vec` a thread moves 8 values per access and keeps its first kStageKeep
// accesses in registers, so rows up to 8 * kStageKeep * blockDim.x values are read once.
constexpr int kStageThreads = 128;
constexpr int kStageKeep = 4;
__global__ void __launch_bounds__(kStageThreads)
stage_x_bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, int M, int K,
                           __half* __restrict__ out, float* __restrict__ row_unscale, int vec) {
  __shared__ float warp_max[kStageThreads / 32];
  pdl_enter(kPdlOverlap);
  const int tid = threadIdx.x, lane = tid & 31;
  for (int m = blockIdx.x; m < M; m += gridDim.x) {
    const __nv_bfloat16* row = x + (size_t)m * ldx;
    const uint4* row8 = reinterpret_cast<const uint4*>(row);
    const int K8 = K >> 3;
    uint4 keep[kStageKeep];
    float amax = 0.f;
    if (vec) {
#pragma unroll
      for (int s = 0; s < kStageKeep; ++s) {
        const int k = tid + s * kStageThreads;
        keep[s] = k < K8 ? row8[k] : make_uint4(0u, 0u, 0u, 0u);
      }
      for (int k = tid + kStageKeep * kStageThreads; k < K8; k += kStageThreads) {
        const uint4 v = row8[k];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[e] << 16)), fabsf(__uint_as_float(w[e] & 0xFFFF0000u))));
      }
#pragma unroll
      for (int s = 0; s < kStageKeep; ++s) {
        const uint32_t w[4] = {keep[s].x, keep[s].y, keep[s].z, keep[s].w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[e] << 16)), fabsf(__uint_as_float(w[e] & 0xFFFF0000u))));
      }
    } else {
      for (int k = tid; k < K; k += kStageThreads) amax = fmaxf(amax, fabsf(__bfloat162float(row[k])));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __syncthreads();                               // the previous row's readers are done with warp_max
    if (lane == 0) warp_max[tid >> 5] = amax;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kStageThreads / 32; ++w) amax = fmaxf(amax, warp_max[w]);
    float scale = 1.f;
    if (amax > 0.f && isfinite(amax)) {
      int e;
      frexpf(amax, &e);                        // amax = f * 2^e, f in [0.5, 1)
      scale = exp2f((float)max(-100, min(100, 14 - e)));
    }
    if (vec) {
      uint4* out8 = reinterpret_cast<uint4*>(out + (size_t)m * K);
      auto convert = [scale](const uint4& v) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t h[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __half2 t = __floats2half2_rn(__uint_as_float(w[e] << 16) * scale,
                                              __uint_as_float(w[e] & 0xFFFF0000u) * scale);
          h[e] = *reinterpret_cast<const uint32_t*>(&t);
        }
        return make_uint4(h[0], h[1], h[2], h[3]);
      };
#pragma unroll
      for (int s = 0; s < kStageKeep; ++s) {
        const int k = tid + s * kStageThreads;
        if (k < K8) out8[k] = convert(keep[s]);
      }
      for (int k = tid + kStageKeep * kStageThreads; k < K8; k += kStageThreads) out8[k] = convert(row8[k]);
    } else {
      for (int k = tid; k < K; k += kStageThreads) out[(size_t)m * K + k] = __float2half_rn(__bfloat162float(row[k]) * scale);
    }
    if (tid == 0) row_unscale[m] = 1.f / scale;
  }
  pdl_exit(kPdlOverlap);
}

// ---- host side -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D row-major [rows][cols] 16-bit tensor, box = box_rows x 64 columns, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, bool bf16, uint64_t rows, uint64_t cols,
                    uint64_t ld_elems, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return BQQ_ERR_CUDA;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)kBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? BQQ_OK : BQQ_ERR_CUDA;
}

static inline size_t up256(size_t v) { return (v + 255) / 256 * 256; }

// workspace: [256 B: status word, bound parts at +16][W parts 2 x N x K 16-bit][x hi M x K][x lo M x K]
size_t prefill_workspace_bytes(const BqqDims* dims, int M) {
  Geom g(*dims);
  const size_t K = g.in_features();
  return 256 + up256((size_t)2 * g.out_features() * K * 2) + 2 * up256((size_t)M * K * 2);
}


static cudaLaunchAttribute pdl_attribute() {
  cudaLaunchAttribute a;
  a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  a.val.programmaticStreamSerializationAllowed = 1;
  return a;
}

// tiles [tile0, tile0 + ntiles) along N, all of M
template <int BN, int MT>
static int launch_gemm(const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b, GemmParams p, int tile0,
                       int ntiles, cudaStream_t st) {
  const size_t smem = 1024 + (size_t)gemm_stages(BN, MT) * (MT * kBM * kBK * 2 + BN * kBK * 2) + 256;
  auto kern = bqq_gemm_kernel<BN, MT>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return BQQ_ERR_CUDA;
  p.n_tile0 = tile0;
  cudaLaunchAttribute attr[1] = {pdl_attribute()};
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ntiles, (p.M + kBM * MT - 1) / (kBM * MT));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, a0, a1, b, p) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return launch_status();
}

static int launch_gemm_bn(int BN, int MT, const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b,
                          const GemmParams& p, int tile0, int ntiles, cudaStream_t st) {
  if (MT == 2) return launch_gemm<256, 2>(a0, a1, b, p, tile0, ntiles, st);
  switch (BN) {
    case 256: return launch_gemm<256, 1>(a0, a1, b, p, tile0, ntiles, st);
    case 128: return launch_gemm<128, 1>(a0, a1, b, p, tile0, ntiles, st);
    case 64: return launch_gemm<64, 1>(a0, a1, b, p, tile0, ntiles, st);
    default: return launch_gemm<32, 1>(a0, a1, b, p, tile0, ntiles, st);
  }
}

int prefill_launch(const BqqLayer* L, const void* x, int x_dtype, int M, int64_t ldx, void* y, int y_dtype,
                   int64_t ldy, void* ws, size_t ws_bytes, cudaStream_t st) {
  Geom g(L->dims);
  const int N = g.out_features(), K = g.in_features();
  if (K % 8 != 0) return BQQ_ERR_UNSUPPORTED;   // 16-byte row pitch for the TMA descriptors
  if (!ws || ws_bytes < prefill_workspace_bytes(&L->dims, M)) return BQQ_ERR_WORKSPACE;
  if (((uintptr_t)ws & 255) != 0) return BQQ_ERR_MISALIGNED;
  uint8_t* wsb = reinterpret_cast<uint8_t*>(ws);
  unsigned* status = reinterpret_cast<unsigned*>(wsb);
  uint16_t* W = reinterpret_cast<uint16_t*>(wsb + 256);              // [2][N][K]: hi rows, then lo rows
  uint16_t* xhi = reinterpret_cast<uint16_t*>(wsb + 256 + up256((size_t)2 * N * K * 2));
  uint16_t* xlo = reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(xhi) + up256((size_t)M * K * 2));
  float* bound_parts = reinterpret_cast<float*>(wsb + 16);

  if (cudaMemsetAsync(status, 0, 32, st) != cudaSuccess) return BQQ_ERR_CUDA;   // status word and bound parts

  const bool f16 = x_dtype != BQQ_F32;
  const bool split_x = x_dtype == BQQ_F32;
  // widest tile that still gives about one CTA per SM: small batches are bound by how many SMs stream W
  int BN = 32;
  for (int cand = 256; cand >= 64; cand >>= 1) {
    const long long ctas = (long long)((N + cand - 1) / cand) * ((M + kBM - 1) / kBM);
    if (ctas >= 118) { BN = cand; break; }
  }
  // two row halves per CTA (256 x 256 outputs on one B tile) where that still gives about one CTA per SM
  const int MT = (BN == 256 && (long long)((N + 255) / 256) * ((M + 2 * kBM - 1) / (2 * kBM)) >= 118) ? 2 : 1;
  // Column panels of W of about one wave of GEMM tiles each (at most 4): the rebuild of panel p+1 runs beside the
  // GEMM of panel p.  A panel border must not cut a row patch (the rebuild works on whole row patches).
  const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + kBM * MT - 1) / (kBM * MT);
  int panels = (int)(((long long)tiles_n * tiles_m + 74) / 148);
  panels = panels < 1 ? 1 : (panels > 4 ? 4 : panels);
  if (panels > tiles_n) panels = tiles_n;
  if (BN % g.P != 0) panels = 1;
  const int tiles_pp = (tiles_n + panels - 1) / panels;
  panels = (tiles_n + tiles_pp - 1) / tiles_pp;
  auto panel_rows = [&](int pnl, int* i0, int* i1) {           // row patches of panel pnl
    const int c0 = pnl * tiles_pp * BN, c1 = std::min(N, (pnl + 1) * tiles_pp * BN);
    *i0 = c0 / g.P;
    *i1 = (c1 + g.P - 1) / g.P;
  };

  // x: fp16 is used in place when its pitch suits TMA; everything else is staged
  const bool direct = x_dtype == BQQ_F16 && (ldx % 8) == 0 && ((uintptr_t)x & 15) == 0;
  const void* a_ptr = direct ? x : (const void*)xhi;
  const int64_t a_ld = direct ? ldx : (int64_t)K;
  float* unscale = reinterpret_cast<float*>(xlo);            // the lo region is free when x has 16 bits
  const float* row_unscale = x_dtype == BQQ_BF16 ? unscale : nullptr;

  CUtensorMap ma0, ma1, mb;
  int rc = make_map(&ma0, a_ptr, !f16, (uint64_t)M, (uint64_t)K, (uint64_t)a_ld, kBM * MT);
  if (rc) return rc;
  rc = make_map(&ma1, split_x ? (const void*)xlo : a_ptr, !f16, (uint64_t)M, (uint64_t)K,
                split_x ? (uint64_t)K : (uint64_t)a_ld, kBM * MT);
  if (rc) return rc;
  rc = make_map(&mb, W, !f16, (uint64_t)(f16 ? N : 2 * N), (uint64_t)K, (uint64_t)K, (uint32_t)BN);
  if (rc) return rc;

  GemmParams p;
  p.y = y; p.bias = L->bias; p.bound_parts = f16 ? bound_parts : nullptr; p.bound_mult = (float)(g.bw * g.r);
  p.status = status;
  p.row_unscale = row_unscale;
  p.ldy = ldy; p.y_dtype = y_dtype; p.bias_dtype = L->bias_dtype;
  p.M = M; p.N = N; p.K = K;
  p.n_tile0 = 0;
  for (int i = 0; i < 3; ++i) { p.a_sel[i] = 0; p.b_row[i] = 0; }
  if (f16) {
    p.passes = 1;
  } else {
    p.passes = 3; p.b_row[1] = N; p.a_sel[2] = 1;       // xhi*Whi + xhi*Wlo + xlo*Whi
  }
  // instruction descriptor: fp32 accumulate, A and B in the same 16-bit format, both K-major
  const uint32_t fmt = f16 ? 0u : 1u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

  // 1. (16-bit x) bound on |W| for the power-of-two scale of the fp16 weight.  fp16 and bf16 activations use one
  //    fp16 W (bf16 rows are re-staged as scaled fp16, exact); fp32 activations use the bf16 hi + lo pair.
  if (f16) {
    rc = coef_bound_launch(L, bound_parts, st);
    if (rc) return rc;
  }
  // 2. panel 0 of W: waits for the bound (and for whatever preceded this call in the stream)
  auto rebuild = [&](int pnl, int pdl) {
    int i0, i1;
    panel_rows(pnl, &i0, &i1);
    return f16 ? reconstruct_launch(L, W, nullptr, BQQ_F16, 1.f, bound_parts, st, i0, i1, pdl)
               : reconstruct_launch(L, W, W + (size_t)N * K, BQQ_BF16, 1.f, nullptr, st, i0, i1, pdl);
  };
  rc = rebuild(0, kPdlWaitFirst);
  if (rc) return rc;
  // 3. x staging, beside the rebuild of panel 0
  if (x_dtype == BQQ_BF16) {
    const int vec = (K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0) ? 1 : 0;
    cudaLaunchAttribute attr[1] = {pdl_attribute()};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(M);
    cfg.blockDim = dim3(kStageThreads);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, stage_x_bf16_to_f16_kernel, reinterpret_cast<const __nv_bfloat16*>(x), ldx, M, K,
                           reinterpret_cast<__half*>(xhi), unscale, vec) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  } else if (!direct) {
    size_t n = (size_t)M * K;
    int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    cudaLaunchAttribute attr[1] = {pdl_attribute()};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, stage_x_kernel, x, x_dtype, ldx, M, K, K, xhi, xlo) != cudaSuccess) {
      cudaGetLastError();
      return BQQ_ERR_CUDA;
    }
  }
  rc = launch_status();
  if (rc) return rc;
  // 4. alternately: multiply panel p (waits for everything before it, then lets its successor start), rebuild
  //    panel p+1 beside it (its last CTA waits for that GEMM, so the next GEMM's wait covers both)
  for (int pnl = 0; pnl < panels; ++pnl) {
    const int tile0 = pnl * tiles_pp, ntiles = std::min(tiles_pp, tiles_n - tile0);
    rc = launch_gemm_bn(BN, MT, ma0, ma1, mb, p, tile0, ntiles, st);
    if (rc) return rc;
    if (pnl + 1 < panels) {
      rc = rebuild(pnl + 1, kPdlOverlap);
      if (rc) return rc;
    }
  }
  return BQQ_OK;
}

}  // namespace bqq
