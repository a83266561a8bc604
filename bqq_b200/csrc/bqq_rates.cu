// Issue rates of the instructions the decode kernel could be built from, measured on the device: the
// mma.sync shapes for 8-bit, 16-bit, fp8, 4-bit and 1-bit operands and the plain ALU instructions
// around them.  The choice of byte operands for the decode kernel (int8 MMAs fed by masked plane
// words, instead of the 1-bit AND+POPC shape that would take the planes as they are) rests on these
// numbers.  A diagnostic of this library; the reference has no counterpart.
#include "bqq_common.cuh"

namespace bqq {

enum {
  kRateMmaS8 = 0, kRateMmaF16, kRateMmaE4M3, kRateMmaU4, kRateMmaB1, kRateLop3, kRateFadd, kRateImad, kRatePopc,
  kRateShfl, kRateKinds
};

__device__ unsigned g_rate_sink[32];

// Every warp runs `iters` rounds of independent instructions of one kind (two accumulator sets for the MMAs, eight
// chains for the others); the result is kept alive through a store that never happens in practice.
template <int KIND>
__global__ void __launch_bounds__(256)
rate_kernel(int iters, unsigned never) {
  const uint32_t a0 = threadIdx.x, a1 = a0 * 3u + 1u, a2 = a0 * 5u + 2u, a3 = a0 * 7u + 3u, b0 = a0 * 11u, b1 = a0 * 13u;
  unsigned result = 0;
  if constexpr (KIND <= kRateMmaB1) {
    uint32_t c[4] = {0, 0, 0, 0}, d[4] = {0, 0, 0, 0};
#define BQQ_RATE_MMA(SHAPE_TYPES, ACC)                                                                               \
  asm volatile("mma.sync.aligned." SHAPE_TYPES " {%0,%1,%2,%3},{%4,%5,%6,%7},{%8,%9},{%0,%1,%2,%3};"                \
               : "+r"(ACC[0]), "+r"(ACC[1]), "+r"(ACC[2]), "+r"(ACC[3])                                             \
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1))
    for (int i = 0; i < iters; ++i) {
      if constexpr (KIND == kRateMmaS8) {
        BQQ_RATE_MMA("m16n8k32.row.col.s32.u8.s8.s32", c);
        BQQ_RATE_MMA("m16n8k32.row.col.s32.u8.s8.s32", d);
      } else if constexpr (KIND == kRateMmaF16) {
        BQQ_RATE_MMA("m16n8k16.row.col.f32.f16.f16.f32", c);
        BQQ_RATE_MMA("m16n8k16.row.col.f32.f16.f16.f32", d);
      } else if constexpr (KIND == kRateMmaE4M3) {
        BQQ_RATE_MMA("m16n8k32.row.col.f32.e4m3.e4m3.f32", c);
        BQQ_RATE_MMA("m16n8k32.row.col.f32.e4m3.e4m3.f32", d);
      } else if constexpr (KIND == kRateMmaU4) {
        BQQ_RATE_MMA("m16n8k64.row.col.s32.u4.s4.s32", c);
        BQQ_RATE_MMA("m16n8k64.row.col.s32.u4.s4.s32", d);
      } else {
        BQQ_RATE_MMA("m16n8k256.row.col.s32.b1.b1.s32.and.popc", c);
        BQQ_RATE_MMA("m16n8k256.row.col.s32.b1.b1.s32.and.popc", d);
      }
    }
#undef BQQ_RATE_MMA
    result = c[0] + c[1] + c[2] + c[3] + d[0] + d[1] + d[2] + d[3];
  } else {
    uint32_t r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = a0 + j;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if constexpr (KIND == kRateLop3) asm volatile("lop3.b32 %0, %0, %1, %2, 0x6A;" : "+r"(r[j]) : "r"(a1), "r"(a2));
        else if constexpr (KIND == kRateFadd) asm volatile("add.f32 %0, %0, %1;" : "+r"(r[j]) : "r"(a1));
        else if constexpr (KIND == kRateImad) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(r[j]) : "r"(a1), "r"(a2));
        else if constexpr (KIND == kRatePopc) asm volatile("popc.b32 %0, %0;" : "+r"(r[j]));
        else asm volatile("shfl.sync.bfly.b32 %0, %0, %1, 0x1f, 0xffffffff;" : "+r"(r[j]) : "r"(1 + j));
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) result += r[j];
  }
  if (result == never) g_rate_sink[threadIdx.x & 31] = result;
}

template <int KIND>
static int rate_run(int iters, double* per_clk, cudaStream_t st) {
  int dev = 0, sms = 0, khz = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev) != cudaSuccess)
    return BQQ_ERR_CUDA;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return BQQ_ERR_CUDA;
  const int ctas = sms * 4;                                  // 8 warps per CTA, 32 warps per SM
  rate_kernel<KIND><<<ctas, 256, 0, st>>>(64, 0x9E3779B9u);  // warm-up
  cudaEventRecord(e0, st);
  rate_kernel<KIND><<<ctas, 256, 0, st>>>(iters, 0x9E3779B9u);
  cudaEventRecord(e1, st);
  float ms = 0.f;
  const bool ok = cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && ms > 0.f;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (!ok) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  const double per_round = KIND <= kRateMmaB1 ? 2.0 : 8.0;
  const double inst = (double)ctas * 8.0 * iters * per_round;          // warp-instructions
  *per_clk = inst / (ms * 1e-3) / ((double)khz * 1e3) / sms;           // per SM and clock of the nominal SM clock
  return BQQ_OK;
}

}  // namespace bqq

extern "C" int bqq_instruction_rate(int kind, int iters, double* warp_inst_per_clk_per_sm, void* stream) {
  using namespace bqq;
  if (!warp_inst_per_clk_per_sm) return BQQ_ERR_NULL;
  if (iters < 1 || iters > (1 << 20)) return BQQ_ERR_BAD_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  switch (kind) {
    case kRateMmaS8: return rate_run<kRateMmaS8>(iters, warp_inst_per_clk_per_sm, st);
    case kRateMmaF16: return rate_run<kRateMmaF16>(iters, warp_inst_per_clk_per_sm, st);
    case kRateMmaE4M3: return rate_run<kRateMmaE4M3>(iters, warp_inst_per_clk_per_sm, st);
    case kRateMmaU4: return rate_run<kRateMmaU4>(iters, warp_inst_per_clk_per_sm, st);
    case kRateMmaB1: return rate_run<kRateMmaB1>(iters, warp_inst_per_clk_per_sm, st);
    case kRateLop3: return rate_run<kRateLop3>(iters, warp_inst_per_clk_per_sm, st);
    case kRateFadd: return rate_run<kRateFadd>(iters, warp_inst_per_clk_per_sm, st);
    case kRateImad: return rate_run<kRateImad>(iters, warp_inst_per_clk_per_sm, st);
    case kRatePopc: return rate_run<kRatePopc>(iters, warp_inst_per_clk_per_sm, st);
    case kRateShfl: return rate_run<kRateShfl>(iters, warp_inst_per_clk_per_sm, st);
    default: return BQQ_ERR_BAD_SHAPE;
  }
}
