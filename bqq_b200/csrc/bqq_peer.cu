// Column gather across the GPUs of one node by peer-to-peer stores (no reduction, no NCCL call).
//
// A column-parallel BinaryQuadratic layer leaves rank g with the output columns
// [g*n, (g+1)*n) of every row.  Each rank owns one region (cudaMalloc + CUDA IPC, mapped by
// all peers): control words and one gather buffer [rows][world*n].  A gather is one kernel
// per rank:
//   1. wait until every peer has acknowledged the previous gather (my old data is consumed),
//   2. store my column slice into every rank's buffer (NVLink stores, 16 bytes per thread),
//      fence, then publish the gather's sequence number in each peer's flag word for me,
//   3. wait until every rank's flag word in MY region carries the sequence number,
//   4. copy the complete rows out of my buffer into the caller's tensor and acknowledge to
//      every peer.
// Every wait is bounded by a clock budget; when one gives up the kernel still finishes, the
// status word is set and the next bqq_peer_status call reports BQQ_ERR_TIMEOUT.  The sequence
// number lives on the device, so a captured CUDA graph can replay the gather.
#include <cuda_runtime.h>
#include <string.h>

#include "bqq_common.cuh"

namespace bqq {

constexpr size_t kPeerCtrlBytes = 512;         // epoch, status, counters | flags | acks
constexpr int kFlagWord = 32;                  // word offset of flags[world] inside the region
constexpr int kAckWord = 64;                   // word offset of acks[world]
constexpr long long kPeerWaitBudget = 2000000000LL;   // clock cycles (~1 s) before a wait gives up
constexpr int kPeerThreads = 256;
constexpr int kPeerMaxBlocks = 32;             // far below the number of SMs: all blocks are co-resident

struct PeerArgs {
  uint8_t* regions[BQQ_MAX_PEERS];             // every rank's region as mapped in this process
  const uint8_t* src;                          // local slice [rows][ld_src] bytes
  uint8_t* out;                                // gathered rows [rows][ld_out] bytes (local), may be NULL
  int rank, world, rows;
  long long row_bytes;                         // bytes of one row of the local slice (n * element size)
  long long ld_src, ld_out;                    // row pitches in bytes
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *p has reached `target` (sequence numbers wrap).
__device__ __forceinline__ bool wait_reached(const unsigned* p, unsigned target) {
  if ((int)(ld_acquire_sys(p) - target) >= 0) return true;
  const long long t0 = clock64();
  while ((int)(ld_acquire_sys(p) - target) < 0) {
    if (clock64() - t0 > kPeerWaitBudget) return false;
    __nanosleep(64);
  }
  return true;
}

// Loads bypass L1 (the source may have been written by another GPU since this SM last read it).
__device__ __forceinline__ void copy_rows(uint8_t* dst, long long ld_dst, const uint8_t* src, long long ld_src,
                                          int rows, long long row_bytes, int tid, int nthreads) {
  const bool vec = ((row_bytes | ld_dst | ld_src | (long long)(uintptr_t)dst | (long long)(uintptr_t)src) & 15) == 0;
  if (vec) {
    const long long per_row = row_bytes >> 4, total = per_row * rows;
    for (long long e = tid; e < total; e += nthreads) {
      const long long r = e / per_row, c = e - r * per_row;
      reinterpret_cast<uint4*>(dst + r * ld_dst)[c] = __ldcg(reinterpret_cast<const uint4*>(src + r * ld_src) + c);
    }
  } else {
    const long long per_row = row_bytes >> 1, total = per_row * rows;      // every element type is >= 2 bytes
    for (long long e = tid; e < total; e += nthreads) {
      const long long r = e / per_row, c = e - r * per_row;
      reinterpret_cast<uint16_t*>(dst + r * ld_dst)[c] = __ldcg(reinterpret_cast<const uint16_t*>(src + r * ld_src) + c);
    }
  }
}

__global__ void __launch_bounds__(kPeerThreads)
bqq_peer_gather_kernel(const PeerArgs a) {
  __shared__ int s_last, s_fail;
  unsigned* mine = reinterpret_cast<unsigned*>(a.regions[a.rank]);
  const int tid = threadIdx.x;
  const int gtid = blockIdx.x * kPeerThreads + tid, gthreads = gridDim.x * kPeerThreads;
  const unsigned e = *reinterpret_cast<volatile unsigned*>(mine) + 1u;    // sequence number of this gather
  const long long gathered_row = a.row_bytes * a.world;
  if (tid == 0) s_fail = 0;
  __syncthreads();

  // 1. every peer has consumed what I stored for the previous gather
  if (tid < a.world && !wait_reached(mine + kAckWord + tid, e - 1u)) s_fail = 1;
  __syncthreads();

  // 2. my slice into every rank's buffer, then publish
  for (int q = 0; q < a.world; ++q)
    copy_rows(a.regions[q] + kPeerCtrlBytes + a.rank * a.row_bytes, gathered_row, a.src, a.ld_src, a.rows,
              a.row_bytes, gtid, gthreads);
  __threadfence_system();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(mine + 2, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (tid < a.world) st_release_sys(reinterpret_cast<unsigned*>(a.regions[tid]) + kFlagWord + a.rank, e);
    if (tid == 0) mine[2] = 0u;
  }

  // 3. every rank's slice has arrived in my buffer
  if (tid < a.world && !wait_reached(mine + kFlagWord + tid, e)) s_fail = 1;
  __syncthreads();

  // 4. copy the rows out and acknowledge
  if (a.out)
    copy_rows(a.out, a.ld_out, reinterpret_cast<const uint8_t*>(mine) + kPeerCtrlBytes, gathered_row, a.rows,
              gathered_row, gtid, gthreads);
  if (s_fail && tid == 0) atomicExch(mine + 1, 1u);
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(mine + 3, 1u) == gridDim.x - 1;
  __syncthreads();
  if (s_last) {
    if (tid < a.world) st_release_sys(reinterpret_cast<unsigned*>(a.regions[tid]) + kAckWord + a.rank, e);
    if (tid == 0) {
      mine[3] = 0u;
      *reinterpret_cast<volatile unsigned*>(mine) = e;
    }
  }
}

}  // namespace bqq

using namespace bqq;

extern "C" {

size_t bqq_peer_region_bytes(size_t gather_bytes) { return kPeerCtrlBytes + (gather_bytes + 255) / 256 * 256; }

int bqq_peer_alloc(size_t gather_bytes, void** region, unsigned char handle[BQQ_PEER_HANDLE_BYTES]) {
  if (!region || !handle) return BQQ_ERR_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == BQQ_PEER_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  const size_t bytes = bqq_peer_region_bytes(gather_bytes);
  if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, bytes) != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return BQQ_ERR_CUDA;
  }
  memcpy(handle, &h, sizeof(h));
  *region = p;
  return BQQ_OK;
}

int bqq_peer_open(const unsigned char handle[BQQ_PEER_HANDLE_BYTES], void** region) {
  if (!region || !handle) return BQQ_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  *region = p;
  return BQQ_OK;
}

int bqq_peer_close(void* region) {
  if (!region) return BQQ_ERR_NULL;
  if (cudaIpcCloseMemHandle(region) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return BQQ_OK;
}

int bqq_peer_free(void* region) {
  if (!region) return BQQ_ERR_NULL;
  if (cudaFree(region) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return BQQ_OK;
}

int bqq_peer_gather(const BqqPeerGroup* g, const void* y_local, int dtype, int rows, int64_t n_local, int64_t ldy,
                    void* gathered, int64_t ld_gathered, void* stream) {
  if (!g || !y_local) return BQQ_ERR_NULL;
  if (g->world < 1 || g->world > BQQ_MAX_PEERS || g->rank < 0 || g->rank >= g->world) return BQQ_ERR_BAD_SHAPE;
  const size_t es = dtype_size(dtype);
  if (!es) return BQQ_ERR_DTYPE;
  if (rows <= 0 || n_local <= 0 || ldy < n_local || (gathered && ld_gathered < n_local * g->world)) return BQQ_ERR_BAD_SHAPE;
  if ((size_t)rows * n_local * g->world * es > g->gather_bytes) return BQQ_ERR_WORKSPACE;
  PeerArgs a;
  for (int q = 0; q < g->world; ++q) {
    if (!g->regions[q]) return BQQ_ERR_NULL;
    a.regions[q] = reinterpret_cast<uint8_t*>(g->regions[q]);
  }
  a.src = reinterpret_cast<const uint8_t*>(y_local);
  a.out = reinterpret_cast<uint8_t*>(gathered);
  a.rank = g->rank; a.world = g->world; a.rows = rows;
  a.row_bytes = (long long)n_local * es;
  a.ld_src = (long long)ldy * es;
  a.ld_out = (long long)ld_gathered * es;
  const long long vec = ((long long)rows * a.row_bytes * g->world + 15) / 16;
  int blocks = (int)((vec + 4 * kPeerThreads - 1) / (4 * kPeerThreads));
  blocks = blocks < 1 ? 1 : (blocks > kPeerMaxBlocks ? kPeerMaxBlocks : blocks);
  bqq_peer_gather_kernel<<<blocks, kPeerThreads, 0, (cudaStream_t)stream>>>(a);
  return launch_status();
}

int bqq_peer_status(const BqqPeerGroup* g, void* stream) {
  if (!g || g->rank < 0 || g->rank >= BQQ_MAX_PEERS || !g->regions[g->rank]) return BQQ_ERR_NULL;
  unsigned st = 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemcpyAsync(&st, reinterpret_cast<unsigned*>(g->regions[g->rank]) + 1, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return st ? BQQ_ERR_TIMEOUT : BQQ_OK;
}

}  // extern "C"
