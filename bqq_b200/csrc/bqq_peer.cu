// Column gather across the GPUs of one node by peer-to-peer stores (no reduction, no NCCL call).
//
// A column-parallel BinaryQuadratic layer leaves rank g with the output columns
// [g*n, (g+1)*n) of every row.  Each rank owns one region (cudaMalloc + CUDA IPC, mapped by
// all peers): control words and two halves of 8-byte slots, one slot per 32-bit word of the
// gathered rows [rows][world*n].  A gather is one kernel per rank:
//   send: every 32-bit word of my slice goes, together with the gather's sequence number, as one
//         scalar 64-bit store (st.relaxed.sys.b64) into the matching slot of every rank's region
//         (NVLink stores; a naturally aligned scalar 64-bit access is single-copy atomic, so data and
//         sequence number arrive together and no fence or separate flag is needed);
//   receive: every slot of my own region is polled until it carries the sequence number, and its
//         data word is written to the caller's tensor.
// Consecutive gathers alternate between the two halves.  A rank can only start gather e+2 after it
// has received gather e+1 from every peer, which the peers send after their gather e has returned,
// so a half is never overwritten while its owner still reads it.
// Every poll is bounded by a clock budget (BqqPeerGroup::wait_cycles, about one second by default);
// when one gives up the kernel still finishes, the status word is set and the next bqq_peer_status
// call reports BQQ_ERR_TIMEOUT.  The sequence number lives
// on the device, so a captured CUDA graph can replay the gather.
#include <cuda_runtime.h>
#include <string.h>

#include "bqq_common.cuh"

// bqq_forward_decode with the peer group handed through to the kernel (bqq_api.cu)
int bqq_forward_decode_peer(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y, int y_dtype,
                            int64_t ldy, void* workspace, size_t workspace_bytes, void* stream, const BqqPeerGroup* peer,
                            const BqqFusion* fusion = nullptr, void* gathered = nullptr, int64_t ld_gathered = 0);

namespace bqq {

constexpr long long kPeerWaitBudget = 2000000000LL;   // default clock cycles (~1 s) before a poll gives up
constexpr int kPeerThreads = 256;
constexpr int kPeerMaxBlocks = 32;

struct PeerArgs {
  uint8_t* regions[BQQ_MAX_PEERS];             // every rank's region as mapped in this process
  const uint32_t* src;                         // local slice, rows of `row_words` words, pitch ld_src words;
                                               // NULL: the producing kernel sends the slice itself
  uint32_t* out;                               // gathered rows, pitch ld_out words
  int rank, world, rows;
  int row_words;                               // 32-bit words of one row of the local slice
  long long ld_src, ld_out;                    // row pitches in words
  unsigned long long half_bytes;               // bytes of one half of the slot area
  long long wait_cycles;                       // clock budget of one poll
};

// slot = one scalar 64-bit word: data in the low half, sequence number in the high half
__device__ __forceinline__ void st_slot(uint2* p, uint32_t data, uint32_t seq) {
  peer_slot_store(p, data, seq);
}
__device__ __forceinline__ uint2 ld_slot(const uint2* p) {
  return peer_slot_load(p);
}

__global__ void __launch_bounds__(kPeerThreads)
bqq_peer_gather_kernel(const PeerArgs a) {
  __shared__ int s_giveup;
  // started as a programmatic dependent of the kernel that produces the slice: wait for the producer
  // before reading the slice.  When the producer sends the slice itself (src == NULL) the polling below
  // may run while the producer still works, and the wait moves to the end.
  if (a.src) asm volatile("griddepcontrol.wait;" ::: "memory");
  unsigned* mine = reinterpret_cast<unsigned*>(a.regions[a.rank]);
  const int tid = threadIdx.x;
  const long long gtid = (long long)blockIdx.x * kPeerThreads + tid, gthreads = (long long)gridDim.x * kPeerThreads;
  const unsigned count = *reinterpret_cast<volatile unsigned*>(mine) + 1u;   // gathers on this group so far
  const unsigned e = count | 0x80000000u;             // sequence number: never the zero of a fresh slot
  const unsigned long long half = (count & 1u) * a.half_bytes;
  const long long grow = (long long)a.row_words * a.world;                // words of one gathered row
  if (tid == 0) s_giveup = 0;
  __syncthreads();

  // send: my words into everybody's slots (my own included)
  const long long nsend = a.src ? (long long)a.rows * a.row_words : 0;
  for (long long w = gtid; w < nsend; w += gthreads) {
    const long long r = w / a.row_words, c = w - r * a.row_words;
    const uint32_t data = a.src[r * a.ld_src + c];
    const long long slot = r * grow + (long long)a.rank * a.row_words + c;
    for (int q = 0; q < a.world; ++q)
      st_slot(reinterpret_cast<uint2*>(a.regions[q] + kPeerCtrlBytes + half) + slot, data, e);
  }

  // receive: poll every slot of my region
  const uint2* slots = reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(mine) + kPeerCtrlBytes + half);
  const long long nrecv = (long long)a.rows * grow;
  // four slots per round, their loads in flight together; a slot that has not arrived yet is polled on its own
  for (long long w0 = gtid; w0 < nrecv; w0 += 4 * gthreads) {
    uint2 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long w = w0 + k * gthreads;
      v[k] = w < nrecv ? ld_slot(slots + w) : make_uint2(0u, e);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long w = w0 + k * gthreads;
      if (w >= nrecv) break;
      if (v[k].y != e) {
        const long long t0 = clock64();
        while (v[k].y != e && !*reinterpret_cast<volatile int*>(&s_giveup)) {
          if (clock64() - t0 > a.wait_cycles) { s_giveup = 1; break; }
          __nanosleep(32);
          v[k] = ld_slot(slots + w);
        }
      }
      const long long r = w / grow, c = w - r * grow;
      a.out[r * a.ld_out + c] = v[k].x;
    }
  }
  __syncthreads();
  // every slot has arrived, so a sending producer has issued all its stores; it must also have ended
  // before this grid ends, because later kernels only wait for this one
  if (!a.src) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the next kernel of the stream may become resident
  if (s_giveup && tid == 0) atomicExch(mine + 1, 1u);

  // the last block to finish advances the sequence number (every block has read it by then)
  __threadfence();
  if (tid == 0 && atomicAdd(mine + 2, 1u) == gridDim.x - 1) {
    mine[2] = 0u;
    *reinterpret_cast<volatile unsigned*>(mine) = count;
  }
}

// a region = control words + two halves of 8-byte slots (one per 32-bit word of the largest gathered result)
size_t peer_half_bytes(size_t gather_bytes) { return (2 * gather_bytes + 255) / 256 * 256; }

}  // namespace bqq

using namespace bqq;

extern "C" {

size_t bqq_peer_region_bytes(size_t gather_bytes) { return kPeerCtrlBytes + 2 * peer_half_bytes(gather_bytes); }

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

// y_local == NULL: receive only (the slices are sent by the kernels that produce them)
static int peer_gather_launch(const BqqPeerGroup* g, const void* y_local, int dtype, int rows, int64_t n_local,
                              int64_t ldy, void* gathered, int64_t ld_gathered, void* stream) {
  if (!g) return BQQ_ERR_NULL;
  if (g->world < 1 || g->world > BQQ_MAX_PEERS || g->rank < 0 || g->rank >= g->world) return BQQ_ERR_BAD_SHAPE;
  const size_t es = dtype_size(dtype);
  if (!es) return BQQ_ERR_DTYPE;
  if (!gathered) return BQQ_ERR_NULL;
  if (rows <= 0 || n_local <= 0 || ldy < n_local || ld_gathered < n_local * g->world) return BQQ_ERR_BAD_SHAPE;
  if ((size_t)rows * n_local * g->world * es > g->gather_bytes) return BQQ_ERR_WORKSPACE;
  if (((size_t)n_local * es) % 4 || ((size_t)ldy * es) % 4 || ((size_t)ld_gathered * es) % 4 ||
      (y_local && ((uintptr_t)y_local & 3)) || ((uintptr_t)gathered & 3))
    return BQQ_ERR_MISALIGNED;                                  // slices travel as 32-bit words
  PeerArgs a;
  for (int q = 0; q < g->world; ++q) {
    if (!g->regions[q]) return BQQ_ERR_NULL;
    a.regions[q] = reinterpret_cast<uint8_t*>(g->regions[q]);
  }
  a.src = reinterpret_cast<const uint32_t*>(y_local);
  a.out = reinterpret_cast<uint32_t*>(gathered);
  a.rank = g->rank; a.world = g->world; a.rows = rows;
  a.row_words = (int)((size_t)n_local * es / 4);
  a.ld_src = (long long)((size_t)ldy * es / 4);
  a.ld_out = (long long)((size_t)ld_gathered * es / 4);
  a.half_bytes = peer_half_bytes(g->gather_bytes);
  a.wait_cycles = g->wait_cycles ? (long long)g->wait_cycles : kPeerWaitBudget;
  const long long words = (long long)rows * a.row_words * g->world;
  int blocks = (int)((words + 2 * kPeerThreads - 1) / (2 * kPeerThreads));
  blocks = blocks < 1 ? 1 : (blocks > kPeerMaxBlocks ? kPeerMaxBlocks : blocks);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kPeerThreads);
  cfg.stream = (cudaStream_t)stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, bqq_peer_gather_kernel, a) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return launch_status();
}

int bqq_peer_gather(const BqqPeerGroup* g, const void* y_local, int dtype, int rows, int64_t n_local, int64_t ldy,
                    void* gathered, int64_t ld_gathered, void* stream) {
  if (!y_local) return BQQ_ERR_NULL;
  return peer_gather_launch(g, y_local, dtype, rows, n_local, ldy, gathered, ld_gathered, stream);
}

int bqq_forward_decode_gathered(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y_local,
                                int y_dtype, int64_t ldy, const BqqFusion* fusion, const BqqPeerGroup* g, void* gathered,
                                int64_t ld_gathered, void* workspace, size_t workspace_bytes, void* stream) {
  if (!layer || !g || !gathered) return BQQ_ERR_NULL;
  if (g->world < 1 || g->world > BQQ_MAX_PEERS || g->rank < 0 || g->rank >= g->world) return BQQ_ERR_BAD_SHAPE;
  if (M <= 0 || M > BQQ_DECODE_MAX_M) return BQQ_ERR_BAD_SHAPE;
  for (int q = 0; q < g->world; ++q)
    if (!g->regions[q]) return BQQ_ERR_NULL;
  Geom geo(layer->dims);
  const size_t es = dtype_size(y_dtype);
  if (!es) return BQQ_ERR_DTYPE;
  if ((size_t)M * geo.out_features() * g->world * es > g->gather_bytes) return BQQ_ERR_WORKSPACE;
  if (ld_gathered < (int64_t)geo.out_features() * g->world) return BQQ_ERR_BAD_SHAPE;
  // same argument checks as bqq_forward_decode, then ONE launch: the decode kernel's computing CTAs store their
  // finished row patches into every rank's region, a few more CTAs of the same grid wait for the peers' row
  // patches and write the gathered rows
  return bqq_forward_decode_peer(layer, x, x_dtype, M, ldx, y_local, y_dtype, ldy, workspace, workspace_bytes, stream, g,
                                 fusion, gathered, ld_gathered);
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
