// Decode forward for callers that cannot allocate device memory.
//
// bqq_forward_decode needs a caller-provided workspace.  Some callers have no way
// to provide one: code that runs inside somebody else's stream-ordered section and
// is not allowed to call cudaMalloc (or an allocating library routine) there,
// plugin hosts that hand an operator only its input and output buffers, and
// start-up paths that run before any allocator is configured.  For them this file
// keeps the workspace in a fixed device array that is part of the loaded library
// image: every GPU that loads the library holds those bytes until the process exits,
// which is why the size is a modest, fixed maximum.
#include <mutex>

#include "bqq_common.cuh"

// argument checks shared with bqq_forward_decode (bqq_api.cu)
int bqq_decode_check_args(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y, int y_dtype,
                          int64_t ldy, const BqqFusion* fusion);

namespace bqq {

constexpr size_t kNoAllocBytes = BQQ_NOALLOC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle for the runtime, not
// a device address: the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

static void* g_scratch_ptr[kMaxDevices];
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device (looked up on first use).
static int scratch_address(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  if (dev < 0 || dev >= kMaxDevices) return BQQ_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_noalloc_scratch) != cudaSuccess || !ptr) {
      cudaGetLastError();
      return BQQ_ERR_CUDA;
    }
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return BQQ_OK;
}

}  // namespace bqq

using namespace bqq;

extern "C" {

size_t bqq_noalloc_scratch_bytes(void) { return kNoAllocBytes; }

int bqq_forward_decode_noalloc(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                               int y_dtype, int64_t ldy, void* stream) {
  // every argument check comes before anything is enqueued: a rejected call leaves the stream untouched
  int rc = bqq_decode_check_args(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, nullptr);
  if (rc) return rc;
  const size_t need = decode_workspace_bytes(&layer->dims, M);
  if (need == 0) return BQQ_ERR_UNSUPPORTED;
  if (need > kNoAllocBytes) return BQQ_ERR_SCRATCH_LIMIT;      // layer / batch too large for the fixed array
  void* scratch = nullptr;
  rc = scratch_address(&scratch);
  if (rc) return rc;
  // The array keeps whatever the previous call left.  The kernels overwrite everything they
  // read except the completion counters, which must start at zero: clear them here.  The last
  // counter word is the "a bounded wait gave up" status; it is left alone, so that it stays set
  // until bqq_noalloc_status has reported it.
  if (cudaMemsetAsync(scratch, 0, decode_counter_bytes() - 4, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return BQQ_ERR_CUDA;
  }
  // same argument checks and launch as the entry point with a caller workspace
  return bqq_forward_decode(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, scratch, kNoAllocBytes, stream);
}

// Synchronises `stream` and reports whether any call on the current device since the last report hit a
// bounded device-side wait that gave up (BQQ_ERR_TIMEOUT: the outputs of those calls are invalid).
// Reporting clears the word.  Like the entry point itself it allocates nothing.
int bqq_noalloc_status(void* stream) {
  void* scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc) return rc;
  unsigned st = 0;
  cudaStream_t s = (cudaStream_t)stream;
  void* word = reinterpret_cast<char*>(scratch) + decode_counter_bytes() - 4;
  if (cudaMemcpyAsync(&st, word, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return BQQ_ERR_CUDA;
  }
  if (st && (cudaMemsetAsync(word, 0, 4, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)) {
    cudaGetLastError();
    return BQQ_ERR_CUDA;
  }
  return st ? BQQ_ERR_TIMEOUT : BQQ_OK;
}

}  // extern "C"
