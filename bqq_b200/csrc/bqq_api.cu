// C ABI of the library: argument checks and dispatch (see include/bqq_b200.h).
#include "bqq_common.cuh"

using namespace bqq;

static int check_layer(const BqqLayer* L) {
  if (!L) return BQQ_ERR_NULL;
  int rc = check_dims(&L->dims);
  if (rc) return rc;
  if (!L->zplanes || !L->yplanes || !L->a || !L->b || !L->c || !L->d) return BQQ_ERR_NULL;
  if (((uintptr_t)L->zplanes & 15) || ((uintptr_t)L->yplanes & 15)) return BQQ_ERR_MISALIGNED;
  if (!dtype_size(L->coef_dtype)) return BQQ_ERR_DTYPE;
  if (L->bias && !dtype_size(L->bias_dtype)) return BQQ_ERR_DTYPE;
  return BQQ_OK;
}

static int check_io(const BqqLayer* L, const void* x, int x_dtype, int M, int64_t ldx, void* y, int y_dtype,
                    int64_t ldy) {
  if (!x || !y) return BQQ_ERR_NULL;
  if (!dtype_size(x_dtype) || !dtype_size(y_dtype)) return BQQ_ERR_DTYPE;
  if (M <= 0) return BQQ_ERR_BAD_SHAPE;
  Geom g(L->dims);
  if (ldx < g.in_features() || ldy < g.out_features()) return BQQ_ERR_BAD_SHAPE;
  if (((uintptr_t)x % dtype_size(x_dtype)) || ((uintptr_t)y % dtype_size(y_dtype))) return BQQ_ERR_MISALIGNED;
  return BQQ_OK;
}

// Argument checks of the decode entry points (nothing is enqueued); not exported in the header.
int bqq_decode_check_args(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y, int y_dtype,
                          int64_t ldy, const BqqFusion* fusion) {
  int rc = check_layer(layer);
  if (rc) return rc;
  rc = check_io(layer, x, x_dtype, M, ldx, y, y_dtype, ldy);
  if (rc) return rc;
  if (M > BQQ_DECODE_MAX_M) return BQQ_ERR_UNSUPPORTED;
  if (fusion) {
    Geom g(layer->dims);
    if (fusion->prologue < BQQ_PRO_NONE || fusion->prologue > BQQ_PRO_SWIGLU) return BQQ_ERR_BAD_SHAPE;
    if (fusion->prologue == BQQ_PRO_RMSNORM && (!fusion->norm_weight || !dtype_size(fusion->norm_dtype)))
      return fusion->norm_weight ? BQQ_ERR_DTYPE : BQQ_ERR_NULL;
    if (fusion->prologue == BQQ_PRO_SWIGLU && ldx < 2 * (int64_t)g.in_features()) return BQQ_ERR_BAD_SHAPE;
    if (fusion->residual && (!dtype_size(fusion->residual_dtype) || fusion->ld_residual < g.out_features()))
      return dtype_size(fusion->residual_dtype) ? BQQ_ERR_BAD_SHAPE : BQQ_ERR_DTYPE;
  }
  return BQQ_OK;
}

// bqq_forward_decode, optionally with the peer stores of bqq_forward_decode_gathered (not exported in the header)
int bqq_forward_decode_peer(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y, int y_dtype,
                            int64_t ldy, void* workspace, size_t workspace_bytes, void* stream, const BqqPeerGroup* peer,
                            const BqqFusion* fusion = nullptr, void* gathered = nullptr, int64_t ld_gathered = 0) {
  const int rc = bqq_decode_check_args(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, fusion);
  if (rc) return rc;
  return decode_launch(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes,
                       (cudaStream_t)stream, peer, fusion, gathered, ld_gathered);
}

extern "C" {

int bqq_abi_version(void) { return BQQ_ABI_VERSION; }

const char* bqq_strerror(int rc) {
  switch (rc) {
    case BQQ_OK: return "ok";
    case BQQ_ERR_NULL: return "a required pointer is NULL";
    case BQQ_ERR_BAD_SHAPE: return "a dimension is non-positive or inconsistent";
    case BQQ_ERR_UNSUPPORTED: return "patch geometry or batch size outside the kernel limits";
    case BQQ_ERR_MISALIGNED: return "a pointer or leading dimension is misaligned";
    case BQQ_ERR_WORKSPACE: return "workspace missing or too small";
    case BQQ_ERR_DTYPE: return "unknown element type code";
    case BQQ_ERR_CUDA: return "a CUDA call failed";
    case BQQ_ERR_TIMEOUT: return "a bounded device-side wait gave up";
    case BQQ_ERR_NO_DEVICE: return "no sm_100 GPU is current";
    case BQQ_ERR_SCRATCH_LIMIT:
      return "layer and batch need more scratch than the built-in array of the no-allocation entry point";
    default: return "unknown bqq error code";
  }
}

int bqq_device_supported(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}

size_t bqq_decode_workspace_bytes(const BqqDims* dims, int M) {
  if (check_dims(dims) != BQQ_OK || M <= 0) return 0;
  return decode_workspace_bytes(dims, M > BQQ_DECODE_MAX_M ? BQQ_DECODE_MAX_M : M);
}

int bqq_forward_decode(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                       int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes, void* stream) {
  return bqq_forward_decode_peer(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes, stream, nullptr);
}

int bqq_forward_decode_fused(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                             int y_dtype, int64_t ldy, const BqqFusion* fusion, void* workspace, size_t workspace_bytes,
                             void* stream) {
  return bqq_forward_decode_peer(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes, stream, nullptr,
                                 fusion);
}

size_t bqq_prefill_workspace_bytes(const BqqDims* dims, int M) {
  if (check_dims(dims) != BQQ_OK || M <= 0) return 0;
  return prefill_workspace_bytes(dims, M);
}

int bqq_forward_prefill(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y,
                        int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  rc = check_io(layer, x, x_dtype, M, ldx, y, y_dtype, ldy);
  if (rc) return rc;
  return prefill_launch(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes,
                        (cudaStream_t)stream);
}

size_t bqq_forward_workspace_bytes(const BqqDims* dims, int M) {
  return M <= BQQ_DECODE_MAX_M ? bqq_decode_workspace_bytes(dims, M) : bqq_prefill_workspace_bytes(dims, M);
}

int bqq_forward(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx, void* y, int y_dtype,
                int64_t ldy, void* workspace, size_t workspace_bytes, void* stream) {
  if (M <= BQQ_DECODE_MAX_M)
    return bqq_forward_decode(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes, stream);
  return bqq_forward_prefill(layer, x, x_dtype, M, ldx, y, y_dtype, ldy, workspace, workspace_bytes, stream);
}

// One 32-bit word of device memory, read back after synchronising the stream.
static int read_status_word(const void* word, void* stream) {
  unsigned st = 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemcpyAsync(&st, word, 4, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return BQQ_ERR_CUDA;
  }
  return st ? BQQ_ERR_TIMEOUT : BQQ_OK;
}

int bqq_decode_status(const void* workspace, void* stream) {
  if (!workspace) return BQQ_ERR_NULL;
  return read_status_word(reinterpret_cast<const char*>(workspace) + decode_counter_bytes() - 4, stream);
}

int bqq_prefill_status(const void* workspace, void* stream) {
  if (!workspace) return BQQ_ERR_NULL;
  return read_status_word(workspace, stream);
}

int bqq_decode_launches(const BqqDims* dims, int M) {
  if (int rc = check_dims(dims)) return rc;
  if (M <= 0 || M > BQQ_DECODE_MAX_M) return BQQ_ERR_BAD_SHAPE;
  return decode_launches(dims, M);
}

// Device-visible address of pinned, mapped host memory (cudaHostAlloc / cudaHostRegister), or NULL.
static void* mapped_device_pointer(const void* host) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, host) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (at.type != cudaMemoryTypeHost || !at.devicePointer) return nullptr;
  return at.devicePointer;
}

// Rows of x from mapped host memory into the device staging buffer: 16 bytes per thread where the
// alignment allows, 2 bytes otherwise.  Waits for the preceding kernel of the stream before writing.
__global__ void __launch_bounds__(256)
stage_host_rows_kernel(const uint8_t* __restrict__ src, long long ld_src, uint8_t* __restrict__ dst, long long row_bytes,
                       int rows, int vec) {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const long long tid = (long long)blockIdx.x * 256 + threadIdx.x, n = (long long)gridDim.x * 256;
  if (vec) {
    const long long per_row = row_bytes >> 4;
    for (long long e = tid; e < per_row * rows; e += n) {
      const long long r = e / per_row, c = e - r * per_row;
      reinterpret_cast<uint4*>(dst + r * row_bytes)[c] = reinterpret_cast<const uint4*>(src + r * ld_src)[c];
    }
  } else {
    const long long per_row = row_bytes >> 1;
    for (long long e = tid; e < per_row * rows; e += n) {
      const long long r = e / per_row, c = e - r * per_row;
      reinterpret_cast<uint16_t*>(dst + r * row_bytes)[c] = reinterpret_cast<const uint16_t*>(src + r * ld_src)[c];
    }
  }
}

static inline size_t host_stage_bytes(size_t rows, size_t cols, int dtype) {
  return (rows * cols * dtype_size(dtype) + 255) / 256 * 256;
}

size_t bqq_forward_host_workspace_bytes(const BqqDims* dims, int M, int x_dtype, int y_dtype) {
  if (check_dims(dims) != BQQ_OK || M <= 0 || !dtype_size(x_dtype) || !dtype_size(y_dtype)) return 0;
  const size_t inner = bqq_forward_workspace_bytes(dims, M);
  if (!inner) return 0;
  Geom g(*dims);
  return inner + host_stage_bytes(M, g.in_features(), x_dtype) + host_stage_bytes(M, g.out_features(), y_dtype);
}

int bqq_forward_host(const BqqLayer* layer, const void* x_host, int x_dtype, int M, int64_t ldx, void* y_host,
                     int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  rc = check_io(layer, x_host, x_dtype, M, ldx, y_host, y_dtype, ldy);
  if (rc) return rc;
  if (!workspace) return BQQ_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 255) return BQQ_ERR_MISALIGNED;
  if (workspace_bytes < bqq_forward_host_workspace_bytes(&layer->dims, M, x_dtype, y_dtype)) return BQQ_ERR_WORKSPACE;
  Geom g(layer->dims);
  const size_t inner = bqq_forward_workspace_bytes(&layer->dims, M);
  const size_t xs = dtype_size(x_dtype), ys = dtype_size(y_dtype);
  char* xd = reinterpret_cast<char*>(workspace) + inner;
  char* yd = xd + host_stage_bytes(M, g.in_features(), x_dtype);
  cudaStream_t st = (cudaStream_t)stream;
  // Small batches with pinned, mapped host buffers skip the copy engines (two DMA copies cost more than the
  // decode kernel itself): the kernels read x from and write y to host memory directly.  Layers whose CTAs
  // each read all of x first get it staged on the device by a small kernel.
  if (M <= BQQ_DECODE_MAX_M) {
    void* xm = mapped_device_pointer(x_host);
    void* ym = mapped_device_pointer(y_host);
    if (xm && ym) {
      const void* xin = xm;
      int64_t ld_in = ldx;
      if (decode_launches(&layer->dims, M) == 1) {
        const long long row_bytes = (long long)g.in_features() * xs;
        const int vec = ((row_bytes | (long long)(ldx * xs) | (long long)(uintptr_t)xm | (long long)(uintptr_t)xd) & 15) == 0;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t cfg = {};
        const long long units = (row_bytes >> (vec ? 4 : 1)) * M;
        cfg.gridDim = dim3((unsigned)((units + 255) / 256 > 64 ? 64 : (units + 255) / 256));
        cfg.blockDim = dim3(256);
        cfg.stream = st;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, stage_host_rows_kernel, (const uint8_t*)xm, (long long)(ldx * xs), (uint8_t*)xd, row_bytes,
                               M, vec) != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
        xin = xd;
        ld_in = g.in_features();
      }
      return bqq_forward(layer, xin, x_dtype, M, ld_in, ym, y_dtype, ldy, workspace, inner, stream);
    }
  }
  // the forward's own workspace comes first so that its zero-initialised counters stay where they were
  const size_t xrow = g.in_features() * xs, yrow = g.out_features() * ys;
  cudaError_t ce = (M == 1 || ldx == g.in_features())
                       ? cudaMemcpyAsync(xd, x_host, xrow * M, cudaMemcpyHostToDevice, st)
                       : cudaMemcpy2DAsync(xd, xrow, x_host, ldx * xs, xrow, M, cudaMemcpyHostToDevice, st);
  if (ce != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  rc = bqq_forward(layer, xd, x_dtype, M, g.in_features(), yd, y_dtype, g.out_features(), workspace, inner, stream);
  if (rc) return rc;
  ce = (M == 1 || ldy == g.out_features())
           ? cudaMemcpyAsync(y_host, yd, yrow * M, cudaMemcpyDeviceToHost, st)
           : cudaMemcpy2DAsync(y_host, ldy * ys, yd, yrow, yrow, M, cudaMemcpyDeviceToHost, st);
  if (ce != cudaSuccess) { cudaGetLastError(); return BQQ_ERR_CUDA; }
  return BQQ_OK;
}

int bqq_reconstruct_weight(const BqqLayer* layer, void* W, int w_dtype, float scale, void* stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if (!W) return BQQ_ERR_NULL;
  if (!dtype_size(w_dtype)) return BQQ_ERR_DTYPE;
  return reconstruct_launch(layer, W, nullptr, w_dtype, scale, nullptr, (cudaStream_t)stream);
}

}  // extern "C"
