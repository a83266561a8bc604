// Load-time packer: bool Y/Z (one byte per entry) <-> 32-bit bit planes, row
// sums, coefficient records.  Device kernels plus single-threaded host twins
// that share the index arithmetic below.
//
// Replaces PackedBinaryQuadratic.from_unpacked / _np_packbits / _unpack_to_bool
// of the reference (neural_network_compression/src/bqq_modules.py:99-169).
#include "bqq_common.cuh"

namespace bqq {

// ---- index arithmetic shared by host and device ---------------------------

// Word of the Z planes at flat index w: which (i, n, qw, k) it holds.
struct ZWordIdx { int i, n, qw, k; };
__host__ __device__ inline ZWordIdx z_word_index(const Geom& g, size_t w) {
  ZWordIdx o;
  int sub = (int)(w % kGroup); w /= kGroup;
  o.k = (int)(w % g.RP); w /= g.RP;
  o.qw = (int)(w % g.QW); w /= g.QW;
  int s = (int)(w % g.NS); w /= g.NS;
  o.i = (int)w;
  o.n = s * kGroup + sub;
  return o;
}
struct YWordIdx { int i, n, kw, p; };
__host__ __device__ inline YWordIdx y_word_index(const Geom& g, size_t w) {
  YWordIdx o;
  int sub = (int)(w % kGroup); w /= kGroup;
  o.p = (int)(w % g.PP); w /= g.PP;
  o.kw = (int)(w % g.RW); w /= g.RW;
  int s = (int)(w % g.NS); w /= g.NS;
  o.i = (int)w;
  o.n = s * kGroup + sub;
  return o;
}
__host__ __device__ inline size_t z_word_offset(const Geom& g, int i, int n, int qw, int k) {
  return ((((size_t)i * g.NS + n / kGroup) * g.QW + qw) * g.RP + k) * kGroup + (n % kGroup);
}
__host__ __device__ inline size_t y_word_offset(const Geom& g, int i, int n, int kw, int p) {
  return ((((size_t)i * g.NS + n / kGroup) * g.RW + kw) * g.PP + p) * kGroup + (n % kGroup);
}
// Offsets into the reference tensors Y [bw,rw,cw,P,r] and Z [bw,rw,cw,r,Q].
__host__ __device__ inline size_t y_bool_offset(const Geom& g, int b, int i, int j, int p, int k) {
  return ((((size_t)b * g.rw + i) * g.cw + j) * g.P + p) * g.r + k;
}
__host__ __device__ inline size_t z_bool_offset(const Geom& g, int b, int i, int j, int k, int q) {
  return ((((size_t)b * g.rw + i) * g.cw + j) * g.r + k) * g.Q + q;
}

__host__ __device__ inline uint32_t make_z_word(const Geom& g, const uint8_t* Z, size_t w) {
  ZWordIdx x = z_word_index(g, w);
  if (x.n >= g.NPB || x.k >= g.r) return 0u;
  int j = x.n / g.bw, b = x.n % g.bw;
  const uint8_t* src = Z + z_bool_offset(g, b, x.i, j, x.k, 0);
  uint32_t word = 0;
  int q0 = x.qw * 32;
  int nq = g.Q - q0 < 32 ? g.Q - q0 : 32;
  for (int t = 0; t < nq; ++t) word |= (uint32_t)(src[q0 + t] != 0) << t;
  return word;
}
__host__ __device__ inline uint32_t make_y_word(const Geom& g, const uint8_t* Y, size_t w) {
  YWordIdx x = y_word_index(g, w);
  if (x.n >= g.NPB || x.p >= g.P) return 0u;
  int j = x.n / g.bw, b = x.n % g.bw;
  const uint8_t* src = Y + y_bool_offset(g, b, x.i, j, x.p, 0);
  uint32_t word = 0;
  int k0 = x.kw * 32;
  int nk = g.r - k0 < 32 ? g.r - k0 : 32;
  for (int t = 0; t < nk; ++t) word |= (uint32_t)(src[k0 + t] != 0) << t;
  return word;
}

// Same words, sourced from the reference's big-endian uint8 packs
// Y_packed [bw,rw,cw,P,k8], Z_packed [bw,rw,cw,Q,k8] (Z transposed: rank packed).
__host__ __device__ inline uint32_t bit_be(const uint8_t* row, int idx) {
  return (row[idx >> 3] >> (7 - (idx & 7))) & 1u;
}
__host__ __device__ inline uint32_t make_z_word_u8(const Geom& g, const uint8_t* Zp8, size_t w) {
  ZWordIdx x = z_word_index(g, w);
  if (x.n >= g.NPB || x.k >= g.r) return 0u;
  int j = x.n / g.bw, b = x.n % g.bw;
  int k8 = (g.r + 7) / 8;
  const uint8_t* patch = Zp8 + (((size_t)b * g.rw + x.i) * g.cw + j) * (size_t)g.Q * k8;
  uint32_t word = 0;
  int q0 = x.qw * 32;
  int nq = g.Q - q0 < 32 ? g.Q - q0 : 32;
  for (int t = 0; t < nq; ++t) word |= bit_be(patch + (size_t)(q0 + t) * k8, x.k) << t;
  return word;
}
__host__ __device__ inline uint32_t make_y_word_u8(const Geom& g, const uint8_t* Yp8, size_t w) {
  YWordIdx x = y_word_index(g, w);
  if (x.n >= g.NPB || x.p >= g.P) return 0u;
  int j = x.n / g.bw, b = x.n % g.bw;
  int k8 = (g.r + 7) / 8;
  const uint8_t* row = Yp8 + ((((size_t)b * g.rw + x.i) * g.cw + j) * g.P + x.p) * (size_t)k8;
  uint32_t word = 0;
  int k0 = x.kw * 32;
  int nk = g.r - k0 < 32 ? g.r - k0 : 32;
  for (int t = 0; t < nk; ++t) word |= bit_be(row, k0 + t) << t;
  return word;
}

// ---- device kernels --------------------------------------------------------

__global__ void pack_z_kernel(Geom g, const uint8_t* __restrict__ Z, uint32_t* __restrict__ zp, size_t nwords) {
  for (size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x; w < nwords; w += (size_t)gridDim.x * blockDim.x)
    zp[w] = make_z_word(g, Z, w);
}
__global__ void pack_y_kernel(Geom g, const uint8_t* __restrict__ Y, uint32_t* __restrict__ yp, size_t nwords) {
  for (size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x; w < nwords; w += (size_t)gridDim.x * blockDim.x)
    yp[w] = make_y_word(g, Y, w);
}
__global__ void repack_z_kernel(Geom g, const uint8_t* __restrict__ Z8, uint32_t* __restrict__ zp, size_t nwords) {
  for (size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x; w < nwords; w += (size_t)gridDim.x * blockDim.x)
    zp[w] = make_z_word_u8(g, Z8, w);
}
__global__ void repack_y_kernel(Geom g, const uint8_t* __restrict__ Y8, uint32_t* __restrict__ yp, size_t nwords) {
  for (size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x; w < nwords; w += (size_t)gridDim.x * blockDim.x)
    yp[w] = make_y_word_u8(g, Y8, w);
}
// ysum [bw,rw,cw,P]: sum over k of Y;  zsum [bw,rw,cw,Q]: sum over k of Z.
__global__ void ysum_kernel(Geom g, const uint8_t* __restrict__ Y, uint8_t* __restrict__ ysum, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    const uint8_t* row = Y + t * g.r;
    int s = 0;
    for (int k = 0; k < g.r; ++k) s += row[k] != 0;
    ysum[t] = (uint8_t)s;
  }
}
__global__ void zsum_kernel(Geom g, const uint8_t* __restrict__ Z, uint8_t* __restrict__ zsum, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    size_t patch = t / g.Q;
    int q = (int)(t % g.Q);
    const uint8_t* base = Z + patch * (size_t)g.r * g.Q + q;
    int s = 0;
    for (int k = 0; k < g.r; ++k) s += base[(size_t)k * g.Q] != 0;
    zsum[t] = (uint8_t)s;
  }
}
__global__ void unpack_y_kernel(Geom g, const uint32_t* __restrict__ yp, uint8_t* __restrict__ Y, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    size_t u = t;
    int k = (int)(u % g.r); u /= g.r;
    int p = (int)(u % g.P); u /= g.P;
    int j = (int)(u % g.cw); u /= g.cw;
    int i = (int)(u % g.rw); u /= g.rw;
    int b = (int)u;
    uint32_t w = yp[y_word_offset(g, i, j * g.bw + b, k >> 5, p)];
    Y[t] = (uint8_t)((w >> (k & 31)) & 1u);
  }
}
__global__ void unpack_z_kernel(Geom g, const uint32_t* __restrict__ zp, uint8_t* __restrict__ Z, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    size_t u = t;
    int q = (int)(u % g.Q); u /= g.Q;
    int k = (int)(u % g.r); u /= g.r;
    int j = (int)(u % g.cw); u /= g.cw;
    int i = (int)(u % g.rw); u /= g.rw;
    int b = (int)u;
    uint32_t w = zp[z_word_offset(g, i, j * g.bw + b, q >> 5, k)];
    Z[t] = (uint8_t)((w >> (q & 31)) & 1u);
  }
}

// coef [rw][NS*4][4] = (a, b, c, d if bit 0 else 0)
__global__ void pack_coef_kernel(Geom g, const void* __restrict__ a, const void* __restrict__ b,
                                 const void* __restrict__ c, const void* __restrict__ d, int dt,
                                 float4* __restrict__ coef, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    int nn = (int)(t % ((size_t)g.NS * kGroup));
    int i = (int)(t / ((size_t)g.NS * kGroup));
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (nn < g.NPB) {
      int j = nn / g.bw, bit = nn % g.bw;
      size_t src = ((size_t)bit * g.rw + i) * g.cw + j;
      v.x = load_as_float(a, src, dt);
      v.y = load_as_float(b, src, dt);
      v.z = load_as_float(c, src, dt);
      if (bit == 0) v.w = load_as_float(d, (size_t)i * g.cw + j, dt);
    }
    coef[t] = v;
    // running maxima for the bound on |W| (non-negative floats order like ints)
    int* tr = reinterpret_cast<int*>(coef + n);
    atomicMax(tr, __float_as_int(fabsf(v.x) + fabsf(v.y) + fabsf(v.z)));
    atomicMax(tr + 1, __float_as_int(fabsf(v.w)));
  }
}

static inline int grid_for(size_t n, int block) {
  size_t gsz = (n + block - 1) / block;
  if (gsz > 148u * 32u) gsz = 148u * 32u;
  if (gsz == 0) gsz = 1;
  return (int)gsz;
}

}  // namespace bqq

using namespace bqq;

extern "C" {

size_t bqq_zplane_words(const BqqDims* dims) {
  if (check_dims(dims) != BQQ_OK) return 0;
  return Geom(*dims).z_words();
}
size_t bqq_yplane_words(const BqqDims* dims) {
  if (check_dims(dims) != BQQ_OK) return 0;
  return Geom(*dims).y_words();
}
size_t bqq_coeff_floats(const BqqDims* dims) {
  if (check_dims(dims) != BQQ_OK) return 0;
  return Geom(*dims).coef_floats();
}
size_t bqq_algorithmic_bytes(const BqqDims* dims) {
  if (check_dims(dims) != BQQ_OK) return 0;
  const BqqDims& d = *dims;
  size_t bits = (size_t)d.bw * d.rw * d.cw * ((size_t)d.P * d.r + (size_t)d.r * d.Q);
  return bits / 8 + 4 * (size_t)d.rw * d.cw * (3 * (size_t)d.bw + 1);
}

int bqq_pack_planes(const uint8_t* Y_bool, const uint8_t* Z_bool, const BqqDims* dims,
                    uint32_t* zplanes, uint32_t* yplanes, uint8_t* ysum, uint8_t* zsum, void* stream) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_bool || !Z_bool || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  cudaStream_t st = (cudaStream_t)stream;
  size_t nz = g.z_words(), ny = g.y_words();
  pack_z_kernel<<<grid_for(nz, 256), 256, 0, st>>>(g, Z_bool, zplanes, nz);
  pack_y_kernel<<<grid_for(ny, 256), 256, 0, st>>>(g, Y_bool, yplanes, ny);
  if (ysum) {
    size_t n = (size_t)g.bw * g.rw * g.cw * g.P;
    ysum_kernel<<<grid_for(n, 256), 256, 0, st>>>(g, Y_bool, ysum, n);
  }
  if (zsum) {
    size_t n = (size_t)g.bw * g.rw * g.cw * g.Q;
    zsum_kernel<<<grid_for(n, 256), 256, 0, st>>>(g, Z_bool, zsum, n);
  }
  return launch_status();
}

int bqq_unpack_planes(const uint32_t* zplanes, const uint32_t* yplanes, const BqqDims* dims,
                      uint8_t* Y_bool, uint8_t* Z_bool, void* stream) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_bool || !Z_bool || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  cudaStream_t st = (cudaStream_t)stream;
  size_t ny = (size_t)g.bw * g.rw * g.cw * g.P * g.r;
  size_t nz = (size_t)g.bw * g.rw * g.cw * g.r * g.Q;
  unpack_y_kernel<<<grid_for(ny, 256), 256, 0, st>>>(g, yplanes, Y_bool, ny);
  unpack_z_kernel<<<grid_for(nz, 256), 256, 0, st>>>(g, zplanes, Z_bool, nz);
  return launch_status();
}

int bqq_repack_u8_planes(const uint8_t* Y_packed, const uint8_t* Z_packed, const BqqDims* dims,
                         uint32_t* zplanes, uint32_t* yplanes, void* stream) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_packed || !Z_packed || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  cudaStream_t st = (cudaStream_t)stream;
  size_t nz = g.z_words(), ny = g.y_words();
  repack_z_kernel<<<grid_for(nz, 256), 256, 0, st>>>(g, Z_packed, zplanes, nz);
  repack_y_kernel<<<grid_for(ny, 256), 256, 0, st>>>(g, Y_packed, yplanes, ny);
  return launch_status();
}

int bqq_pack_planes_host(const uint8_t* Y_bool, const uint8_t* Z_bool, const BqqDims* dims,
                         uint32_t* zplanes, uint32_t* yplanes, uint8_t* ysum, uint8_t* zsum) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_bool || !Z_bool || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  size_t nz = g.z_words(), ny = g.y_words();
  for (size_t w = 0; w < nz; ++w) zplanes[w] = make_z_word(g, Z_bool, w);
  for (size_t w = 0; w < ny; ++w) yplanes[w] = make_y_word(g, Y_bool, w);
  if (ysum) {
    size_t n = (size_t)g.bw * g.rw * g.cw * g.P;
    for (size_t t = 0; t < n; ++t) {
      int s = 0;
      for (int k = 0; k < g.r; ++k) s += Y_bool[t * g.r + k] != 0;
      ysum[t] = (uint8_t)s;
    }
  }
  if (zsum) {
    size_t n = (size_t)g.bw * g.rw * g.cw * g.Q;
    for (size_t t = 0; t < n; ++t) {
      size_t patch = t / g.Q;
      int q = (int)(t % g.Q);
      int s = 0;
      for (int k = 0; k < g.r; ++k) s += Z_bool[patch * (size_t)g.r * g.Q + (size_t)k * g.Q + q] != 0;
      zsum[t] = (uint8_t)s;
    }
  }
  return BQQ_OK;
}

int bqq_unpack_planes_host(const uint32_t* zplanes, const uint32_t* yplanes, const BqqDims* dims,
                           uint8_t* Y_bool, uint8_t* Z_bool) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_bool || !Z_bool || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  for (int b = 0; b < g.bw; ++b)
    for (int i = 0; i < g.rw; ++i)
      for (int j = 0; j < g.cw; ++j) {
        int n = j * g.bw + b;
        for (int p = 0; p < g.P; ++p)
          for (int k = 0; k < g.r; ++k)
            Y_bool[y_bool_offset(g, b, i, j, p, k)] =
                (uint8_t)((yplanes[y_word_offset(g, i, n, k >> 5, p)] >> (k & 31)) & 1u);
        for (int k = 0; k < g.r; ++k)
          for (int q = 0; q < g.Q; ++q)
            Z_bool[z_bool_offset(g, b, i, j, k, q)] =
                (uint8_t)((zplanes[z_word_offset(g, i, n, q >> 5, k)] >> (q & 31)) & 1u);
      }
  return BQQ_OK;
}

int bqq_pack_coeffs(const void* a, const void* b, const void* c, const void* d, int dtype,
                    const BqqDims* dims, float* coef, void* stream) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!a || !b || !c || !d || !coef) return BQQ_ERR_NULL;
  if (!dtype_size(dtype)) return BQQ_ERR_DTYPE;
  if (((uintptr_t)coef & 15) != 0) return BQQ_ERR_MISALIGNED;
  Geom g(*dims);
  size_t n = g.coef_records();
  if (cudaMemsetAsync(coef + n * 4, 0, 16, (cudaStream_t)stream) != cudaSuccess) return BQQ_ERR_CUDA;
  pack_coef_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
      g, a, b, c, d, dtype, reinterpret_cast<float4*>(coef), n);
  return launch_status();
}

}  // extern "C"
