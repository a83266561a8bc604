// Load-time packer: bool Y/Z (one byte per entry) <-> 32-bit bit planes in the
// fragment order documented in bqq_common.cuh, plus row sums.  Device kernels
// and single-threaded host twins share the index arithmetic below.
//
// Replaces PackedBinaryQuadratic.from_unpacked / _np_packbits / _unpack_to_bool
// of the reference (neural_network_compression/src/bqq_modules.py:99-169).
#include "bqq_common.cuh"

namespace bqq {

// Offsets into the reference tensors Y [bw,rw,cw,P,r] and Z [bw,rw,cw,r,Q].
__host__ __device__ inline size_t y_bool_offset(const Geom& g, int b, int i, int j, int p, int k) {
  return ((((size_t)b * g.rw + i) * g.cw + j) * g.P + p) * g.r + k;
}
__host__ __device__ inline size_t z_bool_offset(const Geom& g, int b, int i, int j, int k, int q) {
  return ((((size_t)b * g.rw + i) * g.cw + j) * g.r + k) * g.Q + q;
}
// Bit idx of a big-endian uint8 pack (element 0 is the MSB of byte 0).
__host__ __device__ inline uint32_t bit_be(const uint8_t* row, int idx) {
  return (row[idx >> 3] >> (7 - (idx & 7))) & 1u;
}

// Source of one binary entry: either bool bytes or the reference's uint8 packs
// (Y_packed [bw,rw,cw,P,k8]; Z_packed [bw,rw,cw,Q,k8], Z transposed so the rank is packed).
struct BitSource {
  const uint8_t* Y;
  const uint8_t* Z;
  int packed_u8;
  __host__ __device__ uint32_t y(const Geom& g, int b, int i, int j, int p, int k) const {
    if (!packed_u8) return Y[y_bool_offset(g, b, i, j, p, k)] != 0;
    const int k8 = (g.r + 7) / 8;
    return bit_be(Y + ((((size_t)b * g.rw + i) * g.cw + j) * g.P + p) * (size_t)k8, k);
  }
  __host__ __device__ uint32_t z(const Geom& g, int b, int i, int j, int k, int q) const {
    if (!packed_u8) return Z[z_bool_offset(g, b, i, j, k, q)] != 0;
    const int k8 = (g.r + 7) / 8;
    return bit_be(Z + ((((size_t)b * g.rw + i) * g.cw + j) * g.Q + q) * (size_t)k8, k);
  }
};

// Decompose a flat word index of a plane [rw][NS][B1][B2][32][4].
struct WordIdx { int i, b, j, blk1, blk2, g, t; };
__host__ __device__ inline WordIdx word_index(const Geom& g, size_t w, int B1, int B2) {
  WordIdx o;
  const int sub = (int)(w % kGroup); w /= kGroup;
  const int lane = (int)(w % 32); w /= 32;
  o.blk2 = (int)(w % B2); w /= B2;
  o.blk1 = (int)(w % B1); w /= B1;
  const int s = (int)(w % g.NS); w /= g.NS;
  o.i = (int)w;
  o.b = s / g.JG;
  o.j = (s % g.JG) * kGroup + sub;
  o.g = lane >> 2;
  o.t = lane & 3;
  return o;
}

__host__ __device__ inline uint32_t make_z_word(const Geom& g, const BitSource& src, size_t w) {
  const WordIdx x = word_index(g, w, g.RT, g.QT);   // blk1 = rt, blk2 = qt
  if (x.j >= g.cw) return 0u;
  uint32_t word = 0;
  for (int e = 0; e < 4; ++e)
    for (int qh = 0; qh < 2; ++qh)
      for (int rr = 0; rr < 4; ++rr) {
        const int k = 32 * x.blk1 + 4 * x.g + rr;
        const int q = 32 * x.blk2 + 16 * qh + 4 * x.t + e;
        if (k < g.r && q < g.Q) word |= src.z(g, x.b, x.i, x.j, k, q) << (8 * e + 4 * qh + rr);
      }
  return word;
}
__host__ __device__ inline uint32_t make_y_word(const Geom& g, const BitSource& src, size_t w) {
  const WordIdx x = word_index(g, w, g.PT, g.RT);   // blk1 = pt, blk2 = rt
  if (x.j >= g.cw) return 0u;
  uint32_t word = 0;
  for (int e = 0; e < 4; ++e)
    for (int kh = 0; kh < 2; ++kh)
      for (int rr = 0; rr < 4; ++rr) {
        const int p = 32 * x.blk1 + x.g + 8 * rr;
        const int k = 32 * x.blk2 + 16 * kh + 4 * x.t + e;
        if (p < g.P && k < g.r) word |= src.y(g, x.b, x.i, x.j, p, k) << (8 * e + 4 * kh + rr);
      }
  return word;
}

// ---- device kernels --------------------------------------------------------

__global__ void pack_z_kernel(Geom g, BitSource src, uint32_t* __restrict__ zp, size_t nwords) {
  for (size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x; w < nwords; w += (size_t)gridDim.x * blockDim.x)
    zp[w] = make_z_word(g, src, w);
}
__global__ void pack_y_kernel(Geom g, BitSource src, uint32_t* __restrict__ yp, size_t nwords) {
  for (size_t w = blockIdx.x * (size_t)blockDim.x + threadIdx.x; w < nwords; w += (size_t)gridDim.x * blockDim.x)
    yp[w] = make_y_word(g, src, w);
}
// ysum [bw,rw,cw,P]: sum over k of Y;  zsum [bw,rw,cw,Q]: sum over k of Z.
__global__ void ysum_kernel(Geom g, BitSource src, uint8_t* __restrict__ ysum, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    size_t u = t;
    const int p = (int)(u % g.P); u /= g.P;
    const int j = (int)(u % g.cw); u /= g.cw;
    const int i = (int)(u % g.rw); u /= g.rw;
    int s = 0;
    for (int k = 0; k < g.r; ++k) s += src.y(g, (int)u, i, j, p, k);
    ysum[t] = (uint8_t)s;
  }
}
__global__ void zsum_kernel(Geom g, BitSource src, uint8_t* __restrict__ zsum, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    size_t u = t;
    const int q = (int)(u % g.Q); u /= g.Q;
    const int j = (int)(u % g.cw); u /= g.cw;
    const int i = (int)(u % g.rw); u /= g.rw;
    int s = 0;
    for (int k = 0; k < g.r; ++k) s += src.z(g, (int)u, i, j, k, q);
    zsum[t] = (uint8_t)s;
  }
}
__global__ void unpack_y_kernel(Geom g, const uint32_t* __restrict__ yp, uint8_t* __restrict__ Y, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    size_t u = t;
    const int k = (int)(u % g.r); u /= g.r;
    const int p = (int)(u % g.P); u /= g.P;
    const int j = (int)(u % g.cw); u /= g.cw;
    const int i = (int)(u % g.rw); u /= g.rw;
    int bit;
    const size_t w = g.y_word((int)u, i, j, p, k, &bit);
    Y[t] = (uint8_t)((yp[w] >> bit) & 1u);
  }
}
__global__ void unpack_z_kernel(Geom g, const uint32_t* __restrict__ zp, uint8_t* __restrict__ Z, size_t n) {
  for (size_t t = blockIdx.x * (size_t)blockDim.x + threadIdx.x; t < n; t += (size_t)gridDim.x * blockDim.x) {
    size_t u = t;
    const int q = (int)(u % g.Q); u /= g.Q;
    const int k = (int)(u % g.r); u /= g.r;
    const int j = (int)(u % g.cw); u /= g.cw;
    const int i = (int)(u % g.rw); u /= g.rw;
    int bit;
    const size_t w = g.z_word((int)u, i, j, k, q, &bit);
    Z[t] = (uint8_t)((zp[w] >> bit) & 1u);
  }
}

static inline int grid_for(size_t n, int block) {
  size_t gsz = (n + block - 1) / block;
  if (gsz > 148u * 32u) gsz = 148u * 32u;
  if (gsz == 0) gsz = 1;
  return (int)gsz;
}

static int pack_device(const BitSource& src, const BqqDims* dims, uint32_t* zplanes, uint32_t* yplanes,
                       uint8_t* ysum, uint8_t* zsum, cudaStream_t st) {
  Geom g(*dims);
  const size_t nz = g.z_words(), ny = g.y_words();
  pack_z_kernel<<<grid_for(nz, 256), 256, 0, st>>>(g, src, zplanes, nz);
  pack_y_kernel<<<grid_for(ny, 256), 256, 0, st>>>(g, src, yplanes, ny);
  if (ysum) {
    const size_t n = (size_t)g.bw * g.rw * g.cw * g.P;
    ysum_kernel<<<grid_for(n, 256), 256, 0, st>>>(g, src, ysum, n);
  }
  if (zsum) {
    const size_t n = (size_t)g.bw * g.rw * g.cw * g.Q;
    zsum_kernel<<<grid_for(n, 256), 256, 0, st>>>(g, src, zsum, n);
  }
  return launch_status();
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
  BitSource src{Y_bool, Z_bool, 0};
  return pack_device(src, dims, zplanes, yplanes, ysum, zsum, (cudaStream_t)stream);
}

int bqq_repack_u8_planes(const uint8_t* Y_packed, const uint8_t* Z_packed, const BqqDims* dims,
                         uint32_t* zplanes, uint32_t* yplanes, uint8_t* ysum, uint8_t* zsum, void* stream) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_packed || !Z_packed || !zplanes || !yplanes) return BQQ_ERR_NULL;
  BitSource src{Y_packed, Z_packed, 1};
  return pack_device(src, dims, zplanes, yplanes, ysum, zsum, (cudaStream_t)stream);
}

int bqq_unpack_planes(const uint32_t* zplanes, const uint32_t* yplanes, const BqqDims* dims,
                      uint8_t* Y_bool, uint8_t* Z_bool, void* stream) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_bool || !Z_bool || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t ny = (size_t)g.bw * g.rw * g.cw * g.P * g.r;
  const size_t nz = (size_t)g.bw * g.rw * g.cw * g.r * g.Q;
  unpack_y_kernel<<<grid_for(ny, 256), 256, 0, st>>>(g, yplanes, Y_bool, ny);
  unpack_z_kernel<<<grid_for(nz, 256), 256, 0, st>>>(g, zplanes, Z_bool, nz);
  return launch_status();
}

int bqq_pack_planes_host(const uint8_t* Y_bool, const uint8_t* Z_bool, const BqqDims* dims,
                         uint32_t* zplanes, uint32_t* yplanes, uint8_t* ysum, uint8_t* zsum) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_bool || !Z_bool || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  BitSource src{Y_bool, Z_bool, 0};
  const size_t nz = g.z_words(), ny = g.y_words();
  for (size_t w = 0; w < nz; ++w) zplanes[w] = make_z_word(g, src, w);
  for (size_t w = 0; w < ny; ++w) yplanes[w] = make_y_word(g, src, w);
  if (ysum) {
    const size_t n = (size_t)g.bw * g.rw * g.cw * g.P;
    for (size_t t = 0; t < n; ++t) {
      int s = 0;
      for (int k = 0; k < g.r; ++k) s += Y_bool[t * g.r + k] != 0;
      ysum[t] = (uint8_t)s;
    }
  }
  if (zsum) {
    const size_t n = (size_t)g.bw * g.rw * g.cw * g.Q;
    for (size_t t = 0; t < n; ++t) {
      const size_t patch = t / g.Q;
      const int q = (int)(t % g.Q);
      int s = 0;
      for (int k = 0; k < g.r; ++k) s += Z_bool[patch * (size_t)g.r * g.Q + (size_t)k * g.Q + q] != 0;
      zsum[t] = (uint8_t)s;
    }
  }
  return BQQ_OK;
}

int bqq_pack_patch_host(const uint8_t* mat1, const uint8_t* mat2, const BqqDims* dims, int bit, int i, int j,
                        uint32_t* zplanes, uint32_t* yplanes) {
  if (int rc = check_dims(dims)) return rc;
  if (!mat1 || !mat2 || !zplanes || !yplanes) return BQQ_ERR_NULL;
  if (bit < 0 || bit >= dims->bw || i < 0 || i >= dims->rw || j < 0 || j >= dims->cw) return BQQ_ERR_BAD_SHAPE;
  Geom g(*dims);
  int pos;
  // replace the patch's bits (clear, then set), so a later entry for the same (bit, i, j) wins as in get_matrices
  for (int p = 0; p < g.P; ++p)
    for (int k = 0; k < g.r; ++k) {
      uint32_t& w = yplanes[g.y_word(bit, i, j, p, k, &pos)];
      w = (w & ~(1u << pos)) | ((mat1[(size_t)p * g.r + k] ? 1u : 0u) << pos);
    }
  for (int k = 0; k < g.r; ++k)
    for (int q = 0; q < g.Q; ++q) {
      uint32_t& w = zplanes[g.z_word(bit, i, j, k, q, &pos)];
      w = (w & ~(1u << pos)) | ((mat2[(size_t)k * g.Q + q] ? 1u : 0u) << pos);
    }
  return BQQ_OK;
}

int bqq_unpack_planes_host(const uint32_t* zplanes, const uint32_t* yplanes, const BqqDims* dims,
                           uint8_t* Y_bool, uint8_t* Z_bool) {
  int rc = check_dims(dims);
  if (rc) return rc;
  if (!Y_bool || !Z_bool || !zplanes || !yplanes) return BQQ_ERR_NULL;
  Geom g(*dims);
  int bit;
  for (int b = 0; b < g.bw; ++b)
    for (int i = 0; i < g.rw; ++i)
      for (int j = 0; j < g.cw; ++j) {
        for (int p = 0; p < g.P; ++p)
          for (int k = 0; k < g.r; ++k) {
            const size_t w = g.y_word(b, i, j, p, k, &bit);
            Y_bool[y_bool_offset(g, b, i, j, p, k)] = (uint8_t)((yplanes[w] >> bit) & 1u);
          }
        for (int k = 0; k < g.r; ++k)
          for (int q = 0; q < g.Q; ++q) {
            const size_t w = g.z_word(b, i, j, k, q, &bit);
            Z_bool[z_bool_offset(g, b, i, j, k, q)] = (uint8_t)((zplanes[w] >> bit) & 1u);
          }
      }
  return BQQ_OK;
}

}  // extern "C"
