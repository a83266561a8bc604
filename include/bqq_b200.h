/*
 * bqq_b200 — C ABI of the B200 (sm_100a) BinaryQuadratic linear forward.
 *
 * Plain C: pointers and sizes only, no C++ or torch types.  Unless a function
 * says "host", every data pointer is a DEVICE pointer owned by the caller; the
 * library keeps no pointer after a call returns and never allocates or frees
 * device memory.  Work is enqueued on the CUDA stream passed as `stream`
 * (a cudaStream_t cast to void*; NULL = the legacy default stream).
 *
 * Every function returning int returns BQQ_OK (0) or a negative BQQ_ERR_*;
 * bqq_strerror() turns it into text.  Nothing aborts or traps.
 *
 * Each entry point cites the reference interface it replaces, by path inside
 * the reference project (src/ = neural_network_compression/src/).
 *
 * Tensor conventions of the reference module (src/bqq_modules.py:21-32):
 *   Y bool [bw,rw,cw,P,r], Z bool [bw,rw,cw,r,Q], a/b/c [bw,rw,cw,1,1],
 *   d [rw,cw,1,1]; out feature o = i*P+p, in feature n = j*Q+q (:42).
 */
#ifndef BQQ_B200_H
#define BQQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BQQ_ABI_VERSION 1

/* error codes */
#define BQQ_OK                0
#define BQQ_ERR_NULL         -1   /* a required pointer is NULL                    */
#define BQQ_ERR_BAD_SHAPE    -2   /* a dimension is <= 0 or inconsistent           */
#define BQQ_ERR_UNSUPPORTED  -3   /* patch geometry / batch outside kernel limits  */
#define BQQ_ERR_MISALIGNED   -4   /* a pointer or leading dimension is misaligned  */
#define BQQ_ERR_WORKSPACE    -5   /* workspace missing or too small                */
#define BQQ_ERR_DTYPE        -6   /* unknown element type code                     */
#define BQQ_ERR_CUDA         -7   /* a CUDA runtime / driver call failed           */
#define BQQ_ERR_TIMEOUT      -8   /* a bounded device-side wait gave up            */
#define BQQ_ERR_NO_DEVICE    -9   /* GPU is not an sm_100 device                   */

/* element type codes for activations, outputs, coefficients and bias */
#define BQQ_F32  0
#define BQQ_BF16 1
#define BQQ_F16  2

/* geometry limits of the kernels */
#define BQQ_MAX_P 128
#define BQQ_MAX_Q 128
#define BQQ_MAX_R 64
#define BQQ_DECODE_MAX_M 16     /* rows of X handled by the decode kernel */

/* bw bit layers, rw x cw patches of P x Q, rank r */
typedef struct BqqDims {
  int32_t bw, rw, cw, P, Q, r;
} BqqDims;

/*
 * One packed layer (or one rank's shard of it: a shard is simply a layer with
 * fewer row patches).  Planes and coefficients are in this library's packed
 * formats (see bqq_pack_planes / bqq_pack_coeffs).
 */
typedef struct BqqLayer {
  BqqDims dims;
  const uint32_t* zplanes;   /* bqq_zplane_words() words                     */
  const uint32_t* yplanes;   /* bqq_yplane_words() words                     */
  const float*    coef;      /* bqq_coeff_floats() floats                    */
  const void*     bias;      /* [rw*P] or NULL                               */
  int32_t         bias_dtype;
  int32_t         reserved;
} BqqLayer;

int         bqq_abi_version(void);
const char* bqq_strerror(int rc);

/* 1 if the current device is compute capability 10.x, else 0 (no device: 0) */
int bqq_device_supported(void);

/* ---- packed sizes (host, pure arithmetic) -------------------------------- */
size_t bqq_zplane_words(const BqqDims* dims);
size_t bqq_yplane_words(const BqqDims* dims);
size_t bqq_coeff_floats(const BqqDims* dims);
/* bits + fp32 coefficients actually carrying information, in bytes */
size_t bqq_algorithmic_bytes(const BqqDims* dims);

/* ---- load-time packer -----------------------------------------------------
 * Replaces PackedBinaryQuadratic.from_unpacked / _np_packbits
 * (src/bqq_modules.py:99-148): bool Y [bw,rw,cw,P,r] and Z [bw,rw,cw,r,Q]
 * (one byte per entry, 0/1) become 32-bit bit planes
 *   zplanes [rw][NS][QW][RP][4]  bit q%32 of word q/32 of Z row k
 *   yplanes [rw][NS][RW][PP][4]  bit k%32 of word k/32 of Y row p
 * where a patch-bit n = j*bw+b, NS = ceil(cw*bw/4) super-groups of 4
 * patch-bits (innermost index), QW = ceil(Q/32), RW = ceil(r/32),
 * RP/PP = r/P rounded up to 32; all padding is zero.  ysum [bw,rw,cw,P] and
 * zsum [bw,rw,cw,Q] (uint8; may be NULL) are the row sums of Y and column
 * sums of Z that the reference keeps as Y_sum_i16 / Z_sum_i16 (:140-141).
 */
int bqq_pack_planes(const uint8_t* Y_bool, const uint8_t* Z_bool, const BqqDims* dims,
                    uint32_t* zplanes, uint32_t* yplanes, uint8_t* ysum, uint8_t* zsum,
                    void* stream);
/* Inverse (replaces _unpack_to_bool, src/bqq_modules.py:159-169). */
int bqq_unpack_planes(const uint32_t* zplanes, const uint32_t* yplanes, const BqqDims* dims,
                      uint8_t* Y_bool, uint8_t* Z_bool, void* stream);
/* Same two operations on HOST memory, single-threaded C++ (load-time path
 * for hosts that pack before uploading). */
int bqq_pack_planes_host(const uint8_t* Y_bool, const uint8_t* Z_bool, const BqqDims* dims,
                         uint32_t* zplanes, uint32_t* yplanes, uint8_t* ysum, uint8_t* zsum);
int bqq_unpack_planes_host(const uint32_t* zplanes, const uint32_t* yplanes, const BqqDims* dims,
                           uint8_t* Y_bool, uint8_t* Z_bool);
/*
 * Re-pack the reference's own uint8 checkpoints (PackedBinaryQuadratic buffers
 * Y_packed [bw,rw,cw,P,ceil(r/8)], Z_packed [bw,rw,cw,Q,ceil(r/8)], big-endian,
 * Z transposed; src/bqq_modules.py:70-74) into bit planes.
 */
int bqq_repack_u8_planes(const uint8_t* Y_packed, const uint8_t* Z_packed, const BqqDims* dims,
                         uint32_t* zplanes, uint32_t* yplanes, void* stream);

/*
 * Coefficients a,b,c [bw,rw,cw] and d [rw,cw] (element type `dtype`) to
 * float32 [rw][NS*4][4] = (a, b, c, d if bit 0 else 0) per patch-bit.
 * Replaces the per-call reshape/.to(float32) of src/bqq_cuda.cu:318-323.
 */
int bqq_pack_coeffs(const void* a, const void* b, const void* c, const void* d, int dtype,
                    const BqqDims* dims, float* coef, void* stream);

/* ---- forward ---------------------------------------------------------------
 * y[M, rw*P] = x[M, cw*Q] @ W^T (+ bias), the result of
 * BinaryQuadratic.forward (src/bqq_modules.py:34-46), fp32 accumulation.
 * x rows are ldx elements apart, y rows ldy elements apart; x and y use the
 * same element type codes (y_dtype may differ from x_dtype).
 *
 * bqq_forward_decode: M <= BQQ_DECODE_MAX_M; streams the packed planes once;
 *   replaces bqq_forward_kernel (src/bqq_cuda.cu:47-180).  The workspace
 *   (bqq_decode_workspace_bytes, 256-byte aligned) must be zero-filled once
 *   after allocation; the kernel leaves it zeroed for the next call.  Calls
 *   sharing one workspace must not overlap on the GPU.
 * bqq_forward_prefill: any M; rebuilds W once into the workspace and runs a
 *   tcgen05 tensor-core GEMM; replaces reconstruct_W_kernel + torch::mm
 *   (src/bqq_cuda.cu:198-246, 367-383).
 * bqq_forward: picks decode for M <= 16 and prefill otherwise, the dispatch
 *   of src/bqq_cuda.cu:327,367; workspace must satisfy bqq_forward_workspace_bytes.
 */
size_t bqq_decode_workspace_bytes(const BqqDims* dims, int M);
int bqq_forward_decode(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx,
                       void* y, int y_dtype, int64_t ldy,
                       void* workspace, size_t workspace_bytes, void* stream);

size_t bqq_prefill_workspace_bytes(const BqqDims* dims, int M);
int bqq_forward_prefill(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx,
                        void* y, int y_dtype, int64_t ldy,
                        void* workspace, size_t workspace_bytes, void* stream);

size_t bqq_forward_workspace_bytes(const BqqDims* dims, int M);
int bqq_forward(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx,
                void* y, int y_dtype, int64_t ldy,
                void* workspace, size_t workspace_bytes, void* stream);

/*
 * Dense weight W [rw*P, cw*Q] row-major in element type w_dtype: the value of
 * BinaryQuadratic.get_weight (src/bqq_modules.py:48-55), built with AND +
 * popcount like reconstruct_W_kernel (src/bqq_cuda.cu:198-246) but with
 * coalesced row-major stores.  `scale` multiplies every entry (1.0f for the
 * plain weight).
 */
int bqq_reconstruct_weight(const BqqLayer* layer, void* W, int w_dtype, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BQQ_B200_H */
