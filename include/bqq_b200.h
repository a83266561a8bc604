/*
 * bqq_b200 — C ABI of the B200 (sm_100a) BinaryQuadratic linear forward.
 *
 * Plain C: pointers and sizes only, no C++ or torch types.  Unless a function
 * says "host", every data pointer is a DEVICE pointer owned by the caller; the
 * library keeps no pointer after a call returns and, apart from the explicit
 * bqq_peer_alloc / bqq_peer_free pair, never allocates or frees device memory.  Work is enqueued on the CUDA stream passed as `stream`
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

#define BQQ_ABI_VERSION 2

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
#define BQQ_ERR_SCRATCH_LIMIT -10  /* needs more than the fixed built-in scratch     */

/* element type codes for activations, outputs, coefficients and bias */
#define BQQ_F32  0
#define BQQ_BF16 1
#define BQQ_F16  2

/* geometry limits of the kernels */
#define BQQ_MAX_P 128
#define BQQ_MAX_Q 128
#define BQQ_MAX_R 64
#define BQQ_DECODE_MAX_M 16     /* rows of X handled by the decode kernel */
#define BQQ_NOALLOC_SCRATCH_BYTES (8u << 20)   /* built-in scratch of bqq_forward_decode_noalloc */

/* bw bit layers, rw x cw patches of P x Q, rank r */
typedef struct BqqDims {
  int32_t bw, rw, cw, P, Q, r;
} BqqDims;

/*
 * One layer (or one rank's shard of it: a shard is simply a layer with fewer row
 * patches).  The binary factors are in this library's packed plane format
 * (bqq_pack_planes); the coefficients are read where the module keeps them:
 * the parameter tensors a, b, c [bw,rw,cw] and d [rw,cw] of the reference
 * (src/bqq_modules.py:28-31), contiguous, all of element type coef_dtype.  They
 * are read on every call, so in-place updates of the parameters are always seen.
 */
typedef struct BqqLayer {
  BqqDims dims;
  const uint32_t* zplanes;   /* bqq_zplane_words() words, 16-byte aligned    */
  const uint32_t* yplanes;   /* bqq_yplane_words() words, 16-byte aligned    */
  const void*     a;         /* [bw,rw,cw]                                   */
  const void*     b;         /* [bw,rw,cw]                                   */
  const void*     c;         /* [bw,rw,cw]                                   */
  const void*     d;         /* [rw,cw]                                      */
  const void*     bias;      /* [rw*P] or NULL                               */
  int32_t         coef_dtype;
  int32_t         bias_dtype;
} BqqLayer;

int         bqq_abi_version(void);
const char* bqq_strerror(int rc);

/* 1 if the current device is compute capability 10.x, else 0 (no device: 0) */
int bqq_device_supported(void);

/* ---- packed sizes (host, pure arithmetic) -------------------------------- */
size_t bqq_zplane_words(const BqqDims* dims);
size_t bqq_yplane_words(const BqqDims* dims);
/* bits + fp32 coefficients actually carrying information, in bytes */
size_t bqq_algorithmic_bytes(const BqqDims* dims);

/* ---- load-time packer -----------------------------------------------------
 * Replaces PackedBinaryQuadratic.from_unpacked / _np_packbits
 * (src/bqq_modules.py:99-148): bool Y [bw,rw,cw,P,r] and Z [bw,rw,cw,r,Q]
 * (one byte per entry, 0/1) become 32-bit bit planes.  Patches are padded to
 * PT x QT x RT blocks of 32 (P, Q, r rounded up); for a row patch i the
 * super-group s = b*JG + jg (JG = ceil(cw/4), NS = bw*JG) holds the col patches
 * j = 4*jg + sub of bit layer b, interleaved so that one 128-bit load fetches a
 * word of all four:
 *   zplanes [rw][NS][RT][QT][32 lanes][4 sub]
 *   yplanes [rw][NS][PT][RT][32 lanes][4 sub]
 * With lane = 4*g + t, a word is a 4-row x 8-column fragment in the order of the
 * int8 tensor-core operand that the decode kernel builds from it with byte masks:
 *   Z bit 8e + 4qh + rr = Z[k = 32rt + 4g + rr][q = 32qt + 16qh + 4t + e]
 *   Y bit 8e + 4kh + rr = Y[p = 32pt + g + 8rr][k = 32rt + 16kh + 4t + e]
 * All padding is zero.  ysum [bw,rw,cw,P] and zsum [bw,rw,cw,Q] (uint8; may be
 * NULL) are the row sums of Y and column sums of Z that the reference keeps as
 * Y_sum_i16 / Z_sum_i16 (:140-141).
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
 * One patch straight into HOST planes: mat1 [P,r] and mat2 [r,Q] (one byte per
 * element, non-zero = 1) of bit layer `bit`, row patch i, col patch j replace that
 * patch's bits in zplanes / yplanes (zero-initialised by the caller, sized by
 * bqq_zplane_words / bqq_yplane_words).  Lets a loader stream the reference's
 * patch files ({patch_row, patch_col, coeff, mat1, mat2, bit_idx} dicts, gathered
 * into dense tensors by get_matrices, src/bqq_modules.py:485-507) into planes
 * without the dense Y/Z intermediate (32 times the planes' size as bytes).
 */
int bqq_pack_patch_host(const uint8_t* mat1, const uint8_t* mat2, const BqqDims* dims, int bit, int i, int j,
                        uint32_t* zplanes, uint32_t* yplanes);
/*
 * Re-pack the reference's own uint8 checkpoints (PackedBinaryQuadratic buffers
 * Y_packed [bw,rw,cw,P,ceil(r/8)], Z_packed [bw,rw,cw,Q,ceil(r/8)], big-endian,
 * Z transposed; src/bqq_modules.py:70-74) into bit planes (ysum/zsum optional).
 */
int bqq_repack_u8_planes(const uint8_t* Y_packed, const uint8_t* Z_packed, const BqqDims* dims,
                         uint32_t* zplanes, uint32_t* yplanes, uint8_t* ysum, uint8_t* zsum,
                         void* stream);

/* ---- forward ---------------------------------------------------------------
 * y[M, rw*P] = x[M, cw*Q] @ W^T (+ bias), the result of
 * BinaryQuadratic.forward (src/bqq_modules.py:34-46).
 * x rows are ldx elements apart, y rows ldy elements apart; x and y use the
 * same element type codes (y_dtype may differ from x_dtype).
 *
 * bqq_forward_decode: M <= BQQ_DECODE_MAX_M; streams the packed planes once,
 *   both contractions on the int8 tensor cores with x and the intermediate in
 *   block fixed point (16 and 24 bits), fp32 across patches; replaces
 *   bqq_forward_kernel (src/bqq_cuda.cu:47-180).  The first 256 KiB of the
 *   workspace (bqq_decode_workspace_bytes, 256-byte aligned) are counters that
 *   must be zero-filled once after allocation; the kernel leaves them zeroed,
 *   so one workspace serves layers of any shape (the last counter word turns
 *   non-zero if a bounded device-side wait ever gave up).  A workspace is always
 *   required.  Calls sharing a workspace
 *   must not overlap on the GPU.  Results do not depend on the number of row
 *   patches: a row shard reproduces its slice of the full output bit for bit.
 * bqq_forward_prefill: any M; rebuilds W once into the workspace and runs a
 *   tcgen05 tensor-core GEMM (fp32 accumulate); replaces reconstruct_W_kernel +
 *   torch::mm (src/bqq_cuda.cu:198-246, 367-383).  The first word of the
 *   workspace is a status word: non-zero after the call completes means a
 *   bounded device-side wait gave up (BQQ_ERR_TIMEOUT) and y is invalid.
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
 * bqq_forward_decode with the neighbouring element-wise operations of a decoder
 * block folded in (the reference runs them as separate torch ops around the
 * module; it has no counterpart).  prologue, applied to x as it is read:
 *   BQQ_PRO_NONE     x as is;
 *   BQQ_PRO_RMSNORM  x[m,n] * rsqrt(mean_n x[m,:]^2 + eps) * norm_weight[n];
 *   BQQ_PRO_SWIGLU   silu(x[m,n]) * x[m, in + n]: x has rows [gate | up] of
 *                    2*in elements (ldx >= 2*in).
 * residual (may be NULL, may alias y): [M, out] added to the output before it is
 * stored.  All prologue arithmetic is fp32.  fusion == NULL is bqq_forward_decode.
 */
#define BQQ_PRO_NONE    0
#define BQQ_PRO_RMSNORM 1
#define BQQ_PRO_SWIGLU  2
typedef struct BqqFusion {
  int32_t prologue;
  int32_t norm_dtype;          /* element type of norm_weight */
  const void* norm_weight;     /* [in], BQQ_PRO_RMSNORM only */
  float eps;
  int32_t residual_dtype;
  const void* residual;
  int64_t ld_residual;         /* row pitch of residual in elements */
  int32_t out_segments;        /* bqq_forward_decode_gathered only: 0 or 1 = the gathered row is the ranks'
                                  rows side by side; 2 = every rank's row is two halves [h0 | h1] and the
                                  gathered row is [h0 of all ranks | h1 of all ranks] (a stacked gate / up
                                  layer whose consumer applies BQQ_PRO_SWIGLU to [gate | up]) */
} BqqFusion;
int bqq_forward_decode_fused(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx,
                             void* y, int y_dtype, int64_t ldy, const BqqFusion* fusion,
                             void* workspace, size_t workspace_bytes, void* stream);

/*
 * Status words of the workspaces (the reference has no counterpart: its kernels
 * have no waits).  Both synchronise `stream` and return BQQ_ERR_TIMEOUT when a
 * bounded device-side wait gave up in a call that used the workspace (its outputs
 * are invalid), else BQQ_OK: bqq_decode_status reads the last counter word of a
 * decode workspace (it stays set until the caller zero-fills the counters again),
 * bqq_prefill_status the first word of a prefill workspace (cleared by every
 * prefill call).
 */
int bqq_decode_status(const void* workspace, void* stream);
int bqq_prefill_status(const void* workspace, void* stream);

/*
 * Number of kernels one bqq_forward_decode call enqueues for this layer shape and
 * M (1 or 2: short single-chunk layers at M = 1 prepare x inside the decode
 * kernel, all others launch a preparation kernel first); negative BQQ_ERR_* for
 * bad arguments.  For launch accounting; the reference has no such query.
 */
int bqq_decode_launches(const BqqDims* dims, int M);

/*
 * Glue for decoder blocks built from these layers (no counterpart in the
 * reference, whose host models call torch's scaled_dot_product_attention): the
 * attention of ONE new token per sequence, in one launch.  qkv [B][heads +
 * 2 kv_heads][head_dim] is the row the stacked q/k/v projection produced (ld_qkv
 * elements between sequences); the new q and k heads get the rotary embedding of
 * position lens[b] (pairs (x[2i], x[2i+1]) rotated by cos/sin_table[lens[b]][i],
 * tables [max_seq][head_dim/2]), k and v are written to row lens[b] of the caches
 * [B][max_seq][kv_heads][head_dim] (ld_cache elements between sequences), and out
 * [B][heads][head_dim] (ld_out between sequences) receives softmax(q K^T /
 * sqrt(head_dim)) V over rows 0..lens[b] for every query head (query head h reads
 * kv head h / (heads / kv_heads)).  The key range is split over CTAs and combined
 * in a fixed order, so results are reproducible.  lens is device memory, read by
 * the kernel (the call can be captured in a CUDA graph); sequences with lens[b]
 * outside [0, max_seq) are skipped.  bf16 only (dtype = BQQ_BF16), head_dim 128,
 * at most 16 query heads per kv head; pointers 16-byte aligned, leading dimensions
 * multiples of 8.  workspace: bqq_attention_decode_workspace_bytes bytes,
 * 16-byte aligned, zero-filled once before its first use (the kernel leaves its
 * counters zeroed); one workspace serves one stream.
 */
size_t bqq_attention_decode_workspace_bytes(int B, int heads, int kv_heads);
int bqq_attention_decode(const void* qkv, int64_t ld_qkv, void* k_cache, void* v_cache, int64_t ld_cache,
                         int max_seq, const void* cos_table, const void* sin_table, const int32_t* lens,
                         int B, int heads, int kv_heads, int head_dim, int dtype, void* out, int64_t ld_out,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * Diagnostic: issue rate of one instruction kind on the current device, in
 * warp-instructions per SM and clock (at the device's nominal SM clock), measured
 * with CUDA events over one launch of `iters` rounds per warp on 32 warps per SM.
 * kind: 0 mma.sync m16n8k32 u8*s8, 1 m16n8k16 f16, 2 m16n8k32 e4m3, 3 m16n8k64
 * u4*s4, 4 m16n8k256 b1 and.popc, 5 lop3, 6 add.f32, 7 mad.lo.u32, 8 popc,
 * 9 shfl.  The decode kernel's operand format (bytes masked out of the plane
 * words for int8 MMAs) was chosen from these rates; `bench.py --workload rates`
 * prints them.  Synchronises `stream`.  The reference has no counterpart.
 */
int bqq_instruction_rate(int kind, int iters, double* warp_inst_per_clk_per_sm, void* stream);

/*
 * bqq_forward with HOST activations and outputs: copies x [M, ldx] from host
 * memory into the workspace, runs bqq_forward on the stream and copies y back to
 * host memory, all asynchronously on `stream` (use pinned host buffers; with
 * pageable memory the copies block the host).  It is what the reference module
 * does when it is handed a CPU tensor (`X.to(self.Y.device)`,
 * src/bqq_modules.py:35) without the per-call tensor allocations.  The caller
 * synchronises the stream before reading y_host.  For M <= 16 with pinned and
 * mapped host buffers (cudaHostAlloc, cudaHostRegister, torch pin_memory) the
 * kernels read x from and write y to host memory directly and no copy engine is
 * involved; otherwise the two copies are cudaMemcpyAsync.  The workspace must hold
 * bqq_forward_host_workspace_bytes (the forward's workspace first, then the two
 * staging buffers), be 256-byte aligned and obey the decode workspace's
 * zero-initialisation rule.
 */
size_t bqq_forward_host_workspace_bytes(const BqqDims* dims, int M, int x_dtype, int y_dtype);
int bqq_forward_host(const BqqLayer* layer, const void* x_host, int x_dtype, int M, int64_t ldx,
                     void* y_host, int y_dtype, int64_t ldy,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * bqq_forward_decode without a caller workspace (no counterpart in the reference,
 * whose extension allocates through torch on every call).  It is for callers that
 * cannot allocate device memory at the point of the call: operators hosted by a
 * runtime that passes only input and output buffers, code inside a section where
 * cudaMalloc or an allocating library call is not permitted, and start-up code
 * that runs before an allocator exists.  The workspace is a fixed array of
 * BQQ_NOALLOC_SCRATCH_BYTES (8 MiB) inside the library image, held by every GPU
 * that loads the library until the process exits.  A layer / M whose
 * bqq_decode_workspace_bytes exceeds that returns BQQ_ERR_SCRATCH_LIMIT and
 * launches nothing.  The call performs no cudaMalloc, cudaFree or allocating
 * library call.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress) with that device current, so make that first call
 * outside any stream capture.  All calls share the one array and it keeps the
 * previous call's contents (the call clears the counters it relies on): calls
 * that overlap on the GPU, on any streams, race with each other.
 * The array's last counter word is the decode kernel's "a bounded wait gave up"
 * status; the call does not clear it.  bqq_noalloc_status synchronises `stream`,
 * returns BQQ_ERR_TIMEOUT if any call on the current device since the previous
 * report set it (their outputs are invalid) and clears it; it allocates nothing
 * either.  Arguments are checked before anything is enqueued.
 */
size_t bqq_noalloc_scratch_bytes(void);
int bqq_forward_decode_noalloc(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx,
                               void* y, int y_dtype, int64_t ldy, void* stream);
int bqq_noalloc_status(void* stream);

/*
 * Column gather for row-patch sharded layers by peer-to-peer stores (one process
 * per GPU, all on one node).  The reference has no multi-GPU path; this replaces
 * the all-gather a column-parallel wrapper of its module would issue.
 *
 * Set-up (the only calls of this library that allocate): every rank calls
 * bqq_peer_alloc for its own region (control words + slots for gathered results
 * of up to `gather_bytes`; bqq_peer_region_bytes in all), sends the 64-byte handle to its peers by any host channel,
 * opens theirs with bqq_peer_open, and fills a BqqPeerGroup with the region
 * pointers in rank order (its own allocation at [rank]).  All ranks must finish
 * this before the first gather.  Tear-down: synchronise all ranks, bqq_peer_close
 * the peers' regions, bqq_peer_free the own one.
 *
 * bqq_peer_gather: rank g passes its slice y_local [rows, n_local] (row pitch ldy
 * elements); one kernel stores it into every rank's region, waits for all slices
 * to arrive in the own region and writes the rows [rows, world*n_local] (rank-major
 * columns, i.e. the unsharded column order) to `gathered` (row pitch ld_gathered).
 * Slices travel as 32-bit words: n_local, ldy and ld_gathered times the element
 * size must be multiples of 4 bytes (BQQ_ERR_MISALIGNED otherwise).
 * Every rank must issue the same sequence of gathers on the same group.  Waits on
 * peers are bounded (BqqPeerGroup.wait_cycles, about one second by default); if one gives up the kernel still ends and
 * bqq_peer_status (which synchronises `stream`) returns BQQ_ERR_TIMEOUT.  No
 * reduction is involved, so the gathered rows equal the single-GPU output bit for
 * bit.  The call can be captured in a CUDA graph.
 */
#define BQQ_MAX_PEERS 8
#define BQQ_PEER_HANDLE_BYTES 64
typedef struct BqqPeerGroup {
  int32_t rank, world;
  void* regions[BQQ_MAX_PEERS];   /* every rank's region as mapped in this process */
  uint64_t gather_bytes;          /* largest gathered result, as given to bqq_peer_alloc */
  uint64_t wait_cycles;           /* clock cycles a wait on a peer may take before it gives up;
                                     0 = the default (2e9, about one second) */
} BqqPeerGroup;

size_t bqq_peer_region_bytes(size_t gather_bytes);
int bqq_peer_alloc(size_t gather_bytes, void** region, unsigned char handle[BQQ_PEER_HANDLE_BYTES]);
int bqq_peer_open(const unsigned char handle[BQQ_PEER_HANDLE_BYTES], void** region);
int bqq_peer_close(void* region);
int bqq_peer_free(void* region);
int bqq_peer_gather(const BqqPeerGroup* group, const void* y_local, int dtype, int rows, int64_t n_local,
                    int64_t ldy, void* gathered, int64_t ld_gathered, void* stream);
int bqq_peer_status(const BqqPeerGroup* group, void* stream);

/*
 * bqq_forward_decode of a row-patch shard fused with the gather, in ONE launch:
 * the decode kernel's epilogue stores every finished output row patch into the
 * gather regions of all ranks while the rest of the kernel still runs, and a few
 * additional CTAs of the same grid wait (bounded) for the peers' row patches and
 * write the full rows [M, world*out_local] to `gathered`; the computing CTAs never
 * wait for them.  y_local [M, out_local] still receives this rank's columns.
 * `fusion` (may be NULL) as in bqq_forward_decode_fused; a residual is this rank's
 * column slice [M, out_local] and is added before the outputs are sent.  Same
 * rules as bqq_forward_decode and bqq_peer_gather; 16-bit outputs need an even P.
 * This is the sharded forward a column-parallel wrapper of the reference module
 * would need (the reference has no multi-GPU path).
 */
int bqq_forward_decode_gathered(const BqqLayer* layer, const void* x, int x_dtype, int M, int64_t ldx,
                                void* y_local, int y_dtype, int64_t ldy, const BqqFusion* fusion,
                                const BqqPeerGroup* group, void* gathered, int64_t ld_gathered,
                                void* workspace, size_t workspace_bytes, void* stream);

/*
 * bqq_attention_decode for heads sharded over the ranks of a peer group, with the
 * gather of the outputs in the same launch: every rank passes its local heads
 * (qkv, caches, out_local as in bqq_attention_decode, `heads` and `kv_heads` being
 * the local counts) and receives gathered [B][world * heads][head_dim] (ld_gathered
 * elements between sequences), the ranks' heads side by side in rank order.  The
 * finished output words are stored into every rank's slot region as they are
 * produced; a few more CTAs of the same grid wait (bounded) for all ranks' words.
 * Same rules as bqq_peer_gather: all ranks call in the same order on their streams,
 * B * world * heads * head_dim * 2 <= gather_bytes.  No counterpart in the reference.
 */
int bqq_attention_decode_gathered(const BqqPeerGroup* group, const void* qkv, int64_t ld_qkv, void* k_cache,
                                  void* v_cache, int64_t ld_cache, int max_seq, const void* cos_table,
                                  const void* sin_table, const int32_t* lens, int B, int heads, int kv_heads,
                                  int head_dim, int dtype, void* out_local, int64_t ld_out, void* gathered,
                                  int64_t ld_gathered, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Dense weight W [rw*P, cw*Q] row-major in element type w_dtype: the value of
 * BinaryQuadratic.get_weight (src/bqq_modules.py:48-55).  Replaces
 * reconstruct_W_kernel (src/bqq_cuda.cu:198-246): the per-entry counts
 * popc(Yrow & Zcol) are formed as exact small-integer products on the
 * tensor cores, one 32x32 block per warp, and stored row-major.  `scale`
 * multiplies every entry (1.0f for the plain weight).
 */
int bqq_reconstruct_weight(const BqqLayer* layer, void* W, int w_dtype, float scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BQQ_B200_H */
