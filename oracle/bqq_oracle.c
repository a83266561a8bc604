/*
 * CPU oracle for the BinaryQuadratic linear forward, plain C (TEST INFRASTRUCTURE ONLY).
 *
 * Restates the reference algorithm: rebuild the dense weight of every patch from
 * the binary factors, then multiply (BinaryQuadratic.forward,
 * neural_network_compression/src/bqq_modules.py:34-46):
 *     W_core = Y Z                                  (:37)
 *     W = sum_b a W_core + b rowsum(Y) + c colsum(Z) + d   (:38-41)
 *     y = X W^T (+ bias), out feature i*P+p, in feature j*Q+q (:42-46)
 * Parity status: PINNED through tests/test_oracle.py, which checks this file
 * against fixtures produced by the unmodified reference (tests/golden/).
 *
 * It is the checker and the timed CPU baseline ("port"); the product path never
 * calls it.  Row patches are handed to pthread workers.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

typedef struct {
  const uint8_t *Y, *Z;
  const float *a, *b, *c, *d, *bias, *X;
  float* y;
  int M, bw, rw, cw, P, Q, r, use_double;
  int next_row;   /* next row patch to hand out (atomic) */
  int failed;
} Job;

/* Dense weight rows of row patch i, W [P][cw*Q]: steps :37-42 of the reference forward. */
static void build_row_patch(const Job* J, int i, float* W, float* core) {
  const int bw = J->bw, rw = J->rw, cw = J->cw, P = J->P, Q = J->Q, r = J->r;
  const size_t in_f = (size_t)cw * Q;
  for (int j = 0; j < cw; ++j) {
    for (int p = 0; p < P; ++p)
      for (int q = 0; q < Q; ++q) W[(size_t)p * in_f + (size_t)j * Q + q] = J->d[(size_t)i * cw + j];
    for (int bit = 0; bit < bw; ++bit) {
      const size_t patch = ((size_t)bit * rw + i) * cw + j;
      const uint8_t* Yp = J->Y + patch * (size_t)P * r;
      const uint8_t* Zp = J->Z + patch * (size_t)r * Q;
      const float ca = J->a[patch], cb = J->b[patch], cc = J->c[patch];
      memset(core, 0, sizeof(float) * (size_t)P * Q);
      for (int p = 0; p < P; ++p) {
        float ysum = 0.f;
        float* crow = core + (size_t)p * Q;
        for (int k = 0; k < r; ++k) {
          if (Yp[(size_t)p * r + k]) {
            ysum += 1.f;
            const uint8_t* zrow = Zp + (size_t)k * Q;
            for (int q = 0; q < Q; ++q) crow[q] += (float)zrow[q];
          }
        }
        float* wrow = W + (size_t)p * in_f + (size_t)j * Q;
        for (int q = 0; q < Q; ++q) wrow[q] += ca * crow[q] + cb * ysum;
      }
      for (int q = 0; q < Q; ++q) {
        float zsum = 0.f;
        for (int k = 0; k < r; ++k) zsum += (float)Zp[(size_t)k * Q + q];
        const float t = cc * zsum;
        for (int p = 0; p < P; ++p) W[(size_t)p * in_f + (size_t)j * Q + q] += t;
      }
    }
  }
}

static void* worker(void* arg) {
  Job* J = (Job*)arg;
  const size_t in_f = (size_t)J->cw * J->Q, out_f = (size_t)J->rw * J->P;
  float* W = (float*)malloc(sizeof(float) * (size_t)J->P * in_f);
  float* core = (float*)malloc(sizeof(float) * (size_t)J->P * J->Q);
  if (!W || !core) {
    __atomic_store_n(&J->failed, 1, __ATOMIC_RELAXED);
  } else {
    for (;;) {
      const int i = __atomic_fetch_add(&J->next_row, 1, __ATOMIC_RELAXED);
      if (i >= J->rw) break;
      build_row_patch(J, i, W, core);
      for (int m = 0; m < J->M; ++m) {
        const float* x = J->X + (size_t)m * in_f;
        for (int p = 0; p < J->P; ++p) {
          const float* wrow = W + (size_t)p * in_f;
          float out;
          if (J->use_double) {
            double s = 0.0;
            for (size_t n = 0; n < in_f; ++n) s += (double)wrow[n] * (double)x[n];
            out = (float)s;
          } else {
            float s = 0.f;
            for (size_t n = 0; n < in_f; ++n) s += wrow[n] * x[n];
            out = s;
          }
          if (J->bias) out += J->bias[(size_t)i * J->P + p];
          J->y[(size_t)m * out_f + (size_t)i * J->P + p] = out;
        }
      }
    }
  }
  free(W);
  free(core);
  return NULL;
}

int bqq_oracle_max_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

/* Y u8 [bw,rw,cw,P,r], Z u8 [bw,rw,cw,r,Q] (0/1), a,b,c [bw,rw,cw], d [rw,cw],
 * X [M, cw*Q], y [M, rw*P], bias [rw*P] or NULL.  Dot products accumulate in double
 * when `use_double` is nonzero, else in float like the fp32 reference run.
 * nthreads <= 0 uses every online core.  Returns 0, or -1 on allocation failure. */
int bqq_oracle_forward(const uint8_t* Y, const uint8_t* Z, const float* a, const float* b, const float* c,
                       const float* d, const float* bias, const float* X, int M, int bw, int rw, int cw, int P,
                       int Q, int r, float* y, int use_double, int nthreads) {
  Job J = {Y, Z, a, b, c, d, bias, X, y, M, bw, rw, cw, P, Q, r, use_double, 0, 0};
  if (nthreads <= 0) nthreads = bqq_oracle_max_threads();
  if (nthreads > rw) nthreads = rw;
  if (nthreads > 256) nthreads = 256;
  pthread_t tid[256];
  int started = 0;
  for (int t = 1; t < nthreads; ++t)
    if (pthread_create(&tid[started], NULL, worker, &J) == 0) ++started;
  worker(&J);
  for (int t = 0; t < started; ++t) pthread_join(tid[t], NULL);
  return J.failed ? -1 : 0;
}
