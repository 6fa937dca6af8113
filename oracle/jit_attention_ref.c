/* CPU restatement of the reference's JIT attention sequence.  TEST INFRASTRUCTURE ONLY.
 *
 * The reference (csrc/ops/kernels/attention_kernels.cpp:218-257, "Method 1")
 * runs four library primitives one after another on dense [B,N,S|L,H] tensors:
 *     scores = (Q . K^T) * 1/sqrt(H)      stored in the input dtype   (:222-233, scale :188)
 *     scores += mask (broadcast)          in place                    (:236-238)
 *     scores  = softmax(scores, axis L)   in place                    (:241)
 *     out     = scores . V                                            (:244-252)
 * Each primitive accumulates in fp32 and rounds to bf16 when it stores.  The
 * primitives themselves are oneDNN v3.8 (not vendored in the reference tree);
 * this file restates their documented arithmetic in plain C.
 *
 * Layout: bf16 as uint16_t, row-major [B][N][S][H], [B][N][L][H], mask
 * [B][1][mS][L] with mS in {1,S} (or NULL), out [B][N][S][H].
 * Also: the BMC append copy (pace/llm/cache.py:317-325) on the same layout.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline float bf2f(uint16_t x) {
  uint32_t u = ((uint32_t)x) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f2bf(float f) { /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

typedef struct {
  const uint16_t *q, *k, *v, *mask;
  uint16_t* out;
  int mask_rows, B, N, S, L, H, tid, nthreads, err;
} job_t;

/* one (batch, head) pair: the four primitives for all S query rows */
static int one_head(const job_t* j, int b, int n, uint16_t* sc, float* qf, float* acc) {
  const int N = j->N, S = j->S, L = j->L, H = j->H;
  const float scale = 1.0f / sqrtf((float)H);
  const uint16_t* kb = j->k + ((size_t)b * N + n) * L * H;
  const uint16_t* vb = j->v + ((size_t)b * N + n) * L * H;
  for (int s = 0; s < S; ++s) {
    const uint16_t* qr = j->q + (((size_t)b * N + n) * S + s) * H;
    for (int h = 0; h < H; ++h) qf[h] = bf2f(qr[h]);
    /* primitive 1: matmul with the scale as a post-op, bf16 destination */
    for (int l = 0; l < L; ++l) {
      const uint16_t* kr = kb + (size_t)l * H;
      float d = 0.f;
      for (int h = 0; h < H; ++h) d += qf[h] * bf2f(kr[h]);
      sc[l] = f2bf(d * scale);
    }
    /* primitive 2: binary add of the broadcast mask, in place */
    if (j->mask) {
      const uint16_t* mr =
          j->mask + ((size_t)b * j->mask_rows + (j->mask_rows == 1 ? 0 : s)) * L;
      for (int l = 0; l < L; ++l) sc[l] = f2bf(bf2f(sc[l]) + bf2f(mr[l]));
    }
    /* primitive 3: softmax over L, in place */
    float mx = -INFINITY;
    for (int l = 0; l < L; ++l) { float x = bf2f(sc[l]); if (x > mx) mx = x; }
    float sum = 0.f;
    for (int l = 0; l < L; ++l) sum += expf(bf2f(sc[l]) - mx);
    const float inv = 1.0f / sum;
    for (int l = 0; l < L; ++l) sc[l] = f2bf(expf(bf2f(sc[l]) - mx) * inv);
    /* primitive 4: matmul P . V */
    for (int h = 0; h < H; ++h) acc[h] = 0.f;
    for (int l = 0; l < L; ++l) {
      const float p = bf2f(sc[l]);
      if (p == 0.f) continue;
      const uint16_t* vr = vb + (size_t)l * H;
      for (int h = 0; h < H; ++h) acc[h] += p * bf2f(vr[h]);
    }
    uint16_t* orow = j->out + (((size_t)b * N + n) * S + s) * H;
    for (int h = 0; h < H; ++h) orow[h] = f2bf(acc[h]);
  }
  return 0;
}

static void* worker(void* arg) {
  job_t* j = (job_t*)arg;
  uint16_t* sc = (uint16_t*)malloc((size_t)j->L * sizeof(uint16_t));
  float* qf = (float*)malloc((size_t)j->H * sizeof(float));
  float* acc = (float*)malloc((size_t)j->H * sizeof(float));
  if (!sc || !qf || !acc) { j->err = 1; free(sc); free(qf); free(acc); return NULL; }
  const int total = j->B * j->N;
  for (int i = j->tid; i < total; i += j->nthreads) one_head(j, i / j->N, i % j->N, sc, qf, acc);
  free(sc); free(qf); free(acc);
  return NULL;
}

/* nthreads <= 0 means 1.  Returns 0 on success. */
int pace_ref_attention_bf16(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                            const uint16_t* mask, int mask_rows, uint16_t* out,
                            int B, int N, int S, int L, int H, int nthreads) {
  if (nthreads <= 0) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  job_t jobs[256];
  pthread_t th[256];
  for (int t = 0; t < nthreads; ++t) {
    job_t j = {q, k, v, mask, out, mask_rows, B, N, S, L, H, t, nthreads, 0};
    jobs[t] = j;
    if (t > 0 && pthread_create(&th[t], NULL, worker, &jobs[t]) != 0) return 2;
  }
  worker(&jobs[0]);
  int err = jobs[0].err;
  for (int t = 1; t < nthreads; ++t) { pthread_join(th[t], NULL); err |= jobs[t].err; }
  return err;
}

/* BMC append: copy [B][N][n_new][H] rows into [B][N][cap][H] at token seq_len. */
void pace_ref_bmc_append_bf16(uint16_t* cache, const uint16_t* fresh, int B, int N,
                              int cap, int seq_len, int n_new, int H) {
  for (int b = 0; b < B; ++b)
    for (int n = 0; n < N; ++n)
      memcpy(cache + (((size_t)b * N + n) * cap + seq_len) * H,
             fresh + ((size_t)b * N + n) * n_new * H, (size_t)n_new * H * sizeof(uint16_t));
}
