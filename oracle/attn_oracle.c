/*
 * Plain-C restatement of the operator -- TEST INFRASTRUCTURE ONLY (see oracle.py
 * for who may use it).  Independent of torch: scalar fp32 loops, so it also
 * cross-checks the torch-based oracle's blocked evaluation.
 *
 *   math      out = softmax(q k^T / sqrt(128)) v in fp32 -- the reference's oracle,
 *             examples/basic.py:16-17; inputs are bf16 bit patterns widened to fp32.
 *   rounding  csrc/attention_kernel.hip:110-145 (RTNE / RTNA / RTZ bit formulas),
 *             NaN -> 0x7FFF in every mode.
 *   layouts   0 = [B,H,S,D], 1 = [B,S,H,D] (csrc/attention_kernel.hip:554-566, :1581).
 *
 * Build: make -C oracle   (gcc -O2 -shared -pthread)
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HEAD_DIM 128

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static inline size_t row_offset(int layout, int H, int S, int b, int h, int r) {
  if (layout == 1) return (((size_t)b * S + r) * H + h) * HEAD_DIM;
  return (((size_t)b * H + h) * S + r) * HEAD_DIM;
}

uint16_t oracle_round_one(float f, int mode) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if (f != f) return 0x7FFF;
  if (mode == 0) return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16); /* RTNE */
  if (mode == 1) return (uint16_t)((u + 0x8000u) >> 16);                    /* RTNA */
  return (uint16_t)(u >> 16);                                               /* RTZ  */
}

void oracle_round_bf16(const float* src, uint16_t* dst, size_t n, int mode) {
  for (size_t i = 0; i < n; ++i) dst[i] = oracle_round_one(src[i], mode);
}

typedef struct {
  const uint16_t *q, *k, *v;
  float* out;
  int B, H, Sq, Skv, layout, row_begin, row_end;
  long idx_begin, idx_end;
} job_t;

static void* run_job(void* arg) {
  const job_t* jb = (const job_t*)arg;
  const float scale = 1.0f / sqrtf((float)HEAD_DIM);
  const long nrows = (long)(jb->row_end - jb->row_begin);
  float* s = (float*)malloc(sizeof(float) * (size_t)jb->Skv);
  if (s == NULL) return (void*)1;
  for (long idx = jb->idx_begin; idx < jb->idx_end; ++idx) {
    const int r = jb->row_begin + (int)(idx % nrows);
    const int h = (int)((idx / nrows) % jb->H);
    const int b = (int)(idx / (nrows * jb->H));
    const uint16_t* qr = jb->q + row_offset(jb->layout, jb->H, jb->Sq, b, h, r);
    float qf[HEAD_DIM];
    for (int d = 0; d < HEAD_DIM; ++d) qf[d] = bf16_to_f32(qr[d]);
    float m = -INFINITY;
    for (int j = 0; j < jb->Skv; ++j) {
      const uint16_t* kr = jb->k + row_offset(jb->layout, jb->H, jb->Skv, b, h, j);
      float acc = 0.f;
      for (int d = 0; d < HEAD_DIM; ++d) acc += qf[d] * bf16_to_f32(kr[d]);
      s[j] = acc * scale;
      if (s[j] > m) m = s[j]; /* NaN never wins the comparison, like the max-subtraction of torch.softmax */
    }
    float l = 0.f;
    for (int j = 0; j < jb->Skv; ++j) {
      s[j] = expf(s[j] - m);
      l += s[j];
    }
    float o[HEAD_DIM];
    for (int d = 0; d < HEAD_DIM; ++d) o[d] = 0.f;
    for (int j = 0; j < jb->Skv; ++j) {
      const uint16_t* vr = jb->v + row_offset(jb->layout, jb->H, jb->Skv, b, h, j);
      const float p = s[j] / l;
      for (int d = 0; d < HEAD_DIM; ++d) o[d] += p * bf16_to_f32(vr[d]);
    }
    float* orow = jb->out + row_offset(jb->layout, jb->H, jb->Sq, b, h, r);
    for (int d = 0; d < HEAD_DIM; ++d) orow[d] = o[d];
  }
  free(s);
  return NULL;
}

/* q: [.., Sq, ..], k, v: [.., Skv, ..] as bf16 bits; out fp32 in the same layout as q.
 * Computes query rows [row_begin, row_end) of every (batch, head) on `threads` POSIX threads.
 * Returns 0, or 1 on bad arguments / allocation failure. */
int oracle_attention_f32(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* out, int B, int H, int Sq,
                         int Skv, int layout, int row_begin, int row_end, int threads) {
  if (B <= 0 || H <= 0 || Sq <= 0 || Skv <= 0 || (layout != 0 && layout != 1)) return 1;
  if (row_begin < 0) row_begin = 0;
  if (row_end > Sq) row_end = Sq;
  if (row_end <= row_begin) return 0;
  if (threads < 1) threads = 1;
  if (threads > 256) threads = 256;
  const long total = (long)B * H * (row_end - row_begin);
  pthread_t tid[256];
  job_t jobs[256];
  int started = 0, bad = 0;
  for (int t = 0; t < threads; ++t) {
    job_t jb = {q, k, v, out, B, H, Sq, Skv, layout, row_begin, row_end, total * t / threads, total * (t + 1) / threads};
    jobs[t] = jb;
    if (pthread_create(&tid[t], NULL, run_job, &jobs[t]) != 0) {
      bad = 1;
      break;
    }
    ++started;
  }
  for (int t = 0; t < started; ++t) {
    void* rv = NULL;
    pthread_join(tid[t], &rv);
    if (rv != NULL) bad = 1;
  }
  return bad;
}
