/*
 * CPU oracle for the attention / KV-cache path of rdna4-infer.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the GPU kernels are compared
 * against; it is never linked into, imported by, or called from the product
 * library. Only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg may load it.
 *
 * It is a plain-C restatement (not a copy) of the reference's scalar math. Each
 * function names the reference lines it follows (paths are relative to the
 * reference project root). Build with -ffp-contract=off: the reference
 * quantizers are written as separate multiply and add (`x*id + 8.5f`), and on a
 * baseline x86-64 host that is two roundings, so an FMA here would change bytes
 * when the sum lands within an ulp of an integer.
 *
 * Parity pin: the quantizers, fp16 conversion, RoPE, the merge and the unsplit /
 * split attention walk are checked against the reference's own headers executed
 * on the CPU (see ref_driver.cpp and the Makefile target `ref`); vectors produced
 * by that run are committed under tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

enum { RDO_F32 = 0, RDO_F16 = 1, RDO_Q8_0 = 2, RDO_Q4_0 = 3, RDO_Q5_0 = 4, RDO_Q4_1 = 5 };

/* ------------------------------------------------------------------ fp16 -- */

/* include/rdna4/fp16.h:16-34 (host branch): exact widening, subnormals kept. */
float rdo_fp16_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h >> 15) & 1u;
  const uint32_t e = (uint32_t)(h >> 10) & 0x1fu;
  const uint32_t m = (uint32_t)h & 0x3ffu;
  if (e == 0u) {
    const float v = (float)m * 5.9604644775390625e-8f; /* 2^-24 */
    return sign ? -v : v;
  }
  /* The reference widens e==31 like a normal number (no Inf/NaN special case). */
  union { uint32_t u; float f; } c;
  c.u = (sign << 31) | ((e + 112u) << 23) | (m << 13);
  return c.f;
}

/* include/rdna4/fp16.h:37-57: round-to-nearest-even; NaN and overflow give Inf;
 * anything below half the smallest subnormal flushes to signed zero. */
uint16_t rdo_float_to_fp16(float f) {
  union { float f; uint32_t u; } c;
  c.f = f;
  const uint32_t x = c.u;
  const uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t mant = x & 0x007fffffu;
  const int exp = (int)((x >> 23) & 0xffu) - 127 + 15;
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    mant |= 0x00800000u;
    const uint32_t shift = (uint32_t)(14 - exp);
    uint32_t hm = mant >> shift;
    const uint32_t rb = 1u << (shift - 1);
    if ((mant & rb) && ((mant & (rb - 1)) || (hm & 1u))) ++hm;
    return (uint16_t)(sign | hm);
  }
  if (exp >= 31) return (uint16_t)(sign | 0x7c00u);
  uint32_t half = sign | ((uint32_t)exp << 10) | (mant >> 13);
  const uint32_t rem = mant & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) ++half;
  return (uint16_t)half;
}

/* ------------------------------------------------------------- KV tables -- */

/* include/rdna4/kv.h:155-169. Returns 0 for a type outside the enum (the
 * reference aborts there; the oracle leaves that to its caller). */
uint64_t rdo_kv_row_bytes(int type, int head_dim) {
  const uint64_t blocks = (uint64_t)(head_dim + 31) / 32;
  switch (type) {
    case RDO_F32: return (uint64_t)head_dim * 4;
    case RDO_F16: return (uint64_t)head_dim * 2;
    case RDO_Q8_0: return blocks * 34;
    case RDO_Q4_0: return blocks * 18;
    case RDO_Q5_0: return blocks * 22;
    case RDO_Q4_1: return blocks * 20;
  }
  return 0;
}

static void put16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)(v & 0xff); p[1] = (uint8_t)(v >> 8); }
static uint16_t get16(const uint8_t *p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }

static int clampi(int q, int hi) { return q > hi ? hi : (q < 0 ? 0 : q); }

/* One 32-element block. include/rdna4/kv.h:402-411 (q8_0), :412-444 (q5_0),
 * :445-467 (q4_1), :476-499 (q4_0); host mirror tests/check_rope_gpu.hip:250-326. */
static void quant_block(int type, const float *x, uint8_t *y) {
  if (type == RDO_Q8_0) {
    float amax = 0.0f;
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(x[j]));
    const float d = amax / 127.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    put16(y, rdo_float_to_fp16(d));
    for (int j = 0; j < 32; ++j) y[2 + j] = (uint8_t)(int8_t)roundf(x[j] * id);
    return;
  }
  if (type == RDO_Q4_0 || type == RDO_Q5_0) {
    /* signed value of largest magnitude; strict '<' keeps the first on ties */
    float amax = 0.0f, vmax = 0.0f;
    for (int j = 0; j < 32; ++j) {
      const float v = x[j];
      if (amax < fabsf(v)) { amax = fabsf(v); vmax = v; }
    }
    if (type == RDO_Q4_0) {
      const float d = vmax / -8.0f;
      const float id = d != 0.0f ? 1.0f / d : 0.0f;
      put16(y, rdo_float_to_fp16(d));
      for (int j = 0; j < 16; ++j) {
        const float x0 = x[j] * id;
        const float x1 = x[j + 16] * id;
        const int q0 = clampi((int)(int8_t)(x0 + 8.5f), 15);
        const int q1 = clampi((int)(int8_t)(x1 + 8.5f), 15);
        y[2 + j] = (uint8_t)(q0 | (q1 << 4));
      }
    } else {
      const float d = vmax / -16.0f;
      const float id = d != 0.0f ? 1.0f / d : 0.0f;
      put16(y, rdo_float_to_fp16(d));
      uint32_t qh = 0;
      for (int j = 0; j < 16; ++j) {
        const float x0 = x[j] * id;
        const float x1 = x[j + 16] * id;
        const int q0 = clampi((int)(int8_t)(x0 + 16.5f), 31);
        const int q1 = clampi((int)(int8_t)(x1 + 16.5f), 31);
        y[6 + j] = (uint8_t)((q0 & 0x0f) | ((q1 & 0x0f) << 4));
        qh |= (uint32_t)((q0 & 0x10) >> 4) << j;
        qh |= (uint32_t)((q1 & 0x10) >> 4) << (j + 16);
      }
      y[2] = (uint8_t)(qh & 0xff);
      y[3] = (uint8_t)((qh >> 8) & 0xff);
      y[4] = (uint8_t)((qh >> 16) & 0xff);
      y[5] = (uint8_t)((qh >> 24) & 0xff);
    }
    return;
  }
  if (type == RDO_Q4_1) {
    float vmin = x[0], vmax = x[0];
    for (int j = 1; j < 32; ++j) { vmin = fminf(vmin, x[j]); vmax = fmaxf(vmax, x[j]); }
    const float d = (vmax - vmin) / 15.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    put16(y, rdo_float_to_fp16(d));
    put16(y + 2, rdo_float_to_fp16(vmin));
    for (int j = 0; j < 16; ++j) {
      const float x0 = (x[j] - vmin) * id;
      const float x1 = (x[j + 16] - vmin) * id;
      const int q0 = clampi((int)(int8_t)(x0 + 0.5f), 15);
      const int q1 = clampi((int)(int8_t)(x1 + 0.5f), 15);
      y[4 + j] = (uint8_t)(q0 | (q1 << 4));
    }
  }
}

/* include/rdna4/kv.h:386-501 + launcher :673-694: `width` consecutive f32 values
 * become width/32 blocks (or width scalars). Returns 0, or -1 on a bad type or a
 * width that is not a multiple of 32 for a block type. */
int rdo_kv_store_rows(int type, const float *src, void *dst, int64_t width) {
  uint8_t *out = (uint8_t *)dst;
  if (type == RDO_F32) { memcpy(out, src, (size_t)width * 4); return 0; }
  if (type == RDO_F16) {
    for (int64_t i = 0; i < width; ++i) put16(out + 2 * i, rdo_float_to_fp16(src[i]));
    return 0;
  }
  if (type < RDO_Q8_0 || type > RDO_Q4_1) return -1;
  if (width % 32 != 0) return -1;
  const uint64_t bb = rdo_kv_row_bytes(type, 32);
  const int64_t nb = width / 32;
#pragma omp parallel for schedule(static) if (nb > 4096)
  for (int64_t b = 0; b < nb; ++b) quant_block(type, src + b * 32, out + (uint64_t)b * bb);
  return 0;
}

/* include/rdna4/kv.h:174-229: element `d` of a stored row. */
static float load_elem(int type, const uint8_t *row, int d) {
  switch (type) {
    case RDO_F32: { float f; memcpy(&f, row + 4 * (size_t)d, 4); return f; }
    case RDO_F16: return rdo_fp16_to_float(get16(row + 2 * (size_t)d));
    case RDO_Q8_0: {
      const uint8_t *b = row + (size_t)(d >> 5) * 34;
      return rdo_fp16_to_float(get16(b)) * (float)(int8_t)b[2 + (d & 31)];
    }
    case RDO_Q4_0: {
      const uint8_t *b = row + (size_t)(d >> 5) * 18;
      const int j = d & 31;
      const uint8_t byte = b[2 + (j & 15)];
      const int q = (j < 16) ? (byte & 0x0f) : (byte >> 4);
      return rdo_fp16_to_float(get16(b)) * (float)(q - 8);
    }
    case RDO_Q5_0: {
      const uint8_t *b = row + (size_t)(d >> 5) * 22;
      const int j = d & 31;
      const uint8_t byte = b[6 + (j & 15)];
      const int nib = (j < 16) ? (byte & 0x0f) : (byte >> 4);
      const int hi = (b[2 + (j >> 3)] >> (j & 7)) & 1;
      return rdo_fp16_to_float(get16(b)) * (float)((nib | (hi << 4)) - 16);
    }
    case RDO_Q4_1: {
      const uint8_t *b = row + (size_t)(d >> 5) * 20;
      const int j = d & 31;
      const uint8_t byte = b[4 + (j & 15)];
      const int q = (j < 16) ? (byte & 0x0f) : (byte >> 4);
      return rdo_fp16_to_float(get16(b)) * (float)q + rdo_fp16_to_float(get16(b + 2));
    }
  }
  return 0.0f;
}

int rdo_kv_dequant_rows(int type, const void *src, float *dst, int64_t n_rows, int head_dim) {
  const uint64_t rb = rdo_kv_row_bytes(type, head_dim);
  if (rb == 0) return -1;
#pragma omp parallel for schedule(static) if (n_rows > 1024)
  for (int64_t r = 0; r < n_rows; ++r)
    for (int d = 0; d < head_dim; ++d)
      dst[r * head_dim + d] = load_elem(type, (const uint8_t *)src + (uint64_t)r * rb, d);
  return 0;
}

/* include/rdna4/kv.h:508-513: the synthetic-cache hash. */
float rdo_kv_rand(uint32_t idx, uint32_t seed) {
  uint32_t h = idx * 2654435761u ^ seed * 2246822519u;
  h ^= h >> 13;
  h *= 1274126177u;
  return ((float)(h >> 8) / 8388608.0f) - 1.0f;
}

/* Values the fill kernel feeds to its quantizer: x[row*head_dim + e] =
 * kv_rand(row*head_dim + e, seed), index truncated to 32 bits as in
 * include/rdna4/kv.h:524. */
void rdo_kv_fill_values(float *dst, int64_t n_rows, int head_dim, uint32_t seed) {
  const int64_t n = n_rows * head_dim;
#pragma omp parallel for schedule(static) if (n > 65536)
  for (int64_t i = 0; i < n; ++i) dst[i] = rdo_kv_rand((uint32_t)i, seed);
}

/* include/rdna4/kv.h:515-630 as a contract: a cache whose rows hold the hash
 * values, stored with the real quantizer. For f32/f16/q8_0/q5_0/q4_1 that equals
 * the reference fill byte for byte; the reference's q4_0 fill writes one scale
 * per byte pair from 16 racing lanes (:607-627) and is not a block quantizer, so
 * for q4_0 this deliberately differs and the reference bytes are no fixture. */
int rdo_kv_fill(int type, void *cache, int64_t n_rows, int head_dim, uint32_t seed) {
  const uint64_t rb = rdo_kv_row_bytes(type, head_dim);
  if (rb == 0 || head_dim % 32 != 0) return -1;
#pragma omp parallel for schedule(static) if (n_rows > 256)
  for (int64_t r = 0; r < n_rows; ++r) {
    float tmp[512];
    for (int e = 0; e < head_dim; ++e) tmp[e] = rdo_kv_rand((uint32_t)(r * head_dim + e), seed);
    rdo_kv_store_rows(type, tmp, (uint8_t *)cache + (uint64_t)r * rb, head_dim);
  }
  return 0;
}

/* ------------------------------------------------------------------ RoPE -- */

/* include/rdna4/attn.cuh:30-54, host mirror tests/check_rope_gpu.hip:64-75:
 * split-half pairs (p, p+n_rot/2) of the first n_rot dims, f32 powf/cosf/sinf. */
void rdo_rope(float *x, int n_tok, int n_heads, int head_dim, int n_rot, float freq_base,
              const int32_t *pos) {
  const int pairs = n_rot / 2;
  for (int t = 0; t < n_tok; ++t)
    for (int h = 0; h < n_heads; ++h) {
      float *base = x + ((int64_t)t * n_heads + h) * head_dim;
      for (int p = 0; p < pairs; ++p) {
        const float theta = (float)pos[t] * powf(freq_base, -2.0f * (float)p / (float)n_rot);
        const float c = cosf(theta), s = sinf(theta);
        const float x0 = base[p], x1 = base[p + pairs];
        base[p] = x0 * c - x1 * s;
        base[p + pairs] = x0 * s + x1 * c;
      }
    }
}

/* ------------------------------------------------------------------ gate -- */

/* include/rdna4/nn.cuh:110,405-412: y *= 1/(1+expf(-g)); the sigmoid is written
 * back into g when store_sigmoid is non-zero (the decode path does). */
void rdo_sigmoid_gate(float *g, float *y, int64_t n, int store_sigmoid) {
  for (int64_t i = 0; i < n; ++i) {
    const float s = 1.0f / (1.0f + expf(-g[i]));
    if (store_sigmoid) g[i] = s;
    y[i] = y[i] * s;
  }
}

/* include/rdna4/nn.cuh:23-63: y = x * rsqrt(mean(x^2) + eps) (* w). The sum of squares
 * follows the kernel's order exactly: thread t accumulates elements t, t+256, ... with
 * fmaf, then a shared-memory tree adds partial[t + stride] into partial[t] for stride =
 * 128 .. 1. rsqrt is written as 1/sqrt (the device intrinsic is approximate; this is the
 * value the tests hold the CUDA kernel to). x and y may alias. */
void rdo_rms_norm(const float *x, const float *w, float *y, int64_t nrows, int64_t ncols, float eps) {
  for (int64_t r = 0; r < nrows; ++r) {
    const float *xr = x + r * ncols;
    float *yr = y + r * ncols;
    float partial[256];
    for (int t = 0; t < 256; ++t) {
      float acc = 0.0f;
      for (int64_t i = t; i < ncols; i += 256) acc = fmaf(xr[i], xr[i], acc);
      partial[t] = acc;
    }
    for (int stride = 128; stride > 0; stride >>= 1)
      for (int t = 0; t < stride; ++t) partial[t] += partial[t + stride];
    const float scale = 1.0f / sqrtf(partial[0] / (float)ncols + eps);
    for (int64_t i = 0; i < ncols; ++i) yr[i] = w ? xr[i] * scale * w[i] : xr[i] * scale;
  }
}

/* include/rdna4/gdn.cuh:367-375,838-851: per head [q(hd) | gate(hd)] -> q, gate. */
void rdo_deinterleave_q_gate(const float *yq, float *q, float *gate, int64_t n_tok, int n_head,
                             int head_dim) {
  for (int64_t i = 0; i < n_tok * n_head; ++i) {
    memcpy(q + i * head_dim, yq + i * 2 * head_dim, (size_t)head_dim * 4);
    memcpy(gate + i * head_dim, yq + i * 2 * head_dim + head_dim, (size_t)head_dim * 4);
  }
}

/* ------------------------------------------------------------- attention -- */

/* Causal GQA attention for n_tok query tokens over a stored cache:
 *   q, out [n_tok][n_head][head_dim] f32 (may alias), k/v rows [key][n_head_kv]
 *   of type kt/vt, token i attends keys 0..pos[i] inclusive.
 * Follows tests/check_rope_gpu.hip:103-130 (two-pass softmax over the
 * dequantized stored rows) with the accumulation width chosen by `f64`:
 *   0: f32 dot, f32 expf, f32 sums (the tolerance gates compare against this)
 *   1: double everywhere, as the reference's own host check does (yardstick).
 * Query head h reads kv head h/(n_head/n_head_kv) (include/rdna4/attn.cuh:104).
 * Zero keys (pos[i] < 0) give zeros (attn.cuh:163-166). */
int rdo_attn(const float *q, const void *k, const void *v, float *out, const int32_t *pos,
             int n_tok, int n_head, int n_head_kv, int head_dim, float scale, int kt, int vt,
             int f64) {
  const uint64_t krb = rdo_kv_row_bytes(kt, head_dim), vrb = rdo_kv_row_bytes(vt, head_dim);
  if (!krb || !vrb || n_head_kv <= 0 || n_head % n_head_kv) return -1;
  const int grp = n_head / n_head_kv;
  int maxpos = -1;
  for (int i = 0; i < n_tok; ++i) if (pos[i] > maxpos) maxpos = pos[i];
  const int64_t nkeys = (int64_t)maxpos + 1;
  /* dequantize every needed row once */
  float *kf = (float *)malloc((size_t)(nkeys > 0 ? nkeys : 1) * n_head_kv * head_dim * 4);
  float *vf = (float *)malloc((size_t)(nkeys > 0 ? nkeys : 1) * n_head_kv * head_dim * 4);
  if (!kf || !vf) { free(kf); free(vf); return -2; }
  rdo_kv_dequant_rows(kt, k, kf, nkeys * n_head_kv, head_dim);
  rdo_kv_dequant_rows(vt, v, vf, nkeys * n_head_kv, head_dim);
  float *qc = (float *)malloc((size_t)n_tok * n_head * head_dim * 4);
  memcpy(qc, q, (size_t)n_tok * n_head * head_dim * 4); /* q and out may alias */
  int rc = 0;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int i = 0; i < n_tok; ++i)
    for (int h = 0; h < n_head; ++h) {
      const int t = pos[i];
      const int kvh = h / grp;
      const float *qr = qc + ((int64_t)i * n_head + h) * head_dim;
      float *o = out + ((int64_t)i * n_head + h) * head_dim;
      if (t < 0) { for (int d = 0; d < head_dim; ++d) o[d] = 0.0f; continue; }
      if (!f64) {
        float *sc = (float *)malloc((size_t)(t + 1) * 4);
        float m = -INFINITY;
        for (int j = 0; j <= t; ++j) {
          const float *kr = kf + ((int64_t)j * n_head_kv + kvh) * head_dim;
          float dsum = 0.0f;
          for (int d = 0; d < head_dim; ++d) dsum += qr[d] * kr[d];
          sc[j] = dsum * scale;
          if (sc[j] > m) m = sc[j];
        }
        float sum = 0.0f;
        for (int j = 0; j <= t; ++j) { sc[j] = expf(sc[j] - m); sum += sc[j]; }
        float acc[512];
        for (int d = 0; d < head_dim; ++d) acc[d] = 0.0f;
        for (int j = 0; j <= t; ++j) {
          const float *vr = vf + ((int64_t)j * n_head_kv + kvh) * head_dim;
          const float p = sc[j];
          for (int d = 0; d < head_dim; ++d) acc[d] += p * vr[d];
        }
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
        for (int d = 0; d < head_dim; ++d) o[d] = acc[d] * inv;
        free(sc);
      } else {
        double *sc = (double *)malloc((size_t)(t + 1) * 8);
        double m = -1e300;
        for (int j = 0; j <= t; ++j) {
          const float *kr = kf + ((int64_t)j * n_head_kv + kvh) * head_dim;
          double dsum = 0.0;
          for (int d = 0; d < head_dim; ++d) dsum += (double)qr[d] * kr[d];
          sc[j] = dsum * (double)scale;
          if (sc[j] > m) m = sc[j];
        }
        double sum = 0.0;
        for (int j = 0; j <= t; ++j) { sc[j] = exp(sc[j] - m); sum += sc[j]; }
        double acc[512];
        for (int d = 0; d < head_dim; ++d) acc[d] = 0.0;
        for (int j = 0; j <= t; ++j) {
          const float *vr = vf + ((int64_t)j * n_head_kv + kvh) * head_dim;
          const double p = sc[j];
          for (int d = 0; d < head_dim; ++d) acc[d] += p * vr[d];
        }
        for (int d = 0; d < head_dim; ++d) o[d] = (float)(acc[d] / sum);
        free(sc);
      }
    }
  free(kf); free(vf); free(qc);
  return rc;
}

/* Partial records of a split evaluation, include/rdna4/attn.cuh:445-560 as a
 * contract: record (h, s) = (m, l, acc[head_dim]) with m = max score over the
 * keys split s owns, l = sum exp(score-m), acc = sum exp(score-m)*v; an empty
 * split is (-inf, 0, 0...). Split s of n_splits owns the contiguous key range
 * [key_begin + s*len, key_begin + (s+1)*len) cut to key_end, len =
 * ceil((key_end-key_begin)/n_splits): WHICH keys a split owns is not observable
 * after the merge, so the oracle uses contiguous ranges (what a context sharded
 * over devices holds) rather than the reference's warp-strided walk.
 * q is one token [n_head][head_dim]; f32 accumulation. */
int rdo_attn_partials(const float *q, const void *k, const void *v, float *partial,
                      int key_begin, int key_end, int n_head, int n_head_kv, int head_dim,
                      float scale, int kt, int vt, int n_splits) {
  const uint64_t krb = rdo_kv_row_bytes(kt, head_dim), vrb = rdo_kv_row_bytes(vt, head_dim);
  if (!krb || !vrb || n_splits < 1 || n_head_kv <= 0 || n_head % n_head_kv) return -1;
  const int grp = n_head / n_head_kv;
  const int total = key_end > key_begin ? key_end - key_begin : 0;
  const int len = (total + n_splits - 1) / n_splits;
  const int rec = 2 + head_dim;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int h = 0; h < n_head; ++h)
    for (int s = 0; s < n_splits; ++s) {
      const int kvh = h / grp;
      float *r = partial + ((int64_t)h * n_splits + s) * rec;
      int b = key_begin + s * len, e = b + len;
      if (e > key_end) e = key_end;
      float m = -INFINITY, l = 0.0f;
      for (int d = 0; d < head_dim; ++d) r[2 + d] = 0.0f;
      if (b < e && len > 0) {
        float *sc = (float *)malloc((size_t)(e - b) * 4);
        for (int j = b; j < e; ++j) {
          const uint8_t *kr = (const uint8_t *)k + ((uint64_t)j * n_head_kv + kvh) * krb;
          float dsum = 0.0f;
          for (int d = 0; d < head_dim; ++d) dsum += q[h * head_dim + d] * load_elem(kt, kr, d);
          sc[j - b] = dsum * scale;
          if (sc[j - b] > m) m = sc[j - b];
        }
        for (int j = b; j < e; ++j) {
          const uint8_t *vr = (const uint8_t *)v + ((uint64_t)j * n_head_kv + kvh) * vrb;
          const float p = expf(sc[j - b] - m);
          l += p;
          for (int d = 0; d < head_dim; ++d) r[2 + d] += p * load_elem(vt, vr, d);
        }
        free(sc);
      }
      r[0] = m;
      r[1] = l;
    }
  return 0;
}

/* include/rdna4/attn.cuh:563-590 (f32, same statement order) or, with f64 != 0,
 * the host form of tests/bench_attn_gpu.hip:1287-1322. partial is
 * [n_rows][n_splits][2+head_dim], out [n_rows][head_dim]; a row whose splits are
 * all empty gives zeros. */
void rdo_attn_merge(const float *partial, float *out, int n_rows, int head_dim, int n_splits,
                    int f64) {
  const int rec = 2 + head_dim;
  for (int h = 0; h < n_rows; ++h) {
    const float *base = partial + (int64_t)h * n_splits * rec;
    float *o = out + (int64_t)h * head_dim;
    if (!f64) {
      float mm = -INFINITY;
      for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, base[(int64_t)s * rec]);
      if (mm == -INFINITY) { for (int d = 0; d < head_dim; ++d) o[d] = 0.0f; continue; }
      float ll = 0.0f;
      for (int s = 0; s < n_splits; ++s) ll += base[(int64_t)s * rec + 1] * expf(base[(int64_t)s * rec] - mm);
      const float inv = ll > 0.0f ? 1.0f / ll : 0.0f;
      for (int d = 0; d < head_dim; ++d) {
        float a = 0.0f;
        for (int s = 0; s < n_splits; ++s)
          a += base[(int64_t)s * rec + 2 + d] * expf(base[(int64_t)s * rec] - mm);
        o[d] = a * inv;
      }
    } else {
      double mm = -INFINITY;
      for (int s = 0; s < n_splits; ++s) mm = fmax(mm, (double)base[(int64_t)s * rec]);
      if (mm == -INFINITY) { for (int d = 0; d < head_dim; ++d) o[d] = 0.0f; continue; }
      double ll = 0.0;
      for (int s = 0; s < n_splits; ++s) {
        if (base[(int64_t)s * rec] == -INFINITY) continue;
        ll += (double)base[(int64_t)s * rec + 1] * exp((double)base[(int64_t)s * rec] - mm);
      }
      for (int d = 0; d < head_dim; ++d) {
        double a = 0.0;
        for (int s = 0; s < n_splits; ++s) {
          if (base[(int64_t)s * rec] == -INFINITY) continue;
          a += (double)base[(int64_t)s * rec + 2 + d] * exp((double)base[(int64_t)s * rec] - mm);
        }
        o[d] = (float)(ll > 0 ? a / ll : 0.0);
      }
    }
  }
}

int rdo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void rdo_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
