/*
 * CPU oracle for the decode hot path: a plain-C restatement of the reference's
 * CPU operators.  TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the
 * benchmark's cpu_baseline leg load this; no product code path may.
 *
 * Every function follows one reference routine (cited by file:line, paths
 * relative to the reference project) in the same arithmetic order: the same
 * fp32 accumulators, the same loop nesting, the same libm calls (powf, cosf,
 * sinf, expf, sqrtf).  Parity pin: tests compare these functions bit-for-bit
 * with the reference's own CPU library compiled from its sources
 * (oracle/_ref, built by oracle/Makefile) and with committed golden vectors
 * produced by that library.
 *
 * Build: gcc -O3 -fopenmp -mavx2 -mfma -shared -fPIC (oracle/Makefile): the flags
 * of the reference's own x86-64 build (CMakeLists.txt:40-70), floating-point
 * contraction left at the compiler default in both, so the same expressions
 * contract to the same FMAs.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_OK 0
#define ORC_INVALID_ARGUMENT 1
#define ORC_SHAPE_MISMATCH 4

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ---- fp16 bit conversions: include/axono/core/half.h:14-79 ---------------- */

/* half.h:55-79 (Half2Float): exact widening, subnormals normalised by shifting. */
float orc_half_to_float1(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1Fu;
  const uint32_t man = h & 0x3FFu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) {
      x = sign;
    } else {
      int32_t e = -1;
      uint32_t m = man;
      while ((m & 0x400u) == 0) {
        m <<= 1;
        --e;
      }
      m &= 0x3FFu;
      x = sign | ((uint32_t)(127 - 15 + e + 1) << 23) | (m << 13);
    }
  } else if (exp == 0x1F) {
    x = sign | 0x7F800000u | (man << 13);
  } else {
    x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  }
  float out;
  memcpy(&out, &x, sizeof(out));
  return out;
}

/* half.h:14-52 (Float2Half).  The reference's "round to nearest even" adds 1 to
 * the 23-bit mantissa (not to bit 13), so normal values are in effect truncated;
 * restated as written, because this is what the reference's CPU cast produces. */
uint16_t orc_float_to_half1(float value) {
  uint32_t x;
  memcpy(&x, &value, sizeof(x));
  const uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t exp = (x >> 23) & 0xFFu;
  uint32_t man = x & 0x7FFFFFu;
  if (exp == 0xFF) {
    return (uint16_t)(sign | 0x7C00u | (man ? (man >> 13 ? 0x0200u : 1) : 0));
  }
  int32_t e = (int32_t)exp - 127 + 15;
  if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign;
    man |= 0x800000u;
    const uint32_t shift = (uint32_t)(14 - e);
    const uint32_t round = (1u << (shift - 1));
    uint16_t half_man = (uint16_t)(
        (man >> shift) +
        ((man & round) != 0 && ((man >> shift) & 1 || (man & (round << 1)) != 0) ? 1 : 0));
    return (uint16_t)(sign | half_man);
  }
  const uint32_t round = 0x00001000u;
  uint32_t m = man + (((man & round) != 0 && (man & (round << 1)) != 0) ? 0x1u : 0x0u);
  uint32_t half = ((uint32_t)e << 10) | (m >> 13);
  return (uint16_t)(sign | half);
}

void orc_half_to_float(const uint16_t *h, float *out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = orc_half_to_float1(h[i]);
}

void orc_float_to_half(const float *x, uint16_t *out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = orc_float_to_half1(x[i]);
}

/* ---- attention: src/ops/cpu/sequence.cpp:236-301 -------------------------- */

/* ScaledDotProductAttention with GQA head mapping hk = h / group.  q (sq,hq,d),
 * k/v (skv,hkv,d) token-major, out (sq,hq,d).  Three passes per (t,h): scores
 * with a serial fp32 dot, max, exp+sum, then the weighted V sum with p = e*inv. */
int orc_sdpa_f32(const float *qp, const float *kp, const float *vp, float *rp,
                 size_t sq, size_t hq, size_t hkv, size_t d, size_t skv,
                 int is_causal) {
  if (hkv == 0 || hq % hkv != 0) return ORC_SHAPE_MISMATCH;
  if (skv == 0) return ORC_INVALID_ARGUMENT;
  const size_t group = hq / hkv;
  const float scale = 1.0f / sqrtf((float)d);
  int64_t t, h;
#pragma omp parallel for collapse(2) schedule(static)
  for (t = 0; t < (int64_t)sq; ++t) {
    for (h = 0; h < (int64_t)hq; ++h) {
      const float *qr = qp + ((size_t)t * hq + (size_t)h) * d;
      float *outr = rp + ((size_t)t * hq + (size_t)h) * d;
      const size_t hk = (size_t)h / group;
      size_t kv_end = skv;
      if (is_causal && skv >= (size_t)t + 1) kv_end = (size_t)t + 1;
      float *scores = (float *)malloc(kv_end * sizeof(float));
      for (size_t s = 0; s < kv_end; ++s) {
        const float *kr = kp + (s * hkv + hk) * d;
        float acc = 0.0f;
        for (size_t i = 0; i < d; ++i) acc += qr[i] * kr[i];
        scores[s] = acc * scale;
      }
      float mx = scores[0];
      for (size_t s = 1; s < kv_end; ++s) mx = scores[s] > mx ? scores[s] : mx;
      float sum = 0.0f;
      for (size_t s = 0; s < kv_end; ++s) {
        scores[s] = expf(scores[s] - mx);
        sum += scores[s];
      }
      const float inv = 1.0f / sum;
      for (size_t i = 0; i < d; ++i) outr[i] = 0.0f;
      for (size_t s = 0; s < kv_end; ++s) {
        const float p = scores[s] * inv;
        const float *vr = vp + (s * hkv + hk) * d;
        for (size_t i = 0; i < d; ++i) outr[i] += p * vr[i];
      }
      free(scores);
    }
  }
  return ORC_OK;
}

/* Batched decode attention as the reference would evaluate it: B independent
 * calls of the single-sequence op (the reference has no batch dimension,
 * src/ops/cuda/gqa.cu:139-148).  q/out (B,hq,d); sequence b's keys/values are
 * the first lens[b] rows of k + b*seq_stride (token-major (cap,hkv,d)). */
int orc_gqa_decode_batched_f32(const float *q, const float *k, const float *v,
                               float *out, const int32_t *lens, size_t B,
                               size_t hq, size_t hkv, size_t d,
                               size_t seq_stride_elems) {
  for (size_t b = 0; b < B; ++b) {
    int st = orc_sdpa_f32(q + b * hq * d, k + b * seq_stride_elems,
                          v + b * seq_stride_elems, out + b * hq * d, 1, hq, hkv,
                          d, (size_t)lens[b], 0);
    if (st != ORC_OK) return st;
  }
  return ORC_OK;
}

/* ---- RoPE: src/ops/cpu/sequence.cpp:54-93 --------------------------------- */

/* Rotate-half pairs (i, i+half); freq = powf(theta, -2i/dim); angle =
 * float(pos[r]) * freq; x (rows,heads,dim), pos int64[rows]. */
int orc_rope_f32(const float *xp, const int64_t *pos, float theta, float *rp,
                 size_t rows, size_t heads, size_t dim) {
  if (dim % 2 != 0) return ORC_INVALID_ARGUMENT;
  const size_t half = dim / 2;
  int64_t r, h;
#pragma omp parallel for collapse(2) schedule(static)
  for (r = 0; r < (int64_t)rows; ++r) {
    for (h = 0; h < (int64_t)heads; ++h) {
      const float *src = xp + ((size_t)r * heads + (size_t)h) * dim;
      float *dst = rp + ((size_t)r * heads + (size_t)h) * dim;
      const float p = (float)pos[r];
      for (size_t i = 0; i < half; ++i) {
        const float freq = powf(theta, -2.0f * (float)i / (float)dim);
        const float ang = p * freq;
        const float c = cosf(ang), s = sinf(ang);
        const float a = src[i], b = src[i + half];
        dst[i] = a * c - b * s;
        dst[i + half] = b * c + a * s;
      }
    }
  }
  return ORC_OK;
}

/* The inverse-frequency table the rope op uses internally (sequence.cpp:83-84),
 * exposed so tests can pin the product's host-side table against it. */
void orc_rope_inv_freq(float theta, size_t dim, float *out) {
  for (size_t i = 0; i < dim / 2; ++i)
    out[i] = powf(theta, -2.0f * (float)i / (float)dim);
}

/* RopeWithCosSin: src/ops/cpu/sequence.cpp:96-138.  cos/sin (rows,dim). */
int orc_rope_with_cos_sin_f32(const float *xp, const float *cp, const float *sp,
                              float *rp, size_t rows, size_t heads, size_t dim) {
  if (dim % 2 != 0) return ORC_INVALID_ARGUMENT;
  const size_t half = dim / 2;
  int64_t r, h;
#pragma omp parallel for collapse(2) schedule(static)
  for (r = 0; r < (int64_t)rows; ++r) {
    for (h = 0; h < (int64_t)heads; ++h) {
      const float *src = xp + ((size_t)r * heads + (size_t)h) * dim;
      float *dst = rp + ((size_t)r * heads + (size_t)h) * dim;
      const float *cr = cp + (size_t)r * dim;
      const float *sr = sp + (size_t)r * dim;
      for (size_t i = 0; i < half; ++i) {
        const float a = src[i], b = src[i + half];
        dst[i] = a * cr[i] - b * sr[i];
        dst[i + half] = b * cr[i + half] + a * sr[i + half];
      }
    }
  }
  return ORC_OK;
}

/* The stride-3 M-RoPE position rule shared by MropeCosSin and RopeThd
 * (sequence.cpp:166-171, 222-227): pair i takes the H position when
 * i%3==1 && i<3*h_sec, the W position when i%3==2 && i<3*w_sec, else T. */
static inline float orc_mrope_angle(size_t i, float f, float pt, float ph,
                                    float pw, size_t h_lim, size_t w_lim) {
  float angle = pt * f;
  if (i % 3 == 1 && i < h_lim)
    angle = ph * f;
  else if (i % 3 == 2 && i < w_lim)
    angle = pw * f;
  return angle;
}

/* MropeCosSin: src/ops/cpu/sequence.cpp:140-182.  pos int64 (3,rows) row-major,
 * inv_freq (half); cos/sin out (rows, 2*half) with the halves duplicated. */
int orc_mrope_cos_sin_f32(const int64_t *pp, const float *fp, int h_sec,
                          int w_sec, float *cp, float *sp, size_t rows,
                          size_t half) {
  if (half == 0) return ORC_INVALID_ARGUMENT;
  const size_t h_lim = (size_t)h_sec * 3, w_lim = (size_t)w_sec * 3;
  int64_t r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < (int64_t)rows; ++r) {
    const float pt = (float)pp[r];
    const float ph = (float)pp[rows + (size_t)r];
    const float pw = (float)pp[2 * rows + (size_t)r];
    float *cr = cp + (size_t)r * (2 * half);
    float *sr = sp + (size_t)r * (2 * half);
    for (size_t i = 0; i < half; ++i) {
      const float angle = orc_mrope_angle(i, fp[i], pt, ph, pw, h_lim, w_lim);
      const float c = cosf(angle), sn = sinf(angle);
      cr[i] = c;
      cr[i + half] = c;
      sr[i] = sn;
      sr[i + half] = sn;
    }
  }
  return ORC_OK;
}

/* RopeThd (M-RoPE applied to a tensor): src/ops/cpu/sequence.cpp:184-234.
 * t_sec is accepted and ignored, as in the reference (:206). */
int orc_rope_thd_f32(const float *xp, const int64_t *pp, const float *fp,
                     int t_sec, int h_sec, int w_sec, float *rp, size_t rows,
                     size_t heads, size_t dim) {
  (void)t_sec;
  if (dim % 2 != 0) return ORC_INVALID_ARGUMENT;
  const size_t half = dim / 2;
  const size_t h_lim = (size_t)h_sec * 3, w_lim = (size_t)w_sec * 3;
  int64_t r, h;
#pragma omp parallel for collapse(2) schedule(static)
  for (r = 0; r < (int64_t)rows; ++r) {
    for (h = 0; h < (int64_t)heads; ++h) {
      const float *src = xp + ((size_t)r * heads + (size_t)h) * dim;
      float *dst = rp + ((size_t)r * heads + (size_t)h) * dim;
      const float pt = (float)pp[r];
      const float ph = (float)pp[rows + (size_t)r];
      const float pw = (float)pp[2 * rows + (size_t)r];
      for (size_t i = 0; i < half; ++i) {
        const float angle = orc_mrope_angle(i, fp[i], pt, ph, pw, h_lim, w_lim);
        const float c = cosf(angle), s = sinf(angle);
        const float a = src[i], b = src[i + half];
        dst[i] = a * c - b * s;
        dst[i + half] = b * c + a * s;
      }
    }
  }
  return ORC_OK;
}

/* ---- KV append = Concat: src/ops/cpu/sequence.cpp:303-338 ------------------ */

/* Byte-wise concat of a (outer, a_inner_bytes) and b (outer, b_inner_bytes)
 * along the axis that follows `outer`; axis 0 is outer == 1, which is what
 * DynamicKVCache.update does per layer (axono/python/axono/nn/kv_cache.py:96-102). */
int orc_concat_bytes(const void *a, const void *b, void *out, size_t outer,
                     size_t a_bytes, size_t b_bytes) {
  const char *ap = (const char *)a, *bp = (const char *)b;
  char *rp = (char *)out;
  for (size_t o = 0; o < outer; ++o) {
    memcpy(rp, ap + o * a_bytes, a_bytes);
    rp += a_bytes;
    memcpy(rp, bp + o * b_bytes, b_bytes);
    rp += b_bytes;
  }
  return ORC_OK;
}

/* ---- fused ops: src/ops/cpu/fused.cpp:16-76 -------------------------------- */

/* SiluMul (fused.cpp:16-35): g / (1 + exp(-g)) * u. */
int orc_silu_mul_f32(const float *gp, const float *up, float *yp, size_t n) {
  int64_t i;
#pragma omp parallel for schedule(static)
  for (i = 0; i < (int64_t)n; ++i) {
    const float g = gp[i];
    yp[i] = g / (1.0f + expf(-g)) * up[i];
  }
  return ORC_OK;
}

/* AddRmsNorm (fused.cpp:37-76): y = x + res stored, serial fp32 sum of y*y,
 * rms = 1/sqrt(sum/hidden + eps), out = y * rms * w (left to right). */
int orc_add_rms_norm_f32(const float *xp, const float *rp, const float *wp,
                         float eps, float *yp, float *op, size_t rows,
                         size_t hidden) {
  int64_t r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < (int64_t)rows; ++r) {
    const float *xr = xp + (size_t)r * hidden;
    const float *rr = rp + (size_t)r * hidden;
    float *yr = yp + (size_t)r * hidden;
    float *orr = op + (size_t)r * hidden;
    float sum = 0.0f;
    for (size_t i = 0; i < hidden; ++i) {
      const float v = xr[i] + rr[i];
      yr[i] = v;
      sum += v * v;
    }
    const float rms = 1.0f / sqrtf(sum / (float)hidden + eps);
    for (size_t i = 0; i < hidden; ++i) orr[i] = yr[i] * rms * wp[i];
  }
  return ORC_OK;
}

/* RmsNorm: src/ops/cpu/llm.cpp:57-92 (NormRows, rms_mode) and :240-264.
 * weight may be NULL (no scale). */
int orc_rms_norm_f32(const float *x, const float *weight, float eps, float *out,
                     size_t rows, size_t cols) {
  int64_t r;
#pragma omp parallel for schedule(static)
  for (r = 0; r < (int64_t)rows; ++r) {
    const float *xr = x + (size_t)r * cols;
    float *orr = out + (size_t)r * cols;
    float ss = 0.0f;
    for (size_t c = 0; c < cols; ++c) ss += xr[c] * xr[c];
    const float inv = 1.0f / sqrtf(ss / (float)cols + eps);
    for (size_t c = 0; c < cols; ++c) {
      const float normed = xr[c] * inv;
      orr[c] = weight ? normed * weight[c] : normed;
    }
  }
  return ORC_OK;
}

/* ---- M-RoPE positions: examples/vlm/qwen3vl/model.py:49-61 ----------------- */

/* build_mrope_pos3 for one image: text before the image counts 0..img_start-1 on
 * all three axes; image token j gets T=img_start, H=img_start+j/llm_w,
 * W=img_start+j%llm_w; text after resumes at img_start+max(llm_h,llm_w).
 * pos3 is int64 (3,n) row-major. */
void orc_build_mrope_pos3(int64_t *pos3, size_t n, size_t img_start, size_t want,
                          size_t llm_h, size_t llm_w) {
  for (size_t ax = 0; ax < 3; ++ax)
    for (size_t i = 0; i < img_start && i < n; ++i) pos3[ax * n + i] = (int64_t)i;
  const int64_t cur = (int64_t)img_start;
  for (size_t j = 0; j < want && img_start + j < n; ++j) {
    pos3[0 * n + img_start + j] = cur;
    pos3[1 * n + img_start + j] = cur + (int64_t)(j / llm_w);
    pos3[2 * n + img_start + j] = cur + (int64_t)(j % llm_w);
  }
  const int64_t after = cur + (int64_t)(llm_h > llm_w ? llm_h : llm_w);
  for (size_t ax = 0; ax < 3; ++ax)
    for (size_t i = img_start + want; i < n; ++i)
      pos3[ax * n + i] = after + (int64_t)(i - (img_start + want));
}

/* ---- Embedding / ArgmaxLastDim: src/ops/cpu/sequence.cpp:18-52, 370-400 ---------------------- */

/* table (vocab,hidden) fp32; ids int64[n]; out (n,hidden): row copy per id. */
int orc_embedding_f32(const int64_t *ids, const float *table, float *out, size_t n, size_t hidden) {
  for (size_t i = 0; i < n; ++i)
    memcpy(out + i * hidden, table + (size_t)ids[i] * hidden, hidden * sizeof(float));
  return ORC_OK;
}

/* First maximum wins: best = 0; for c >= 1: if (row[c] > row[best]) best = c. */
int orc_argmax_last_dim_f32(const float *x, int64_t *out, size_t rows, size_t cols) {
  for (size_t r = 0; r < rows; ++r) {
    const float *row = x + r * cols;
    int64_t best = 0;
    for (size_t c = 1; c < cols; ++c)
      if (row[c] > row[best]) best = (int64_t)c;
    out[r] = best;
  }
  return ORC_OK;
}
