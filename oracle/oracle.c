/*
 * CPU restatement of the attention hot path of bonsai-pot (Rust + WGSL).
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA kernels are
 * compared against and the timed CPU baseline; no product code path may call
 * into it.
 *
 * PARITY UNPINNED: the reference ships no golden vectors for this path and
 * cannot be built or run where this oracle runs (Rust + wgpu/Vulkan). What IS
 * pinned by the reference's own unit tests, and re-checked by the tests of
 * this repository: the snapshot payload sizes and offsets
 * (src/kv_snapshot.rs:430-468), the 32-byte header (src/kv_snapshot.rs:69-80)
 * and the RoPE-table sample values (src/model.rs:2021-2045).
 *
 * Every function cites the reference lines it restates (paths are relative to
 * the reference repository).
 *
 * Evaluation rules fixed here, because WGSL leaves them to the driver:
 *   - IEEE binary32, round-to-nearest-even, no FMA contraction (compile with
 *     -ffp-contract=off; the optional `contract` switch re-enables it on
 *     purpose for the sensitivity report);
 *   - inverseSqrt(x) is the correctly rounded 1/sqrt(x);
 *   - `/` is correctly rounded; round() is ties-to-even;
 *   - f32 -> f16 casts round to nearest even; f16 -> f32 is exact;
 *   - the 128-lane sum of squares is an xor butterfly (offsets 16,8,4,2,1)
 *     inside each aligned group of 32 lanes, then (w0 + w1) + (w2 + w3).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HEAD_DIM 128u
#define HALF_DIM 64u
#define QK8_0 32u
#define ATTN_CHUNK 16u      /* src/model.rs:511 ATTN_CHUNK_SIZE */
#define PARTIAL_STRIDE 130u /* attention_split.wgsl:57 */

/* ------------------------------------------------------------------ f16 -- */

float orc_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        e++;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | (exp + 112u) << 23 | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t orc_f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t abs = x & 0x7FFFFFFFu;
  if (abs >= 0x7F800000u) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((abs > 0x7F800000u) ? 0x200u : 0u));
  }
  if (abs >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (abs < 0x33000001u) { /* < 2^-25 (or exactly 2^-25: tie to even -> 0) */
    return (uint16_t)sign;
  }
  int32_t e = (int32_t)(abs >> 23) - 127;
  uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
  uint32_t shift, half_bits;
  if (e < -14) { /* subnormal result */
    shift = (uint32_t)(13 + (-14 - e));
    half_bits = 0;
  } else {
    shift = 13;
    half_bits = (uint32_t)(e + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t q = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  uint32_t out = half_bits + q;
  if (rem > halfway || (rem == halfway && (q & 1u))) out += 1u;
  return (uint16_t)(sign | out);
}

/* --------------------------------------------------------------- layout -- */
/* src/forward.rs:48-58 (kv_qs_byte_base, kv_layer_offsets);
 * src/kv_snapshot.rs:172-180 (buf_d_offset, buf_qs_offset). */

uint64_t orc_kv_d_total(uint32_t n_layer, uint32_t max_seq, uint32_t kv_dim) {
  return (uint64_t)n_layer * max_seq * (kv_dim / QK8_0) * 4u;
}
uint64_t orc_kv_total_bytes(uint32_t n_layer, uint32_t max_seq, uint32_t kv_dim) {
  return orc_kv_d_total(n_layer, max_seq, kv_dim) + (uint64_t)n_layer * max_seq * kv_dim;
}
uint64_t orc_buf_d_offset(uint32_t max_seq, uint32_t kv_dim, uint32_t il) {
  return (uint64_t)il * max_seq * (kv_dim / QK8_0) * 4u;
}
uint64_t orc_buf_qs_offset(uint32_t n_layer, uint32_t max_seq, uint32_t kv_dim, uint32_t il) {
  return orc_kv_d_total(n_layer, max_seq, kv_dim) + (uint64_t)il * max_seq * kv_dim;
}
/* src/kv_snapshot.rs:150-154 */
uint64_t orc_payload_bytes(uint32_t n_layer, uint32_t kv_dim, uint32_t pos) {
  uint64_t d_layer = (uint64_t)pos * (kv_dim / QK8_0) * 4u;
  uint64_t qs_layer = (uint64_t)pos * kv_dim;
  return 2u * (uint64_t)n_layer * (d_layer + qs_layer);
}
/* src/kv_snapshot.rs:158-169; kind 0 = K, 1 = V; sect 0 = d, 1 = qs */
uint64_t orc_payload_offset(uint32_t n_layer, uint32_t kv_dim, uint32_t pos, uint32_t kind,
                            uint32_t il, uint32_t sect) {
  uint64_t d_layer = (uint64_t)pos * (kv_dim / QK8_0) * 4u;
  uint64_t qs_layer = (uint64_t)pos * kv_dim;
  uint64_t layer_bytes = d_layer + qs_layer;
  uint64_t base = (uint64_t)kind * n_layer * layer_bytes + (uint64_t)il * layer_bytes;
  return sect == 0 ? base : base + d_layer;
}

/* ----------------------------------------------------------------- RoPE -- */
/* src/model.rs:1756-1769 build_rope_table: f64 pow/cos/sin, cast to f32;
 * src/model.rs:1148-1149 then casts the table to f16. */

void orc_build_rope_table_f32(uint32_t head_dim, float freq_base, uint32_t max_seq, float* out) {
  uint32_t half = head_dim / 2;
  for (uint32_t p = 0; p < max_seq; p++) {
    for (uint32_t j = 0; j < half; j++) {
      double theta = pow((double)freq_base, -2.0 * (double)j / (double)head_dim);
      double angle = (double)p * theta;
      out[(size_t)p * head_dim + 2 * j] = (float)cos(angle);
      out[(size_t)p * head_dim + 2 * j + 1] = (float)sin(angle);
    }
  }
}

void orc_build_rope_table_f16(uint32_t head_dim, float freq_base, uint32_t max_seq, uint16_t* out) {
  uint32_t half = head_dim / 2;
#pragma omp parallel for schedule(static)
  for (uint32_t p = 0; p < max_seq; p++) {
    for (uint32_t j = 0; j < half; j++) {
      double theta = pow((double)freq_base, -2.0 * (double)j / (double)head_dim);
      double angle = (double)p * theta;
      out[(size_t)p * head_dim + 2 * j] = orc_f32_to_f16((float)cos(angle));
      out[(size_t)p * head_dim + 2 * j + 1] = orc_f32_to_f16((float)sin(angle));
    }
  }
}

/* --------------------------------------------- norm + RoPE + quantise ---- */

/* Sign of mid^2 * x - 1, exactly, for a positive `mid` with at most 26 significant bits (a float
 * or the midpoint of two adjacent floats) and a positive normal float x: integer mantissas, one
 * 128-bit product, a power-of-two comparison. mid^2 * x > 1 is the same as 1/sqrt(x) < mid. */
static int mid2x_vs_one(double mid, float x) {
  int e1, e2;
  const double fm = frexp(mid, &e1);       /* mid = fm * 2^e1, fm in [0.5, 1) */
  const float fx = frexpf(x, &e2);
  const uint64_t m = (uint64_t)ldexp(fm, 26); /* exact: at most 26 bits */
  const uint64_t xm = (uint64_t)ldexpf(fx, 24);
  const unsigned __int128 p = (unsigned __int128)(m * m) * xm; /* < 2^76 */
  const int s = -(2 * (e1 - 26) + (e2 - 24));                  /* compare p with 2^s */
  if (s < 0) return 1;
  if (s > 126) return -1;
  const unsigned __int128 one = (unsigned __int128)1 << s;
  return p > one ? 1 : (p < one ? -1 : 0);
}

/* Correctly rounded 1/sqrt(x) for positive normal x (CUDA's __frsqrt_rn, WGSL's inverseSqrt taken
 * at its best): a binary64 estimate picks the candidate, and the exact comparison above moves it to
 * a neighbour when 1/sqrt(x) lies on the other side of the midpoint. No tie exists: a midpoint of
 * two floats has an odd 25-bit mantissa, and 1/mid^2 is then not a dyadic number, so it cannot be x. */
static float rsqrt_rn(float x) {
  float c = (float)(1.0 / sqrt((double)x));
  for (int iter = 0; iter < 2; iter++) {
    const float lo = nextafterf(c, 0.0f), hi = nextafterf(c, INFINITY);
    if (mid2x_vs_one(((double)lo + (double)c) * 0.5, x) > 0) c = lo;       /* 1/sqrt(x) below the lower midpoint */
    else if (mid2x_vs_one(((double)c + (double)hi) * 0.5, x) < 0) c = hi;  /* above the upper midpoint */
    else break;
  }
  return c;
}

/* For the tests: the function above; the earlier evaluation through an 80-bit long double (two
 * roundings); and a sweep over `count` inputs from bit pattern `first` in steps of `stride` that
 * returns how many of them the two evaluate differently (and checks on each that the exact result
 * has 1/sqrt(x) between its two midpoints: a violation returns UINT64_MAX). */
float orc_rsqrt_rn(float x) { return rsqrt_rn(x); }
float orc_rsqrt_long_double(float x) { return (float)(1.0L / sqrtl((long double)x)); }
uint64_t orc_rsqrt_sweep(uint32_t first, uint64_t count, uint32_t stride) {
  uint64_t differ = 0, bad = 0;
#pragma omp parallel for schedule(static) reduction(+ : differ, bad)
  for (uint64_t i = 0; i < count; i++) {
    const uint32_t bits = first + (uint32_t)(i * stride);
    float x;
    memcpy(&x, &bits, 4);
    if (!(x >= 1.17549435e-38f) || !(x <= 3.0e38f)) continue; /* positive normal inputs only */
    const float r = rsqrt_rn(x);
    const float lo = nextafterf(r, 0.0f), hi = nextafterf(r, INFINITY);
    if (mid2x_vs_one(((double)lo + (double)r) * 0.5, x) > 0 || mid2x_vs_one(((double)r + (double)hi) * 0.5, x) < 0) bad++;
    if (r != orc_rsqrt_long_double(x)) differ++;
  }
  return bad ? UINT64_MAX : differ;
}

/* Sum of 128 squares. tree 0: the canonical order (see the file header).
 * tree 1: one 64-lane butterfly per half, then h0 + h1 (a wave64 device).
 * tree 2: plain left-to-right sum. Trees 1 and 2 exist only so the tests can
 * report how many cache bytes depend on this choice. */
static float sumsq128(const float* x, int tree) {
  float sq[128];
  for (int i = 0; i < 128; i++) sq[i] = x[i] * x[i];
  if (tree == 2) {
    float s = 0.0f;
    for (int i = 0; i < 128; i++) s = s + sq[i];
    return s;
  }
  int width = (tree == 1) ? 64 : 32;
  float tmp[128];
  for (int off = width / 2; off >= 1; off >>= 1) {
    for (int i = 0; i < 128; i++) tmp[i] = sq[i] + sq[i ^ off];
    memcpy(sq, tmp, sizeof sq);
  }
  if (tree == 1) return sq[0] + sq[64];
  return (sq[0] + sq[32]) + (sq[64] + sq[96]);
}

/* Steps 1-4 shared by kv_writeback_fused.wgsl:65-108 and
 * q_norm_rope_fused.wgsl:49-93: RMS-norm over the head, times the norm
 * weight, NEOX rotation with the (cos, sin) pair of j = dim mod 64. */
static void norm_rope_head(const uint16_t* x_f16, const uint16_t* w_f16, const uint16_t* rope_row,
                           float eps, int tree, int contract, float* post) {
  float raw[128], xn[128];
  for (int i = 0; i < 128; i++) raw[i] = orc_f16_to_f32(x_f16[i]);
  float total = sumsq128(raw, tree);
  float inv_h = rsqrt_rn(total / 128.0f + eps);
  for (int i = 0; i < 128; i++) xn[i] = (raw[i] * inv_h) * orc_f16_to_f32(w_f16[i]);
  for (int i = 0; i < 128; i++) {
    int j = i & 63;
    float c = orc_f16_to_f32(rope_row[2 * j]);
    float s = orc_f16_to_f32(rope_row[2 * j + 1]);
    if (i < 64) {
      post[i] = contract ? fmaf(xn[i], c, -(xn[i + 64] * s)) : xn[i] * c - xn[i + 64] * s;
    } else {
      post[i] = contract ? fmaf(xn[j], s, xn[i] * c) : xn[j] * s + xn[i] * c;
    }
  }
}

/* Block-32 absmax quantiser: kv_writeback_fused.wgsl:118-166 (the same
 * formula as quantize_q8_0.wgsl:67-70). */
static void quant_block32(const float* x, float* d_out, int8_t* q_out) {
  float amax = 0.0f;
  for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
  float d = amax / 127.0f;
  float inv = d > 0.0f ? 1.0f / d : 0.0f;
  for (int i = 0; i < 32; i++) {
    float r = rintf(x[i] * inv); /* ties to even in the default rounding mode */
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    q_out[i] = (int8_t)(int32_t)r;
  }
  *d_out = d;
}

/* kv_writeback_fused.wgsl:52-201, launched per (kv_head, token) by
 * dispatch_kv_writeback_fused (src/forward.rs:359-388). kv_k / kv_v are whole
 * cache buffers (d-section then qs-section). tree/contract: see sumsq128. */
void orc_kv_writeback(const uint16_t* k_cur, const uint16_t* v_cur, const uint16_t* w_k_norm,
                      const uint16_t* rope, uint8_t* kv_k, uint8_t* kv_v, uint32_t n_layer,
                      uint32_t max_seq, uint32_t n_kv_head, uint32_t layer, uint32_t pos_base,
                      uint32_t m, float eps, int tree, int contract) {
  const uint32_t kv_dim = n_kv_head * HEAD_DIM;
  const uint32_t nb = kv_dim / QK8_0;
  const uint64_t d_base = orc_buf_d_offset(max_seq, kv_dim, layer);
  const uint64_t qs_base = orc_buf_qs_offset(n_layer, max_seq, kv_dim, layer);
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t tok = 0; tok < m; tok++) {
    for (uint32_t head = 0; head < n_kv_head; head++) {
      const uint32_t pos_abs = pos_base + tok;
      const size_t src = (size_t)tok * kv_dim + (size_t)head * HEAD_DIM;
      float k_post[128], v_raw[128];
      norm_rope_head(k_cur + src, w_k_norm, rope + (size_t)pos_abs * HEAD_DIM, eps, tree, contract,
                     k_post);
      for (int i = 0; i < 128; i++) v_raw[i] = orc_f16_to_f32(v_cur[src + i]);
      for (uint32_t b = 0; b < 4; b++) {
        float dk, dv;
        int8_t qk[32], qv[32];
        quant_block32(k_post + 32 * b, &dk, qk);
        quant_block32(v_raw + 32 * b, &dv, qv);
        uint64_t d_off = d_base + ((uint64_t)pos_abs * nb + head * 4u + b) * 4u;
        uint64_t q_off = qs_base + (uint64_t)pos_abs * kv_dim + head * HEAD_DIM + 32u * b;
        memcpy(kv_k + d_off, &dk, 4);
        memcpy(kv_v + d_off, &dv, 4);
        memcpy(kv_k + q_off, qk, 32);
        memcpy(kv_v + q_off, qv, 32);
      }
    }
  }
}

/* Plain block-32 quantiser over raw f16 rows (the V path of the kernel above,
 * applied to any [m][kv_dim] f16 matrix). Used to fill "past" cache rows. */
void orc_quantize_rows(const uint16_t* x, uint8_t* kv, uint32_t n_layer, uint32_t max_seq,
                       uint32_t kv_dim, uint32_t layer, uint32_t pos_base, uint32_t m) {
  const uint32_t nb = kv_dim / QK8_0;
  const uint64_t d_base = orc_buf_d_offset(max_seq, kv_dim, layer);
  const uint64_t qs_base = orc_buf_qs_offset(n_layer, max_seq, kv_dim, layer);
#pragma omp parallel for schedule(static)
  for (uint32_t tok = 0; tok < m; tok++) {
    for (uint32_t b = 0; b < nb; b++) {
      float xs[32], d;
      int8_t q[32];
      for (int i = 0; i < 32; i++) xs[i] = orc_f16_to_f32(x[(size_t)tok * kv_dim + 32u * b + i]);
      quant_block32(xs, &d, q);
      uint64_t row = (uint64_t)(pos_base + tok);
      memcpy(kv + d_base + (row * nb + b) * 4u, &d, 4);
      memcpy(kv + qs_base + row * kv_dim + 32u * b, q, 32);
    }
  }
}

/* q_norm_rope_fused.wgsl:37-96, launched per (head, token) by
 * dispatch_q_norm_rope_fused (src/forward.rs:392-413). In place on q. */
void orc_q_norm_rope(uint16_t* q, const uint16_t* w_q_norm, const uint16_t* rope, uint32_t n_head,
                     uint32_t pos_base, uint32_t m, float eps, int tree, int contract) {
  const uint32_t q_dim = n_head * HEAD_DIM;
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t tok = 0; tok < m; tok++) {
    for (uint32_t head = 0; head < n_head; head++) {
      float post[128];
      uint16_t* row = q + (size_t)tok * q_dim + (size_t)head * HEAD_DIM;
      norm_rope_head(row, w_q_norm, rope + (size_t)(pos_base + tok) * HEAD_DIM, eps, tree, contract,
                     post);
      for (int i = 0; i < 128; i++) row[i] = orc_f32_to_f16(post[i]);
    }
  }
}

/* ------------------------------------------------------------ attention -- */

typedef struct {
  const float* d;   /* layer base of the d-section */
  const int8_t* qs; /* layer base of the qs-section */
  uint32_t kv_dim;
} kv_view;

static kv_view view_of(const uint8_t* kv, uint32_t n_layer, uint32_t max_seq, uint32_t kv_dim,
                       uint32_t layer) {
  kv_view v;
  v.d = (const float*)(kv + orc_buf_d_offset(max_seq, kv_dim, layer));
  v.qs = (const int8_t*)(kv + orc_buf_qs_offset(n_layer, max_seq, kv_dim, layer));
  v.kv_dim = kv_dim;
  return v;
}

/* load_k / load_v: attention_split.wgsl:87-109, attention.wgsl:95-117. */
static inline float kv_load(const kv_view* v, uint32_t t, uint32_t e) {
  size_t idx = (size_t)t * v->kv_dim + e;
  return v->d[idx >> 5] * (float)v->qs[idx];
}

/* Workgroup sum over `n` lanes (n = 64 here): xor butterfly inside aligned
 * groups of 32 lanes, then the group sums added left to right. This is one
 * admissible order of subgroupAdd + the cross-subgroup merge of wg_sum_v4
 * (attention_split.wgsl:63-78). */
static float wg_sum(float* v, int n) {
  float tmp[128];
  for (int off = 16; off >= 1; off >>= 1) {
    for (int i = 0; i < n; i++) tmp[i] = v[i] + v[i ^ off];
    memcpy(v, tmp, (size_t)n * sizeof(float));
  }
  float s = v[0];
  for (int g = 32; g < n; g += 32) s = s + v[g];
  return s;
}

/* attention_split.wgsl:111-199, launched per (kv head, 16-token chunk) by
 * layer_post_kv_in_pass (src/forward.rs:822-844). q: f16 [n_head][128];
 * partials: f32 [n_head][n_chunks][130], n_chunks = ceil(cur_pos / 16). */
void orc_attn_split(const uint16_t* q, const uint8_t* kv_k, const uint8_t* kv_v, float* partials,
                    uint32_t n_layer, uint32_t max_seq, uint32_t n_head, uint32_t n_kv_head,
                    uint32_t layer, uint32_t cur_pos) {
  const uint32_t kv_dim = n_kv_head * HEAD_DIM;
  const uint32_t qpg = n_head / n_kv_head;
  const uint32_t n_chunks = (cur_pos + ATTN_CHUNK - 1) / ATTN_CHUNK;
  const kv_view K = view_of(kv_k, n_layer, max_seq, kv_dim, layer);
  const kv_view V = view_of(kv_v, n_layer, max_seq, kv_dim, layer);
  const float scale = 1.0f / sqrtf((float)HEAD_DIM);
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t g = 0; g < n_kv_head; g++) {
    for (uint32_t chunk = 0; chunk < n_chunks; chunk++) {
      const uint32_t t0 = chunk * ATTN_CHUNK;
      const uint32_t t1 = (t0 + ATTN_CHUNK < cur_pos) ? t0 + ATTN_CHUNK : cur_pos;
      for (uint32_t hq = 0; hq < qpg; hq++) {
        const uint32_t h = g * qpg + hq;
        float qf[128], o[128];
        for (int i = 0; i < 128; i++) {
          qf[i] = orc_f16_to_f32(q[(size_t)h * HEAD_DIM + i]);
          o[i] = 0.0f;
        }
        float mrun = -1e30f, lrun = 0.0f;
        for (uint32_t t = t0; t < t1; t++) {
          float lane[64];
          for (int tid = 0; tid < 64; tid++) {
            float acc = 0.0f;
            for (int d = tid; d < 128; d += 64) acc = acc + kv_load(&K, t, g * HEAD_DIM + d) * qf[d];
            lane[tid] = acc;
          }
          float s = wg_sum(lane, 64) * scale;
          float m_new = fmaxf(mrun, s);
          float corr = expf(mrun - m_new);
          float w = expf(s - m_new);
          lrun = lrun * corr + w;
          mrun = m_new;
          for (int d = 0; d < 128; d++) o[d] = o[d] * corr + w * kv_load(&V, t, g * HEAD_DIM + d);
        }
        float* dst = partials + ((size_t)h * n_chunks + chunk) * PARTIAL_STRIDE;
        memcpy(dst, o, 128 * sizeof(float));
        dst[128] = mrun;
        dst[129] = lrun;
      }
    }
  }
}

/* attention_merge.wgsl:70-130, launched per Q head (src/forward.rs:846-856).
 * out: f16 [n_head][128]. */
void orc_attn_merge(const float* partials, uint16_t* out, uint32_t n_head, uint32_t n_chunks) {
#pragma omp parallel for schedule(static)
  for (uint32_t h = 0; h < n_head; h++) {
    const float* base = partials + (size_t)h * n_chunks * PARTIAL_STRIDE;
    float m_global = -1e30f;
    for (uint32_t c = 0; c < n_chunks; c++) m_global = fmaxf(m_global, base[c * PARTIAL_STRIDE + 128]);
    /* Phase B: lane tid sums its strided chunks, then a 128-lane workgroup sum. */
    float lane[128];
    for (uint32_t tid = 0; tid < 128; tid++) {
      float acc = 0.0f;
      for (uint32_t c = tid; c < n_chunks; c += 128) {
        float w = expf(base[c * PARTIAL_STRIDE + 128] - m_global);
        acc = acc + base[c * PARTIAL_STRIDE + 129] * w;
      }
      lane[tid] = acc;
    }
    float l_global = wg_sum(lane, 128);
    float inv_l = 1.0f / l_global;
    for (uint32_t d = 0; d < 128; d++) {
      float o = 0.0f;
      for (uint32_t c = 0; c < n_chunks; c++) {
        float w = expf(base[c * PARTIAL_STRIDE + 128] - m_global);
        o = o + base[c * PARTIAL_STRIDE + d] * w;
      }
      out[(size_t)h * HEAD_DIM + d] = orc_f32_to_f16(o * inv_l);
    }
  }
}

/* Decode attention = split + merge with the reference's 16-token chunks. */
void orc_attn_decode(const uint16_t* q, const uint8_t* kv_k, const uint8_t* kv_v, uint16_t* out,
                     uint32_t n_layer, uint32_t max_seq, uint32_t n_head, uint32_t n_kv_head,
                     uint32_t layer, uint32_t cur_pos) {
  const uint32_t n_chunks = (cur_pos + ATTN_CHUNK - 1) / ATTN_CHUNK;
  float* partials = (float*)malloc((size_t)n_head * n_chunks * PARTIAL_STRIDE * sizeof(float));
  orc_attn_split(q, kv_k, kv_v, partials, n_layer, max_seq, n_head, n_kv_head, layer, cur_pos);
  orc_attn_merge(partials, out, n_head, n_chunks);
  free(partials);
}

/* attention.wgsl:119-214 with is_prefill = 1 (dispatch_attention,
 * src/forward.rs:501-532): token m_tok of head h attends to keys [0, m_tok].
 * q, out: f16 [m][n_head][128]. The 4-way unrolled dot and the sequential
 * online-softmax update follow attention.wgsl:148-205. */
void orc_attn_prefill(const uint16_t* q, const uint8_t* kv_k, const uint8_t* kv_v, uint16_t* out,
                      uint32_t n_layer, uint32_t max_seq, uint32_t n_head, uint32_t n_kv_head,
                      uint32_t layer, uint32_t m) {
  const uint32_t kv_dim = n_kv_head * HEAD_DIM;
  const uint32_t q_dim = n_head * HEAD_DIM;
  const uint32_t qpg = n_head / n_kv_head;
  const kv_view K = view_of(kv_k, n_layer, max_seq, kv_dim, layer);
  const kv_view V = view_of(kv_v, n_layer, max_seq, kv_dim, layer);
  const float scale = 1.0f / sqrtf((float)HEAD_DIM);
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
  for (uint32_t m_tok = 0; m_tok < m; m_tok++) {
    for (uint32_t h = 0; h < n_head; h++) {
      const uint32_t g = h / qpg;
      const uint32_t cur_pos = m_tok + 1;
      float qf[128], o[128];
      for (int i = 0; i < 128; i++) {
        qf[i] = orc_f16_to_f32(q[(size_t)m_tok * q_dim + (size_t)h * HEAD_DIM + i]);
        o[i] = 0.0f;
      }
      float mrun = -1e30f, lrun = 0.0f;
      for (uint32_t t = 0; t < cur_pos; t++) {
        float lane[64];
        for (int tid = 0; tid < 64; tid++) {
          float acc = 0.0f;
          for (int d = tid; d < 128; d += 64) acc = acc + qf[d] * kv_load(&K, t, g * HEAD_DIM + d);
          lane[tid] = acc;
        }
        float s = wg_sum(lane, 64) * scale;
        float m_new = fmaxf(mrun, s);
        float corr = expf(mrun - m_new);
        float w = expf(s - m_new);
        lrun = lrun * corr + w;
        mrun = m_new;
        for (int d = 0; d < 128; d++) o[d] = o[d] * corr + w * kv_load(&V, t, g * HEAD_DIM + d);
      }
      float inv_l = 1.0f / lrun;
      for (int d = 0; d < 128; d++)
        out[(size_t)m_tok * q_dim + (size_t)h * HEAD_DIM + d] = orc_f32_to_f16(o[d] * inv_l);
    }
  }
}

/* Ground truth for the tolerance test: a two-pass softmax over the
 * dequantised cache (scale * int8, as load_k/load_v compute it) and the f16
 * query, accumulated in binary64 and returned unrounded as f32. `causal` = 1:
 * row i of q ([m][n_head][128]) attends to keys [0, key_base + i]; with m = 1
 * and key_base = cur_pos - 1 this is the decode case. */
void orc_attn_exact(const uint16_t* q, const uint8_t* kv_k, const uint8_t* kv_v, float* out,
                    uint32_t n_layer, uint32_t max_seq, uint32_t n_head, uint32_t n_kv_head,
                    uint32_t layer, uint32_t m, uint32_t key_base) {
  const uint32_t kv_dim = n_kv_head * HEAD_DIM;
  const uint32_t q_dim = n_head * HEAD_DIM;
  const uint32_t qpg = n_head / n_kv_head;
  const kv_view K = view_of(kv_k, n_layer, max_seq, kv_dim, layer);
  const kv_view V = view_of(kv_v, n_layer, max_seq, kv_dim, layer);
  const double scale = 1.0 / sqrt((double)HEAD_DIM);
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
  for (uint32_t i = 0; i < m; i++) {
    for (uint32_t h = 0; h < n_head; h++) {
      const uint32_t g = h / qpg;
      const uint32_t n_keys = key_base + i + 1;
      double* s = (double*)malloc((size_t)n_keys * sizeof(double));
      double qd[128], acc[128];
      for (int d = 0; d < 128; d++) {
        qd[d] = (double)orc_f16_to_f32(q[(size_t)i * q_dim + (size_t)h * HEAD_DIM + d]);
        acc[d] = 0.0;
      }
      double smax = -INFINITY;
      for (uint32_t t = 0; t < n_keys; t++) {
        double dot = 0.0;
        for (int d = 0; d < 128; d++) dot += qd[d] * (double)kv_load(&K, t, g * HEAD_DIM + d);
        s[t] = dot * scale;
        if (s[t] > smax) smax = s[t];
      }
      double l = 0.0;
      for (uint32_t t = 0; t < n_keys; t++) {
        double w = exp(s[t] - smax);
        l += w;
        for (int d = 0; d < 128; d++) acc[d] += w * (double)kv_load(&V, t, g * HEAD_DIM + d);
      }
      for (int d = 0; d < 128; d++)
        out[(size_t)i * q_dim + (size_t)h * HEAD_DIM + d] = (float)(acc[d] / l);
      free(s);
    }
  }
}

/* Number of OpenMP threads the parallel loops above use from now on (n >= 1). A
 * launcher may export OMP_NUM_THREADS=1 for its children; the timed CPU baseline
 * sets the count it wants explicitly. No-op in a build without OpenMP. */
void orc_set_threads(int n) {
#ifdef _OPENMP
  extern void omp_set_num_threads(int);
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_num_threads(void) {
#ifdef _OPENMP
  extern int omp_get_max_threads(void);
  return omp_get_max_threads();
#else
  return 1;
#endif
}
