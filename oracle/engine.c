/*
 * engine.c - CPU restatement of the reference's NON-attention operators, the rest of
 * one decode / prefill layer around the attention path restated in oracle.c.
 *
 * TEST INFRASTRUCTURE ONLY, like oracle.c: the thing the CUDA kernels of
 * bonsai_pot_b200/csrc/bp_q1_ops.cu are compared against and the CPU arm of the
 * end-to-end comparison; no product code path may call, link or load it.
 *
 * PARITY UNPINNED for numerics (the reference cannot be built or run here and holds
 * no golden vectors for these operators). What the shaders leave to the driver is
 * FIXED here, in the spirit of the rules in oracle.c's header:
 *   - f16 arithmetic (`vec4<f16>` adds and multiplies) rounds to nearest even after
 *     every operation (computed in binary32 and rounded to binary16: innocuous
 *     double rounding, 24 >= 2 * 11 + 2);
 *   - binary32 operations round separately, left to right as written (no FMA
 *     contraction); `inverseSqrt` and `/` are correctly rounded; `round()` is ties to even;
 *   - `subgroupAdd` over a subgroup of 32 is the xor butterfly 16, 8, 4, 2, 1; the
 *     cross-subgroup merge puts the partial of subgroup s in lane s of subgroup 0,
 *     zero elsewhere, and runs the same butterfly;
 *   - `exp(x)` in silu is orc_exp_det below (Cody-Waite reduction, degree-6 Horner
 *     polynomial in fused multiply-adds, under 3 ulp): an algorithm both sides can
 *     run bit for bit, since neither WGSL nor libm fixes one.
 * Each function cites the shader lines it follows (paths inside the reference).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

float orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);

/* a value rounded to binary16 and held as binary32 */
static inline float hr(float x) { return orc_f16_to_f32(orc_f32_to_f16(x)); }
static inline float hadd(float a, float b) { return hr(a + b); }
static inline float hmul(float a, float b) { return hr(a * b); }

static inline float load_f16(const uint8_t* p) {
  uint16_t h;
  memcpy(&h, p, 2);
  return orc_f16_to_f32(h);
}

/* 1/sqrt(x), correctly rounded (the exact routine lives in oracle.c) */
float orc_rsqrt_rn(float x);

/* exp(x) as both sides evaluate it. n = rint(x * log2(e)); r = x - n * ln2 (two-step, fused);
 * p(r) = sum r^k / k!, k <= 6, Horner in fused multiply-adds; result = p * 2^n. x is clamped to
 * [-87.3, 88.7]: the result stays finite and normal. */
float orc_exp_det(float x) {
  x = fminf(fmaxf(x, -87.3f), 88.7f);
  const float n = rintf(x * 1.44269504088896341f);
  float r = fmaf(n, -0.693359375f, x);
  r = fmaf(n, 2.12194440e-4f, r);
  float p = fmaf(r, 1.0f / 720.0f, 1.0f / 120.0f);
  p = fmaf(r, p, 1.0f / 24.0f);
  p = fmaf(r, p, 1.0f / 6.0f);
  p = fmaf(r, p, 0.5f);
  p = fmaf(r, p, 1.0f);
  p = fmaf(r, p, 1.0f);
  return ldexpf(p, (int)n);
}

/* silu(g) * up as silu_mul.wgsl:22-26 and matvec_q1_0_silu.wgsl:77-95 compute it:
 * g / (1 + exp(-g)) in binary32, cast to f16, times up in f16. */
static inline float silu_times_up(uint16_t gate, uint16_t up) {
  const float g = orc_f16_to_f32(gate);
  const float s = g / (1.0f + orc_exp_det(-g));
  return hmul(hr(s), orc_f16_to_f32(up));
}

/* subgroupAdd over `n_sub` subgroups of 32 lanes, then the cross-subgroup merge
 * (rms_norm.wgsl:62-78, matvec_q1_0_fused_normed.wgsl:131-146). lanes[] has 32 * n_sub values. */
static float workgroup_sum(float* lanes, int n_sub) {
  float part[32];
  for (int i = 0; i < 32; i++) part[i] = 0.0f;
  for (int s = 0; s < n_sub; s++) {
    float v[32], t[32];
    memcpy(v, lanes + 32 * s, sizeof v);
    for (int off = 16; off >= 1; off >>= 1) {
      for (int i = 0; i < 32; i++) t[i] = v[i] + v[i ^ off];
      memcpy(v, t, sizeof v);
    }
    part[s] = v[0];
  }
  if (n_sub == 1) return part[0];
  float t[32];
  for (int off = 16; off >= 1; off >>= 1) {
    for (int i = 0; i < 32; i++) t[i] = part[i] + part[i ^ off];
    memcpy(part, t, sizeof part);
  }
  return part[0];
}

/* One 128-weight block of a Q1_0 row against 128 activations held as f16 values:
 * matvec_q1_0.wgsl:92-112. Four f16 accumulators (element 4 g + c goes to component c, groups
 * g = 0..31 in order), then ((a0 + a1) + a2) + a3 in f16, widened to binary32. */
static float block_sum(const uint8_t* qs16, const float* x128) {
  float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int g = 0; g < 32; g++) {
    const uint32_t bits = (qs16[g >> 1] >> ((g & 1) * 4)) & 0xFu;
    for (int c = 0; c < 4; c++) {
      const float xv = x128[4 * g + c];
      a[c] = hadd(a[c], (bits >> c) & 1u ? xv : -xv);
    }
  }
  return hadd(hadd(hadd(a[0], a[1]), a[2]), a[3]);
}

/* The eight "tx" lanes of a row and their butterfly (matvec_q1_0.wgsl:84-133): lane tx takes the
 * blocks b = tx (mod 8) in increasing order, acc = acc + d_eff * lane_sum in binary32; then
 * acc += shuffleXor(acc, 1), 2, 4. d_scale multiplies every block scale (1 or inv_rms). */
static float row_dot(const uint8_t* d_row, const uint8_t* qs_row, uint32_t nb, const float* x, float d_scale,
                     int scale_d) {
  float acc[8], t[8];
  for (int tx = 0; tx < 8; tx++) {
    float a = 0.0f;
    for (uint32_t b = (uint32_t)tx; b < nb; b += 8) {
      float d = load_f16(d_row + 2u * b);
      if (scale_d) d = d * d_scale;
      const float lane_sum = block_sum(qs_row + 16u * b, x + 128u * b);
      const float prod = d * lane_sum;
      a = a + prod;
    }
    acc[tx] = a;
  }
  for (int off = 1; off <= 4; off <<= 1) {
    for (int i = 0; i < 8; i++) t[i] = acc[i] + acc[i ^ off];
    memcpy(acc, t, sizeof acc);
  }
  return acc[0];
}

static void store_row(uint16_t* y, float acc, int accumulate) {
  *y = accumulate ? orc_f32_to_f16(orc_f16_to_f32(*y) + acc) : orc_f32_to_f16(acc);
}

/* embed.wgsl:37-52: row `token` of a Q1_0 matrix as f16 (+d or -d per sign bit). */
void orc_embed(const uint8_t* w, uint64_t d_off, uint64_t qs_off, uint32_t k, const uint32_t* tokens, uint32_t m,
               uint16_t* x_out) {
  const uint32_t nb = k / 128u;
  for (uint32_t t = 0; t < m; t++) {
    const uint64_t row = tokens[t];
    for (uint32_t b = 0; b < nb; b++) {
      uint16_t dh;
      memcpy(&dh, w + d_off + (row * nb + b) * 2u, 2);
      const uint16_t pos = orc_f32_to_f16(orc_f16_to_f32(dh)), neg = orc_f32_to_f16(-orc_f16_to_f32(dh));
      const uint8_t* qs = w + qs_off + (row * nb + b) * 16u;
      for (uint32_t e = 0; e < 128; e++)
        x_out[(size_t)t * k + 128u * b + e] = (qs[e >> 3] >> (e & 7)) & 1u ? pos : neg;
    }
  }
}

/* rms_norm.wgsl:41-85: 512 invocations per group; invocation tid sums v * v over i = tid, tid + 512, ...;
 * workgroup sum; inv_h = f16(inverseSqrt(total / n + eps)); out = (x * inv_h) * w in f16. In place is allowed. */
void orc_rms_norm(const uint16_t* in, uint16_t* out, const uint16_t* w, uint32_t group_size, uint32_t n_groups,
                  float eps) {
#pragma omp parallel for schedule(static)
  for (uint32_t gi = 0; gi < n_groups; gi++) {
    float lanes[512];
    for (uint32_t tid = 0; tid < 512; tid++) {
      float s = 0.0f;
      for (uint32_t i = tid; i < group_size; i += 512) {
        const float v = orc_f16_to_f32(in[(size_t)gi * group_size + i]);
        const float sq = v * v;
        s = s + sq;
      }
      lanes[tid] = s;
    }
    const float total = workgroup_sum(lanes, 16);
    const float inv_h = hr(orc_rsqrt_rn(total / (float)group_size + eps));
    for (uint32_t i = 0; i < group_size; i++) {
      const float x = orc_f16_to_f32(in[(size_t)gi * group_size + i]);
      out[(size_t)gi * group_size + i] = orc_f32_to_f16(hmul(hmul(x, inv_h), orc_f16_to_f32(w[i])));
    }
  }
}

/* matvec_q1_0.wgsl:53-133 (dispatch_matvec_q1_0, src/forward.rs:188-240): y[n] (+)= W[n][k] x[k]. */
void orc_matvec_q1_0(const uint8_t* w, uint64_t d_off, uint64_t qs_off, uint32_t k, uint32_t n, const uint16_t* x,
                     uint16_t* y, int accumulate) {
  const uint32_t nb = k / 128u;
  float* xf = (float*)malloc((size_t)k * sizeof(float));
  for (uint32_t i = 0; i < k; i++) xf[i] = orc_f16_to_f32(x[i]);
#pragma omp parallel for schedule(static)
  for (uint32_t row = 0; row < n; row++) {
    const float acc = row_dot(w + d_off + (uint64_t)row * nb * 2u, w + qs_off + (uint64_t)row * nb * 16u, nb, xf, 1.0f, 0);
    store_row(y + row, acc, accumulate);
  }
  free(xf);
}

/* matvec_q1_0_fused_normed.wgsl:80-207 (src/forward.rs:776-790, 871-885): up to three Q1_0 tensors
 * over the same rms-normed input. 128 invocations: invocation tid sums the squares of the vec4s
 * v = tid, tid + 128, ... as ((((ssq + xx) + yy) + zz) + ww); the staged input is x * w_norm in f16;
 * every block scale is d * inv_rms. */
void orc_matvec_q1_0_fused_normed(const uint8_t* w, uint32_t k, const uint16_t* x, const uint16_t* w_norm, float eps,
                                  uint32_t n_ranges, const uint64_t* d_off, const uint64_t* qs_off,
                                  const uint32_t* n, uint16_t* const* out) {
  const uint32_t nb = k / 128u, k_v4 = k / 4u;
  float lanes[128];
  for (uint32_t tid = 0; tid < 128; tid++) {
    float ssq = 0.0f;
    for (uint32_t v = tid; v < k_v4; v += 128)
      for (int c = 0; c < 4; c++) {
        const float xv = orc_f16_to_f32(x[4u * v + (uint32_t)c]);
        const float sq = xv * xv;
        ssq = ssq + sq;
      }
    lanes[tid] = ssq;
  }
  const float total = workgroup_sum(lanes, 4);
  const float inv_rms = orc_rsqrt_rn(total / (float)k + eps);
  float* xs = (float*)malloc((size_t)k * sizeof(float));
  for (uint32_t i = 0; i < k; i++) xs[i] = hmul(orc_f16_to_f32(x[i]), orc_f16_to_f32(w_norm[i]));
  for (uint32_t r = 0; r < n_ranges; r++) {
#pragma omp parallel for schedule(static)
    for (uint32_t row = 0; row < n[r]; row++) {
      const float acc = row_dot(w + d_off[r] + (uint64_t)row * nb * 2u, w + qs_off[r] + (uint64_t)row * nb * 16u, nb,
                                xs, inv_rms, 1);
      out[r][row] = orc_f32_to_f16(acc);
    }
  }
  free(xs);
}

/* matvec_q1_0_silu.wgsl:53-138 (src/forward.rs:891-906): y (+)= W (silu(gate) * up). */
void orc_matvec_q1_0_silu(const uint8_t* w, uint64_t d_off, uint64_t qs_off, uint32_t k, uint32_t n,
                          const uint16_t* gate, const uint16_t* up, uint16_t* y, int accumulate) {
  const uint32_t nb = k / 128u;
  float* xs = (float*)malloc((size_t)k * sizeof(float));
#pragma omp parallel for schedule(static)
  for (uint32_t i = 0; i < k; i++) xs[i] = silu_times_up(gate[i], up[i]);
#pragma omp parallel for schedule(static)
  for (uint32_t row = 0; row < n; row++) {
    const float acc = row_dot(w + d_off + (uint64_t)row * nb * 2u, w + qs_off + (uint64_t)row * nb * 16u, nb, xs, 1.0f, 0);
    store_row(y + row, acc, accumulate);
  }
  free(xs);
}

/* silu_mul.wgsl:18-27 */
void orc_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, uint64_t n) {
#pragma omp parallel for schedule(static)
  for (uint64_t i = 0; i < n; i++) out[i] = orc_f32_to_f16(silu_times_up(gate[i], up[i]));
}

/* quantize_q8_0.wgsl:49-106: per 32 values d = amax / 127 (binary32), q = clamp(round(v * (1 / d))). */
void orc_quantize_q8_0(const uint16_t* x, uint32_t k, uint32_t m, float* d_out, int8_t* qs_out) {
  const uint32_t nbq = k / 32u;
#pragma omp parallel for schedule(static)
  for (uint64_t blk = 0; blk < (uint64_t)m * nbq; blk++) {
    float v[32], amax = 0.0f;
    for (int i = 0; i < 32; i++) {
      v[i] = orc_f16_to_f32(x[blk * 32u + (uint32_t)i]);
      amax = fmaxf(amax, fabsf(v[i]));
    }
    const float d = amax / 127.0f;
    const float id = d > 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < 32; i++) {
      float r = rintf(v[i] * id);
      r = fminf(fmaxf(r, -127.0f), 127.0f);
      qs_out[blk * 32u + (uint32_t)i] = (int8_t)(int32_t)r;
    }
    d_out[blk] = d;
  }
}

/* matmul_q1_0_q8_0.wgsl:57-293 (src/forward.rs:415-499): y[m][n] (+)= sum over the Q1_0 blocks b and their
 * four Q8_0 sub-blocks s, in that order, of (a_d[m][4 b + s] * w_d[n][b]) * f32(sumi), sumi the exact
 * integer dot of 32 signs (+1 / -1) with 32 int8 activations. */
void orc_matmul_q1_0_q8_0(const uint8_t* w, uint64_t d_off, uint64_t qs_off, uint32_t k, uint32_t n, uint32_t m,
                          const float* a_d, const int8_t* a_qs, uint16_t* y, int accumulate) {
  const uint32_t nb1 = k / 128u, nb8 = k / 32u;
#pragma omp parallel for collapse(2) schedule(static)
  for (uint32_t mi = 0; mi < m; mi++) {
    for (uint32_t ni = 0; ni < n; ni++) {
      float acc = 0.0f;
      for (uint32_t b = 0; b < nb1; b++) {
        const float wd = load_f16(w + d_off + ((uint64_t)ni * nb1 + b) * 2u);
        const uint8_t* qs = w + qs_off + ((uint64_t)ni * nb1 + b) * 16u;
        for (uint32_t s = 0; s < 4; s++) {
          const int8_t* a = a_qs + (uint64_t)mi * k + 128u * b + 32u * s;
          int32_t sumi = 0;
          for (uint32_t e = 0; e < 32; e++) {
            const uint32_t bit = (qs[4u * s + (e >> 3)] >> (e & 7)) & 1u;
            sumi += bit ? (int32_t)a[e] : -(int32_t)a[e];
          }
          const float scale = a_d[(uint64_t)mi * nb8 + 4u * b + s] * wd;
          const float v = scale * (float)sumi;
          acc = acc + v;
        }
      }
      store_row(y + (uint64_t)mi * n + ni, acc, accumulate);
    }
  }
}

/* topk_reduce.wgsl:59-196, restated step by step (ties fall where the shader's comparisons put them):
 * 256 invocations keep a 32-entry min-heap each over the logits words w = tid, tid + 256, ...; heapsort to
 * descending; then log2(256) rounds that merge list j + s into list j by a bitonic "keep the larger half"
 * step and a bitonic sort. vals / idx receive min(k, 32) entries, descending. */
#define TK_WG 256u
#define TK_K 32u
static void tk_sift(float* val, uint32_t* idx, uint32_t limit) {
  uint32_t i = 0;
  for (;;) {
    const uint32_t l = 2u * i + 1u, r = l + 1u;
    uint32_t smallest = i;
    if (l < limit && val[l] < val[smallest]) smallest = l;
    if (r < limit && val[r] < val[smallest]) smallest = r;
    if (smallest == i) break;
    const float tv = val[i]; val[i] = val[smallest]; val[smallest] = tv;
    const uint32_t ti = idx[i]; idx[i] = idx[smallest]; idx[smallest] = ti;
    i = smallest;
  }
}

void orc_topk_reduce(const uint16_t* logits, uint32_t n, uint32_t k, float* vals, uint32_t* idx_out) {
  float* sv = (float*)malloc(TK_WG * TK_K * sizeof(float));
  uint32_t* si = (uint32_t*)malloc(TK_WG * TK_K * sizeof(uint32_t));
  const uint32_t n_words = (n + 1u) >> 1;
  for (uint32_t tid = 0; tid < TK_WG; tid++) {
    float* val = sv + tid * TK_K;
    uint32_t* idx = si + tid * TK_K;
    for (uint32_t i = 0; i < TK_K; i++) { val[i] = -1e30f; idx[i] = 0; }
    for (uint32_t w = tid; w < n_words; w += TK_WG) {
      for (uint32_t h = 0; h < 2; h++) {
        const uint32_t i = 2u * w + h;
        if (i >= n) break;
        const float v = orc_f16_to_f32(logits[i]);
        if (v > val[0]) { val[0] = v; idx[0] = i; tk_sift(val, idx, TK_K); }
      }
    }
    for (uint32_t active = TK_K - 1u; active > 0; active--) {
      const float tv = val[0]; val[0] = val[active]; val[active] = tv;
      const uint32_t ti = idx[0]; idx[0] = idx[active]; idx[active] = ti;
      tk_sift(val, idx, active);
    }
  }
  for (uint32_t s = TK_WG / 2u; s > 0; s /= 2u) {
    for (uint32_t kk = 0; kk < s * TK_K; kk++) { /* keep the larger of a[i] and b[31 - i] */
      const uint32_t pair = kk / TK_K, i = kk % TK_K;
      float* a = sv + pair * TK_K; uint32_t* ai = si + pair * TK_K;
      const float* b = sv + (pair + s) * TK_K; const uint32_t* bi = si + (pair + s) * TK_K;
      if (b[TK_K - 1u - i] > a[i]) { a[i] = b[TK_K - 1u - i]; ai[i] = bi[TK_K - 1u - i]; }
    }
    for (uint32_t stride = TK_K / 2u; stride > 0; stride /= 2u) {
      for (uint32_t kk = 0; kk < s * (TK_K / 2u); kk++) {
        const uint32_t pair = kk / (TK_K / 2u), local = kk % (TK_K / 2u);
        const uint32_t lo = ((local & ~(stride - 1u)) << 1) | (local & (stride - 1u)), hi = lo | stride;
        float* a = sv + pair * TK_K; uint32_t* ai = si + pair * TK_K;
        if (a[hi] > a[lo]) {
          const float tv = a[lo]; a[lo] = a[hi]; a[hi] = tv;
          const uint32_t ti = ai[lo]; ai[lo] = ai[hi]; ai[hi] = ti;
        }
      }
    }
  }
  const uint32_t kk = k < TK_K ? k : TK_K;
  for (uint32_t i = 0; i < kk; i++) { vals[i] = sv[i]; idx_out[i] = si[i]; }
  free(sv);
  free(si);
}
