/*
 * hy3_oracle.c -- CPU restatement of the Hy3 attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels: it is
 * linked by the tests, by the smoke check and by the CPU-baseline leg of the
 * benchmark, never by the product library.  Every function restates, in plain
 * C99 without -ffast-math, a piece of the reference engine (yuhai-china/hy3) and
 * cites the reference file:line it follows.  Parity of this restatement with the
 * reference itself is pinned two ways: (1) live, against the reference's own
 * sources compiled into oracle/_ref/ (tests/test_oracle_vs_ref.py), and (2) by the
 * committed fixtures under tests/golden/, which were produced by that compiled
 * reference (tests/golden/make_golden.py).
 *
 * Layout convention used here ("layer view"): K and V of one layer are dense
 * [ntok][n_kv_heads][128] fp32 arrays.  The reference interleaves all 80 layers
 * in one slot array (slot = token*80 + layer, hy3.c:631); the index arithmetic is
 * the only difference.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define HY3O_HEAD_DIM 128

/* ---------------------------------------------------------------- fp16 <-> fp32 */

/* IEEE binary16 -> binary32 (what __half2float does, hy3_gpu.cu:206). */
float hy3o_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round-to-nearest-even (what __float2half does,
 * hy3_gpu.cu:262). */
uint16_t hy3o_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or == 2^-25 exactly -> ties to even 0) */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q)); /* carry into the exponent is correct */
}

/* ---------------------------------------------------------------- RoPE table */

/* hy3.c:484-502 (yarn_correction_dim / yarn_correction_range) and hy3.c:538-556
 * (table loop).  Arguments are the values hy3_rope_init resolves from GGUF
 * metadata and the HY3_ROPE_* environment (hy3.c:506-536); the caller passes them
 * explicitly.  attn_factor_override < 0 means "not set".                        */
void hy3o_rope_table(double base, int yarn, double factor, double orig_ctx,
                     double beta_fast, double beta_slow, double attn_factor_override,
                     float *inv_freq /*[64]*/, float *attn_factor_out) {
    const int half = HY3O_HEAD_DIM / 2;
    double attn_factor = 1.0;
    if (yarn && factor > 1.0) attn_factor = 0.1 * log(factor) + 1.0; /* hy3.c:533 */
    if (attn_factor_override >= 0.0) attn_factor = attn_factor_override; /* :534 */
    if (!(yarn && factor > 1.0)) { yarn = 0; attn_factor = 1.0; factor = 1.0; } /* :535 */

    double lo = 0, hi = 0;
    if (yarn) { /* hy3.c:488-502 */
        double dlo = ((double)HY3O_HEAD_DIM * log(orig_ctx / (beta_fast * 2.0 * M_PI))) / (2.0 * log(base));
        double dhi = ((double)HY3O_HEAD_DIM * log(orig_ctx / (beta_slow * 2.0 * M_PI))) / (2.0 * log(base));
        lo = floor(dlo);
        hi = ceil(dhi);
        if (lo < 0) lo = 0;
        if (hi > HY3O_HEAD_DIM - 1) hi = HY3O_HEAD_DIM - 1;
    }
    double denom = hi - lo;
    if (denom < 1e-3) denom = 1e-3;
    for (int i = 0; i < half; i++) {
        double pos_freq = pow(base, (double)(2 * i) / (double)HY3O_HEAD_DIM);
        double inv_extrap = 1.0 / pos_freq;
        double invf = inv_extrap;
        if (yarn) {
            double inv_interp = 1.0 / (factor * pos_freq);
            double ramp = ((double)i - lo) / denom;
            if (ramp < 0) ramp = 0;
            if (ramp > 1) ramp = 1;
            double extrap_w = 1.0 - ramp;
            invf = inv_interp * (1.0 - extrap_w) + inv_extrap * extrap_w;
        }
        inv_freq[i] = (float)invf;
    }
    *attn_factor_out = (float)attn_factor;
}

/* ---------------------------------------------------------------- norm + rope */

/* hy3.c:435-444. */
void hy3o_rms_norm(float *out, const float *x, const float *w, int n, float eps) {
    float ss = 0.0f;
    for (int i = 0; i < n; i++) ss += x[i] * x[i];
    float r = 1.0f / sqrtf(ss / (float)n + eps);
    for (int i = 0; i < n; i++) out[i] = x[i] * r * w[i];
}

/* hy3.c:585-615, for one tensor of n_heads heads (the reference runs the same loop
 * over q and then k).  pos is the token index; the jump/stride probes are applied
 * as at hy3.c:588-589.                                                            */
void hy3o_rope(float *x, int n_heads, int pos, const float *inv_freq, float af,
               int pos_stride, int pos_jump, int pos_jump_at) {
    if (pos >= pos_jump_at) pos += pos_jump;
    pos *= pos_stride;
    const int half = HY3O_HEAD_DIM / 2;
    for (int h = 0; h < n_heads; h++) {
        float *xh = x + (size_t)h * HY3O_HEAD_DIM;
        for (int d = 0; d < half; d++) {
            float freq = (float)pos * inv_freq[d];
            float c = cosf(freq) * af;
            float s = sinf(freq) * af;
            float x0 = xh[d], x1 = xh[d + half];
            xh[d] = x0 * c - x1 * s;
            xh[d + half] = x1 * c + x0 * s;
        }
    }
}

/* ---------------------------------------------------------------- quantisers */

/* hy3_gpu.cu:250-270 for one head of 128 values: absmax, s = absmax/127 + 1e-8,
 * inv = 1/s (all IEEE fp32), code = (int8)roundf(clamp(x*inv)), stored scale =
 * fp16(s).  The codes are computed with the fp32 scale, the stored scale is the
 * fp16 rounding of it (the asymmetry is the reference's and is kept).            */
void hy3o_quant_int8(const float *x, uint16_t *scale_h, int8_t *codes) {
    float m = 0.0f;
    for (int i = 0; i < HY3O_HEAD_DIM; i++) m = fmaxf(m, fabsf(x[i]));
    volatile float s = m / 127.0f + 1e-8f;
    volatile float inv = 1.0f / s;
    *scale_h = hy3o_float_to_half(s);
    for (int i = 0; i < HY3O_HEAD_DIM; i++) {
        volatile float f = x[i] * inv;
        codes[i] = (int8_t)roundf(fmaxf(-127.0f, fminf(127.0f, f)));
    }
}

/* hy3_gpu.cu:329-352: same with /7, clamp +-7, two codes per byte, even dim in the
 * low nibble.                                                                     */
void hy3o_quant_int4(const float *x, uint16_t *scale_h, uint8_t *packed /*[64]*/) {
    float m = 0.0f;
    for (int i = 0; i < HY3O_HEAD_DIM; i++) m = fmaxf(m, fabsf(x[i]));
    volatile float s = m / 7.0f + 1e-8f;
    volatile float inv = 1.0f / s;
    *scale_h = hy3o_float_to_half(s);
    for (int b = 0; b < HY3O_HEAD_DIM / 2; b++) {
        volatile float f0 = x[2 * b] * inv, f1 = x[2 * b + 1] * inv;
        int q0 = (int)roundf(fmaxf(-7.0f, fminf(7.0f, f0))) & 0xF;
        int q1 = (int)roundf(fmaxf(-7.0f, fminf(7.0f, f1))) & 0xF;
        packed[b] = (uint8_t)(q0 | (q1 << 4));
    }
}

/* hy3_gpu.cu:206-215: value = (float)code * half2float(scale). */
void hy3o_dequant_int8(const int8_t *codes, uint16_t scale_h, float *out) {
    float s = hy3o_half_to_float(scale_h);
    for (int i = 0; i < HY3O_HEAD_DIM; i++) out[i] = (float)codes[i] * s;
}

/* hy3_gpu.cu:300-310: nibble n>7 -> n-16. */
void hy3o_dequant_int4(const uint8_t *packed, uint16_t scale_h, float *out) {
    float s = hy3o_half_to_float(scale_h);
    for (int b = 0; b < HY3O_HEAD_DIM / 2; b++) {
        int n0 = packed[b] & 0xF, n1 = (packed[b] >> 4) & 0xF;
        if (n0 > 7) n0 -= 16;
        if (n1 > 7) n1 -= 16;
        out[2 * b] = (float)n0 * s;
        out[2 * b + 1] = (float)n1 * s;
    }
}

/* Metal kv_cache_write (hy3.metal:285-297): the FP16 cache stores (half)x. */
void hy3o_round_fp16(const float *x, float *out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = hy3o_half_to_float(hy3o_float_to_half(x[i]));
}

/* ---------------------------------------------------------------- attention */

/* hy3.c:617-652 without the 4096-key stack cap (hy3.c:628-629): two-pass fp32
 * softmax, scale 1/sqrtf(128) applied after the dot, inv_sum = 1/(sum+1e-10).
 * Same loop order as the reference so a strict-IEEE build of both is bit-equal
 * for ntok <= 4096.  k, v: [ntok][n_kv_heads][128].                              */
void hy3o_attention(float *out, const float *q, const float *k, const float *v,
                    int n_heads, int n_kv_heads, int ntok) {
    const int hd = HY3O_HEAD_DIM;
    float scale = 1.0f / sqrtf((float)hd);
    int kv_group = n_heads / n_kv_heads;
    float *scores = (float *)malloc(sizeof(float) * (size_t)(ntok > 0 ? ntok : 1));
    for (int h = 0; h < n_heads; h++) {
        int kv_h = h / kv_group;
        const float *q_h = q + (size_t)h * hd;
        float max_score = -FLT_MAX;
        for (int t = 0; t < ntok; t++) {
            const float *k_t = k + ((size_t)t * n_kv_heads + kv_h) * hd;
            float s = 0.0f;
            for (int d = 0; d < hd; d++) s += q_h[d] * k_t[d];
            s *= scale;
            scores[t] = s;
            if (s > max_score) max_score = s;
        }
        float sum = 0.0f;
        for (int t = 0; t < ntok; t++) {
            scores[t] = expf(scores[t] - max_score);
            sum += scores[t];
        }
        float inv_sum = 1.0f / (sum + 1e-10f);
        float *out_h = out + (size_t)h * hd;
        memset(out_h, 0, hd * sizeof(float));
        for (int t = 0; t < ntok; t++) {
            float a = scores[t] * inv_sum;
            const float *v_t = v + ((size_t)t * n_kv_heads + kv_h) * hd;
            for (int d = 0; d < hd; d++) out_h[d] += a * v_t[d];
        }
    }
    free(scores);
}

/* Same attention in fp64 with an online softmax; used as the high-precision
 * yardstick for long contexts where fp32 two-pass sums lose bits.              */
void hy3o_attention_f64(double *out, const float *q, const float *k, const float *v,
                        int n_heads, int n_kv_heads, int ntok) {
    const int hd = HY3O_HEAD_DIM;
    double scale = 1.0 / sqrt((double)hd);
    int kv_group = n_heads / n_kv_heads;
    for (int h = 0; h < n_heads; h++) {
        int kv_h = h / kv_group;
        const float *q_h = q + (size_t)h * hd;
        double m = -INFINITY, l = 0.0, acc[HY3O_HEAD_DIM];
        for (int d = 0; d < hd; d++) acc[d] = 0.0;
        for (int t = 0; t < ntok; t++) {
            const float *k_t = k + ((size_t)t * n_kv_heads + kv_h) * hd;
            const float *v_t = v + ((size_t)t * n_kv_heads + kv_h) * hd;
            double s = 0.0;
            for (int d = 0; d < hd; d++) s += (double)q_h[d] * (double)k_t[d];
            s *= scale;
            double nm = s > m ? s : m;
            double corr = exp(m - nm), p = exp(s - nm);
            l = l * corr + p;
            for (int d = 0; d < hd; d++) acc[d] = acc[d] * corr + p * (double)v_t[d];
            m = nm;
        }
        for (int d = 0; d < hd; d++) out[(size_t)h * hd + d] = l > 0.0 ? acc[d] / l : 0.0;
    }
}

/* Unnormalised partial {m, l, acc[128]} per head over keys [t0, t1): the record a
 * split / shard emits (hy3_gpu.cu:183-230: p[0]=m, p[1]=l, p[2..129]=acc; an empty
 * range gives {-inf, 0, 0...}, hy3_gpu.cu:197-199).  partial: [n_heads][130].    */
void hy3o_attention_partial(float *partial, const float *q, const float *k, const float *v,
                            int n_heads, int n_kv_heads, int t0, int t1) {
    const int hd = HY3O_HEAD_DIM;
    double scale = 1.0 / sqrt((double)hd);
    int kv_group = n_heads / n_kv_heads;
    for (int h = 0; h < n_heads; h++) {
        int kv_h = h / kv_group;
        const float *q_h = q + (size_t)h * hd;
        float *p = partial + (size_t)h * 130;
        double m = -INFINITY, l = 0.0, acc[HY3O_HEAD_DIM];
        for (int d = 0; d < hd; d++) acc[d] = 0.0;
        for (int t = t0; t < t1; t++) {
            const float *k_t = k + ((size_t)t * n_kv_heads + kv_h) * hd;
            const float *v_t = v + ((size_t)t * n_kv_heads + kv_h) * hd;
            double s = 0.0;
            for (int d = 0; d < hd; d++) s += (double)q_h[d] * (double)k_t[d];
            s *= scale;
            double nm = s > m ? s : m;
            double corr = exp(m - nm), pr = exp(s - nm);
            l = l * corr + pr;
            for (int d = 0; d < hd; d++) acc[d] = acc[d] * corr + pr * (double)v_t[d];
            m = nm;
        }
        p[0] = (float)m;
        p[1] = (float)l;
        for (int d = 0; d < hd; d++) p[2 + d] = (float)acc[d];
    }
}

/* hy3_gpu.cu:233-247: fold n_parts partials per head in order; skip l<=0;
 * out = acc/l (0 when l==0).  partials: [n_parts][n_heads][130].                 */
void hy3o_merge_partials(float *out, const float *partials, int n_parts, int n_heads) {
    const int hd = HY3O_HEAD_DIM;
    for (int h = 0; h < n_heads; h++) {
        float ms = -INFINITY, ss = 0.0f, ov[HY3O_HEAD_DIM];
        for (int d = 0; d < hd; d++) ov[d] = 0.0f;
        for (int s = 0; s < n_parts; s++) {
            const float *p = partials + ((size_t)s * n_heads + h) * 130;
            float pms = p[0], pss = p[1];
            if (pss <= 0.0f) continue;
            float nm = fmaxf(ms, pms), os = expf(ms - nm), rs = expf(pms - nm);
            ss = ss * os + pss * rs;
            for (int d = 0; d < hd; d++) ov[d] = ov[d] * os + p[2 + d] * rs;
            ms = nm;
        }
        float inv = ss > 0.0f ? 1.0f / ss : 0.0f;
        for (int d = 0; d < hd; d++) out[(size_t)h * hd + d] = ov[d] * inv;
    }
}

/* Causal chunked prefill as the reference defines it (hy3_gpu.cu:379-382, :402):
 * query i of the chunk has global index base_tok+i and attends keys
 * [0 .. base_tok+i]; i.e. one decode attention per token.  q: [nq][n_heads][128]
 * (row stride q_stride floats), out: [nq][n_heads][128] (row stride o_stride).
 * rows: optional list of n_rows chunk-local query indices to evaluate (NULL = all). */
void hy3o_prefill_causal(float *out, const float *q, const float *k, const float *v,
                         int n_heads, int n_kv_heads, int base_tok, int nq,
                         size_t q_stride, size_t o_stride, const int *rows, int n_rows) {
    int n = rows ? n_rows : nq;
    for (int r = 0; r < n; r++) {
        int i = rows ? rows[r] : r;
        hy3o_attention(out + (size_t)i * o_stride, q + (size_t)i * q_stride, k, v,
                       n_heads, n_kv_heads, base_tok + i + 1);
    }
}

/* ---------------------------------------------------------------- fused append */

/* The per-token pipeline the reference runs before attention for one layer:
 * per-head RMSNorm of q and k with one shared 128-weight vector each
 * (hy3.c:1238-1247), rotate_half RoPE on q and k (hy3.c:1249), v untouched.
 * In place on q [n_heads*128] and k [n_kv_heads*128].                            */
void hy3o_qk_norm_rope(float *q, float *k, const float *qw, const float *kw, float eps,
                       int n_heads, int n_kv_heads, int pos, const float *inv_freq, float af,
                       int pos_stride, int pos_jump, int pos_jump_at) {
    for (int h = 0; h < n_heads; h++)
        hy3o_rms_norm(q + (size_t)h * HY3O_HEAD_DIM, q + (size_t)h * HY3O_HEAD_DIM, qw, HY3O_HEAD_DIM, eps);
    for (int h = 0; h < n_kv_heads; h++)
        hy3o_rms_norm(k + (size_t)h * HY3O_HEAD_DIM, k + (size_t)h * HY3O_HEAD_DIM, kw, HY3O_HEAD_DIM, eps);
    hy3o_rope(q, n_heads, pos, inv_freq, af, pos_stride, pos_jump, pos_jump_at);
    hy3o_rope(k, n_kv_heads, pos, inv_freq, af, pos_stride, pos_jump, pos_jump_at);
}

/* ---------------------------------------------------------------- seeded inputs */

/* Counter-based N(0,1) generator shared by host tests and the benchmark:
 * splitmix64(seed ^ (tensor_id << 40) ^ index) -> two 24-bit uniforms ->
 * Box-Muller (cos branch).  Host-only; device data is never regenerated here.    */
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

void hy3o_fill_normal(float *out, size_t n, uint64_t seed, uint64_t tensor_id) {
    for (size_t i = 0; i < n; i++) {
        uint64_t r = splitmix64(seed ^ (tensor_id << 40) ^ (uint64_t)i);
        double u1 = ((double)((r >> 40) & 0xFFFFFFu) + 1.0) / 16777217.0;
        double u2 = (double)((r >> 8) & 0xFFFFFFu) / 16777216.0;
        out[i] = (float)(sqrt(-2.0 * log(u1)) * cos(2.0 * M_PI * u2));
    }
}
