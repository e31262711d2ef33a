/*
 * ref_model_harness.c -- the REFERENCE engine (its own hy3.c, included from where it lies) as a shared
 * library, plus helpers that build a small in-memory model for it.
 *
 * TEST INFRASTRUCTURE ONLY.  Two purposes:
 *   1. the library exports the engine's public API (hy3_eval, hy3_rope_init, hy3_rope_get_params,
 *      forward_layer_dense / forward_layer_moe, ...), i.e. it plays the host program the drop-in backend
 *      (hy3_gpu_init / hy3_eval_gpu) is linked into;
 *   2. hy3h_model_new() fills a calloc'd hy3_model with seeded weights WITHOUT a checkpoint: all tensors live in
 *      memory, layer 0 is the dense layer, layers 1..79 share one set of MoE tensors and the 192 experts share a
 *      few distinct weight sets, so the whole 80-layer model is about a gigabyte.  hy3h_eval_cpu() then runs the
 *      engine's own CPU path (hy3_eval with no backend attached, hy3.c:1379-1412) on it.
 * No reference source is copied into this repository; the compiled result goes to oracle/_ref/ only.
 */
#ifndef HY3_REF_SRC
#error "compile with -DHY3_REF_SRC=\"/path/to/reference/hy3.c\""
#endif
#include HY3_REF_SRC

#define HY3H_POOL 4194301u            /* prime: tiled tensors never repeat a row exactly */
typedef struct {
    float *pool;                        /* HY3H_POOL seeded N(0,1) values; tensors are tiled from it at seeded offsets */
    hy3_tensor_info *infos;
    int n_infos, cap_infos;
    void **bufs;
    int n_bufs, cap_bufs;
    uint64_t rng;
} hy3h_arena;

static hy3h_arena *arena_of(hy3_model *m) { return (hy3h_arena *)m->gguf.kv; }   /* unused by an in-memory model */

static uint64_t h_next(uint64_t *s) {
    uint64_t x = (*s += 0x9E3779B97F4A7C15ull);
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
static float h_normal(uint64_t *s) {
    const double u1 = ((double)(h_next(s) >> 11) + 1.0) / 9007199254740993.0, u2 = (double)(h_next(s) >> 11) / 9007199254740992.0;
    return (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2));
}
static void *arena_alloc(hy3h_arena *a, size_t bytes) {
    if (a->n_bufs == a->cap_bufs) { a->cap_bufs = a->cap_bufs ? 2 * a->cap_bufs : 64; a->bufs = realloc(a->bufs, (size_t)a->cap_bufs * sizeof(void *)); }
    void *p = malloc(bytes);
    a->bufs[a->n_bufs++] = p;
    return p;
}
static hy3_weight make_weight(hy3h_arena *a, void *data, uint32_t type, uint64_t rows, uint64_t cols) {
    hy3_tensor_info *t = &a->infos[a->n_infos++];
    memset(t, 0, sizeof *t);
    t->ndim = cols > 1 ? 2 : 1;
    t->dim[0] = rows; t->dim[1] = cols;
    t->ggml_type = type;
    t->elements = rows * cols;
    hy3_weight w;
    w.t = t; w.data = (const uint8_t *)data;
    return w;
}
static inline float pool_at(const hy3h_arena *a, uint64_t off, uint64_t i) { return a->pool[(off + i) % HY3H_POOL]; }
/* fp32 tensor [rows][cols] ~ N(0, scale^2 / cols) (mean `mean`) */
static hy3_weight dense_f32(hy3h_arena *a, uint64_t rows, uint64_t cols, float scale, float mean) {
    float *p = arena_alloc(a, rows * cols * sizeof(float));
    const float s = scale / sqrtf((float)(cols > 1 ? cols : 1));
    const uint64_t off = h_next(&a->rng) % HY3H_POOL;
    for (uint64_t i = 0; i < rows * cols; i++) p[i] = mean + s * pool_at(a, off, i);
    return make_weight(a, p, 0, rows, cols);
}
#define HY3H_MIN_NORMAL_HALF 6.2e-5f
static uint16_t f2h(float f) {   /* round-to-nearest-even float -> half (subnormal halves included) */
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    int e = (int)((x >> 23) & 0xFF) - 127 + 15;
    uint32_t m = x & 0x7FFFFFu;
    if (e >= 31) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        m |= 0x800000u;                          /* the implicit one becomes explicit: value = m * 2^(e - 1 - 23 - 14) halves' ulps */
        const int shift = 14 - e;                /* 14 .. 24 */
        uint32_t h = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1u))) h++;
        return (uint16_t)(sign | h);
    }
    uint32_t h = (uint32_t)(e << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)(sign | h);
}
static hy3_weight dense_f16(hy3h_arena *a, uint64_t rows, uint64_t cols, float scale) {
    uint16_t *p = arena_alloc(a, rows * cols * sizeof(uint16_t));
    const float s = scale / sqrtf((float)cols);
    const uint64_t off = h_next(&a->rng) % HY3H_POOL;
    for (uint64_t i = 0; i < rows * cols; i++) {
        /* kept in the normal half range: the engine's own half decoder (hy3.c:354-369) reads zero and subnormal halves as
         * (1 + mantissa / 1024) * 2^-15, the device reads them as IEEE does -- such values would only compare the decoders */
        float v = s * pool_at(a, off, i);
        if (fabsf(v) < HY3H_MIN_NORMAL_HALF) v = copysignf(HY3H_MIN_NORMAL_HALF, v);
        p[i] = f2h(v);
    }
    return make_weight(a, p, 1, rows, cols);
}
/* Q4_K tensor of random blocks whose values have mean ~0 and rms ~ scale / sqrt(cols) */
static hy3_weight dense_q4k(hy3h_arena *a, uint64_t rows, uint64_t cols, float scale) {
    const uint64_t nb = rows * cols / 256;
    uint8_t *p = arena_alloc(a, nb * 144);
    float d = scale / sqrtf((float)cols) / 143.f;            /* code * sc has rms ~ 143 around its mean */
    if (d < HY3H_MIN_NORMAL_HALF / 0.75f) d = HY3H_MIN_NORMAL_HALF / 0.75f;   /* d and dmin stay normal halves (see dense_f16) */
    for (uint64_t b = 0; b < nb; b++) {
        uint8_t *blk = p + b * 144;
        const uint16_t hd = f2h(d * (0.75f + 0.5f * (float)(h_next(&a->rng) & 0xFF) / 255.f)), hm = f2h(d * 7.5f);
        memcpy(blk, &hd, 2); memcpy(blk + 2, &hm, 2);
        for (int i = 4; i < 144; i += 8) { const uint64_t r = h_next(&a->rng); memcpy(blk + i, &r, i + 8 <= 144 ? 8 : 144 - i); }
    }
    return make_weight(a, p, 12, rows, cols);
}

/* out_scale: size of the projections that write into the residual stream (attention output, FFN / expert down) relative
 * to a unit-variance projection; small values make every layer a small perturbation of the stream, so that the model
 * does not amplify rounding differences chaotically through its 80 layers */
hy3_model *hy3h_model_new(uint64_t seed, int vocab, int n_distinct_experts, int expert_type, int dense_f16_attn, float out_scale) {
    if (vocab < 1 || vocab > HY3_N_VOCAB || n_distinct_experts < 1 || n_distinct_experts > HY3_N_EXPERT) return NULL;
    hy3_model *m = calloc(1, sizeof(hy3_model));
    hy3h_arena *a = calloc(1, sizeof(hy3h_arena));
    if (!m || !a) return NULL;
    a->cap_infos = 64 + 3 * HY3_N_EXPERT;
    a->infos = calloc((size_t)a->cap_infos, sizeof(hy3_tensor_info));
    a->rng = seed;
    a->pool = malloc((size_t)HY3H_POOL * sizeof(float));
    for (uint32_t i = 0; i < HY3H_POOL; i++) a->pool[i] = h_normal(&a->rng);
    m->gguf.fd = -1;
    m->gguf.kv = (hy3_kv *)a;              /* parked here: nothing reads gguf.kv when n_kv is 0 */
    m->n_threads = 1;
    m->n_expert_used = HY3_N_EXPERT_USED;
    const int E = HY3_N_EMBD, QS = HY3_N_HEAD * HY3_HEAD_DIM, KVD = HY3_N_KV_HEAD * HY3_HEAD_DIM;
    m->w.token_embd = dense_f32(a, (uint64_t)vocab, E, sqrtf((float)E), 0.f);     /* rows ~ N(0, 1) */
    m->w.output_norm = dense_f32(a, E, 1, 0.05f, 1.f);
    m->w.output = dense_f32(a, (uint64_t)vocab, E, 1.f, 0.f);
    m->w.n_layer = HY3_N_LAYER;
    hy3_layer_weights proto[2];
    memset(proto, 0, sizeof proto);
    for (int k = 0; k < 2; k++) {
        hy3_layer_weights *l = &proto[k];
        l->attn_norm = dense_f32(a, E, 1, 0.05f, 1.f);
        l->ffn_norm = dense_f32(a, E, 1, 0.05f, 1.f);
        l->attn_q = dense_f16_attn ? dense_f16(a, QS, E, 1.f) : dense_f32(a, QS, E, 1.f, 0.f);
        l->attn_k = dense_f32(a, KVD, E, 1.f, 0.f);
        l->attn_v = dense_f32(a, KVD, E, 1.f, 0.f);
        l->attn_output = dense_f32(a, E, QS, out_scale, 0.f);
        l->attn_q_norm = dense_f32(a, HY3_HEAD_DIM, 1, 0.05f, 1.f);
        l->attn_k_norm = dense_f32(a, HY3_HEAD_DIM, 1, 0.05f, 1.f);
    }
    proto[0].ffn_gate = dense_f32(a, HY3_DENSE_INTERMED, E, 1.f, 0.f);
    proto[0].ffn_up = dense_f32(a, HY3_DENSE_INTERMED, E, 1.f, 0.f);
    proto[0].ffn_down = dense_f32(a, E, HY3_DENSE_INTERMED, out_scale, 0.f);
    {
        hy3_layer_weights *l = &proto[1];
        l->ffn_gate_inp = dense_f32(a, HY3_N_EXPERT, E, 2.f, 0.f);
        l->ffn_gate_shexp = dense_f32(a, HY3_MOE_INTERMED, E, 1.f, 0.f);
        l->ffn_up_shexp = dense_f32(a, HY3_MOE_INTERMED, E, 1.f, 0.f);
        l->ffn_down_shexp = dense_f32(a, E, HY3_MOE_INTERMED, out_scale, 0.f);
        hy3_weight g[HY3_N_EXPERT], u[HY3_N_EXPERT], d[HY3_N_EXPERT];
        for (int e = 0; e < n_distinct_experts; e++) {
            if (expert_type == 12) {
                g[e] = dense_q4k(a, HY3_MOE_INTERMED, E, 1.f); u[e] = dense_q4k(a, HY3_MOE_INTERMED, E, 1.f); d[e] = dense_q4k(a, E, HY3_MOE_INTERMED, out_scale);
            } else if (expert_type == 1) {
                g[e] = dense_f16(a, HY3_MOE_INTERMED, E, 1.f); u[e] = dense_f16(a, HY3_MOE_INTERMED, E, 1.f); d[e] = dense_f16(a, E, HY3_MOE_INTERMED, out_scale);
            } else {
                g[e] = dense_f32(a, HY3_MOE_INTERMED, E, 1.f, 0.f); u[e] = dense_f32(a, HY3_MOE_INTERMED, E, 1.f, 0.f); d[e] = dense_f32(a, E, HY3_MOE_INTERMED, out_scale, 0.f);
            }
        }
        for (int e = 0; e < HY3_N_EXPERT; e++) {
            l->ffn_gate_exps[e] = g[e % n_distinct_experts]; l->ffn_up_exps[e] = u[e % n_distinct_experts]; l->ffn_down_exps[e] = d[e % n_distinct_experts];
            l->expert_bias[e] = 0.05f * pool_at(a, 12345, (uint64_t)e);
        }
        l->has_expert_bias = true;
    }
    for (int il = 0; il < HY3_N_LAYER; il++) m->w.layers[il] = proto[il < HY3_N_LAYER_DENSE ? 0 : 1];
    hy3_rope_init(m);                      /* default table, or YaRN / probes from the HY3_ROPE_* / HY3_POS_* environment */
    m->embed = xcalloc(HY3_N_EMBD, sizeof(float));
    m->scratch = xcalloc(HY3_DENSE_INTERMED * 2 + HY3_N_EMBD * 4 + HY3_N_HEAD * HY3_HEAD_DIM * 4, sizeof(float));   /* hy3.c:904 */
    m->scratch2 = xcalloc(HY3_N_EXPERT + HY3_MOE_INTERMED * 4 + HY3_N_EMBD * 2, sizeof(float));                     /* hy3.c:905 */
    return m;
}

void hy3h_model_free(hy3_model *m) {
    if (!m) return;
    hy3h_arena *a = arena_of(m);
    for (int i = 0; i < a->n_bufs; i++) free(a->bufs[i]);
    free(a->bufs); free(a->infos); free(a->pool); free(a);
    free(m->embed); free(m->scratch); free(m->scratch2); free(m->cache_k); free(m->cache_v); free(m->cache_tokens);
    free(m);
}

/* the engine's CPU path on n tokens: returns hy3_eval's status, logits of the last token */
int hy3h_eval_cpu(hy3_model *m, const int *tok, int n, float *logits, int *pos) {
    hy3_tokens t;
    t.v = (int *)tok; t.len = n; t.cap = n;
    void *g = m->gpu_ctx;
    m->gpu_ctx = NULL;
    const int rc = hy3_eval(m, &t, logits, pos);
    m->gpu_ctx = g;
    return rc;
}
int hy3h_get_cache_len(const hy3_model *m) { return m->cache_len; }
void hy3h_set_cache_len(hy3_model *m, int v) { m->cache_len = v; }
void hy3h_set_expert_used(hy3_model *m, int k) { m->n_expert_used = k; }
int hy3h_gpu_layers(const hy3_model *m) { return m->gpu_layers; }
int hy3h_has_gpu_ctx(const hy3_model *m) { return m->gpu_ctx != NULL; }
