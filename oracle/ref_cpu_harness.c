/*
 * ref_cpu_harness.c -- thin exported wrappers around the REFERENCE's own CPU code.
 *
 * TEST INFRASTRUCTURE ONLY.  This translation unit textually includes the
 * reference engine's hy3.c from where it lies (path given by -DHY3_REF_SRC=...)
 * so that its file-static functions rms_norm (hy3.c:441), rope (hy3.c:585) and
 * attention (hy3.c:617) can be called unmodified.  No reference source is copied
 * into this repository; the compiled result goes to oracle/_ref/ only.
 *
 * The wrappers translate between the dense "layer view" the tests use
 * ([ntok][8][128] fp32 per layer) and the reference's interleaved slot layout
 * (slot = token*80 + layer, hy3.c:631).  The slot arrays are sparse anonymous
 * mappings so that a single layer only touches its own pages.
 */
#ifndef HY3_REF_SRC
#error "compile with -DHY3_REF_SRC=\"/path/to/reference/hy3.c\""
#endif
#include HY3_REF_SRC

#include <sys/mman.h>

#define REF_KV_ROW (HY3_N_KV_HEAD * HY3_HEAD_DIM)

static float *g_slot_k, *g_slot_v;
static size_t g_slot_tokens;

static int ensure_slots(size_t ntok) {
    if (ntok <= g_slot_tokens) return 0;
    if (g_slot_k) {
        munmap(g_slot_k, g_slot_tokens * HY3_N_LAYER * REF_KV_ROW * sizeof(float));
        munmap(g_slot_v, g_slot_tokens * HY3_N_LAYER * REF_KV_ROW * sizeof(float));
    }
    size_t bytes = ntok * HY3_N_LAYER * REF_KV_ROW * sizeof(float);
    g_slot_k = (float *)mmap(NULL, bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    g_slot_v = (float *)mmap(NULL, bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (g_slot_k == MAP_FAILED || g_slot_v == MAP_FAILED) { g_slot_k = g_slot_v = NULL; g_slot_tokens = 0; return -1; }
    g_slot_tokens = ntok;
    return 0;
}

/* Scatter a dense layer view into the reference slot layout (layer `layer`). */
int hy3ref_load_layer(const float *k, const float *v, int ntok, int layer) {
    if (ensure_slots((size_t)ntok)) return -1;
    for (int t = 0; t < ntok; t++) {
        size_t slot = (size_t)t * HY3_N_LAYER + (size_t)layer;
        memcpy(g_slot_k + slot * REF_KV_ROW, k + (size_t)t * REF_KV_ROW, REF_KV_ROW * sizeof(float));
        memcpy(g_slot_v + slot * REF_KV_ROW, v + (size_t)t * REF_KV_ROW, REF_KV_ROW * sizeof(float));
    }
    return 0;
}

/* The reference attention() over the first ntok tokens of the loaded layer.
 * cache_len is chosen so that the reference's own ntok formula (hy3.c:622) gives
 * ntok.  Note the reference silently caps at 4096 keys (hy3.c:628-629).          */
void hy3ref_attention(float *out, const float *q, int ntok, int layer) {
    int cache_len = (ntok - 1) * HY3_N_LAYER + layer + 1;
    attention(out, q, g_slot_k, g_slot_v, HY3_N_KV_HEAD, HY3_N_HEAD, HY3_HEAD_DIM, cache_len,
              HY3_N_HEAD / HY3_N_KV_HEAD, layer);
}

/* The reference attention() for one KV group only (8 query heads), used to run
 * the unmodified function from several threads at once: pointers are pre-offset
 * to the group, n_heads = 8 and kv_group = 8 make kv_h evaluate to 0 while the
 * row stride still uses n_kv_heads = 8.                                          */
void hy3ref_attention_group(float *out, const float *q, int ntok, int layer, int group) {
    int cache_len = (ntok - 1) * HY3_N_LAYER + layer + 1;
    int gq = HY3_N_HEAD / HY3_N_KV_HEAD;
    attention(out + (size_t)group * gq * HY3_HEAD_DIM, q + (size_t)group * gq * HY3_HEAD_DIM,
              g_slot_k + (size_t)group * HY3_HEAD_DIM, g_slot_v + (size_t)group * HY3_HEAD_DIM,
              HY3_N_KV_HEAD, gq, HY3_HEAD_DIM, cache_len, gq, layer);
}

/* All 8 groups of hy3ref_attention_group on OpenMP threads. */
void hy3ref_attention_mt(float *out, const float *q, int ntok, int layer) {
#pragma omp parallel for schedule(static)
    for (int g = 0; g < HY3_N_KV_HEAD; g++) hy3ref_attention_group(out, q, ntok, layer, g);
}

/* Several layers of the loaded slot arrays at once: (layer, group) pairs spread over all
 * OpenMP threads, each pair one call of the unmodified attention().  q/out: [n_layers][64][128]. */
void hy3ref_attention_layers_mt(float *out, const float *q, int ntok, int n_layers) {
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int l = 0; l < n_layers; l++)
        for (int g = 0; g < HY3_N_KV_HEAD; g++)
            hy3ref_attention_group(out + (size_t)l * HY3_N_HEAD * HY3_HEAD_DIM, q + (size_t)l * HY3_N_HEAD * HY3_HEAD_DIM, ntok, l, g);
}

void hy3ref_rms_norm(float *out, const float *x, const float *w, int n, float eps) { rms_norm(out, x, w, n, eps); }

/* hy3_rope_init on a zeroed model (no GGUF: every metadata lookup falls back to
 * its default); the HY3_ROPE_* / HY3_POS_* environment is read by the reference
 * itself.  Returns the table the backends would get from hy3_rope_get_params.    */
static hy3_model *g_model;
void hy3ref_rope_init(float *inv_freq /*[64]*/, float *attn_factor) {
    if (!g_model) g_model = (hy3_model *)calloc(1, sizeof(hy3_model));
    hy3_rope_init(g_model);
    hy3_rope_get_params(g_model, inv_freq, attn_factor);
}

/* The reference rope() on q [64][128] and k [8][128] with the table from the last
 * hy3ref_rope_init call.                                                         */
void hy3ref_rope(float *q, float *k, int pos) {
    rope(g_model, q, k, pos, HY3_HEAD_DIM, HY3_N_HEAD, HY3_N_KV_HEAD);
}

int hy3ref_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the OpenMP team size the *_mt entry points use (the benchmark's reference arm passes the host's core count, so
 * the team does not depend on OMP_NUM_THREADS of the launching shell); returns the size in effect. */
int hy3ref_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}
