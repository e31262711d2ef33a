/*
 * capi.cu -- the C ABI declared in include/hy3_attn.h: context, KV block pool, per-step
 * batch descriptor, and the thin wrappers that enqueue the kernels.
 *
 * Host-side counterpart of the KV / scratch / position plumbing in the reference's
 * hy3_gpu_init, gpu_ensure_kv_capacity and hy3_eval_gpu (hy3_gpu.cu:598-627, :692-698,
 * :868-889).  Differences that matter to a caller: no exit() on errors (codes + message),
 * every launch is checked, growth never copies or moves the cache, and positions are an
 * argument of every step (no hidden counter), so a rolled-back cache_len just works.
 */
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ctx.h"

static thread_local char g_create_err[512];   /* message of the last failed hy3a_create of this thread */

int hy3a_fail(hy3a_ctx *ctx, int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx ? ctx->err : g_create_err, 512, fmt, ap);
    va_end(ap);
    return code;
}

extern "C" {

const char *hy3a_version(void) { return "hy3attn sm_100a " __DATE__; }

const char *hy3a_last_error(const hy3a_ctx *ctx) { return ctx ? ctx->err : g_create_err; }

void hy3a_default_config(hy3a_config *cfg) {
    memset(cfg, 0, sizeof(*cfg));
    cfg->kv_dtype = HY3A_KV_INT8;
    cfg->n_layers = 80;
    cfg->kv_head_begin = 0;
    cfg->kv_head_count = HY3A_N_KV_HEAD;
    cfg->max_seqs = 1;
    cfg->max_batch = 512;
    cfg->max_blocks = 8192 / HY3A_PAGE_TOKENS;
    cfg->max_blocks_per_seq = 8192 / HY3A_PAGE_TOKENS;
    cfg->device = -1;
    cfg->rms_eps = 1e-5f;
}

int hy3a_slot_bytes(int kv_dtype) { return kv_dtype == HY3A_KV_INT8 ? 1040 : (kv_dtype == HY3A_KV_INT4 ? 528 : (kv_dtype == HY3A_KV_FP16 ? 2048 : -1)); }

static int check_config(const hy3a_config *c) {
    if (!c) return hy3a_fail(NULL, HY3A_EINVAL, "config is NULL");
    if (c->kv_dtype < 0 || c->kv_dtype > 2) return hy3a_fail(NULL, HY3A_EINVAL, "kv_dtype %d not in {0,1,2}", c->kv_dtype);
    if (c->n_layers < 1 || c->n_layers > HY3A_MAX_LAYERS) return hy3a_fail(NULL, HY3A_EINVAL, "n_layers %d out of range", c->n_layers);
    if (c->kv_head_count < 1 || c->kv_head_begin < 0 || c->kv_head_begin + c->kv_head_count > HY3A_N_KV_HEAD)
        return hy3a_fail(NULL, HY3A_EINVAL, "kv head range [%d,+%d) outside [0,8)", c->kv_head_begin, c->kv_head_count);
    if (c->max_seqs < 1 || c->max_batch < 1 || c->max_blocks < 1 || c->max_blocks_per_seq < 1)
        return hy3a_fail(NULL, HY3A_EINVAL, "max_seqs/max_batch/max_blocks/max_blocks_per_seq must be >= 1");
    if (!(c->rms_eps > 0.f)) return hy3a_fail(NULL, HY3A_EINVAL, "rms_eps must be > 0");
    return 0;
}

size_t hy3a_block_bytes(const hy3a_config *cfg) {
    if (check_config(cfg)) return 0;
    hy3a_geom g = hy3a_make_geom(cfg->kv_dtype);
    return (size_t)cfg->n_layers * cfg->kv_head_count * g.page_bytes;
}

int hy3a_decode_schedule(int n, const int *kv_lens, int kv_heads, int n_ctas, int cta, long long *total_units, long long *u0,
                         long long *u1) {
    /* the same arithmetic as the head of hy3a_decode_kernel (the INT8 kernel moves a few pages between the pieces of the last
     * segment of a single-row grid on top of it: decode_umma.cu) */
    if (n < 0 || kv_heads < 1 || n_ctas < 1 || cta < 0 || cta >= n_ctas) return HY3A_EINVAL;
    long long P = 0;
    int rows_ne = 0;
    for (int i = 0; i < n; i++) { long long p = kv_lens[i] > 0 ? (kv_lens[i] + HY3A_PAGE_TOKENS - 1) / HY3A_PAGE_TOKENS : 0; P += p; rows_ne += p > 0; }
    const long long U = P * kv_heads;
    if (total_units) *total_units = U;
    long long b = U, e = U;
    bool aligned = U > 0 && (long long)n * kv_heads < n_ctas;
    if (aligned && (long long)n * kv_heads * 4 > n_ctas) {
        /* the aligned split is kept only while its rounding leaves no CTA more than 5/4 of the even share */
        const long long spare = (long long)n_ctas - (long long)rows_ne * kv_heads, PG = P * kv_heads;
        long long worst = 0;
        for (int r = 0; r < n; r++) {
            long long p = kv_lens[r] > 0 ? (kv_lens[r] + HY3A_PAGE_TOKENS - 1) / HY3A_PAGE_TOKENS : 0;
            if (p == 0) continue;
            long long c = 1 + spare * p / PG;
            if (c > p) c = p;
            if ((p + c - 1) / c > worst) worst = (p + c - 1) / c;
        }
        aligned = worst * 4 <= (PG + n_ctas - 1) / n_ctas * 5 + 4;
    }
    if (aligned) {
        const long long spare = (long long)n_ctas - (long long)rows_ne * kv_heads;
        long long base = 0, pre = 0;
        for (int r = 0; r < n; r++) {
            long long p = kv_lens[r] > 0 ? (kv_lens[r] + HY3A_PAGE_TOKENS - 1) / HY3A_PAGE_TOKENS : 0;
            if (p == 0) continue;
            long long c = 1 + spare * p / (P * kv_heads);
            if (c > p) c = p;
            if (cta < base + kv_heads * c) {
                long long idx = cta - base, hl = idx / c, k = idx % c, seg0 = kv_heads * pre + hl * p;
                b = seg0 + k * p / c; e = seg0 + (k + 1) * p / c;
                break;
            }
            base += kv_heads * c; pre += p;
        }
    } else if (U > 0) {
        const int C = U < n_ctas ? (int)U : n_ctas;
        if (cta < C) { b = (long long)cta * U / C; e = (long long)(cta + 1) * U / C; }
    }
    if (u0) *u0 = b;
    if (u1) *u1 = e;
    return 0;
}

void hy3a_destroy(hy3a_ctx *ctx) {
    if (!ctx) return;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->pool); cudaFree(ctx->d_block_table); cudaFree(ctx->d_vs_max); cudaFree(ctx->d_inv_freq);
    cudaFree(ctx->d_norm_w); cudaFree(ctx->d_batch); cudaFree(ctx->d_partials); cudaFree(ctx->d_counters); cudaFree(ctx->d_err);
    cudaFree(ctx->d_pf_k); cudaFree(ctx->d_pf_v);
    for (int l = 0; l < HY3A_MAX_LAYERS; l++) { cudaFree(ctx->pf_mk[l]); cudaFree(ctx->pf_mv[l]); }
    hy3a_shard_disconnect(ctx);
    cudaFree(ctx->shard_local);
    if (ctx->h_ring) cudaFreeHost(ctx->h_ring);
    if (ctx->h_err) cudaFreeHost(ctx->h_err);
    for (int i = 0; i < HY3A_RING_SLOTS; i++) if (ctx->ring_ev[i]) cudaEventDestroy(ctx->ring_ev[i]);
    if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    free(ctx->h_block_table); free(ctx->h_seq_blocks); free(ctx->h_free);
    free(ctx);
    if (prev >= 0) cudaSetDevice(prev);
}

#define CREATE_CUDA(call)                                                                                            \
    do {                                                                                                             \
        cudaError_t e_ = (call);                                                                                     \
        if (e_ != cudaSuccess) {                                                                                     \
            hy3a_fail(NULL, HY3A_ECUDA, "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__);         \
            hy3a_destroy(ctx);                                                                                       \
            return e_ == cudaErrorMemoryAllocation ? HY3A_ENOMEM : HY3A_ECUDA;                                        \
        }                                                                                                            \
    } while (0)

int hy3a_selftest(hy3a_ctx *ctx);

int hy3a_create(const hy3a_config *cfg, hy3a_ctx **out) {
    if (!out) return hy3a_fail(NULL, HY3A_EINVAL, "out is NULL");
    *out = NULL;
    int rc = check_config(cfg);
    if (rc) return rc;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        return hy3a_fail(NULL, HY3A_ECUDA, "no CUDA device: this library has no CPU path");
    int dev = cfg->device;
    if (dev < 0 && cudaGetDevice(&dev) != cudaSuccess) return hy3a_fail(NULL, HY3A_ECUDA, "cudaGetDevice failed");
    if (dev >= ndev) return hy3a_fail(NULL, HY3A_EINVAL, "device %d of %d", dev, ndev);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return hy3a_fail(NULL, HY3A_ECUDA, "cudaGetDeviceProperties failed");
    if (prop.major != 10 || prop.minor != 0)
        return hy3a_fail(NULL, HY3A_EDEVICE, "device %d (%s) is compute capability %d.%d; the kernels are built for sm_100a (10.0) only",
                         dev, prop.name, prop.major, prop.minor);

    hy3a_ctx *ctx = (hy3a_ctx *)calloc(1, sizeof(hy3a_ctx));
    if (!ctx) return hy3a_fail(NULL, HY3A_ENOMEM, "calloc failed");
    ctx->cfg = *cfg;
    ctx->shard_slot = -1;
    ctx->cfg.device = dev;
    ctx->device = dev;
    ctx->geom = hy3a_make_geom(cfg->kv_dtype);
    ctx->sm_count = prop.multiProcessorCount;
    ctx->decode_ctas = prop.multiProcessorCount;
    { const char *e = getenv("HY3A_DECODE_CTAS"); if (e && atoi(e) > 0) ctx->decode_ctas = atoi(e); }
    if (ctx->decode_ctas > hy3a_decode_max_ctas()) ctx->decode_ctas = hy3a_decode_max_ctas();
    if (ctx->decode_ctas > 512) ctx->decode_ctas = 512;
    { const char *e = getenv("HY3A_NO_PDL"); ctx->use_pdl = !(e && atoi(e)); }
    /* fp16 operand mirrors of the chunked prefill: at most this much device memory beside the pool */
    { const char *e = getenv("HY3A_PF_MIRROR_MB"); ctx->pf_mbudget = (size_t)(e ? (atoll(e) > 0 ? atoll(e) : 0) : 8192) << 20; }
    ctx->pf_mseq = -1;
    {   /* ring depth: as many pages as fit in shared memory beside the merge buffers, at most 8 */
        ctx->decode_stages = hy3a_decode_ring_capacity(ctx->geom.page_bytes, cfg->max_batch);
        const char *e = getenv("HY3A_DECODE_STAGES");
        if (e) { int v = atoi(e); if (v < ctx->decode_stages) ctx->decode_stages = v; }
    }
    struct device_guard {   /* the caller's current device is put back on every way out */
        int prev;
        device_guard() : prev(-1) { cudaGetDevice(&prev); }
        ~device_guard() { if (prev >= 0) cudaSetDevice(prev); }
    } guard;
    CREATE_CUDA(cudaSetDevice(dev));
    CREATE_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    ctx->own_stream = 1;

    const size_t block_bytes = (size_t)cfg->n_layers * cfg->kv_head_count * ctx->geom.page_bytes;
    ctx->pool_bytes = block_bytes * (size_t)cfg->max_blocks;
    CREATE_CUDA(cudaMalloc(&ctx->pool, ctx->pool_bytes));
    if (hy3a_launch_init_pages(ctx, 0, (size_t)cfg->max_blocks * cfg->n_layers * cfg->kv_head_count)) {
        hy3a_fail(NULL, HY3A_ECUDA, "%s", ctx->err); hy3a_destroy(ctx); return HY3A_ECUDA;
    }
    const size_t bt = (size_t)cfg->max_seqs * cfg->max_blocks_per_seq;
    CREATE_CUDA(cudaMalloc(&ctx->d_block_table, bt * sizeof(int)));
    CREATE_CUDA(cudaMemsetAsync(ctx->d_block_table, 0, bt * sizeof(int), ctx->stream));
    CREATE_CUDA(cudaMalloc(&ctx->d_vs_max, (size_t)cfg->n_layers * cfg->kv_head_count * sizeof(unsigned)));
    CREATE_CUDA(cudaMemsetAsync(ctx->d_vs_max, 0, (size_t)cfg->n_layers * cfg->kv_head_count * sizeof(unsigned), ctx->stream));
    CREATE_CUDA(cudaMalloc(&ctx->d_inv_freq, 64 * sizeof(float)));
    CREATE_CUDA(cudaMalloc(&ctx->d_norm_w, (size_t)cfg->n_layers * 2 * HY3A_D * sizeof(float)));
    CREATE_CUDA(cudaMalloc(&ctx->d_batch, (size_t)3 * cfg->max_batch * sizeof(int)));
    ctx->partial_records = (size_t)ctx->decode_ctas + (size_t)cfg->max_batch * cfg->kv_head_count;
    CREATE_CUDA(cudaMalloc(&ctx->d_partials, ctx->partial_records * 8 * HY3A_REC_FLOATS * sizeof(float)));
    CREATE_CUDA(cudaMalloc(&ctx->d_counters, (size_t)2 * cfg->max_batch * cfg->kv_head_count * sizeof(unsigned)));
    CREATE_CUDA(cudaMemsetAsync(ctx->d_counters, 0, (size_t)2 * cfg->max_batch * cfg->kv_head_count * sizeof(unsigned), ctx->stream));
    CREATE_CUDA(cudaMalloc(&ctx->d_err, HY3A_ERR_WORDS * sizeof(unsigned)));
    CREATE_CUDA(cudaMemsetAsync(ctx->d_err, 0, HY3A_ERR_WORDS * sizeof(unsigned), ctx->stream));
    /* operand mirrors of the chunked prefill, sized for a whole sequence, when a context that takes chunks (max_batch >= 16:
     * one query tile) can hold all layers' mirrors within the budget: hy3a_prefill then never allocates.  Zeroed once:
     * columns past a sequence's end are read by the last tile (and masked), so they must never hold a NaN or Inf pattern. */
    if (ctx->pf_mbudget && cfg->max_batch >= 16) {
        const int seq_cap = (cfg->max_blocks_per_seq * HY3A_PT + 1023) / 1024 * 1024;
        const size_t per_layer = 2 * (size_t)cfg->kv_head_count * seq_cap * HY3A_D * 2 /* fp16 */;
        if (per_layer * (size_t)cfg->n_layers <= ctx->pf_mbudget) {
            bool ok = true;
            for (int l = 0; l < cfg->n_layers && ok; l++) {
                ok = cudaMalloc(&ctx->pf_mk[l], per_layer / 2) == cudaSuccess && cudaMalloc(&ctx->pf_mv[l], per_layer / 2) == cudaSuccess &&
                     cudaMemsetAsync(ctx->pf_mk[l], 0, per_layer / 2, ctx->stream) == cudaSuccess &&
                     cudaMemsetAsync(ctx->pf_mv[l], 0, per_layer / 2, ctx->stream) == cudaSuccess;
                if (ok) { ctx->pf_mcap[l] = seq_cap; ctx->pf_mbytes += per_layer; }
            }
            if (!ok) {   /* no room beside the pool: the mirrors are then grown on demand, or the shared workspace is used */
                cudaGetLastError();
                for (int l = 0; l < cfg->n_layers; l++) {
                    cudaFree(ctx->pf_mk[l]); cudaFree(ctx->pf_mv[l]);
                    ctx->pf_mk[l] = ctx->pf_mv[l] = NULL; ctx->pf_mcap[l] = 0;
                }
                ctx->pf_mbytes = 0;
            }
        }
    }
    CREATE_CUDA(cudaHostAlloc((void **)&ctx->h_err, HY3A_ERR_WORDS * sizeof(unsigned), cudaHostAllocDefault));

    ctx->ring_slot_bytes = (size_t)3 * cfg->max_batch * sizeof(int);
    if (ctx->ring_slot_bytes < 4096) ctx->ring_slot_bytes = 4096;
    CREATE_CUDA(cudaHostAlloc((void **)&ctx->h_ring, ctx->ring_slot_bytes * HY3A_RING_SLOTS, cudaHostAllocDefault));
    for (int i = 0; i < HY3A_RING_SLOTS; i++) CREATE_CUDA(cudaEventCreateWithFlags(&ctx->ring_ev[i], cudaEventDisableTiming));

    ctx->h_block_table = (int *)malloc(bt * sizeof(int));
    ctx->h_seq_blocks = (int *)calloc(cfg->max_seqs, sizeof(int));
    ctx->h_free = (int *)malloc((size_t)cfg->max_blocks * sizeof(int));
    if (!ctx->h_block_table || !ctx->h_seq_blocks || !ctx->h_free) { hy3a_destroy(ctx); return hy3a_fail(NULL, HY3A_ENOMEM, "host allocation failed"); }
    for (size_t i = 0; i < bt; i++) ctx->h_block_table[i] = -1;
    for (int i = 0; i < cfg->max_blocks; i++) ctx->h_free[i] = cfg->max_blocks - 1 - i; /* pop order 0,1,2,... */
    ctx->n_free = cfg->max_blocks;

    /* defaults: native RoPE table (theta 11158840, hy3.c:26, :542-545), unit norm weights */
    {
        float inv[64];
        for (int i = 0; i < 64; i++) inv[i] = (float)(1.0 / pow(11158840.0, (double)(2 * i) / 128.0));
        rc = hy3a_set_rope(ctx, inv, 1.0f, 1, 0, 0);
        if (rc) { hy3a_fail(NULL, rc, "%s", ctx->err); hy3a_destroy(ctx); return rc; }
        float ones[HY3A_D];
        for (int i = 0; i < HY3A_D; i++) ones[i] = 1.0f;
        for (int l = 0; l < cfg->n_layers; l++) {
            rc = hy3a_set_norm_weights(ctx, l, ones, ones);
            if (rc) { hy3a_fail(NULL, rc, "%s", ctx->err); hy3a_destroy(ctx); return rc; }
        }
    }
    CREATE_CUDA(cudaStreamSynchronize(ctx->stream));
    { const char *e = getenv("HY3A_NO_SELFTEST");
      if (!(e && atoi(e))) {
          rc = hy3a_selftest(ctx);
          if (rc) { hy3a_fail(NULL, rc, "self-test failed: %s", ctx->err); hy3a_destroy(ctx); return rc; }
      } }
    *out = ctx;
    return HY3A_OK;
}

int hy3a_set_stream(hy3a_ctx *ctx, void *s) {
    if (!ctx) return HY3A_EINVAL;
    if (ctx->own_stream && ctx->stream) { cudaStreamSynchronize(ctx->stream); cudaStreamDestroy(ctx->stream); }
    ctx->own_stream = 0;
    ctx->stream = (cudaStream_t)s;
    return HY3A_OK;
}
void *hy3a_get_stream(hy3a_ctx *ctx) { return ctx ? (void *)ctx->stream : NULL; }

int hy3a_sync(hy3a_ctx *ctx) {
    if (!ctx) return HY3A_EINVAL;
    HY3A_CUDA(ctx, cudaMemcpyAsync(ctx->h_err, ctx->d_err, HY3A_ERR_WORDS * sizeof(unsigned), cudaMemcpyDeviceToHost, ctx->stream));
    HY3A_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->h_err[0]) {
        unsigned code = ctx->h_err[0], where = ctx->h_err[1], w2 = ctx->h_err[2], w3 = ctx->h_err[3];
        cudaMemsetAsync(ctx->d_err, 0, HY3A_ERR_WORDS * sizeof(unsigned), ctx->stream);
        /* a kernel that gave up may have left merge counters behind */
        cudaMemsetAsync(ctx->d_counters, 0, (size_t)2 * ctx->cfg.max_batch * ctx->cfg.kv_head_count * sizeof(unsigned), ctx->stream);
        return hy3a_fail(ctx, HY3A_ETIMEOUT, "device-side bounded wait or bounds check failed (code %u, where %u, detail %u %u)", code, where, w2, w3);
    }
    return HY3A_OK;
}

/* Copy a small host buffer to the device through a ring of pinned slots, so the caller's
 * buffer may be reused at once and no slot is overwritten before its copy has run (the
 * hazard the reference met with its single pinned h_pos, hy3_gpu.cu:361-364).           */
static int stage_h2d(hy3a_ctx *ctx, void *dst, const void *src, size_t bytes) {
    const char *s = (const char *)src;
    char *d = (char *)dst;
    while (bytes) {
        size_t n = bytes < ctx->ring_slot_bytes ? bytes : ctx->ring_slot_bytes;
        int slot = ctx->ring_next;
        ctx->ring_next = (slot + 1) % HY3A_RING_SLOTS;
        if (ctx->ring_used[slot]) HY3A_CUDA(ctx, cudaEventSynchronize(ctx->ring_ev[slot]));
        char *stage = ctx->h_ring + (size_t)slot * ctx->ring_slot_bytes;
        memcpy(stage, s, n);
        HY3A_CUDA(ctx, cudaMemcpyAsync(d, stage, n, cudaMemcpyHostToDevice, ctx->stream));
        HY3A_CUDA(ctx, cudaEventRecord(ctx->ring_ev[slot], ctx->stream));
        ctx->ring_used[slot] = 1;
        s += n; d += n; bytes -= n;
    }
    return HY3A_OK;
}

int hy3a_set_rope(hy3a_ctx *ctx, const float *inv_freq, float attn_factor, int pos_stride, int pos_jump, int pos_jump_at) {
    if (!ctx || !inv_freq) return hy3a_fail(ctx, HY3A_EINVAL, "set_rope: NULL argument");
    if (pos_stride < 1) return hy3a_fail(ctx, HY3A_EINVAL, "set_rope: pos_stride must be >= 1");
    int rc = stage_h2d(ctx, ctx->d_inv_freq, inv_freq, 64 * sizeof(float));
    if (rc) return rc;
    ctx->rope.inv_freq = ctx->d_inv_freq;
    ctx->rope.attn_factor = attn_factor;
    ctx->rope.pos_stride = pos_stride;
    ctx->rope.pos_jump = pos_jump;
    ctx->rope.pos_jump_at = pos_jump_at;
    return HY3A_OK;
}

int hy3a_set_norm_weights(hy3a_ctx *ctx, int layer, const float *qw, const float *kw) {
    if (!ctx || !qw || !kw) return hy3a_fail(ctx, HY3A_EINVAL, "set_norm_weights: NULL argument");
    if (layer < 0 || layer >= ctx->cfg.n_layers) return hy3a_fail(ctx, HY3A_EINVAL, "set_norm_weights: layer %d out of range", layer);
    int rc = stage_h2d(ctx, ctx->d_norm_w + (size_t)layer * 2 * HY3A_D, qw, HY3A_D * sizeof(float));
    if (rc) return rc;
    return stage_h2d(ctx, ctx->d_norm_w + (size_t)layer * 2 * HY3A_D + HY3A_D, kw, HY3A_D * sizeof(float));
}

/* ---- block pool -------------------------------------------------------------------- */
int hy3a_seq_reserve(hy3a_ctx *ctx, int seq, int ntok) {
    if (!ctx) return HY3A_EINVAL;
    if (seq < 0 || seq >= ctx->cfg.max_seqs) return hy3a_fail(ctx, HY3A_EINVAL, "seq %d out of range [0,%d)", seq, ctx->cfg.max_seqs);
    if (ntok < 0) return hy3a_fail(ctx, HY3A_EINVAL, "ntok %d < 0", ntok);
    int need = (ntok + HY3A_PAGE_TOKENS - 1) / HY3A_PAGE_TOKENS;
    int have = ctx->h_seq_blocks[seq];
    if (need <= have) return HY3A_OK;
    if (need > ctx->cfg.max_blocks_per_seq)
        return hy3a_fail(ctx, HY3A_ENOMEM, "sequence %d needs %d blocks, max_blocks_per_seq is %d", seq, need, ctx->cfg.max_blocks_per_seq);
    if (need - have > ctx->n_free)
        return hy3a_fail(ctx, HY3A_ENOMEM, "KV pool exhausted: need %d more blocks, %d free", need - have, ctx->n_free);
    int *row = ctx->h_block_table + (size_t)seq * ctx->cfg.max_blocks_per_seq;
    for (int b = have; b < need; b++) row[b] = ctx->h_free[--ctx->n_free];
    ctx->h_seq_blocks[seq] = need;
    return stage_h2d(ctx, ctx->d_block_table + (size_t)seq * ctx->cfg.max_blocks_per_seq + have, row + have, (size_t)(need - have) * sizeof(int));
}

int hy3a_seq_release(hy3a_ctx *ctx, int seq, int keep_ntok) {
    if (!ctx) return HY3A_EINVAL;
    if (seq < 0 || seq >= ctx->cfg.max_seqs) return hy3a_fail(ctx, HY3A_EINVAL, "seq %d out of range", seq);
    if (keep_ntok < 0) keep_ntok = 0;
    int keep = (keep_ntok + HY3A_PAGE_TOKENS - 1) / HY3A_PAGE_TOKENS;
    hy3a_mirror_truncate(ctx, seq, -1, keep_ntok);
    int *row = ctx->h_block_table + (size_t)seq * ctx->cfg.max_blocks_per_seq;
    while (ctx->h_seq_blocks[seq] > keep) {
        int b = --ctx->h_seq_blocks[seq];
        ctx->h_free[ctx->n_free++] = row[b];
        row[b] = -1;
    }
    return HY3A_OK;
}

int hy3a_seq_capacity(hy3a_ctx *ctx, int seq) {
    if (!ctx || seq < 0 || seq >= ctx->cfg.max_seqs) return HY3A_EINVAL;
    return ctx->h_seq_blocks[seq] * HY3A_PAGE_TOKENS;
}
int hy3a_free_blocks(hy3a_ctx *ctx) { return ctx ? ctx->n_free : HY3A_EINVAL; }

int hy3a_batch_set(hy3a_ctx *ctx, int n, const int *seq_ids, const int *slots, const int *rope_pos) {
    if (!ctx || !seq_ids || !slots || !rope_pos) return hy3a_fail(ctx, HY3A_EINVAL, "batch_set: NULL argument");
    if (n < 1 || n > ctx->cfg.max_batch) return hy3a_fail(ctx, HY3A_EINVAL, "batch_set: n=%d not in [1,%d]", n, ctx->cfg.max_batch);
    for (int i = 0; i < n; i++) {
        if (seq_ids[i] < 0 || seq_ids[i] >= ctx->cfg.max_seqs) return hy3a_fail(ctx, HY3A_EINVAL, "batch_set: row %d seq %d out of range", i, seq_ids[i]);
        if (slots[i] < -1) return hy3a_fail(ctx, HY3A_EINVAL, "batch_set: row %d slot %d < -1", i, slots[i]);
        int rc = hy3a_seq_reserve(ctx, seq_ids[i], slots[i] + 1);
        if (rc) return rc;
        if (slots[i] >= 0) hy3a_mirror_truncate(ctx, seq_ids[i], -1, slots[i]);   /* the slot is about to be written */
    }
    /* one staging copy of [seq | slot | pos], each padded to max_batch */
    size_t mb = (size_t)ctx->cfg.max_batch;
    int *tmp = (int *)malloc(3 * mb * sizeof(int));
    if (!tmp) return hy3a_fail(ctx, HY3A_ENOMEM, "batch_set: malloc failed");
    memset(tmp, 0, 3 * mb * sizeof(int));
    memcpy(tmp, seq_ids, n * sizeof(int));
    memcpy(tmp + mb, slots, n * sizeof(int));
    memcpy(tmp + 2 * mb, rope_pos, n * sizeof(int));
    int rc = stage_h2d(ctx, ctx->d_batch, tmp, 3 * mb * sizeof(int));
    free(tmp);
    if (rc) return rc;
    ctx->batch_n = n;
    ctx->batch_seq0 = seq_ids[0]; ctx->batch_slot0 = slots[0]; ctx->batch_contig = slots[0] >= 0;
    for (int i = 1; i < n && ctx->batch_contig; i++) ctx->batch_contig = seq_ids[i] == seq_ids[0] && slots[i] == slots[0] + i;
    ctx->batch_seq_uniform = 1; ctx->batch_slot_min = slots[0] < 0 ? 0 : slots[0];
    for (int i = 1; i < n; i++) {
        if (seq_ids[i] != seq_ids[0]) ctx->batch_seq_uniform = 0;
        if (slots[i] >= 0 && slots[i] < ctx->batch_slot_min) ctx->batch_slot_min = slots[i];
    }
    return HY3A_OK;
}

/* ---- hot path wrappers --------------------------------------------------------------- */
static int check_layer(hy3a_ctx *ctx, int layer, const char *who) {
    if (!ctx) return HY3A_EINVAL;
    if (layer < 0 || layer >= ctx->cfg.n_layers) return hy3a_fail(ctx, HY3A_EINVAL, "%s: layer %d out of range [0,%d)", who, layer, ctx->cfg.n_layers);
    if (ctx->batch_n < 1) return hy3a_fail(ctx, HY3A_ESTATE, "%s: no batch set (call hy3a_batch_set first)", who);
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != ctx->device)
        return hy3a_fail(ctx, HY3A_ESTATE, "%s: the context lives on device %d but device %d is current (cudaSetDevice first)", who, ctx->device, cur);
    return 0;
}

int hy3a_append(hy3a_ctx *ctx, int layer, const float *q_in, size_t q_stride, const float *k_in, size_t k_stride, const float *v_in,
                size_t v_stride, float *q_out, size_t q_out_stride, void *q_out16) {
    int rc = check_layer(ctx, layer, "append");
    if (rc) return rc;
    if (!q_in || (!k_in) != (!v_in)) return hy3a_fail(ctx, HY3A_EINVAL, "append: NULL input (k_in and v_in may only be NULL together)");
    if (((uintptr_t)q_in | (uintptr_t)k_in | (uintptr_t)v_in | (uintptr_t)q_out | (uintptr_t)q_out16) & 15)
        return hy3a_fail(ctx, HY3A_EINVAL, "append: pointers must be 16-byte aligned");
    if ((q_stride | k_stride | v_stride | q_out_stride) & 3) return hy3a_fail(ctx, HY3A_EINVAL, "append: strides must be multiples of 4 floats");
    return hy3a_launch_append(ctx, layer, q_in, q_stride, k_in, k_stride, v_in, v_stride, q_out, q_out_stride, q_out16);
}

int hy3a_decode(hy3a_ctx *ctx, int layer, const float *q, size_t q_stride, float *out, size_t out_stride, float *partials) {
    int rc = check_layer(ctx, layer, "decode");
    if (rc) return rc;
    if (!q || (!out && !partials)) return hy3a_fail(ctx, HY3A_EINVAL, "decode: NULL argument");
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)partials) & 15) return hy3a_fail(ctx, HY3A_EINVAL, "decode: pointers must be 16-byte aligned");
    if ((q_stride | out_stride) & 3) return hy3a_fail(ctx, HY3A_EINVAL, "decode: strides must be multiples of 4 floats");
    return hy3a_launch_decode(ctx, layer, q, q_stride, out, out_stride, partials, NULL);
}

int hy3a_decode_step(hy3a_ctx *ctx, int layer, const float *q_in, size_t q_stride, const float *k_in, size_t k_stride, const float *v_in,
                     size_t v_stride, float *q_out, size_t q_out_stride, float *out, size_t out_stride, float *partials) {
    int rc = check_layer(ctx, layer, "decode_step");
    if (rc) return rc;
    if (!q_in || (!k_in) != (!v_in) || (!out && !partials)) return hy3a_fail(ctx, HY3A_EINVAL, "decode_step: NULL argument");
    if (((uintptr_t)q_in | (uintptr_t)k_in | (uintptr_t)v_in | (uintptr_t)q_out | (uintptr_t)out | (uintptr_t)partials) & 15)
        return hy3a_fail(ctx, HY3A_EINVAL, "decode_step: pointers must be 16-byte aligned");
    if ((q_stride | k_stride | v_stride | q_out_stride | out_stride) & 3) return hy3a_fail(ctx, HY3A_EINVAL, "decode_step: strides must be multiples of 4 floats");
    if (ctx->decode_stages < 2) {
        /* no shared-memory ring (tuning knob): run the two kernels one after the other */
        if (!q_out) return hy3a_fail(ctx, HY3A_EINVAL, "decode_step: q_out is required when the page ring is disabled");
        rc = hy3a_launch_append(ctx, layer, q_in, q_stride, k_in, k_stride, v_in, v_stride, q_out, q_out_stride, NULL);
        if (rc) return rc;
        return hy3a_launch_decode(ctx, layer, q_out, q_out_stride, out, out_stride, partials, NULL);
    }
    hy3a_step_inputs st;
    st.q_in = q_in; st.k_in = k_in; st.v_in = v_in; st.q_stride = q_stride; st.k_stride = k_stride; st.v_stride = v_stride;
    st.q_out = q_out; st.q_out_stride = q_out_stride;
    return hy3a_launch_decode(ctx, layer, NULL, 0, out, out_stride, partials, &st);
}

/* ---- sequence-shard exchange over peer memory ------------------------------------------------ */
int hy3a_shard_init(hy3a_ctx *ctx, int rank, int world, int n_slots, int n_rows, unsigned char *handle_out) {
    if (!ctx) return HY3A_EINVAL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || n_slots < 1 || n_rows < 1 || n_rows > ctx->cfg.max_batch || !handle_out)
        return hy3a_fail(ctx, HY3A_EINVAL, "shard_init: bad argument (rank %d of %d, %d slots, %d rows)", rank, world, n_slots, n_rows);
    if (ctx->shard_local) return hy3a_fail(ctx, HY3A_ESTATE, "shard_init: already initialised");
    const size_t n_seg = (size_t)n_rows * ctx->cfg.kv_head_count;
    const size_t slice = n_seg * 8 * (HY3A_PARTIAL_FLOATS / 2) * 16;    /* flagged 16-byte lines: 2 values each */
    ctx->shard_state_off = ((size_t)n_slots * world * slice + 255) & ~(size_t)255;
    ctx->shard_bytes = ctx->shard_state_off + (size_t)n_slots * n_seg * 8 * sizeof(unsigned);   /* use count per (slot, segment, head) */
    HY3A_CUDA(ctx, cudaMalloc(&ctx->shard_local, ctx->shard_bytes));
    HY3A_CUDA(ctx, cudaMemset(ctx->shard_local, 0, ctx->shard_bytes));
    cudaIpcMemHandle_t h;
    HY3A_CUDA(ctx, cudaIpcGetMemHandle(&h, ctx->shard_local));
    memcpy(handle_out, &h, sizeof(h));
    ctx->shard_rank = rank; ctx->shard_world = world; ctx->shard_slots = n_slots; ctx->shard_rows = n_rows;
    for (int r = 0; r < 8; r++) ctx->shard_peer[r] = NULL;
    ctx->shard_peer[rank] = ctx->shard_local;
    return HY3A_OK;
}

int hy3a_shard_connect(hy3a_ctx *ctx, const unsigned char *handles) {
    if (!ctx || !handles) return HY3A_EINVAL;
    if (!ctx->shard_local) return hy3a_fail(ctx, HY3A_ESTATE, "shard_connect: call hy3a_shard_init first");
    for (int r = 0; r < ctx->shard_world; r++) {
        if (r == ctx->shard_rank || ctx->shard_peer[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * sizeof(h), sizeof(h));
        void *p = NULL;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return hy3a_fail(ctx, HY3A_ECUDA, "shard_connect: cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e));
        ctx->shard_peer[r] = (unsigned char *)p;
    }
    return HY3A_OK;
}

int hy3a_shard_connect_local(hy3a_ctx *ctx) {
    if (!ctx) return HY3A_EINVAL;
    if (!ctx->shard_local) return hy3a_fail(ctx, HY3A_ESTATE, "shard_connect_local: call hy3a_shard_init first");
    for (int r = 0; r < ctx->shard_world; r++) {
        if (r == ctx->shard_rank || ctx->shard_peer[r]) continue;
        void *p = NULL;
        HY3A_CUDA(ctx, cudaMalloc(&p, ctx->shard_bytes));
        HY3A_CUDA(ctx, cudaMemset(p, 0, ctx->shard_bytes));
        ctx->shard_peer[r] = (unsigned char *)p;
        ctx->shard_standin |= 1 << r;
    }
    return HY3A_OK;
}

int hy3a_shard_disconnect(hy3a_ctx *ctx) {
    if (!ctx) return HY3A_EINVAL;
    for (int r = 0; r < ctx->shard_world; r++) {
        if (r == ctx->shard_rank || !ctx->shard_peer[r]) continue;
        if (ctx->shard_standin & (1 << r)) cudaFree(ctx->shard_peer[r]);
        else cudaIpcCloseMemHandle(ctx->shard_peer[r]);
        ctx->shard_peer[r] = NULL;
    }
    ctx->shard_standin = 0;
    return HY3A_OK;
}

int hy3a_decode_step_sharded(hy3a_ctx *ctx, int layer, int slot, const float *q_in, size_t q_stride, const float *k_in, size_t k_stride,
                             const float *v_in, size_t v_stride, float *out, size_t out_stride) {
    int rc = check_layer(ctx, layer, "decode_step_sharded");
    if (rc) return rc;
    if (!ctx->shard_local) return hy3a_fail(ctx, HY3A_ESTATE, "decode_step_sharded: call hy3a_shard_init / hy3a_shard_connect first");
    for (int r = 0; r < ctx->shard_world; r++) if (!ctx->shard_peer[r]) return hy3a_fail(ctx, HY3A_ESTATE, "decode_step_sharded: rank %d not connected", r);
    if (slot < 0 || slot >= ctx->shard_slots) return hy3a_fail(ctx, HY3A_EINVAL, "decode_step_sharded: slot %d out of range", slot);
    if (ctx->batch_n != ctx->shard_rows) return hy3a_fail(ctx, HY3A_EINVAL, "decode_step_sharded: batch has %d rows, the exchange was set up for %d", ctx->batch_n, ctx->shard_rows);
    if (!q_in || !out || (!k_in) != (!v_in)) return hy3a_fail(ctx, HY3A_EINVAL, "decode_step_sharded: NULL argument");
    if (((uintptr_t)q_in | (uintptr_t)k_in | (uintptr_t)v_in | (uintptr_t)out) & 15 || ((q_stride | k_stride | v_stride | out_stride) & 3))
        return hy3a_fail(ctx, HY3A_EINVAL, "decode_step_sharded: pointers must be 16-byte aligned, strides multiples of 4");
    if (ctx->decode_stages < 2) return hy3a_fail(ctx, HY3A_ESTATE, "decode_step_sharded: needs the page ring (HY3A_DECODE_STAGES >= 2)");
    hy3a_step_inputs st;
    st.q_in = q_in; st.k_in = k_in; st.v_in = v_in; st.q_stride = q_stride; st.k_stride = k_stride; st.v_stride = v_stride;
    st.q_out = NULL; st.q_out_stride = 0;
    ctx->shard_slot = slot;
    rc = hy3a_launch_decode(ctx, layer, NULL, 0, out, out_stride, NULL, &st);
    ctx->shard_slot = -1;
    return rc;
}

int hy3a_merge_partials(hy3a_ctx *ctx, const float *partials, int n_parts, int n_rows, int n_heads, float *out, size_t out_stride) {
    if (!ctx) return HY3A_EINVAL;
    if (!partials || !out || n_parts < 1 || n_rows < 1 || n_heads < 1) return hy3a_fail(ctx, HY3A_EINVAL, "merge_partials: bad argument");
    if (((uintptr_t)out & 15) || (out_stride & 3)) return hy3a_fail(ctx, HY3A_EINVAL, "merge_partials: out must be 16-byte aligned");
    return hy3a_launch_merge(ctx, partials, n_parts, n_rows, n_heads, out, out_stride);
}

int hy3a_prefill(hy3a_ctx *ctx, int layer, int seq, int base_slot, int nq, const void *q16, float *out, size_t out_stride) {
    if (!ctx) return HY3A_EINVAL;
    if (layer < 0 || layer >= ctx->cfg.n_layers) return hy3a_fail(ctx, HY3A_EINVAL, "prefill: layer %d out of range", layer);
    if (seq < 0 || seq >= ctx->cfg.max_seqs) return hy3a_fail(ctx, HY3A_EINVAL, "prefill: seq %d out of range", seq);
    if (base_slot < 0 || nq < 1) return hy3a_fail(ctx, HY3A_EINVAL, "prefill: base_slot=%d nq=%d", base_slot, nq);
    if (base_slot + nq > ctx->h_seq_blocks[seq] * HY3A_PAGE_TOKENS) return hy3a_fail(ctx, HY3A_ESTATE, "prefill: keys [0,%d) are not all appended", base_slot + nq);
    if (!q16 || !out || (((uintptr_t)q16 | (uintptr_t)out) & 15) || (out_stride & 3)) return hy3a_fail(ctx, HY3A_EINVAL, "prefill: bad pointer");
    return hy3a_launch_prefill(ctx, layer, seq, base_slot, nq, q16, out, out_stride);
}

/* ---- import / export ------------------------------------------------------------------ */
static int xport(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint8_t *k_slots, uint8_t *v_slots, int import) {
    if (!ctx) return HY3A_EINVAL;
    if (layer < 0 || layer >= ctx->cfg.n_layers || seq < 0 || seq >= ctx->cfg.max_seqs || t0 < 0 || n < 1 || !k_slots || !v_slots)
        return hy3a_fail(ctx, HY3A_EINVAL, "%s: bad argument", import ? "import_kv" : "export_kv");
    if (import) { int rc = hy3a_seq_reserve(ctx, seq, t0 + n); if (rc) return rc; hy3a_mirror_truncate(ctx, seq, layer, t0); }
    else if (t0 + n > ctx->h_seq_blocks[seq] * HY3A_PAGE_TOKENS) return hy3a_fail(ctx, HY3A_EINVAL, "export_kv: tokens [%d,%d) not mapped", t0, t0 + n);
    size_t bytes = (size_t)n * hy3a_slot_bytes(ctx->cfg.kv_dtype);
    uint8_t *dk = NULL, *dv = NULL;
    HY3A_CUDA(ctx, cudaMalloc(&dk, bytes));
    if (cudaMalloc(&dv, bytes) != cudaSuccess) { cudaFree(dk); return hy3a_fail(ctx, HY3A_ENOMEM, "xport: cudaMalloc failed"); }
    int rc = HY3A_OK;
    cudaError_t e = cudaSuccess;
    if (import) {
        e = cudaMemcpyAsync(dk, k_slots, bytes, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dv, v_slots, bytes, cudaMemcpyHostToDevice, ctx->stream);
    }
    if (e == cudaSuccess) rc = hy3a_launch_export(ctx, layer, seq, t0, n, dk, dv, import);
    if (e == cudaSuccess && rc == HY3A_OK && !import) {
        e = cudaMemcpyAsync(k_slots, dk, bytes, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(v_slots, dv, bytes, cudaMemcpyDeviceToHost, ctx->stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(dk); cudaFree(dv);
    if (e != cudaSuccess) return hy3a_fail(ctx, HY3A_ECUDA, "xport: %s", cudaGetErrorString(e));
    return rc;
}
int hy3a_export_kv(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint8_t *k_slots, uint8_t *v_slots) { return xport(ctx, layer, seq, t0, n, k_slots, v_slots, 0); }
int hy3a_import_kv(hy3a_ctx *ctx, int layer, int seq, int t0, int n, const uint8_t *k_slots, const uint8_t *v_slots) {
    return xport(ctx, layer, seq, t0, n, (uint8_t *)k_slots, (uint8_t *)v_slots, 1);
}

int hy3a_fill_random(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint64_t seed) {
    if (!ctx) return HY3A_EINVAL;
    if (layer < 0 || layer >= ctx->cfg.n_layers || seq < 0 || seq >= ctx->cfg.max_seqs || t0 < 0 || n < 1) return hy3a_fail(ctx, HY3A_EINVAL, "fill_random: bad argument");
    int rc = hy3a_seq_reserve(ctx, seq, t0 + n);
    if (rc) return rc;
    hy3a_mirror_truncate(ctx, seq, layer, t0);
    return hy3a_launch_fill_random(ctx, layer, seq, t0, n, seed);
}

uint64_t hy3a_launch_count(const hy3a_ctx *ctx) { return ctx ? ctx->launches : 0; }

} /* extern "C" */
