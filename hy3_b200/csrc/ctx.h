/* ctx.h -- the context object behind the C ABI, and the parameter blocks of the kernels. */
#ifndef HY3A_CTX_H
#define HY3A_CTX_H

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hy3_attn.h"
#include "layout.h"

#define HY3A_MAX_LAYERS 128
#ifndef HY3A_DECODE_WARPS
#define HY3A_DECODE_WARPS 11
#endif
#ifndef HY3A_UMMA_STAGES
#define HY3A_UMMA_STAGES 6    /* pages in the shared-memory ring of the INT8 decode kernel */
#endif
#define HY3A_ERR_WORDS 4
#define HY3A_REC_FLOATS 132   /* a head's {m, l, acc[128]} record in the merge scratch, padded to a multiple of 16 bytes */
#define HY3A_RING_SLOTS 16

/* Everything a kernel needs to address the cache; passed by value. */
struct hy3a_cache_view {
    uint8_t *pool;           /* base of the block pool */
    const int *block_table;  /* [max_seqs][max_blocks_per_seq] */
    int max_blocks_per_seq;
    int n_layers;
    int kv_heads;            /* owned KV heads */
    int kv_head_begin;
    int page_bytes;
    unsigned int *vs_max;    /* [n_layers][kv_heads] running max of V scale bits (fp16 as uint) */
};

__host__ __device__ __forceinline__ size_t hy3a_page_index(const hy3a_cache_view &c, int block, int layer, int head_local) {
    return ((size_t)block * c.n_layers + layer) * c.kv_heads + head_local;
}

/* Per-step batch descriptor, device resident (struct of arrays in one allocation). */
struct hy3a_batch_view {
    const int *seq;   /* [n] */
    const int *slot;  /* [n] */
    const int *pos;   /* [n] */
    int n;
};

struct hy3a_rope_params {
    const float *inv_freq; /* device float[64] */
    float attn_factor;
    int pos_stride, pos_jump, pos_jump_at;
};

struct hy3a_ctx {
    hy3a_config cfg;
    hy3a_geom geom;
    int device;
    int sm_count;
    cudaStream_t stream;
    int own_stream;

    /* device memory */
    uint8_t *pool;
    size_t pool_bytes;
    int *d_block_table;
    unsigned int *d_vs_max;
    float *d_inv_freq;
    float *d_norm_w;      /* [n_layers][2][128] */
    int *d_batch;         /* [3][max_batch] seq, slot, pos */
    float *d_partials;    /* decode scratch: [(ctas + max_batch*kv_heads)][8][HY3A_REC_FLOATS] */
    unsigned int *d_counters; /* decode scratch: [2][max_batch*kv_heads] arrival / finished-fold counters (self-resetting) */
    void *d_pf_k, *d_pf_v; /* prefill: fp16 operands shared by all layers, rebuilt per call (used when a layer has no mirror) */
    size_t pf_bytes;
    /* prefill operand mirrors: per layer, the fp16 tensor-core image (K rows, V transposed) of ONE sequence's tokens
     * [0, pf_mntok[layer]), kept across chunks so that a chunk only converts the pages it appended.  Any call that
     * can write a slot below pf_mntok (batch_set rows, import, fill, release) lowers pf_mntok first. */
    void *pf_mk[HY3A_MAX_LAYERS], *pf_mv[HY3A_MAX_LAYERS];
    int pf_mcap[HY3A_MAX_LAYERS];   /* tokens of capacity (multiple of 1024) */
    int pf_mntok[HY3A_MAX_LAYERS];  /* tokens converted and still valid */
    int pf_mseq;                    /* the sequence all mirrors belong to, -1 = none */
    size_t pf_mbytes, pf_mbudget;   /* allocated / allowed bytes of mirrors (HY3A_PF_MIRROR_MB, 0 = no mirrors) */
    unsigned int *d_err;  /* HY3A_ERR_WORDS words: kernels record bounded-wait timeouts / bad indices here */
    size_t partial_records;

    /* host mirrors */
    int *h_block_table;   /* [max_seqs][max_blocks_per_seq], -1 = unmapped */
    int *h_seq_blocks;    /* [max_seqs] mapped block count */
    int *h_free;          /* free-list stack */
    int n_free;
    char *h_ring;         /* pinned staging ring for small host->device copies */
    size_t ring_slot_bytes;
    cudaEvent_t ring_ev[HY3A_RING_SLOTS];
    int ring_used[HY3A_RING_SLOTS];
    int ring_next;
    unsigned int *h_err;  /* pinned */
    int batch_n;
    int batch_contig, batch_seq0, batch_slot0;   /* the batch is rows slot0, slot0+1, ... of one sequence (a prefill chunk) */
    int batch_seq_uniform, batch_slot_min;       /* all rows belong to batch_seq0; lowest slot >= 0 of the batch */
    int decode_ctas;
    int bulk_write_pending; /* a kernel that wrote many KV slots was enqueued and no decode launch has followed it yet */
    int use_pdl;          /* launch kernels with programmatic stream serialization (HY3A_NO_PDL=1 turns it off) */
    int decode_stages;    /* pages in the decode kernel's shared-memory ring; < 2 selects the direct-load variant */

    /* sequence-shard exchange over peer memory (hy3a_shard_*): one allocation per rank =
     * [n_slots][world][rows*heads][65] flagged 16-byte lines {value, flag, value, flag} of gathered records,
     * then one use count per (slot, row, KV head) */
    unsigned char *shard_local;
    unsigned char *shard_peer[8];     /* every rank's allocation as mapped into this process ([rank] = shard_local) */
    size_t shard_state_off, shard_bytes;
    int shard_rank, shard_world, shard_slots, shard_rows;
    int shard_standin;                /* bit r: shard_peer[r] is a stand-in allocated by this process */
    int shard_slot;                   /* >= 0 while hy3a_decode_step_sharded is launching */

    hy3a_rope_params rope;
    uint64_t launches;
    char err[512];
};

/* internal kernel launchers (defined in the .cu files) */
int hy3a_launch_append(hy3a_ctx *ctx, int layer, const float *q_in, size_t q_stride, const float *k_in, size_t k_stride,
                       const float *v_in, size_t v_stride, float *q_out, size_t q_out_stride, void *q_out16);
/* inputs of the fused step (pre-norm rows of the new token per batch row); NULL = plain decode */
struct hy3a_step_inputs {
    const float *q_in, *k_in, *v_in;
    size_t q_stride, k_stride, v_stride;
    float *q_out;
    size_t q_out_stride;
};
int hy3a_launch_decode(hy3a_ctx *ctx, int layer, const float *q, size_t q_stride, float *out, size_t out_stride,
                       float *partials, const hy3a_step_inputs *step);
int hy3a_launch_merge(hy3a_ctx *ctx, const float *partials, int n_parts, int n_rows, int n_heads, float *out,
                      size_t out_stride);
int hy3a_launch_export(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint8_t *d_kslots, uint8_t *d_vslots, int import);
int hy3a_launch_fill_random(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint64_t seed);
int hy3a_launch_prefill(hy3a_ctx *ctx, int layer, int seq, int base_slot, int nq, const void *q16, float *out,
                        size_t out_stride);
int hy3a_launch_init_pages(hy3a_ctx *ctx, size_t first_page, size_t n_pages);
int hy3a_decode_ring_capacity(int page_bytes, int max_batch);
int hy3a_decode_max_ctas(void);
int hy3a_fail(hy3a_ctx *ctx, int code, const char *fmt, ...);

/* slots >= ntok of sequence seq (all layers, or one layer if layer >= 0) are about to be rewritten or dropped */
static inline void hy3a_mirror_truncate(hy3a_ctx *c, int seq, int layer, int ntok) {
    if (seq != c->pf_mseq) return;
    if (ntok < 0) ntok = 0;
    if (layer >= 0) { if (c->pf_mntok[layer] > ntok) c->pf_mntok[layer] = ntok; return; }
    for (int l = 0; l < c->cfg.n_layers; l++) if (c->pf_mntok[l] > ntok) c->pf_mntok[l] = ntok;
}

static inline hy3a_cache_view hy3a_view(const hy3a_ctx *c) {
    hy3a_cache_view v;
    v.pool = c->pool; v.block_table = c->d_block_table; v.max_blocks_per_seq = c->cfg.max_blocks_per_seq;
    v.n_layers = c->cfg.n_layers; v.kv_heads = c->cfg.kv_head_count; v.kv_head_begin = c->cfg.kv_head_begin;
    v.page_bytes = c->geom.page_bytes; v.vs_max = c->d_vs_max;
    return v;
}
static inline hy3a_batch_view hy3a_bview(const hy3a_ctx *c) {
    hy3a_batch_view b;
    b.seq = c->d_batch; b.slot = c->d_batch + c->cfg.max_batch; b.pos = c->d_batch + 2 * c->cfg.max_batch; b.n = c->batch_n;
    return b;
}

#define HY3A_CUDA(ctx, call)                                                                                   \
    do {                                                                                                       \
        cudaError_t e_ = (call);                                                                               \
        if (e_ != cudaSuccess) return hy3a_fail((ctx), HY3A_ECUDA, "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

#endif
