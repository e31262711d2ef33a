/*
 * hy3_attn.h -- C ABI of the B200 (sm_100a) attention path for the Hy3 architecture.
 *
 * GQA, 64 query heads over 8 KV heads, head_dim 128, per-head QK RMSNorm, rotate_half
 * RoPE (theta 11158840, YaRN optional), FP16 / INT8 / INT4 KV caches.
 *
 * This is the layer that the reference engine's CUDA backend implements inline in
 * hy3_gpu.cu between its QKV projection and its O projection; every entry point
 * below names the reference code it replaces.  The three symbols of the reference's
 * own backend API (hy3_gpu_init / hy3_gpu_free / hy3_eval_gpu) are declared in
 * hy3_gpu_dropin.h and are implemented on top of this ABI.
 *
 * Conventions
 *   - All functions return 0 on success and a negative HY3A_E* code on failure; they
 *     never call exit().  hy3a_last_error() returns a human-readable message.
 *   - Unless stated otherwise, data pointers are DEVICE pointers (plain void* / float*),
 *     sizes and strides are in elements, and all work is enqueued on the context's
 *     stream (hy3a_set_stream) without synchronising.
 *   - One host thread per context.  A context is bound to one CUDA device.
 *   - q rows are [64][128] fp32 (query heads of all KV groups, head-major); k and v rows
 *     are [8][128] fp32.  With KV-head sharding (kv_head_count < 8) the context still
 *     takes full rows and only touches the heads it owns.
 */
#ifndef HY3_ATTN_H
#define HY3_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HY3A_N_HEAD 64
#define HY3A_N_KV_HEAD 8
#define HY3A_HEAD_DIM 128
#define HY3A_GROUP 8           /* query heads per KV head */
#define HY3A_PAGE_TOKENS 128   /* tokens per KV page */
#define HY3A_PARTIAL_FLOATS 130 /* {m, l, acc[128]} -- the record of hy3_gpu.cu:183-230 */

enum { HY3A_KV_FP16 = 0, HY3A_KV_INT8 = 1, HY3A_KV_INT4 = 2 };

enum {
    HY3A_OK = 0,
    HY3A_EINVAL = -1,   /* bad argument */
    HY3A_ENOMEM = -2,   /* host or device allocation failed / KV pool exhausted */
    HY3A_ECUDA = -3,    /* a CUDA call or kernel launch failed */
    HY3A_EDEVICE = -4,  /* device is not compute capability 10.0 (sm_100a code cannot run) */
    HY3A_ESTATE = -5,   /* call sequence error (e.g. no batch set) */
    HY3A_ETIMEOUT = -6  /* a bounded device-side wait ran out; the kernel returned early */
};

typedef struct hy3a_ctx hy3a_ctx;

typedef struct {
    int kv_dtype;           /* HY3A_KV_*; reference: HY3_KV_INT4 env, hy3_gpu.cu:598 (FP16: hy3.metal:285) */
    int n_layers;           /* layers that own a cache (80 in the model, hy3.h:32) */
    int kv_head_begin;      /* first KV head owned by this context (KV-head sharding); 0 */
    int kv_head_count;      /* KV heads owned; 8 when unsharded */
    int max_seqs;           /* sequences that can hold KV at once (1 for the reference's loop) */
    int max_batch;          /* rows per hy3a_batch_set (decode batch or prefill chunk) */
    int max_blocks;         /* pool capacity in 128-token blocks (a block spans all layers and owned heads) */
    int max_blocks_per_seq; /* longest sequence, in blocks */
    int device;             /* CUDA device ordinal, -1 = current device */
    float rms_eps;          /* QK RMSNorm epsilon; the reference uses 1e-5 (hy3.c:25, hy3_gpu.cu:158) */
} hy3a_config;

/* Fill *cfg with the reference's behaviour: INT8 KV, 80 layers, all 8 KV heads, one
 * sequence, room for 8192 tokens (hy3_gpu.cu:607), eps 1e-5.                          */
void hy3a_default_config(hy3a_config *cfg);

/* Replaces the KV / scratch part of hy3_gpu_init (hy3_gpu.cu:598-627).  Refuses devices
 * whose compute capability is not 10.0 and runs a known-answer self-test of the decode
 * path before returning (the reference never checks a launch, hy3_gpu.cu:750-758).     */
int hy3a_create(const hy3a_config *cfg, hy3a_ctx **out);
/* Replaces the KV part of hy3_gpu_free (hy3_gpu.cu:632-642). */
void hy3a_destroy(hy3a_ctx *ctx);
/* Message of the last failure on ctx (or of the last failed hy3a_create when ctx is NULL). */
const char *hy3a_last_error(const hy3a_ctx *ctx);
/* Bytes of device memory one 128-token block occupies for this configuration. */
size_t hy3a_block_bytes(const hy3a_config *cfg);

/* Work is enqueued on this cudaStream_t (default: a stream the context owns). */
int hy3a_set_stream(hy3a_ctx *ctx, void *cuda_stream);
void *hy3a_get_stream(hy3a_ctx *ctx);
/* cudaStreamSynchronize on the context stream + read of the device error word. */
int hy3a_sync(hy3a_ctx *ctx);

/* RoPE table and position probes.  Replaces the hy3_rope_get_params upload and the
 * HY3_POS_* fields (hy3_gpu.cu:602-606, :625-627).  inv_freq: HOST float[64].          */
int hy3a_set_rope(hy3a_ctx *ctx, const float *inv_freq, float attn_factor, int pos_stride, int pos_jump,
                  int pos_jump_at);
/* Per-layer QK-norm weights, HOST float[128] each (attn_q_norm / attn_k_norm uploads,
 * hy3_gpu.cu:568-569).  Layers never set use all-ones.                                 */
int hy3a_set_norm_weights(hy3a_ctx *ctx, int layer, const float *q_weight, const float *k_weight);

/* ---- sequences and capacity (host side) -------------------------------------------
 * Replaces gpu_ensure_kv_capacity (hy3_gpu.cu:692-698): growth allocates pool blocks,
 * nothing is copied and no pointer a captured graph holds ever changes.               */
int hy3a_seq_reserve(hy3a_ctx *ctx, int seq, int ntok);  /* make slots [0, ntok) addressable */
int hy3a_seq_release(hy3a_ctx *ctx, int seq, int keep_ntok); /* give back blocks past keep_ntok */
int hy3a_seq_capacity(hy3a_ctx *ctx, int seq);           /* addressable slots */
int hy3a_free_blocks(hy3a_ctx *ctx);

/* ---- the per-step batch descriptor -------------------------------------------------
 * Row i of the next append / decode calls belongs to sequence seq_ids[i], writes KV slot
 * slots[i] (local token index in that sequence's cache) and is rotated with RoPE
 * position rope_pos[i] (global token index; differs from the slot under sequence
 * sharding).  After the append the row attends keys [0, slots[i]].  HOST int arrays.
 * Replaces the h_pos -> d_pos hand-off (hy3_gpu.cu:872-873) and iota_kernel (:364);
 * like there, the position is supplied by the caller on every call -- the context keeps
 * no private counter, so rolling back (hy3.c:1514) is just passing smaller positions.
 * Reserves capacity for the slots.                                                    */
int hy3a_batch_set(hy3a_ctx *ctx, int n, const int *seq_ids, const int *slots, const int *rope_pos);

/* ---- hot path ----------------------------------------------------------------------*/

/* Fused per-head QK RMSNorm + RoPE + KV quantise + append for the n rows of the current
 * batch.  Replaces qk_norm_rope_fused_kernel + kv_quantize_int8/int4_kernel
 * (hy3_gpu.cu:144, :250, :329) and their per-token launch loop (:823-829).
 * q_in/k_in/v_in: fp32 rows with the given row strides (floats) -- the reference keeps
 * them inside one 10240-float QKV row (hy3_gpu.cu:748).  q_out: normalised + rotated
 * queries, fp32 [n][64][128] with row stride q_out_stride (may alias q_in; may be NULL
 * when only q_out16 is wanted, as in a prefill chunk); q_out16 (optional, may be NULL):
 * the same values as IEEE fp16 [n][64][128] dense, the operand format of hy3a_prefill.  k_in and v_in may both be NULL: only the queries are
 * normalised and rotated and nothing is stored (a rank that does not own the tail of a
 * sequence-sharded cache still needs the rotated query).                               */
int hy3a_append(hy3a_ctx *ctx, int layer, const float *q_in, size_t q_stride, const float *k_in, size_t k_stride,
                const float *v_in, size_t v_stride, float *q_out, size_t q_out_stride, void *q_out16);

/* Split-KV GQA decode attention for the n rows of the current batch: row i attends keys
 * [0, slots[i]] of its sequence.  Replaces attention_split_kv[_int4]_kernel +
 * attention_reduce_kernel (hy3_gpu.cu:183, :274, :233) and the split heuristic / graph
 * recapture coupling (:766-789): lengths are read from device memory, one launch shape
 * serves every length.  q: fp32 [n][64][128] (row stride q_stride), out the same shape
 * (row stride out_stride).  Only the owned KV groups' 8*kv_head_count heads are written.
 * partials (optional, may be NULL): instead of normalised outputs, write one
 * unnormalised {m, l, acc[128]} record per owned head, [n][8*kv_head_count][130] fp32,
 * for a cross-GPU merge (sequence sharding).                                          */
int hy3a_decode(hy3a_ctx *ctx, int layer, const float *q, size_t q_stride, float *out, size_t out_stride,
                float *partials);

/* The decode step as ONE kernel: hy3a_append (for one new token per batch row) fused into
 * hy3a_decode.  Replaces the four launches per layer of the reference's decode loop --
 * qk_norm_rope_fused_kernel, kv_quantize_*, attention_split_kv_*, attention_reduce_kernel
 * (hy3_gpu.cu:750-758).  q_in/k_in/v_in: pre-norm fp32 rows of the new token as for
 * hy3a_append (k_in and v_in may both be NULL: nothing is appended, see there); q_out
 * (optional): the normalised + rotated queries; out / partials as for hy3a_decode.  Each
 * CTA normalises and rotates the 8 queries of its KV head itself; the one CTA that streams
 * the page holding the newest slot quantises and stores the new K / V row (bit-identical to
 * hy3a_append) and attends over it from shared memory.                                   */
int hy3a_decode_step(hy3a_ctx *ctx, int layer, const float *q_in, size_t q_stride, const float *k_in, size_t k_stride,
                     const float *v_in, size_t v_stride, float *q_out, size_t q_out_stride, float *out, size_t out_stride,
                     float *partials);

/* hy3a_decode for callers that must not allocate.  (No counterpart in the reference: this entry
 * point exists only in this library.)  Some callers cannot tolerate a device allocation on the
 * decode path -- code that runs while the rest of the process has the allocator locked or has
 * handed all free memory to another pool, or that may not take the implicit device-wide
 * synchronisation an allocation or free can cause.  hy3a_decode itself never allocates either,
 * but it leans on scratch buffers that hy3a_create allocated; this variant keeps the scratch of
 * the cross-CTA merge (the {m, l, acc} records and their arrival counters) in a fixed array that
 * is part of the library image, so it works on a context whatever happened to those buffers and
 * never calls cudaMalloc, cudaFree or any allocating routine.  Same arguments and results as
 * hy3a_decode without `partials`.
 * Limits: at most 64 (batch row, owned KV head) pairs per call, i.e. 8 rows with all 8 KV heads;
 * larger batches are refused with HY3A_EINVAL.  The array (2.4 MB) is held by every GPU that
 * loads the library until the process exits.  The first call on a device looks the array's
 * device address up (cudaGetSymbolAddress) -- make that first call outside any stream capture.
 * All contexts on a device share the array, and it keeps the last call's contents (the counters
 * are cleared at each call): calls that can overlap on the GPU -- different streams, or different
 * contexts -- race with each other; serialise them.                                          */
int hy3a_decode_noalloc(hy3a_ctx *ctx, int layer, const float *q, size_t q_stride, float *out, size_t out_stride);

/* Merge n_parts partial records per head in index order with the online-softmax rule of
 * attention_reduce_kernel (hy3_gpu.cu:233-247).  partials: [n_parts][n_rows*n_heads][130]
 * (the layout an all-gather of hy3a_decode partials produces), out: [n_rows][out_stride]
 * with head h at out + h*128.                                                         */
int hy3a_merge_partials(hy3a_ctx *ctx, const float *partials, int n_parts, int n_rows, int n_heads, float *out,
                        size_t out_stride);

/* ---- sequence sharding with the exchange fused into the decode kernel (peer memory over NVLink) ----
 * New functionality (the reference is single-GPU).  Rank r of `world` processes (one per GPU of one
 * box, world <= 8) holds a contiguous token range of every sequence.  hy3a_shard_init allocates this
 * rank's gather buffer ([n_slots][world][n_rows*heads] records of 65 flagged 16-byte lines) and returns its 64-byte CUDA IPC handle; the caller exchanges the handles (any
 * transport) and passes all of them, in rank order, to hy3a_shard_connect.
 *
 * hy3a_decode_step_sharded is hy3a_decode_step over this rank's tokens (k_in = v_in = NULL on ranks that
 * do not own the tail of the sequences) whose epilogue IS the collective: the CTA that completes a
 * (row, KV head) stores the rank's {m, l, acc} records straight into every other rank's gather buffer
 * through the peer mappings, as 16-byte lines that carry their own validity flag (no fence, no separate
 * signal), polls the lines the other ranks store into its own buffer, folds all records in rank order
 * (identical bits on all ranks) and writes the final attention output -- one launch per layer, no
 * second kernel, no NCCL call.  The
 * wait is bounded (about one second; hy3a_sync then reports HY3A_ETIMEOUT and the context stays usable).
 * All ranks must launch the same (layer, slot) sequence.  A slot may be reused once every rank has
 * finished the call that used it: two slots suffice when layer l+1's query depends on layer l's output;
 * callers that run independent layers back to back use one slot per layer.
 * hy3a_shard_connect_local replaces the missing ranks by silent stand-in buffers in this process (for
 * bring-up and for testing the bounded wait on one GPU: with world > 1 every wait runs out).
 * Teardown: every rank calls hy3a_shard_disconnect (unmaps the peers' buffers; enqueues nothing), the
 * ranks meet at a barrier of their own, then hy3a_destroy frees the local buffer.                     */
int hy3a_shard_init(hy3a_ctx *ctx, int rank, int world, int n_slots, int n_rows, unsigned char *handle_out /*[64]*/);
int hy3a_shard_connect(hy3a_ctx *ctx, const unsigned char *handles /*[world][64]*/);
int hy3a_shard_connect_local(hy3a_ctx *ctx);
int hy3a_shard_disconnect(hy3a_ctx *ctx);
int hy3a_decode_step_sharded(hy3a_ctx *ctx, int layer, int slot, const float *q_in, size_t q_stride, const float *k_in,
                             size_t k_stride, const float *v_in, size_t v_stride, float *out, size_t out_stride);

/* Causal chunk attention on tcgen05 tensor cores: query i (global index base_slot + i)
 * of sequence seq attends keys [0, base_slot + i]; the chunk's own K/V must already have
 * been appended (the reference does the same, hy3_gpu.cu:823-832).  Replaces
 * prefill_attn_int8/int4_kernel (hy3_gpu.cu:383, :415).  q16: IEEE fp16 [nq][64][128]
 * dense (hy3a_append's q_out16); out: fp32 [nq][64][128] with row stride out_stride.   */
int hy3a_prefill(hy3a_ctx *ctx, int layer, int seq, int base_slot, int nq, const void *q16, float *out,
                 size_t out_stride);

/* ---- cache import / export (parity and benchmarks) ---------------------------------
 * Export n tokens starting at slot t0 of (layer, seq) in the REFERENCE's slot format,
 * one slot per token: INT8 1040 B = [8 x fp16 scale][8 x 128 int8] (hy3_gpu.cu:26-29),
 * INT4 528 B = [8 x fp16][8 x 64 B] (:30-35), FP16 2048 B = [8 x 128 half]
 * (hy3.metal:285-297).  Heads this context does not own are zero.  HOST buffers;
 * synchronises.                                                                       */
int hy3a_export_kv(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint8_t *k_slots, uint8_t *v_slots);
/* Inverse of export: load n tokens of already-quantised data.  HOST buffers. */
int hy3a_import_kv(hy3a_ctx *ctx, int layer, int seq, int t0, int n, const uint8_t *k_slots, const uint8_t *v_slots);
/* Bytes per token of the slot format above for a KV dtype. */
int hy3a_slot_bytes(int kv_dtype);
/* Fill slots [t0, t0+n) of (layer, seq) on the device with seeded N(0,1) K and V passed
 * through this cache's quantiser (benchmark set-up; no host traffic).                 */
int hy3a_fill_random(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint64_t seed);

/* ---- introspection ------------------------------------------------------------------*/
/* Number of kernels this library has launched on ctx since creation. */
uint64_t hy3a_launch_count(const hy3a_ctx *ctx);
/* Decode schedule for a batch (pure host arithmetic, no GPU): given n lengths, the number
 * of page units, and for CTA `cta` of `n_ctas` its unit range [*u0, *u1).               */
int hy3a_decode_schedule(int n, const int *kv_lens, int kv_heads, int n_ctas, int cta, long long *total_units,
                         long long *u0, long long *u1);
/* Library build info, e.g. "hy3attn sm_100a <date>". */
const char *hy3a_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HY3_ATTN_H */
