/*
 * hy3_gpu_dropin.h -- the reference engine's CUDA backend API, implemented on the B200 attention library
 * (hy3_attn.h).  Include the engine's own hy3.h first: the model and token types are its types, nothing of
 * them is restated here.  The object that defines these symbols is linked into the engine in place of the
 * object built from its hy3_gpu.cu; hy3.c and hy3_cli.c need no change.
 */
#ifndef HY3_GPU_DROPIN_H
#define HY3_GPU_DROPIN_H

#ifndef HY3_H
#error "include the engine's hy3.h before hy3_gpu_dropin.h"
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Replaces hy3_gpu_init (hy3_gpu.cu:544-630; declared in hy3_gpu.h:6, called from hy3_cli.c:280): uploads the
 * weights of the first n_gpu_layers layers (<= 0 or > 81: all), reads HY3_KV_INT4 / HY3_KV_FP16 / HY3_KV_TOKENS /
 * HY3_PREFILL_CHUNK / HY3_POS_STRIDE / HY3_POS_JUMP[_AT] once, creates the paged KV cache, stores the context in
 * m->gpu_ctx and prints "hy3_gpu: initialized (N layers, INT8|INT4|FP16 KV, online attn)".  0, or -1 with a
 * message on stderr; never exits.                                                                          */
int hy3_gpu_init(hy3_model *m, int n_gpu_layers);

/* Replaces hy3_gpu_free (hy3_gpu.cu:632-642; called from hy3_model_free, hy3.c:926-929). */
void hy3_gpu_free(hy3_model *m);

/* Replaces hy3_eval_gpu (hy3_gpu.cu:844-961; declared in hy3.h:79, called from hy3_eval, hy3.c:1370): feeds
 * tokens->v[0 .. len) as positions m->cache_len / 80 ..., appends their K/V, writes the logits of the LAST token
 * to `logits` (host memory), advances m->cache_len by 80 per token and stores it in *pos.  cache_len belongs to
 * the caller, who may set it back between calls (prefix reuse, hy3.c:1514; reset, hy3.c:960); K/V below it
 * persist.  0, or -1 with a message on stderr.  One calling thread per model.                               */
int hy3_eval_gpu(hy3_model *m, const hy3_tokens *tokens, float *logits, int *pos);

/* The name hy3_gpu.h:8 declares for the same function. */
int hy3_gpu_eval(hy3_model *m, const hy3_tokens *tokens, float *logits, int *pos);

/* Message of the last failure of this model's backend ("" if none).  No counterpart in the reference, which
 * exits on errors (hy3_gpu.cu:17-20). */
const char *hy3_gpu_last_error(const hy3_model *m);

#ifdef __cplusplus
}
#endif
#endif /* HY3_GPU_DROPIN_H */
