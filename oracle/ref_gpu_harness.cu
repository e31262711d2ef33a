/*
 * ref_gpu_harness.cu -- exported wrappers around the REFERENCE's own CUDA kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  This translation unit textually includes the
 * reference engine's hy3_gpu.cu from where it lies (-DHY3_REF_GPU_SRC=...) so its
 * attention kernels can be launched unmodified on synthetic inputs:
 *   qk_norm_rope_fused_kernel (hy3_gpu.cu:144), kv_quantize_int8/int4_kernel
 *   (:250/:329), attention_split_kv[_int4]_kernel (:183/:274),
 *   attention_reduce_kernel (:233), prefill_attn_int8/int4_kernel (:383/:415).
 * It is built with the reference's own architecture flags (plain sm_100) into
 * oracle/_ref/ and is used (a) to pin the quantiser codes/scales bit-for-bit and
 * (b) as a speed comparison point.  No reference source is copied.
 *
 * All entry points take HOST pointers, allocate what they need, and return 0 or a
 * negative/CUDA error code; they never exit().
 */
#ifndef HY3_REF_GPU_SRC
#error "compile with -DHY3_REF_GPU_SRC=\"/path/to/reference/hy3_gpu.cu\""
#endif
#include HY3_REF_GPU_SRC

#define RCHK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "hy3refgpu: %s (%s:%d)\n", cudaGetErrorString(e_), __FILE__, __LINE__); return -(int)e_; } } while (0)

extern "C" {

/* Fused per-head RMSNorm (eps fixed at 1e-5 by the kernel) + RoPE, in place on
 * q [64*128] and k [8*128].                                                      */
int hy3refgpu_qk_norm_rope(float *q, float *k, const float *qw, const float *kw, int pos,
                           const float *inv_freq, float af, int stride, int jump, int jump_at) {
    float *dq, *dk, *dqw, *dkw, *dif; int *dpos;
    RCHK(cudaMalloc(&dq, 8192 * 4)); RCHK(cudaMalloc(&dk, 1024 * 4));
    RCHK(cudaMalloc(&dqw, 512)); RCHK(cudaMalloc(&dkw, 512)); RCHK(cudaMalloc(&dif, 256)); RCHK(cudaMalloc(&dpos, 4));
    RCHK(cudaMemcpy(dq, q, 8192 * 4, cudaMemcpyHostToDevice)); RCHK(cudaMemcpy(dk, k, 1024 * 4, cudaMemcpyHostToDevice));
    RCHK(cudaMemcpy(dqw, qw, 512, cudaMemcpyHostToDevice)); RCHK(cudaMemcpy(dkw, kw, 512, cudaMemcpyHostToDevice));
    RCHK(cudaMemcpy(dif, inv_freq, 256, cudaMemcpyHostToDevice)); RCHK(cudaMemcpy(dpos, &pos, 4, cudaMemcpyHostToDevice));
    qk_norm_rope_fused_kernel<<<HY3_N_HEAD + HY3_N_KV_HEAD, BLOCK_DIM, BLOCK_DIM * sizeof(float)>>>(
        dq, dk, dqw, dkw, HY3_HEAD_DIM, HY3_N_HEAD, HY3_N_KV_HEAD, dpos, dif, af, stride, jump, jump_at);
    RCHK(cudaGetLastError());
    RCHK(cudaMemcpy(q, dq, 8192 * 4, cudaMemcpyDeviceToHost)); RCHK(cudaMemcpy(k, dk, 1024 * 4, cudaMemcpyDeviceToHost));
    cudaFree(dq); cudaFree(dk); cudaFree(dqw); cudaFree(dkw); cudaFree(dif); cudaFree(dpos);
    return 0;
}

/* Quantise n tokens: k, v are [n][8*128] fp32; kslots/vslots receive n reference
 * slots (1040 B each for INT8, 528 B for INT4) for a single-layer cache.         */
int hy3refgpu_kv_quantize(int int4, const float *k, const float *v, int n, uint8_t *kslots, uint8_t *vslots) {
    int stride = int4 ? KV_INT4_STRIDE : KV_INT8_STRIDE;
    float *dk, *dv; uint8_t *kc, *vc; int *dpos;
    RCHK(cudaMalloc(&dk, (size_t)n * 4096)); RCHK(cudaMalloc(&dv, (size_t)n * 4096));
    RCHK(cudaMalloc(&kc, (size_t)n * stride)); RCHK(cudaMalloc(&vc, (size_t)n * stride)); RCHK(cudaMalloc(&dpos, (size_t)n * 4));
    RCHK(cudaMemcpy(dk, k, (size_t)n * 4096, cudaMemcpyHostToDevice)); RCHK(cudaMemcpy(dv, v, (size_t)n * 4096, cudaMemcpyHostToDevice));
    iota_kernel<<<(n + 255) / 256, 256>>>(dpos, 0, n);
    for (int t = 0; t < n; t++) {
        if (int4) kv_quantize_int4_kernel<<<HY3_N_KV_HEAD, 32>>>(kc, vc, dk + (size_t)t * 1024, dv + (size_t)t * 1024, dpos + t, 0, 1);
        else      kv_quantize_int8_kernel<<<HY3_N_KV_HEAD, 32>>>(kc, vc, dk + (size_t)t * 1024, dv + (size_t)t * 1024, dpos + t, 0, 1);
    }
    RCHK(cudaGetLastError());
    RCHK(cudaMemcpy(kslots, kc, (size_t)n * stride, cudaMemcpyDeviceToHost)); RCHK(cudaMemcpy(vslots, vc, (size_t)n * stride, cudaMemcpyDeviceToHost));
    cudaFree(dk); cudaFree(dv); cudaFree(kc); cudaFree(vc); cudaFree(dpos);
    return 0;
}

/* Split-KV decode + reduce over a single-layer cache of ntok reference slots. */
int hy3refgpu_decode(int int4, const float *q, const uint8_t *kslots, const uint8_t *vslots, int ntok, int nsplits, float *out) {
    int stride = int4 ? KV_INT4_STRIDE : KV_INT8_STRIDE;
    if (nsplits < 1 || nsplits > ATTN_SPLITS_MAX) return -1;
    float *dq, *dout, *dpart; uint8_t *kc, *vc; int *dpos; int pos = ntok - 1;
    RCHK(cudaMalloc(&dq, 8192 * 4)); RCHK(cudaMalloc(&dout, 8192 * 4));
    RCHK(cudaMalloc(&dpart, (size_t)HY3_N_HEAD * ATTN_SPLITS_MAX * 130 * 4));
    RCHK(cudaMalloc(&kc, (size_t)ntok * stride)); RCHK(cudaMalloc(&vc, (size_t)ntok * stride)); RCHK(cudaMalloc(&dpos, 4));
    RCHK(cudaMemcpy(dq, q, 8192 * 4, cudaMemcpyHostToDevice));
    RCHK(cudaMemcpy(kc, kslots, (size_t)ntok * stride, cudaMemcpyHostToDevice)); RCHK(cudaMemcpy(vc, vslots, (size_t)ntok * stride, cudaMemcpyHostToDevice));
    RCHK(cudaMemcpy(dpos, &pos, 4, cudaMemcpyHostToDevice));
    if (int4) attention_split_kv_int4_kernel<<<HY3_N_HEAD * nsplits, 32>>>(dq, kc, vc, HY3_N_HEAD, HY3_N_KV_HEAD, HY3_HEAD_DIM, dpos, 8, 0, 1, nsplits, dpart);
    else      attention_split_kv_kernel<<<HY3_N_HEAD * nsplits, 32>>>(dq, kc, vc, HY3_N_HEAD, HY3_N_KV_HEAD, HY3_HEAD_DIM, dpos, 8, 0, 1, nsplits, dpart);
    attention_reduce_kernel<<<HY3_N_HEAD, 32>>>(dout, dpart, HY3_N_HEAD, HY3_HEAD_DIM, nsplits);
    RCHK(cudaGetLastError());
    RCHK(cudaMemcpy(out, dout, 8192 * 4, cudaMemcpyDeviceToHost));
    cudaFree(dq); cudaFree(dout); cudaFree(dpart); cudaFree(kc); cudaFree(vc); cudaFree(dpos);
    return 0;
}

/* Chunk prefill attention: q [nq][64*128] fp32, out same shape. */
int hy3refgpu_prefill(int int4, const float *q, const uint8_t *kslots, const uint8_t *vslots, int base_tok, int nq, float *out) {
    int stride = int4 ? KV_INT4_STRIDE : KV_INT8_STRIDE; int ntok = base_tok + nq;
    float *dq, *dout; uint8_t *kc, *vc;
    RCHK(cudaMalloc(&dq, (size_t)nq * 8192 * 4)); RCHK(cudaMalloc(&dout, (size_t)nq * 8192 * 4));
    RCHK(cudaMalloc(&kc, (size_t)ntok * stride)); RCHK(cudaMalloc(&vc, (size_t)ntok * stride));
    RCHK(cudaMemcpy(dq, q, (size_t)nq * 8192 * 4, cudaMemcpyHostToDevice));
    RCHK(cudaMemcpy(kc, kslots, (size_t)ntok * stride, cudaMemcpyHostToDevice)); RCHK(cudaMemcpy(vc, vslots, (size_t)ntok * stride, cudaMemcpyHostToDevice));
    dim3 g(HY3_N_HEAD, (nq + PF_QB - 1) / PF_QB);
    if (int4) prefill_attn_int4_kernel<<<g, 32>>>(dq, dout, kc, vc, HY3_N_HEAD, HY3_HEAD_DIM, 8, 0, 1, base_tok, nq, 8192, 8192);
    else      prefill_attn_int8_kernel<<<g, 32>>>(dq, dout, kc, vc, HY3_N_HEAD, HY3_HEAD_DIM, 8, 0, 1, base_tok, nq, 8192, 8192);
    RCHK(cudaGetLastError());
    RCHK(cudaMemcpy(out, dout, (size_t)nq * 8192 * 4, cudaMemcpyDeviceToHost));
    cudaFree(dq); cudaFree(dout); cudaFree(kc); cudaFree(vc);
    return 0;
}

/* Time the reference decode (split + reduce) on a cache of nl interleaved layers
 * and ntok tokens filled with a fixed byte pattern (scales set to a sane fp16
 * value); layer il cycles 0..nl-1 per launch pair so successive launches do not
 * hit the same L2-resident lines.  Returns the average ms per layer-step.        */
int hy3refgpu_decode_bench(int int4, int ntok, int nl, int iters, float *ms_per_layer) {
    int stride = int4 ? KV_INT4_STRIDE : KV_INT8_STRIDE;
    size_t bytes = (size_t)ntok * nl * stride;
    float *dq, *dout, *dpart; uint8_t *kc, *vc; int *dpos; int pos = ntok - 1;
    RCHK(cudaMalloc(&dq, 8192 * 4)); RCHK(cudaMalloc(&dout, 8192 * 4));
    RCHK(cudaMalloc(&dpart, (size_t)HY3_N_HEAD * ATTN_SPLITS_MAX * 130 * 4));
    RCHK(cudaMalloc(&kc, bytes)); RCHK(cudaMalloc(&vc, bytes)); RCHK(cudaMalloc(&dpos, 4));
    RCHK(cudaMemset(dq, 0, 8192 * 4));
    RCHK(cudaMemset(kc, 0x11, bytes)); RCHK(cudaMemset(vc, 0x11, bytes));   /* scale bits 0x1111 ~ 6.5e-4 */
    RCHK(cudaMemcpy(dpos, &pos, 4, cudaMemcpyHostToDevice));
    int ns = gpu_optimal_splits(ntok);
    cudaEvent_t a, b; cudaEventCreate(&a); cudaEventCreate(&b);
    for (int it = -3; it < iters; it++) {
        if (it == 0) cudaEventRecord(a);
        int il = ((it % nl) + nl) % nl;
        if (int4) attention_split_kv_int4_kernel<<<HY3_N_HEAD * ns, 32>>>(dq, kc, vc, HY3_N_HEAD, HY3_N_KV_HEAD, HY3_HEAD_DIM, dpos, 8, il, nl, ns, dpart);
        else      attention_split_kv_kernel<<<HY3_N_HEAD * ns, 32>>>(dq, kc, vc, HY3_N_HEAD, HY3_N_KV_HEAD, HY3_HEAD_DIM, dpos, 8, il, nl, ns, dpart);
        attention_reduce_kernel<<<HY3_N_HEAD, 32>>>(dout, dpart, HY3_N_HEAD, HY3_HEAD_DIM, ns);
    }
    cudaEventRecord(b); RCHK(cudaEventSynchronize(b)); RCHK(cudaGetLastError());
    float ms = 0; cudaEventElapsedTime(&ms, a, b); *ms_per_layer = ms / iters;
    cudaEventDestroy(a); cudaEventDestroy(b);
    cudaFree(dq); cudaFree(dout); cudaFree(dpart); cudaFree(kc); cudaFree(vc); cudaFree(dpos);
    return 0;
}

} /* extern "C" */
