/*
 * selftest.cu -- known-answer check run by hy3a_create.
 *
 * The reference never checks a kernel launch (hy3_gpu.cu:750-758), which is how a build
 * for the wrong architecture can return all-zero logits without any error.  Here context
 * creation runs the real append + decode kernels on three fixed tokens and compares the
 * result with a double-precision evaluation on the host of the same formulas over the
 * cache contents read back; a wrong-architecture image, a failed launch or a broken
 * layout makes hy3a_create fail loudly.
 */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_fp16.h>

#include "ctx.h"

static float st_val(int i, int salt) { /* deterministic pseudo-data in [-1.5, 1.5] */
    unsigned x = (unsigned)i * 2654435761u + (unsigned)salt * 40503u + 12345u;
    x ^= x >> 13; x *= 2246822519u; x ^= x >> 16;
    return ((float)(x & 0xFFFF) / 65535.0f - 0.5f) * 3.0f;
}

extern "C" int hy3a_selftest(hy3a_ctx *ctx) {
    const int NT = 3, QF = HY3A_N_HEAD * HY3A_D, KF = HY3A_N_KV_HEAD * HY3A_D;
    if (ctx->cfg.max_batch < 1) return HY3A_OK;
    const int nb = ctx->cfg.max_batch >= NT ? NT : 1;
    int rc = HY3A_OK;
    float *hq = (float *)malloc(sizeof(float) * NT * (QF + 2 * KF)), *hqo = (float *)malloc(sizeof(float) * QF), *hout = (float *)malloc(sizeof(float) * QF);
    const int sb = hy3a_slot_bytes(ctx->cfg.kv_dtype);
    uint8_t *ks = (uint8_t *)malloc((size_t)NT * sb), *vs = (uint8_t *)malloc((size_t)NT * sb);
    float *dq = NULL, *dqo = NULL, *dout = NULL;
    if (!hq || !hqo || !hout || !ks || !vs) { rc = hy3a_fail(ctx, HY3A_ENOMEM, "selftest: malloc"); goto done; }
    for (int i = 0; i < NT * (QF + 2 * KF); i++) hq[i] = st_val(i, 7);
    if (cudaMalloc(&dq, sizeof(float) * NT * (QF + 2 * KF)) != cudaSuccess || cudaMalloc(&dqo, sizeof(float) * NT * QF) != cudaSuccess ||
        cudaMalloc(&dout, sizeof(float) * QF) != cudaSuccess) { rc = hy3a_fail(ctx, HY3A_ENOMEM, "selftest: cudaMalloc"); goto done; }
    if (cudaMemcpyAsync(dq, hq, sizeof(float) * NT * (QF + 2 * KF), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) { rc = hy3a_fail(ctx, HY3A_ECUDA, "selftest: H2D"); goto done; }
    if (cudaMemsetAsync(dout, 0, sizeof(float) * QF, ctx->stream) != cudaSuccess) { rc = hy3a_fail(ctx, HY3A_ECUDA, "selftest: memset"); goto done; }
    /* append NT tokens (row layout [q 8192 | k 1024 | v 1024]) in batches of nb rows */
    for (int t = 0; t < NT && rc == HY3A_OK; t += nb) {
        int seqs[NT] = {0, 0, 0}, slots[NT], pos[NT];
        for (int i = 0; i < nb; i++) { slots[i] = t + i; pos[i] = 100 + t + i; }
        rc = hy3a_batch_set(ctx, nb, seqs, slots, pos);
        if (rc == HY3A_OK)
            rc = hy3a_append(ctx, 0, dq + (size_t)t * (QF + 2 * KF), QF + 2 * KF, dq + (size_t)t * (QF + 2 * KF) + QF, QF + 2 * KF,
                             dq + (size_t)t * (QF + 2 * KF) + QF + KF, QF + 2 * KF, dqo + (size_t)t * QF, QF, NULL);
    }
    if (rc) goto done;
    { int seqs[1] = {0}, slots[1] = {NT - 1}, pos[1] = {100 + NT - 1};
      rc = hy3a_batch_set(ctx, 1, seqs, slots, pos);
      if (rc == HY3A_OK) rc = hy3a_decode(ctx, 0, dqo + (size_t)(NT - 1) * QF, QF, dout, QF, NULL);
      if (rc) goto done; }
    if (cudaMemcpyAsync(hqo, dqo + (size_t)(NT - 1) * QF, sizeof(float) * QF, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess ||
        cudaMemcpyAsync(hout, dout, sizeof(float) * QF, cudaMemcpyDeviceToHost, ctx->stream) != cudaSuccess) { rc = hy3a_fail(ctx, HY3A_ECUDA, "selftest: D2H"); goto done; }
    rc = hy3a_export_kv(ctx, 0, 0, 0, NT, ks, vs);
    if (rc) goto done;
    rc = hy3a_sync(ctx);
    if (rc) goto done;
    {
        /* (1) the last token's q: per-head RMSNorm (unit weights) + rotate_half RoPE at pos 102, in double */
        double worst_q = 0, worst_o = 0;
        const float *qin = hq + (size_t)(NT - 1) * (QF + 2 * KF);
        for (int h = 0; h < HY3A_N_HEAD; h++) {
            double ss = 0;
            for (int d = 0; d < HY3A_D; d++) ss += (double)qin[h * HY3A_D + d] * qin[h * HY3A_D + d];
            double r = 1.0 / sqrt(ss / HY3A_D + (double)ctx->cfg.rms_eps);
            for (int d = 0; d < 64; d++) {
                double fr = (double)(float)((float)(100 + NT - 1) * (float)(1.0 / pow(11158840.0, (double)(2 * d) / 128.0)));
                double c = cos(fr), s = sin(fr), x0 = qin[h * HY3A_D + d] * r, x1 = qin[h * HY3A_D + d + 64] * r;
                double e0 = fabs(x0 * c - x1 * s - hqo[h * HY3A_D + d]), e1 = fabs(x1 * c + x0 * s - hqo[h * HY3A_D + d + 64]);
                if (e0 > worst_q) worst_q = e0;
                if (e1 > worst_q) worst_q = e1;
            }
        }
        /* (2) attention of that q over the cache as stored */
        const int dt = ctx->cfg.kv_dtype, hdr = dt == 0 ? 0 : 16, hb = dt == 1 ? 128 : (dt == 2 ? 64 : 256);
        for (int h = 0; h < HY3A_N_HEAD; h++) {
            int kvh = h / 8;
            if (kvh < ctx->cfg.kv_head_begin || kvh >= ctx->cfg.kv_head_begin + ctx->cfg.kv_head_count) continue;
            double sc[NT], mx = -1e300, sum = 0, o[HY3A_D];
            double kv[2][NT][HY3A_D];
            for (int w = 0; w < 2; w++)
                for (int t = 0; t < NT; t++) {
                    const uint8_t *slot = (w ? vs : ks) + (size_t)t * sb;
                    double scale = 1.0;
                    if (dt != 0) { __half_raw hr; memcpy(&hr.x, slot + kvh * 2, 2); scale = (double)__half2float(__half(hr)); }
                    const uint8_t *body = slot + hdr + kvh * hb;
                    for (int d = 0; d < HY3A_D; d++) {
                        double v;
                        if (dt == 1) v = (double)(int8_t)body[d];
                        else if (dt == 2) { int nib = (body[d / 2] >> ((d & 1) * 4)) & 0xF; v = nib > 7 ? nib - 16 : nib; }
                        else { __half_raw hr; memcpy(&hr.x, body + 2 * d, 2); v = (double)__half2float(__half(hr)); }
                        kv[w][t][d] = v * scale;
                    }
                }
            for (int t = 0; t < NT; t++) {
                double s = 0;
                for (int d = 0; d < HY3A_D; d++) s += (double)hqo[h * HY3A_D + d] * kv[0][t][d];
                sc[t] = s / sqrt(128.0);
                if (sc[t] > mx) mx = sc[t];
            }
            for (int d = 0; d < HY3A_D; d++) o[d] = 0;
            for (int t = 0; t < NT; t++) { double p = exp(sc[t] - mx); sum += p; for (int d = 0; d < HY3A_D; d++) o[d] += p * kv[1][t][d]; }
            for (int d = 0; d < HY3A_D; d++) { double e = fabs(o[d] / sum - hout[h * HY3A_D + d]); if (!(e <= worst_o)) worst_o = e; }
        }
        if (!(worst_q < 1e-4) || !(worst_o < 2e-3))
            rc = hy3a_fail(ctx, HY3A_ECUDA, "known-answer mismatch: norm+rope max err %.3g (limit 1e-4), attention max err %.3g (limit 2e-3)", worst_q, worst_o);
    }
done:
    cudaFree(dq); cudaFree(dqo); cudaFree(dout);
    free(hq); free(hqo); free(hout); free(ks); free(vs);
    hy3a_seq_release(ctx, 0, 0);
    ctx->batch_n = 0;
    /* the block the test used (the first one handed out) goes back zeroed */
    hy3a_launch_init_pages(ctx, 0, (size_t)ctx->cfg.n_layers * ctx->cfg.kv_head_count);
    cudaMemsetAsync(ctx->d_vs_max, 0, (size_t)ctx->cfg.n_layers * ctx->cfg.kv_head_count * sizeof(unsigned), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    ctx->launches = 0;
    return rc;
}
