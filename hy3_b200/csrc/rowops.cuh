/*
 * rowops.cuh -- device functions shared by the append kernel and the fused decode step:
 * per-head RMSNorm + rotate_half RoPE of one 128-wide row held by a warp, and the quantise +
 * store of a row into a KV page.  One warp owns one row: lane = 16*half + idx holds dims
 * half*64 + idx*4 .. +3, so the rotate_half partner d+64 is lane^16.
 *
 * Arithmetic follows the reference CUDA kernels operation for operation (hy3_gpu.cu:144-164,
 * :250-270, :329-352); see append.cu for the list.
 */
#ifndef HY3A_ROWOPS_CUH
#define HY3A_ROWOPS_CUH

#include <cuda_fp16.h>
#include <math.h>

#include "ctx.h"

namespace hy3a_rowops {

__device__ __forceinline__ uint8_t *page_ptr(const hy3a_cache_view &c, int seq, int slot, int layer, int head_local) {
    int block = c.block_table[(size_t)seq * c.max_blocks_per_seq + (slot >> 7)];
    return c.pool + hy3a_page_index(c, block, layer, head_local) * (size_t)c.page_bytes;
}

/* Quantise (or round to fp16) the warp's 128 values y[4] (dims d0..d0+3 per lane) and
 * store them as row `tok` (0..127) of the page.  is_v selects the V area / pair layout.
 * Returns the fp16 scale bits (0 for FP16 caches).                                    */
template <int DT>
__device__ __forceinline__ unsigned store_row(uint8_t *page, const hy3a_geom &g, int tok, bool is_v, const float y[4], int d0, int lane,
                                              uint8_t *scale_page = nullptr /* where the scale goes, if not into `page` (a shared-memory copy split in two) */,
                                              int *codes_out = nullptr /* the lane's 4 codes (quantised caches) */) {
    if (DT == 0) {
        __half2 h01 = __floats2half2_rn(y[0], y[1]);
        __half2 h23 = __floats2half2_rn(y[2], y[3]);
        uint2 w;
        w.x = *reinterpret_cast<unsigned *>(&h01);
        w.y = *reinterpret_cast<unsigned *>(&h23);
        int off = is_v ? g.v_off + hy3a_v16_dim_off(tok, d0) : hy3a_k_dim_off<0>(tok, d0);
        *reinterpret_cast<uint2 *>(page + off) = w;
        return 0u;
    }
    float m = fmaxf(fmaxf(fabsf(y[0]), fabsf(y[1])), fmaxf(fabsf(y[2]), fabsf(y[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float qmax = DT == 1 ? 127.f : 7.f;
    float s = __fadd_rn(__fdiv_rn(m, qmax), 1e-8f);
    float inv = __fdiv_rn(1.f, s);
    int c[4];
#pragma unroll
    for (int j = 0; j < 4; j++) c[j] = (int)roundf(fmaxf(-qmax, fminf(qmax, __fmul_rn(y[j], inv))));
    if (codes_out) { codes_out[0] = c[0]; codes_out[1] = c[1]; codes_out[2] = c[2]; codes_out[3] = c[3]; }
    __half sh = __float2half(s);
    unsigned sbits = (unsigned)__half_as_ushort(sh);
    if (lane == 0) *reinterpret_cast<unsigned short *>((scale_page ? scale_page : page) + (is_v ? g.vs_off : g.ks_off) + tok * 2) = (unsigned short)sbits;
    if (DT == 1) {
        if (!is_v) {
            unsigned w = (unsigned)(c[0] & 0xFF) | ((unsigned)(c[1] & 0xFF) << 8) | ((unsigned)(c[2] & 0xFF) << 16) | ((unsigned)(c[3] & 0xFF) << 24);
            *reinterpret_cast<unsigned *>(page + hy3a_k_dim_off<1>(tok, d0)) = w;
        } else {
            /* V codes go into the transposed tile: one byte per (head dim, token) */
#pragma unroll
            for (int j = 0; j < 4; j++) page[g.v_off + hy3a_vt_off(d0 + j, tok)] = (uint8_t)(c[j] & 0xFF);
        }
    } else {
        unsigned short u = (unsigned short)((c[0] & 0xF) | ((c[1] & 0xF) << 4) | ((c[2] & 0xF) << 8) | ((c[3] & 0xF) << 12));
        if (is_v) u ^= 0x8888;   /* V nibbles offset-binary (n + 8): the decode kernel's nibble -> fp16 conversion then needs no sign fix-up */
        int off = is_v ? g.v_off + hy3a_v_unit_off<2>(tok, d0) : hy3a_k_dim_off<2>(tok, d0);
        *reinterpret_cast<unsigned short *>(page + off) = u;
    }
    return sbits;
}

/* cos/sin (times attn_factor) of the RoPE angles of this lane's 4 dim pairs at token index ti
 * (hy3_gpu.cu:152, :161-162). */
__device__ __forceinline__ void rope_coeffs(float c[4], float s[4], const hy3a_rope_params &rope, int ti, int lane) {
    const int idx = lane & 15;
    const int pos = (ti + (ti >= rope.pos_jump_at ? rope.pos_jump : 0)) * rope.pos_stride;
    const float4 fv = *reinterpret_cast<const float4 *>(rope.inv_freq + idx * 4);
    const float fr4[4] = {fv.x, fv.y, fv.z, fv.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float fr = (float)pos * fr4[j];
        c[j] = cosf(fr) * rope.attn_factor;
        s[j] = sinf(fr) * rope.attn_factor;
    }
}

/* RMSNorm (this lane's 4 weights wv, eps) + RoPE with precomputed coefficients of the warp's row y[4]. */
__device__ __forceinline__ void norm_rope_apply(float y[4], const float4 wv, float eps, const float c[4], const float s[4], int lane) {
    const int half = lane >> 4;
    /* sum of squares in the reference's shared-memory tree order (hy3_gpu.cu:155-157) */
    float sq[4];
#pragma unroll
    for (int j = 0; j < 4; j++) sq[j] = __fmul_rn(y[j], y[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int j = 0; j < 4; j++) sq[j] = __fadd_rn(sq[j], __shfl_xor_sync(0xffffffffu, sq[j], o));
    }
    float ss = __fadd_rn(__fadd_rn(sq[0], sq[2]), __fadd_rn(sq[1], sq[3]));
    float r = rsqrtf(ss / (float)HY3A_D + eps);
    y[0] = y[0] * r * wv.x; y[1] = y[1] * r * wv.y; y[2] = y[2] * r * wv.z; y[3] = y[3] * r * wv.w;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float other = __shfl_xor_sync(0xffffffffu, y[j], 16);
        float v0 = half ? other : y[j], v1 = half ? y[j] : other;
        y[j] = half ? (v1 * c[j] + v0 * s[j]) : (v0 * c[j] - v1 * s[j]);
    }
}

/* RMSNorm (weights w[128], eps) + RoPE at token index ti of the warp's row y[4], in place. */
__device__ __forceinline__ void norm_rope_row(float y[4], const float *w, float eps, const hy3a_rope_params &rope, int ti, int lane) {
    const int d0 = (lane >> 4) * 64 + (lane & 15) * 4;
    float c[4], s[4];
    rope_coeffs(c, s, rope, ti, lane);
    norm_rope_apply(y, *reinterpret_cast<const float4 *>(w + d0), eps, c, s, lane);
}

} /* namespace hy3a_rowops */
#endif
