/*
 * append.cu -- fused per-head QK RMSNorm + rotate_half RoPE + KV quantise + append,
 * plus the cache import/export/fill utilities that share its store path.
 *
 * One warp owns one 128-wide head row (4 dims per lane, lanes 0-15 hold dims 0..63 and
 * lanes 16-31 hold dims 64..127, so the rotate_half partner d+64 is lane^16).  One launch
 * covers every row of the step's batch: 64 Q heads + 8 K heads + 8 V heads per token,
 * where the reference launches qk_norm_rope_fused_kernel and kv_quantize_* once per token
 * (hy3_gpu.cu:823-829).  HBM-bound, a few KB per token: the job of this kernel is to be one
 * launch, coalesced (512 B per warp load, 128 B per warp code store) and bit-faithful.
 *
 * Arithmetic follows the reference CUDA kernels operation for operation:
 *   - sum of squares in the reference's shared-memory tree order (hy3_gpu.cu:155-157):
 *     (d, d+64), then (d, d+32), ... reproduced with xor-shuffles 16,8,4,2,1 and the
 *     last two levels in registers;
 *   - r = rsqrtf(ss/128 + eps), y = x*r*w (hy3_gpu.cu:158-159);
 *   - RoPE angle (float)pos*inv_freq[d], full-range cosf/sinf, attn_factor on both
 *     (hy3_gpu.cu:161-163), position probe (ti + (ti>=jump_at ? jump : 0))*stride (:152);
 *   - quantiser: s = absmax/127 (or /7) + 1e-8, inv = 1/s, code = roundf(clamp(x*inv)),
 *     stored scale = fp16(s) (hy3_gpu.cu:260-269, :338-351), IEEE division (no fast-math).
 */
#include <cuda_fp16.h>
#include <math.h>

#include "ctx.h"
#include "rowops.cuh"

namespace {
using namespace hy3a_rowops;

struct append_args {
    const float *q_in, *k_in, *v_in;
    size_t q_stride, k_stride, v_stride;
    float *q_out;
    size_t q_out_stride;
    __half *q_out16;
    const float *norm_w; /* [2][128] for this layer */
    float eps;
    int layer;
    /* write-through into the layer's fp16 prefill operands (NULL = none): K rows [head][token][128] and V transposed
     * [head][128][mirror_stride], the values the conversion kernel of the chunked prefill would produce */
    __half *mirror_k, *mirror_v;
    int mirror_stride;
};

/* grid (10, n_rows), block 256: warp (blockIdx.x*8 + warp) in [0,80) = 64 Q, 8 K, 8 V heads. */
template <int DT>
__global__ void __launch_bounds__(256) hy3a_append_kernel(hy3a_cache_view cache, hy3a_batch_view batch, hy3a_rope_params rope, append_args a) {
    /* programmatic dependent launch: wait until the preceding kernel's results are complete, then
     * let the next kernel start its prologue (no-ops without the launch attribute)              */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int row = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hr = blockIdx.x * 8 + warp;
    /* the RoPE coefficients depend on the row only: 64 threads compute them once for the block's 8 heads (full-range
     * cosf/sinf are most of this kernel's instructions when every warp computes its own) */
    __shared__ float s_cos[64], s_sin[64];
    if (row < batch.n && blockIdx.x < 9 && threadIdx.x < 64) {
        const int ti = batch.pos[row];
        const int pos = (ti + (ti >= rope.pos_jump_at ? rope.pos_jump : 0)) * rope.pos_stride;
        const float fr = (float)pos * rope.inv_freq[threadIdx.x];
        s_cos[threadIdx.x] = cosf(fr) * rope.attn_factor;
        s_sin[threadIdx.x] = sinf(fr) * rope.attn_factor;
    }
    __syncthreads();
    if (row >= batch.n || hr >= 80) return;
    const hy3a_geom g = hy3a_make_geom(DT);
    const int half = lane >> 4, idx = lane & 15;
    const int d0 = half * 64 + idx * 4;
    const int seq = batch.seq[row], slot = batch.slot[row];

    const bool is_q = hr < 64, is_k = (hr >= 64 && hr < 72);
    const int head = is_q ? hr : (is_k ? hr - 64 : hr - 72);
    const bool owned = is_q || (head >= cache.kv_head_begin && head < cache.kv_head_begin + cache.kv_heads);
    if (!owned || (!is_q && a.k_in == nullptr)) return; /* k_in == NULL: query-only mode */
    const float *src = is_q ? a.q_in + (size_t)row * a.q_stride : (is_k ? a.k_in + (size_t)row * a.k_stride : a.v_in + (size_t)row * a.v_stride);
    float4 xv = *reinterpret_cast<const float4 *>(src + (size_t)head * HY3A_D + d0);
    float y[4] = {xv.x, xv.y, xv.z, xv.w};

    if (is_q || is_k) {
        const float4 cv4 = *reinterpret_cast<const float4 *>(s_cos + idx * 4), sv4 = *reinterpret_cast<const float4 *>(s_sin + idx * 4);
        const float c[4] = {cv4.x, cv4.y, cv4.z, cv4.w}, sn[4] = {sv4.x, sv4.y, sv4.z, sv4.w};
        norm_rope_apply(y, *reinterpret_cast<const float4 *>(a.norm_w + (is_k ? HY3A_D : 0) + d0), a.eps, c, sn, lane);
    }
    if (is_q) {
        if (a.q_out) *reinterpret_cast<float4 *>(a.q_out + (size_t)row * a.q_out_stride + (size_t)head * HY3A_D + d0) = make_float4(y[0], y[1], y[2], y[3]);
        if (a.q_out16) {
            __half2 h01 = __floats2half2_rn(y[0], y[1]), h23 = __floats2half2_rn(y[2], y[3]);
            uint2 w2;
            w2.x = *reinterpret_cast<unsigned *>(&h01);
            w2.y = *reinterpret_cast<unsigned *>(&h23);
            *reinterpret_cast<uint2 *>(a.q_out16 + ((size_t)row * 64 + head) * HY3A_D + d0) = w2;
        }
        return;
    }
    const int hl = head - cache.kv_head_begin;
    uint8_t *page = page_ptr(cache, seq, slot, a.layer, hl);
    int codes[4];
    unsigned sb = store_row<DT>(page, g, slot & 127, !is_k, y, d0, lane, nullptr, codes);
    if (DT != 0 && !is_k && lane == 0) atomicMax(cache.vs_max + a.layer * cache.kv_heads + hl, sb);
    if (a.mirror_k) {
        /* value = code * stored fp16 scale (hy3_gpu.cu:206-215), or the fp16 value itself; rounded to fp16 */
        __half hv[4];
        const float sc = DT == 0 ? 0.f : __half2float(__ushort_as_half((unsigned short)sb));
#pragma unroll
        for (int j = 0; j < 4; j++) hv[j] = DT == 0 ? __float2half_rn(y[j]) : __float2half_rn((float)codes[j] * sc);
        if (is_k) {
            *reinterpret_cast<uint2 *>(a.mirror_k + ((size_t)hl * a.mirror_stride + slot) * HY3A_D + d0) = *reinterpret_cast<uint2 *>(hv);
        } else {
#pragma unroll
            for (int j = 0; j < 4; j++) a.mirror_v[((size_t)hl * HY3A_D + d0 + j) * a.mirror_stride + slot] = hv[j];
        }
    }
}

/* ---- the same work for a chunk of rows (prefill): blocks shaped for throughput -----------------------------------
 * With hundreds of rows the per-row blocks above are bound by their own latency (5 120 blocks for 512 rows, each with a
 * cosf/sinf stage in front of one 512-byte load per warp).  Here all blocks of a chunk are resident at once:
 *   blocks [0, n)            one row each: the 64 query heads, 8 per warp, loads issued up front, RoPE coefficients once
 *                            per row;
 *   blocks [n, n + kvh*ng)   one owned KV head x 8 consecutive rows (ng = ceil(n / 8)), warp = row: K and V of that head.
 *                            Eight consecutive tokens of one head in one block make the write-through of the
 *                            TRANSPOSED V operand a 16-byte store per head dim (staged in shared memory).
 * The arithmetic is the per-row kernel's (same rowops functions), so codes, scales and queries are identical bits. */
template <int DT>
__global__ void __launch_bounds__(256) hy3a_append_chunk_kernel(hy3a_cache_view cache, hy3a_batch_view batch, hy3a_rope_params rope, append_args a, int aligned8) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = batch.n;
    const int half = lane >> 4, idx = lane & 15, d0 = half * 64 + idx * 4;
    const hy3a_geom g = hy3a_make_geom(DT);
    if ((int)blockIdx.x < n) {
        /* ---- query block */
        const int row = blockIdx.x;
        __shared__ float s_cos[64], s_sin[64];
        if (threadIdx.x < 64) {
            const int ti = batch.pos[row];
            const int pos = (ti + (ti >= rope.pos_jump_at ? rope.pos_jump : 0)) * rope.pos_stride;
            const float fr = (float)pos * rope.inv_freq[threadIdx.x];
            s_cos[threadIdx.x] = cosf(fr) * rope.attn_factor;
            s_sin[threadIdx.x] = sinf(fr) * rope.attn_factor;
        }
        float4 xv[8];
        const float *src = a.q_in + (size_t)row * a.q_stride + d0;
#pragma unroll
        for (int i = 0; i < 8; i++) xv[i] = *reinterpret_cast<const float4 *>(src + (size_t)(warp + 8 * i) * HY3A_D);
        const float4 wv = *reinterpret_cast<const float4 *>(a.norm_w + d0);
        __syncthreads();
        const float4 cv4 = *reinterpret_cast<const float4 *>(s_cos + idx * 4), sv4 = *reinterpret_cast<const float4 *>(s_sin + idx * 4);
        const float c[4] = {cv4.x, cv4.y, cv4.z, cv4.w}, sn[4] = {sv4.x, sv4.y, sv4.z, sv4.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int head = warp + 8 * i;
            float y[4] = {xv[i].x, xv[i].y, xv[i].z, xv[i].w};
            norm_rope_apply(y, wv, a.eps, c, sn, lane);
            if (a.q_out) *reinterpret_cast<float4 *>(a.q_out + (size_t)row * a.q_out_stride + (size_t)head * HY3A_D + d0) = make_float4(y[0], y[1], y[2], y[3]);
            if (a.q_out16) {
                __half2 h01 = __floats2half2_rn(y[0], y[1]), h23 = __floats2half2_rn(y[2], y[3]);
                uint2 w2;
                w2.x = *reinterpret_cast<unsigned *>(&h01);
                w2.y = *reinterpret_cast<unsigned *>(&h23);
                *reinterpret_cast<uint2 *>(a.q_out16 + ((size_t)row * 64 + head) * HY3A_D + d0) = w2;
            }
        }
        return;
    }
    /* ---- K/V block: owned head hl, rows 8 grp .. 8 grp + 7 (warp = row) */
    const int kb = blockIdx.x - n, hl = kb % cache.kv_heads, grp = kb / cache.kv_heads;
    const int head = cache.kv_head_begin + hl, row = grp * 8 + warp;
    const bool live = row < n;
    __shared__ __align__(16) __half s_vt[HY3A_D][8];
    int slot = 0;
    if (live) {
        const int seq = batch.seq[row], ti = batch.pos[row];
        slot = batch.slot[row];
        const float4 kx = *reinterpret_cast<const float4 *>(a.k_in + (size_t)row * a.k_stride + (size_t)head * HY3A_D + d0);
        const float4 vx = *reinterpret_cast<const float4 *>(a.v_in + (size_t)row * a.v_stride + (size_t)head * HY3A_D + d0);
        uint8_t *page = page_ptr(cache, seq, slot, a.layer, hl);
        int codes[4];
        {
            float y[4] = {kx.x, kx.y, kx.z, kx.w};
            norm_rope_row(y, a.norm_w + HY3A_D, a.eps, rope, ti, lane);
            const unsigned sb = store_row<DT>(page, g, slot & 127, false, y, d0, lane, nullptr, codes);
            if (a.mirror_k) {
                __half hv[4];
                const float sc = DT == 0 ? 0.f : __half2float(__ushort_as_half((unsigned short)sb));
#pragma unroll
                for (int j = 0; j < 4; j++) hv[j] = DT == 0 ? __float2half_rn(y[j]) : __float2half_rn((float)codes[j] * sc);
                *reinterpret_cast<uint2 *>(a.mirror_k + ((size_t)hl * a.mirror_stride + slot) * HY3A_D + d0) = *reinterpret_cast<uint2 *>(hv);
            }
        }
        {
            float y[4] = {vx.x, vx.y, vx.z, vx.w};
            const unsigned sb = store_row<DT>(page, g, slot & 127, true, y, d0, lane, nullptr, codes);
            if (DT != 0 && lane == 0) atomicMax(cache.vs_max + a.layer * cache.kv_heads + hl, sb);
            if (a.mirror_k) {
                const float sc = DT == 0 ? 0.f : __half2float(__ushort_as_half((unsigned short)sb));
#pragma unroll
                for (int j = 0; j < 4; j++) s_vt[d0 + j][warp] = DT == 0 ? __float2half_rn(y[j]) : __float2half_rn((float)codes[j] * sc);
            }
        }
    }
    if (!a.mirror_k) return;      /* uniform over the block */
    __syncthreads();
    if (threadIdx.x < HY3A_D) {
        /* rows of a mirrored chunk are consecutive slots of one sequence: the block's 8 tokens are 8 adjacent columns */
        const int d = threadIdx.x, slot_base = batch.slot[grp * 8];
        __half *dst = a.mirror_v + ((size_t)hl * HY3A_D + d) * a.mirror_stride + slot_base;
        const int nrow = min(8, n - grp * 8);
        if (aligned8 && nrow == 8) {
            *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(&s_vt[d][0]);
        } else {
            for (int t = 0; t < nrow; t++) dst[t] = s_vt[d][t];
        }
    }
}

/* ---- device-side seeded fill (benchmark set-up) ----------------------------------- */
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__device__ __forceinline__ float normal_from(unsigned long long r) {
    float u1 = ((float)((r >> 40) & 0xFFFFFFull) + 1.0f) * (1.0f / 16777217.0f);
    float u2 = (float)((r >> 8) & 0xFFFFFFull) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * __logf(u1)) * __cosf(6.283185307179586f * u2);
}
/* grid (2, n): block 256 = 8 warps = the 8 heads of K (blockIdx.x 0) or V (1) of one token. */
template <int DT>
__global__ void __launch_bounds__(256) hy3a_fill_random_kernel(hy3a_cache_view cache, int layer, int seq, int t0, int n, unsigned long long seed) {
    const int t = t0 + blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool is_v = blockIdx.x == 1;
    if (blockIdx.y >= n || warp >= cache.kv_heads) return;
    const hy3a_geom g = hy3a_make_geom(DT);
    const int half = lane >> 4, idx = lane & 15, d0 = half * 64 + idx * 4;
    float y[4];
    unsigned long long base = seed ^ ((unsigned long long)(layer * 2 + (is_v ? 1 : 0) + 1) << 40);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        unsigned long long index = ((unsigned long long)t * 8ull + (unsigned long long)(warp + cache.kv_head_begin)) * 128ull + (unsigned long long)(d0 + j);
        y[j] = normal_from(splitmix64(base ^ (index + ((unsigned long long)seq << 34))));
    }
    uint8_t *page = page_ptr(cache, seq, t, layer, warp);
    unsigned sb = store_row<DT>(page, g, t & 127, is_v, y, d0, lane);
    if (DT != 0 && is_v && lane == 0) atomicMax(cache.vs_max + layer * cache.kv_heads + warp, sb);
}

/* ---- import / export in the reference's slot format ---------------------------------
 * One thread per (token, head, 4-dim group).  import=0: page -> slot, import=1: slot -> page. */
template <int DT>
__global__ void hy3a_xport_kernel(hy3a_cache_view cache, int layer, int seq, int t0, int n, uint8_t *kslots, uint8_t *vslots, int import) {
    const hy3a_geom g = hy3a_make_geom(DT);
    const int slot_bytes = DT == 1 ? 1040 : (DT == 2 ? 528 : 2048);
    const int hdr = DT == 0 ? 0 : 16;
    const int head_bytes = DT == 1 ? 128 : (DT == 2 ? 64 : 256);
    long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = (long long)n * 8 * 32 * 2;
    if (gid >= total) return;
    int is_v = (int)(gid & 1); gid >>= 1;
    int q4 = (int)(gid & 31); gid >>= 5;
    int head = (int)(gid & 7); gid >>= 3;
    int ti = (int)gid, t = t0 + ti;
    uint8_t *slot = (is_v ? vslots : kslots) + (size_t)ti * slot_bytes;
    int hl = head - cache.kv_head_begin;
    bool owned = hl >= 0 && hl < cache.kv_heads;
    int d0 = q4 * 4;
    int sbytes = DT == 1 ? 4 : (DT == 2 ? 2 : 8); /* bytes of 4 dims in slot format */
    uint8_t *sp = slot + hdr + head * head_bytes + (DT == 1 ? d0 : (DT == 2 ? d0 / 2 : d0 * 2));
    if (!owned) {
        if (!import) { for (int b = 0; b < sbytes; b++) sp[b] = 0; if (DT != 0 && q4 == 0) { slot[head * 2] = 0; slot[head * 2 + 1] = 0; } }
        return;
    }
    uint8_t *page = page_ptr(cache, seq, t, layer, hl);
    int tok = t & 127;
    /* byte locations of these 4 dims inside the page */
    uint8_t *pp[8];
    if (DT == 0) { int off = is_v ? g.v_off + hy3a_v16_dim_off(tok, d0) : hy3a_k_dim_off<0>(tok, d0); for (int b = 0; b < 8; b++) pp[b] = page + off + b; }
    else if (DT == 1) {
        if (!is_v) { int off = hy3a_k_dim_off<1>(tok, d0); for (int b = 0; b < 4; b++) pp[b] = page + off + b; }
        else { for (int b = 0; b < 4; b++) pp[b] = page + g.v_off + hy3a_vt_off(d0 + b, tok); }
    } else {
        int off = is_v ? g.v_off + hy3a_v_unit_off<2>(tok, d0) : hy3a_k_dim_off<2>(tok, d0); pp[0] = page + off; pp[1] = page + off + 1;
    }
    const uint8_t flip = (is_v && DT == 2) ? 0x88 : 0x00;   /* INT4 V nibbles are stored offset-binary */
    for (int b = 0; b < sbytes; b++) { if (import) *pp[b] = sp[b] ^ flip; else sp[b] = *pp[b] ^ flip; }
    if (DT != 0 && q4 == 0) {
        uint8_t *sc = page + (is_v ? g.vs_off : g.ks_off) + tok * 2;
        if (import) {
            sc[0] = slot[head * 2]; sc[1] = slot[head * 2 + 1];
            if (is_v) atomicMax(cache.vs_max + layer * cache.kv_heads + hl, (unsigned)slot[head * 2] | ((unsigned)slot[head * 2 + 1] << 8));
        } else { slot[head * 2] = sc[0]; slot[head * 2 + 1] = sc[1]; }
    }
}

/* Reset pages to the "all codes zero" state: zero bytes everywhere except the V code area of
 * INT4 pages, whose offset-binary zero is 0x88.  grid = pages, block 256.       */
__global__ void hy3a_init_pages_kernel(uint8_t *pool, size_t first_page, int page_bytes, int v_off, int v_end, unsigned flip_word) {
    uint4 *page = reinterpret_cast<uint4 *>(pool + (first_page + blockIdx.x) * (size_t)page_bytes);
    const int lo = v_off / 16, hi = v_end / 16;
    for (int i = threadIdx.x; i < page_bytes / 16; i += blockDim.x) {
        const unsigned w = (i >= lo && i < hi) ? flip_word : 0u;
        page[i] = make_uint4(w, w, w, w);
    }
}

} /* namespace */

int hy3a_launch_init_pages(hy3a_ctx *ctx, size_t first_page, size_t n_pages) {
    const hy3a_geom g = ctx->geom;
    const unsigned flip = g.dtype == 2 ? 0x88888888u : 0u;
    const int v_end = g.dtype == 0 ? g.page_bytes : g.ks_off;
    for (size_t done = 0; done < n_pages;) {
        size_t chunk = n_pages - done > 1048576 ? 1048576 : n_pages - done;
        hy3a_init_pages_kernel<<<(unsigned)chunk, 256, 0, ctx->stream>>>(ctx->pool, first_page + done, g.page_bytes, g.v_off, v_end, flip);
        HY3A_CUDA(ctx, cudaGetLastError());
        done += chunk;
    }
    return HY3A_OK;
}

int hy3a_launch_append(hy3a_ctx *ctx, int layer, const float *q_in, size_t q_stride, const float *k_in, size_t k_stride,
                       const float *v_in, size_t v_stride, float *q_out, size_t q_out_stride, void *q_out16) {
    append_args a;
    a.q_in = q_in; a.k_in = k_in; a.v_in = v_in; a.q_stride = q_stride; a.k_stride = k_stride; a.v_stride = v_stride;
    a.q_out = q_out; a.q_out_stride = q_out_stride; a.q_out16 = (__half *)q_out16;
    a.norm_w = ctx->d_norm_w + (size_t)layer * 2 * HY3A_D; a.eps = ctx->cfg.rms_eps; a.layer = layer;
    /* rows that extend the sequence whose prefill operands this layer keeps, gap-free: convert them here, where they are
     * in registers, instead of reading the pages back in the conversion kernel */
    a.mirror_k = a.mirror_v = NULL; a.mirror_stride = 0;
    if (k_in && ctx->batch_n > 0) {
        /* rows that rewrite slots the layer's operands already cover (a second append of the same batch, corrected K/V):
         * the covered part is stale from the lowest rewritten slot on */
        int lowest = ctx->batch_slot0;
        if (!ctx->batch_contig) lowest = ctx->batch_slot_min;
        if (ctx->batch_seq_uniform) hy3a_mirror_truncate(ctx, ctx->batch_seq0, layer, lowest);
        else { ctx->pf_mntok[layer] = 0; }
    }
    if (k_in && ctx->pf_mseq < 0 && ctx->pf_mk[layer] && ctx->batch_contig && ctx->batch_slot0 == 0)
        ctx->pf_mseq = ctx->batch_seq0;     /* mirrors allocated at create belong to the first sequence that is ingested from slot 0 */
    if (k_in && ctx->pf_mk[layer] && ctx->batch_contig && ctx->batch_seq0 == ctx->pf_mseq && ctx->batch_slot0 == ctx->pf_mntok[layer] &&
        ctx->batch_slot0 + ctx->batch_n <= ctx->pf_mcap[layer]) {
        a.mirror_k = (__half *)ctx->pf_mk[layer]; a.mirror_v = (__half *)ctx->pf_mv[layer]; a.mirror_stride = ctx->pf_mcap[layer];
        ctx->pf_mntok[layer] = ctx->batch_slot0 + ctx->batch_n;
    }
    hy3a_cache_view cv = hy3a_view(ctx);
    hy3a_batch_view bv = hy3a_bview(ctx);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(10, ctx->batch_n); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    cudaError_t e;
    if (ctx->batch_n >= 32) {      /* a chunk: the throughput-shaped kernel */
        const int n = ctx->batch_n, kv_blocks = k_in ? ctx->cfg.kv_head_count * ((n + 7) / 8) : 0;
        const int aligned8 = a.mirror_k && (ctx->batch_slot0 % 8 == 0) && (ctx->pf_mcap[layer] % 8 == 0);
        cfg.gridDim = dim3(n + kv_blocks);
        switch (ctx->geom.dtype) {
            case 0: e = cudaLaunchKernelEx(&cfg, hy3a_append_chunk_kernel<0>, cv, bv, ctx->rope, a, aligned8); break;
            case 1: e = cudaLaunchKernelEx(&cfg, hy3a_append_chunk_kernel<1>, cv, bv, ctx->rope, a, aligned8); break;
            default: e = cudaLaunchKernelEx(&cfg, hy3a_append_chunk_kernel<2>, cv, bv, ctx->rope, a, aligned8); break;
        }
        ctx->launches++;
        ctx->bulk_write_pending = 1;
        HY3A_CUDA(ctx, e);
        return HY3A_OK;
    }
    switch (ctx->geom.dtype) {
        case 0: e = cudaLaunchKernelEx(&cfg, hy3a_append_kernel<0>, cv, bv, ctx->rope, a); break;
        case 1: e = cudaLaunchKernelEx(&cfg, hy3a_append_kernel<1>, cv, bv, ctx->rope, a); break;
        default: e = cudaLaunchKernelEx(&cfg, hy3a_append_kernel<2>, cv, bv, ctx->rope, a); break;
    }
    ctx->launches++;
    if (ctx->batch_n > 1) ctx->bulk_write_pending = 1;
    HY3A_CUDA(ctx, e);
    return HY3A_OK;
}

int hy3a_launch_fill_random(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint64_t seed) {
    hy3a_cache_view cv = hy3a_view(ctx);
    ctx->bulk_write_pending = 1;
    for (int done = 0; done < n;) {
        int chunk = n - done > 32768 ? 32768 : n - done;
        dim3 grid(2, chunk), block(256);
        switch (ctx->geom.dtype) {
            case 0: hy3a_fill_random_kernel<0><<<grid, block, 0, ctx->stream>>>(cv, layer, seq, t0 + done, chunk, seed); break;
            case 1: hy3a_fill_random_kernel<1><<<grid, block, 0, ctx->stream>>>(cv, layer, seq, t0 + done, chunk, seed); break;
            default: hy3a_fill_random_kernel<2><<<grid, block, 0, ctx->stream>>>(cv, layer, seq, t0 + done, chunk, seed); break;
        }
        ctx->launches++;
        HY3A_CUDA(ctx, cudaGetLastError());
        done += chunk;
    }
    return HY3A_OK;
}

int hy3a_launch_export(hy3a_ctx *ctx, int layer, int seq, int t0, int n, uint8_t *d_kslots, uint8_t *d_vslots, int import) {
    hy3a_cache_view cv = hy3a_view(ctx);
    if (import) ctx->bulk_write_pending = 1;
    long long total = (long long)n * 8 * 32 * 2;
    int block = 256;
    unsigned grid = (unsigned)((total + block - 1) / block);
    switch (ctx->geom.dtype) {
        case 0: hy3a_xport_kernel<0><<<grid, block, 0, ctx->stream>>>(cv, layer, seq, t0, n, d_kslots, d_vslots, import); break;
        case 1: hy3a_xport_kernel<1><<<grid, block, 0, ctx->stream>>>(cv, layer, seq, t0, n, d_kslots, d_vslots, import); break;
        default: hy3a_xport_kernel<2><<<grid, block, 0, ctx->stream>>>(cv, layer, seq, t0, n, d_kslots, d_vslots, import); break;
    }
    ctx->launches++;
    HY3A_CUDA(ctx, cudaGetLastError());
    return HY3A_OK;
}
