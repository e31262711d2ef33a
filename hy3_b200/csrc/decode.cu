/*
 * decode.cu -- split-KV GQA decode attention over the paged FP16 / INT8 / INT4 cache.
 *
 * Replaces attention_split_kv[_int4]_kernel + attention_reduce_kernel of the reference
 * (hy3_gpu.cu:183-247, :274-325).  The reference runs one warp per (query head, split),
 * so every KV byte is fetched once per query head of its group (8x) with 4-byte loads at
 * an 83 KB stride.  Here a warp processes 16 tokens of one KV head for ALL 8 query heads
 * of the group at once, on tensor cores, so each KV byte is read exactly once:
 *
 *   S[16 x 8]  = Qsplit[16 x 128] . K^T      mma.sync m16n8k16, rows 0-7 = fp16(q) of the 8
 *                                            heads, rows 8-15 = the fp16 residual q - fp16(q)
 *                                            (M=16 is the MMA's minimum, so the second half
 *                                            of the tile buys ~fp32-accurate queries for free)
 *   O[16 x 128] += Psplit[16 x 16] . V       same trick: rows 8-15 carry the fp16 residual of P
 *
 * INT8/INT4 codes are converted to fp16 exactly (|code| <= 127) in registers with
 * byte-permute / lop3 magic-number tricks; the per-token scales are applied once per
 * score (K) and once per probability (V), never per element.  The contraction dimension
 * of Q.K^T and the output dimension of P.V are permuted so that every thread's MMA
 * operands are exactly the 16-byte chunks it loads -- no shuffles, no transposes.
 *
 * Scheduling: unit = one 128-token page of one (batch row, KV head); units are laid out
 * row-major, head, page and cut into `gridDim.x` contiguous ranges, so one launch shape
 * serves every length (lengths come from device memory; nothing is baked into a captured
 * graph, cf. hy3_gpu.cu:774-789).  A CTA's 8 warps each take 16 tokens of the current
 * page.  The piece a CTA computes for a (row, head) segment is merged in shared memory;
 * if the segment spans several CTAs each writes an {m, l, acc} record and the LAST CTA to
 * arrive (atomic counter) folds them -- the LSE-merge epilogue, no second launch.
 *
 * Roofline: HBM.  Algorithmic bytes per (token, KV head): 4 x 128 (FP16), 260 (INT8),
 * 132 (INT4); per token and layer x8.
 */
#include <cuda_fp16.h>
#include <math.h>

#include "ctx.h"

namespace {

constexpr int kWarps = HY3A_DECODE_WARPS;
constexpr int kThreads = kWarps * 32;
constexpr int kFixedO = kWarps * 8 * HY3A_D * 4;
constexpr int kFixedML = ((kWarps * 8 * 2 * 4) + 127) / 128 * 128;
constexpr int kFixedQ = 8 * 32 * 16;
constexpr int kFixed = kFixedO + kFixedML + kFixedQ;   /* bytes of shared memory in front of the page-count prefix */
constexpr int kSmemMax = 232448 - 1024;                /* opt-in limit per block minus the driver's reserve */
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ uint4 ld16(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned ld4(const uint8_t *p) {
    unsigned v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ unsigned hsub2(unsigned a, unsigned b) {
    unsigned r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ unsigned hfma2(unsigned a, unsigned b, unsigned c) {
    unsigned r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ unsigned pack_h2(float lo, float hi) {
    unsigned r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float2 unpack_h2(unsigned v) {
    __half2 h = *reinterpret_cast<__half2 *>(&v);
    return __half22float2(h);
}
__device__ __forceinline__ void mma16816(float c[4], const unsigned a[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

/* ---- exact integer-code -> fp16x2 conversions ---------------------------------------
 * INT8: xs = word ^ 0x80808080 turns each two's-complement byte into c+128; placing it
 * under the exponent byte 0x64 gives the fp16 number 1024 + (c+128); subtracting 1152
 * leaves c exactly.  sel picks which two bytes become the (low, high) halves.           */
__device__ __forceinline__ unsigned cvt_i8(unsigned xs, unsigned sel) { return hsub2(prmt(xs, 0x64646464u, sel), 0x64806480u); }
/* INT4: xs = word ^ 0x88888888 turns each nibble into n+8.  Nibbles (i, i+4) become one
 * fp16x2.  Low-position nibbles: (xs & 0x000f000f) | 0x6400 = 1024 + (n+8), minus 1032.
 * High-position nibbles: (xs & 0x00f000f0) | 0x6400 = 1024 + 16(n+8); *1/16 - 72 = n.    */
__device__ __forceinline__ unsigned cvt_i4_lo(unsigned xs) {
    unsigned v;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(v) : "r"(xs));
    return hsub2(v, 0x64086408u);
}
__device__ __forceinline__ unsigned cvt_i4_hi(unsigned xs) {
    unsigned v;
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(v) : "r"(xs));
    return hfma2(v, 0x2c002c00u /* 1/16 */, 0xd480d480u /* -72 */);
}

/* ---- contraction-dimension map of Q.K^T ---------------------------------------------
 * For k-step j (0..7) and thread-in-group tig, the four MMA k-slots
 * (2tig, 2tig+1, 2tig+8, 2tig+9) carry head dims kdim(j, tig, 0..3): exactly the dims
 * whose codes the thread gets out of its own 16-byte loads.                             */
template <int DT> __device__ __forceinline__ int kdim(int j, int tig, int s) {
    if (DT == 1) { int c = tig + 4 * (j >> 2); return 16 * c + 4 * (j & 3) + s; }
    if (DT == 2) { int base = 32 * tig + 8 * (j >> 1) + 2 * (j & 1); return base + (s >> 1) + 4 * (s & 1); }
    { int c = tig + 4 * (j >> 1); return 8 * c + 4 * (j & 1) + s; }
}
/* ---- output-dimension map of P.V: n-block jn (0..15), column n (0..7) -> head dim. */
template <int DT> __device__ __forceinline__ int vdim(int jn, int n) {
    if (DT == 2) return 16 * n + jn;
    return 8 * n + 64 * (jn >> 3) + (jn & 7);
}

struct decode_args {
    const float *q;
    size_t q_stride;
    float *out;
    size_t out_stride;
    float *user_partials; /* NULL or [n][8*kv_heads][130] */
    float *scratch;       /* [(gridDim.x + n*kv_heads)][8][130] */
    unsigned int *counters;
    unsigned int *err;
    int layer;
    int stages;           /* staged variant: pages in the shared-memory ring (2..8) */
    int prefix_bytes;     /* staged variant: bytes reserved for the page-count prefix */
};

struct warp_state {
    float m;      /* running max (base-2 logits), identical in the 4 lanes of a head */
    float l;      /* this lane's share of the denominator */
    float o[16][4];
};

struct segment {
    int row, hl, pages, p_begin, p_end, sidx, len, seq;
    long long seg_u0, seg_u1;
};

/* Locate the (row, local head) segment that contains unit u and the page range of it that
 * falls into [u, u_end).                                                                   */
__device__ __forceinline__ segment locate(const int *s_prefix, const hy3a_batch_view &batch, int n, int G, long long u, long long u_end) {
    segment sg;
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if ((long long)G * s_prefix[mid] <= u) lo = mid; else hi = mid - 1;
    }
    sg.row = lo;
    sg.pages = s_prefix[lo + 1] - s_prefix[lo];
    const long long row_u0 = (long long)G * s_prefix[lo];
    sg.hl = (int)((u - row_u0) / sg.pages);
    sg.seg_u0 = row_u0 + (long long)sg.hl * sg.pages;
    sg.seg_u1 = sg.seg_u0 + sg.pages;
    sg.p_begin = (int)(u - sg.seg_u0);
    sg.p_end = (int)((sg.seg_u1 < u_end ? sg.seg_u1 : u_end) - sg.seg_u0);
    sg.sidx = lo * G + sg.hl;
    sg.len = batch.slot[lo] + 1;
    sg.seq = batch.seq[lo];
    return sg;
}

/* ---- shared-memory / mbarrier / bulk-copy primitives (staged variant) ---------------- */
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds16(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ unsigned lds4(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_arrive(unsigned bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void *src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
/* Bounded wait: gives up after ~2^22 polls (far beyond any legitimate wait), records the
 * failure in the device error word and raises the CTA-wide abort flag; once the flag is up
 * every later wait returns at once, so all warps keep the same control flow and the kernel
 * runs to its end (with a meaningless result that the host discards on seeing the error). */
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int *abort_flag, unsigned *err, unsigned where) {
    if (mbar_test(bar, parity)) return true;
    for (unsigned i = 0; i < (1u << 22); i++) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 255u) == 255u) { if (*abort_flag) return false; __nanosleep(64); }
    }
    *abort_flag = 1;
    if (atomicCAS(err, 0u, 1u) == 0u) err[1] = where;
    return false;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

/* One 16-token granule of one warp: loads, S = Q.K^T, online softmax, O += P.V.
 * SM: operands come from a shared-memory copy of the page (addresses are 32-bit shared
 * addresses) instead of global memory.                                                  */
template <int DT, bool SM>
__device__ __forceinline__ void granule(warp_state &st, unsigned sq, const uint8_t *gpage, unsigned spage, const hy3a_geom &geom,
                                        const int (&k_off)[2][4], const int (&v_off)[8], const int (&sc_off)[2], int gi, int tig, int valid,
                                        float pscale) {
    /* page-relative byte offsets of granule gi (16 tokens = 16 K rows = 8 V pair-rows) */
    const int gk = gi * 16 * geom.k_row, gv = geom.v_off + gi * (DT == 0 ? 16 : 8) * geom.v_prow, gs = gi * 32;
    gpage += 0;
    constexpr int NK = DT == 0 ? 4 : (DT == 1 ? 2 : 1);
    constexpr int NV = DT == 0 ? 8 : (DT == 1 ? 4 : 2);
    uint4 kr[2][NK];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) {
#pragma unroll
        for (int i = 0; i < NK; i++) kr[nb][i] = SM ? lds16(spage + gk + k_off[nb][i]) : ld16(gpage + gk + k_off[nb][i]);
    }
    unsigned ksw[2] = {0, 0}, vsw[2] = {0, 0};
    if (DT != 0) {
#pragma unroll
        for (int nb = 0; nb < 2; nb++) {
            ksw[nb] = SM ? lds4(spage + geom.ks_off + gs + sc_off[nb]) : ld4(gpage + geom.ks_off + gs + sc_off[nb]);
            vsw[nb] = SM ? lds4(spage + geom.vs_off + gs + sc_off[nb]) : ld4(gpage + geom.vs_off + gs + sc_off[nb]);
        }
    }
    uint4 vr[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) vr[i] = SM ? lds16(spage + gv + v_off[i]) : ld16(gpage + gv + v_off[i]);
    /* Q operand fragments of this thread for the 8 k-steps, pre-packed in shared memory */
    unsigned qa[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++) { uint4 t = lds16(sq + j * 512); qa[j][0] = t.x; qa[j][1] = t.y; qa[j][2] = t.z; qa[j][3] = t.w; }

    /* ---- S = Q.K^T for the two 8-token n-blocks; even and odd k-steps accumulate separately so
     * that four independent MMA chains are in flight instead of two                              */
    float sc[2][4], sd[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) { sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f; sd[nb][0] = sd[nb][1] = sd[nb][2] = sd[nb][3] = 0.f; }
    if (DT == 1) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
#pragma unroll
            for (int r = 0; r < 4; r += 2) {
#pragma unroll
                for (int nb = 0; nb < 2; nb++) {
                    const unsigned w0 = (r == 0 ? kr[nb][i].x : kr[nb][i].z) ^ 0x80808080u;
                    const unsigned w1 = (r == 0 ? kr[nb][i].y : kr[nb][i].w) ^ 0x80808080u;
                    mma16816(sc[nb], qa[4 * i + r], cvt_i8(w0, 0x4140u), cvt_i8(w0, 0x4342u));
                    mma16816(sd[nb], qa[4 * i + r + 1], cvt_i8(w1, 0x4140u), cvt_i8(w1, 0x4342u));
                }
            }
        }
    } else if (DT == 2) {
#pragma unroll
        for (int r = 0; r < 4; r++) {
#pragma unroll
            for (int nb = 0; nb < 2; nb++) {
                const unsigned w = (r == 0 ? kr[nb][0].x : (r == 1 ? kr[nb][0].y : (r == 2 ? kr[nb][0].z : kr[nb][0].w)));
                const unsigned xs = w ^ 0x88888888u, xh = xs >> 8;
                mma16816(sc[nb], qa[2 * r], cvt_i4_lo(xs), cvt_i4_hi(xs));
                mma16816(sd[nb], qa[2 * r + 1], cvt_i4_lo(xh), cvt_i4_hi(xh));
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < NK; i++) {
#pragma unroll
            for (int nb = 0; nb < 2; nb++) {
                mma16816(sc[nb], qa[2 * i], kr[nb][i].x, kr[nb][i].y);
                mma16816(sd[nb], qa[2 * i + 1], kr[nb][i].z, kr[nb][i].w);
            }
        }
    }
#pragma unroll
    for (int nb = 0; nb < 2; nb++) { sc[nb][0] += sd[nb][0]; sc[nb][1] += sd[nb][1]; sc[nb][2] += sd[nb][2]; sc[nb][3] += sd[nb][3]; }
    /* ---- scores of head g for tokens 16w + 8nb + 2tig + e */
    float s[2][2], vs[2][2];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) {
        float2 kf = make_float2(1.f, 1.f), vf = make_float2(1.f, 1.f);
        if (DT != 0) { kf = unpack_h2(ksw[nb]); vf = unpack_h2(vsw[nb]); }
        int t0 = 16 * gi + 8 * nb + 2 * tig;
        float r0 = sc[nb][0] + sc[nb][2], r1 = sc[nb][1] + sc[nb][3];
        s[nb][0] = (t0 < valid) ? r0 * kf.x : -INFINITY;
        s[nb][1] = (t0 + 1 < valid) ? r1 * kf.y : -INFINITY;
        vs[nb][0] = (t0 < valid) ? vf.x * pscale : 0.f;
        vs[nb][1] = (t0 + 1 < valid) ? vf.y * pscale : 0.f;
    }
    float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m, mx); /* finite: token 16w of this granule is valid */
    if (__any_sync(0xffffffffu, m_new > st.m)) {
        const float alpha = ex2(st.m - m_new); /* 0 on the first granule (m = -inf) */
        st.l *= alpha;
#pragma unroll
        for (int jn = 0; jn < 16; jn++) { st.o[jn][0] *= alpha; st.o[jn][1] *= alpha; st.o[jn][2] *= alpha; st.o[jn][3] *= alpha; }
        st.m = m_new;
    }
    unsigned pa[4];
    {
        float w[2][2];
#pragma unroll
        for (int nb = 0; nb < 2; nb++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                float pe = ex2(s[nb][e] - st.m); /* -inf -> 0 */
                st.l += pe;
                w[nb][e] = pe * vs[nb][e];
            }
        }
        pa[0] = pack_h2(w[0][0], w[0][1]);
        pa[2] = pack_h2(w[1][0], w[1][1]);
        float2 h0 = unpack_h2(pa[0]), h1 = unpack_h2(pa[2]);
        pa[1] = pack_h2(w[0][0] - h0.x, w[0][1] - h0.y);
        pa[3] = pack_h2(w[1][0] - h1.x, w[1][1] - h1.y);
    }
    /* ---- O += P.V over 16 n-blocks of 8 output dims */
    if (DT == 1) {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            unsigned a4[4] = {vr[half].x, vr[half].y, vr[half].z, vr[half].w};
            unsigned b4[4] = {vr[2 + half].x, vr[2 + half].y, vr[2 + half].z, vr[2 + half].w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                unsigned xa = a4[k] ^ 0x80808080u, xb = b4[k] ^ 0x80808080u;
                mma16816(st.o[8 * half + 2 * k], pa, cvt_i8(xa, 0x4240u), cvt_i8(xb, 0x4240u));
                mma16816(st.o[8 * half + 2 * k + 1], pa, cvt_i8(xa, 0x4341u), cvt_i8(xb, 0x4341u));
            }
        }
    } else if (DT == 2) {
        unsigned a4[4] = {vr[0].x, vr[0].y, vr[0].z, vr[0].w};
        unsigned b4[4] = {vr[1].x, vr[1].y, vr[1].z, vr[1].w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            unsigned xa = a4[k] ^ 0x88888888u, xb = b4[k] ^ 0x88888888u, xah = xa >> 8, xbh = xb >> 8;
            mma16816(st.o[4 * k + 0], pa, cvt_i4_lo(xa), cvt_i4_lo(xb));
            mma16816(st.o[4 * k + 1], pa, cvt_i4_hi(xa), cvt_i4_hi(xb));
            mma16816(st.o[4 * k + 2], pa, cvt_i4_lo(xah), cvt_i4_lo(xbh));
            mma16816(st.o[4 * k + 3], pa, cvt_i4_hi(xah), cvt_i4_hi(xbh));
        }
    } else {
#pragma unroll
        for (int half = 0; half < 2; half++) {
            /* vr[2t + half]: token t (A,B = b0 pair; C,D = b1 pair), chunk g + 8*half */
            unsigned tA[4] = {vr[0 + half].x, vr[0 + half].y, vr[0 + half].z, vr[0 + half].w};
            unsigned tB[4] = {vr[2 + half].x, vr[2 + half].y, vr[2 + half].z, vr[2 + half].w};
            unsigned tC[4] = {vr[4 + half].x, vr[4 + half].y, vr[4 + half].z, vr[4 + half].w};
            unsigned tD[4] = {vr[6 + half].x, vr[6 + half].y, vr[6 + half].z, vr[6 + half].w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                mma16816(st.o[8 * half + 2 * k], pa, prmt(tA[k], tB[k], 0x5410u), prmt(tC[k], tD[k], 0x5410u));
                mma16816(st.o[8 * half + 2 * k + 1], pa, prmt(tA[k], tB[k], 0x7632u), prmt(tC[k], tD[k], 0x7632u));
            }
        }
    }
}

/* DIRECT variant: 8 warps, operands fetched straight from global memory with 128-bit loads.
 * STAGED variant: 8 consumer warps + 1 producer warp; the producer streams whole pages into a
 * shared-memory ring with bulk asynchronous copies (cp.async.bulk + mbarrier transaction
 * counts), consumers read their fragments from the ring.  Same arithmetic, same results.  */
template <int DT, bool STAGED>
__global__ void __launch_bounds__(kThreads + (STAGED ? 32 : 0), 1) hy3a_decode_kernel(hy3a_cache_view cache, hy3a_batch_view batch, decode_args a) {
    /* dynamic shared memory: [s_o | s_ml | s_q | page-count prefix | full[8] empty[8] | ring of pages] */
    extern __shared__ __align__(128) uint8_t s_dyn[];
    float (*s_o)[8][HY3A_D] = reinterpret_cast<float (*)[8][HY3A_D]>(s_dyn);                       /* per-warp unnormalised outputs */
    float (*s_ml)[8][2] = reinterpret_cast<float (*)[8][2]>(s_dyn + kFixedO);                      /* per-warp {m, l} */
    uint4 (*s_q)[32] = reinterpret_cast<uint4 (*)[32]>(s_dyn + kFixedO + kFixedML);                /* Q fragments: [k-step][lane] */
    __shared__ int s_flag;
    __shared__ int s_abort;

    const hy3a_geom geom = hy3a_make_geom(DT);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int n = batch.n, G = cache.kv_heads;
    const int cta = blockIdx.x;
    int *s_prefix = reinterpret_cast<int *>(s_dyn + kFixed);
    const unsigned bar_base = smem_u32(s_dyn + kFixed + a.prefix_bytes);
    const unsigned ring_base = bar_base + 128;

    /* ---- schedule: prefix of pages per row */
    for (int i = tid; i < n; i += blockDim.x) {
        int len = batch.slot[i] + 1;
        s_prefix[i + 1] = len > 0 ? (len + HY3A_PT - 1) / HY3A_PT : 0;
    }
    if (tid == 0) {
        s_prefix[0] = 0;
        s_abort = 0;
        if (STAGED) {
            for (int i = 0; i < a.stages; i++) { mbar_init(bar_base + 8 * i, 1); mbar_init(bar_base + 64 + 8 * i, 256); }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < n; base += 32) {
            int i = base + lane;
            int v = i < n ? s_prefix[i + 1] : 0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            if (i < n) s_prefix[i + 1] = v + carry;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();

    /* rows with no keys on this rank: zero output / empty partial (hy3_gpu.cu:197-199) */
    for (int i = cta; i < n; i += gridDim.x) {
        if (s_prefix[i + 1] != s_prefix[i]) continue;
        for (int e = tid; e < G * 8 * HY3A_D; e += blockDim.x) {
            int hq = e / HY3A_D, d = e % HY3A_D;
            if (a.user_partials) {
                float *p = a.user_partials + ((size_t)i * G * 8 + hq) * HY3A_PARTIAL_FLOATS;
                p[2 + d] = 0.f;
                if (d == 0) { p[0] = -INFINITY; p[1] = 0.f; }
            } else {
                a.out[(size_t)i * a.out_stride + (size_t)(cache.kv_head_begin * 8 + hq) * HY3A_D + d] = 0.f;
            }
        }
    }

    const long long U = (long long)G * s_prefix[n];
    /* never more CTAs than units, so that every participating CTA owns at least one unit and the
     * CTAs that share a segment are exactly the contiguous range [c_first, c_last]              */
    const int C = (long long)gridDim.x < U ? (int)gridDim.x : (int)U;
    if (cta >= C) return;
    const long long u_begin = (long long)cta * U / C, u_end = (long long)(cta + 1) * U / C;

    if (STAGED && warp == kWarps) {
        /* ================= producer warp: one lane streams the CTA's pages into the ring */
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            for (long long u = u_begin; u < u_end && ok;) {
                segment sg = locate(s_prefix, batch, n, G, u, u_end);
                const int *bt = cache.block_table + (size_t)sg.seq * cache.max_blocks_per_seq;
                int block_next = bt[sg.p_begin];
                for (int p = sg.p_begin; p < sg.p_end && ok; p++, it++) {
                    const unsigned stage = it % (unsigned)a.stages, phase = (it / (unsigned)a.stages) & 1u;
                    const int block = block_next;
                    if (p + 1 < sg.p_end) block_next = bt[p + 1];   /* in flight while we wait for the stage */
                    ok = mbar_wait(bar_base + 64 + 8 * stage, phase ^ 1u, &s_abort, a.err, 1u);
                    if (!ok) break;
                    const uint8_t *page = cache.pool + hy3a_page_index(cache, block, a.layer, sg.hl) * (size_t)cache.page_bytes;
                    mbar_expect_tx(bar_base + 8 * stage, (unsigned)geom.page_bytes);
                    bulk_g2s(ring_base + stage * (unsigned)geom.page_bytes, page, (unsigned)geom.page_bytes, bar_base + 8 * stage);
                }
                u = sg.seg_u0 + sg.p_end;
            }
            if (!ok) {
                /* gave up: let the copies already issued land before the CTA's shared memory goes away */
                const unsigned first = it > (unsigned)a.stages ? it - (unsigned)a.stages : 0u;
                for (unsigned j = first; j < it; j++) {
                    const unsigned stage = j % (unsigned)a.stages, phase = (j / (unsigned)a.stages) & 1u;
                    for (unsigned spin = 0; spin < (1u << 20) && !mbar_test(bar_base + 8 * stage, phase); spin++) __nanosleep(64);
                }
            }
        }
        return;
    }

    /* ================= consumer warps */
    int k_off[2][4];   /* [n-block][chunk], page-relative, loop invariant */
    int v_off[8];
    int sc_off[2];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) {
        int tok = 8 * nb + g;
        if (DT == 1) { k_off[nb][0] = hy3a_k_chunk_off<1>(tok, tig); k_off[nb][1] = hy3a_k_chunk_off<1>(tok, tig + 4); k_off[nb][2] = k_off[nb][3] = 0; }
        else if (DT == 2) { k_off[nb][0] = hy3a_k_chunk_off<2>(tok, tig); k_off[nb][1] = k_off[nb][2] = k_off[nb][3] = 0; }
        else { for (int i = 0; i < 4; i++) k_off[nb][i] = hy3a_k_chunk_off<0>(tok, tig + 4 * i); }
        sc_off[nb] = 2 * (8 * nb + 2 * tig);
    }
    {
        int pr0 = tig, pr1 = pr0 + 4;
        if (DT == 1) {
            v_off[0] = hy3a_v_chunk_off<1>(pr0, g); v_off[1] = hy3a_v_chunk_off<1>(pr0, g + 8);
            v_off[2] = hy3a_v_chunk_off<1>(pr1, g); v_off[3] = hy3a_v_chunk_off<1>(pr1, g + 8);
            v_off[4] = v_off[5] = v_off[6] = v_off[7] = 0;
        } else if (DT == 2) {
            v_off[0] = hy3a_v_chunk_off<2>(pr0, g); v_off[1] = hy3a_v_chunk_off<2>(pr1, g);
            for (int i = 2; i < 8; i++) v_off[i] = 0;
        } else {
            int tA = 2 * tig;
            for (int t = 0; t < 4; t++) {
                int tok = tA + (t & 1) + 8 * (t >> 1);
                v_off[2 * t] = hy3a_v16_chunk_off(tok, g);
                v_off[2 * t + 1] = hy3a_v16_chunk_off(tok, g + 8);
            }
        }
    }

    unsigned it = 0; /* pages consumed by this CTA so far (ring position) */
    long long u = u_begin;
    while (u < u_end) {
        const segment sg = locate(s_prefix, batch, n, G, u, u_end);
        const int row = sg.row, hl = sg.hl, sidx = sg.sidx;

        /* ---- Q operand fragments: fp16 value in rows 0-7, fp16 residual in rows 8-15.
         * softmax scale 1/sqrt(128) (hy3_gpu.cu:193) and log2(e) are folded into Q.  Thread t < 256
         * packs the entry of k-step t/32 for lane t%32; every warp then reads its lanes' entries. */
        if (tid < 256) {
            const int j = tid >> 5;
            const float *qh = a.q + (size_t)row * a.q_stride + (size_t)((cache.kv_head_begin + hl) * 8 + g) * HY3A_D;
            const float qs = 0.08838834764831845f * kLog2e;
            float x[4], hi4[4], lo4[4];
#pragma unroll
            for (int s = 0; s < 4; s++) x[s] = qh[kdim<DT>(j, tig, s)] * qs;
#pragma unroll
            for (int s = 0; s < 4; s++) { hi4[s] = __half2float(__float2half_rn(x[s])); lo4[s] = x[s] - hi4[s]; }
            s_q[j][lane] = make_uint4(pack_h2(hi4[0], hi4[1]), pack_h2(lo4[0], lo4[1]), pack_h2(hi4[2], hi4[3]), pack_h2(lo4[2], lo4[3]));
        }
        consumer_sync();
        const unsigned sq = smem_u32(&s_q[0][lane]);
        /* P scale: w = p * vscale * 2^E with vs_max * 2^E <= 2^14, so fp16 P never
         * overflows and its subnormal floor sits 2^-38 below the row maximum.          */
        float pscale;
        {
            int E = 14;
            if (DT != 0) {
                unsigned vb = cache.vs_max[a.layer * G + hl];
                __half_raw hr; hr.x = (unsigned short)vb;
                float vmax = __half2float(__half(hr));
                int ex;
                frexpf(fmaxf(vmax, 1e-30f), &ex); /* vmax < 2^ex */
                E = 14 - ex;
                E = E > 60 ? 60 : (E < -60 ? -60 : E);
            }
            pscale = exp2f((float)E);
        }

        warp_state st;
        st.m = -INFINITY; st.l = 0.f;
#pragma unroll
        for (int jn = 0; jn < 16; jn++) { st.o[jn][0] = st.o[jn][1] = st.o[jn][2] = st.o[jn][3] = 0.f; }

        /* granule slot x = 8*(ring position of the page) + granule-in-page; warp w takes slots
         * x = w (mod kWarps), so any number of consumer warps shares the 8 granules of a page and
         * each page is released by exactly 8 warps (one arrival per thread per slot).            */
        const unsigned it_end = it + (unsigned)(sg.p_end - sg.p_begin);
        for (unsigned x = it * 8u + ((unsigned)warp + kWarps - (it * 8u) % kWarps) % kWarps; x < it_end * 8u; x += kWarps) {
            const unsigned pit = x >> 3;
            const int gi = (int)(x & 7u), p = sg.p_begin + (int)(pit - it);
            const int valid = min(HY3A_PT, sg.len - p * HY3A_PT);
            if (STAGED) {
                const unsigned stage = pit % (unsigned)a.stages, phase = (pit / (unsigned)a.stages) & 1u;
                mbar_wait(bar_base + 8 * stage, phase, &s_abort, a.err, 2u);
                if (16 * gi < valid)
                    granule<DT, true>(st, sq, nullptr, ring_base + stage * (unsigned)geom.page_bytes, geom, k_off, v_off, sc_off, gi, tig, valid, pscale);
                mbar_arrive(bar_base + 64 + 8 * stage); /* every thread of the 8 warps that share a page releases it */
            } else {
                if (16 * gi >= valid) continue; /* warp-uniform */
                const int block = cache.block_table[(size_t)sg.seq * cache.max_blocks_per_seq + p];
                const uint8_t *page = cache.pool + hy3a_page_index(cache, block, a.layer, hl) * (size_t)cache.page_bytes;
                granule<DT, false>(st, sq, page, 0u, geom, k_off, v_off, sc_off, gi, tig, valid, pscale);
            }
        }
        it = it_end;

        /* ---- fold the 8 warps of this CTA (shared memory) */
        {
            float l = st.l;
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            if (tig == 0) { s_ml[warp][g][0] = st.m; s_ml[warp][g][1] = l; }
            const float inv_ps = 1.f / pscale;
#pragma unroll
            for (int jn = 0; jn < 16; jn++) {
                s_o[warp][g][vdim<DT>(jn, 2 * tig)] = (st.o[jn][0] + st.o[jn][2]) * inv_ps;
                s_o[warp][g][vdim<DT>(jn, 2 * tig + 1)] = (st.o[jn][1] + st.o[jn][3]) * inv_ps;
            }
        }
        consumer_sync();
        const bool red = tid < 256;                            /* the first 8 warps do the reductions */
        const int h = (tid >> 5) & 7, d4 = (tid & 31) * 4;    /* thread -> (head, 4 dims) */
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; w++) M = fmaxf(M, s_ml[w][h][0]);
        float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < kWarps; w++) {
            float mw = s_ml[w][h][0];
            if (mw == -INFINITY) continue;
            float f = ex2(mw - M);
            L += s_ml[w][h][1] * f;
            float4 o4 = *reinterpret_cast<const float4 *>(&s_o[w][h][d4]);
            acc[0] += o4.x * f; acc[1] += o4.y * f; acc[2] += o4.z * f; acc[3] += o4.w * f;
        }
        consumer_sync(); /* s_o / s_ml free for the next segment */

        /* ---- how many CTAs share this segment? */
        const int c_first = (int)(((sg.seg_u0 + 1) * C + U - 1) / U) - 1;
        const int c_last = (int)((sg.seg_u1 * C + U - 1) / U) - 1;
        const int npieces = c_last - c_first + 1;
        const size_t head_q = (size_t)(cache.kv_head_begin + hl) * 8 + h; /* global query head */
        u = sg.seg_u0 + sg.p_end;

        if (npieces > 1) {
            float *rec = a.scratch + ((size_t)(cta + sidx) * 8 + h) * HY3A_PARTIAL_FLOATS;
            if (red) {
                if (d4 == 0) { rec[0] = M; rec[1] = L; }
                rec[2 + d4] = acc[0]; rec[3 + d4] = acc[1]; rec[4 + d4] = acc[2]; rec[5 + d4] = acc[3];
            }
            __threadfence();
            consumer_sync();
            if (tid == 0) {
                unsigned old = atomicAdd(a.counters + sidx, 1u);
                s_flag = (old == (unsigned)(npieces - 1));
            }
            consumer_sync();
            if (!s_flag || !red) continue;
            __threadfence();
            /* last arrival: fold all pieces (hy3_gpu.cu:233-247 rule).  Two passes so that the
             * loads of different pieces are independent and overlap: first the maxima, then the
             * rescaled sums.  __ldcg reads L2, where the other CTAs' records are after their fence. */
            M = -INFINITY;
            for (int c = c_first; c <= c_last; c++) {
                const float *pr = a.scratch + ((size_t)(c + sidx) * 8 + h) * HY3A_PARTIAL_FLOATS;
                const float pm = __ldcg(pr), pl = __ldcg(pr + 1);
                M = fmaxf(M, pl > 0.f ? pm : -INFINITY);
            }
            L = 0.f; acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll 4
            for (int c = c_first; c <= c_last; c++) {
                const float *pr = a.scratch + ((size_t)(c + sidx) * 8 + h) * HY3A_PARTIAL_FLOATS;
                const float pm = __ldcg(pr), pl = __ldcg(pr + 1);
                const float2 a01 = __ldcg(reinterpret_cast<const float2 *>(pr + 2 + d4)), a23 = __ldcg(reinterpret_cast<const float2 *>(pr + 4 + d4));
                const float rs = pl > 0.f ? ex2(pm - M) : 0.f;
                L += pl * rs;
                acc[0] += a01.x * rs; acc[1] += a01.y * rs; acc[2] += a23.x * rs; acc[3] += a23.y * rs;
            }
            if (tid == 0) a.counters[sidx] = 0u; /* self-reset for the next launch */
        }
        if (!red) continue;
        if (a.user_partials) {
            float *rec = a.user_partials + ((size_t)row * G * 8 + (size_t)hl * 8 + h) * HY3A_PARTIAL_FLOATS;
            if (d4 == 0) { rec[0] = M * kLn2; rec[1] = L; } /* m in natural-log units like the reference record */
            rec[2 + d4] = acc[0]; rec[3 + d4] = acc[1]; rec[4 + d4] = acc[2]; rec[5 + d4] = acc[3];
        } else {
            float inv = L > 0.f ? 1.f / L : 0.f;
            float4 o4 = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
            *reinterpret_cast<float4 *>(a.out + (size_t)row * a.out_stride + head_q * HY3A_D + d4) = o4;
        }
    }
}

/* Merge kernel for cross-GPU partials: grid (n_rows*n_heads), block 32; lane -> 4 dims. */
__global__ void hy3a_merge_kernel(const float *partials, int n_parts, int n_rows, int n_heads, float *out, size_t out_stride) {
    int rh = blockIdx.x, lane = threadIdx.x;
    int row = rh / n_heads, h = rh % n_heads;
    float ms = -INFINITY, ss = 0.f, ov[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n_parts; s++) {
        const float *p = partials + ((size_t)s * n_rows * n_heads + rh) * HY3A_PARTIAL_FLOATS;
        float pms = p[0], pss = p[1];
        if (!(pss > 0.f)) continue;
        float nm = fmaxf(ms, pms), os = __expf(ms - nm), rs = __expf(pms - nm);
        ss = ss * os + pss * rs;
#pragma unroll
        for (int j = 0; j < 4; j++) ov[j] = ov[j] * os + p[2 + lane * 4 + j] * rs;
        ms = nm;
    }
    float inv = ss > 0.f ? 1.f / ss : 0.f;
    *reinterpret_cast<float4 *>(out + (size_t)row * out_stride + (size_t)h * HY3A_D + lane * 4) = make_float4(ov[0] * inv, ov[1] * inv, ov[2] * inv, ov[3] * inv);
}

} /* namespace */

template <int DT>
static cudaError_t launch_decode_dt(hy3a_ctx *ctx, const hy3a_cache_view &cv, const hy3a_batch_view &bv, decode_args &a) {
    const size_t prefix = ((size_t)(ctx->batch_n + 1) * sizeof(int) + 127) & ~(size_t)127;
    dim3 grid(ctx->decode_ctas);
    static bool attr_set[3][2] = {{false, false}, {false, false}, {false, false}};
    a.prefix_bytes = (int)prefix;
    if (ctx->decode_stages >= 2) {
        a.stages = ctx->decode_stages;
        const size_t smem = kFixed + prefix + 128 + (size_t)a.stages * ctx->geom.page_bytes;
        if (!attr_set[DT][1]) {
            cudaError_t e = cudaFuncSetAttribute(hy3a_decode_kernel<DT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
            if (e != cudaSuccess) return e;
            attr_set[DT][1] = true;
        }
        hy3a_decode_kernel<DT, true><<<grid, kThreads + 32, smem, ctx->stream>>>(cv, bv, a);
    } else {
        a.stages = 0;
        if (!attr_set[DT][0]) {
            cudaError_t e = cudaFuncSetAttribute(hy3a_decode_kernel<DT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
            if (e != cudaSuccess) return e;
            attr_set[DT][0] = true;
        }
        hy3a_decode_kernel<DT, false><<<grid, kThreads, kFixed + prefix + 128, ctx->stream>>>(cv, bv, a);
    }
    return cudaGetLastError();
}

/* Pages that fit in the ring for a given page size and batch capacity. */
int hy3a_decode_ring_capacity(int page_bytes, int max_batch) {
    const size_t prefix = ((size_t)(max_batch + 1) * sizeof(int) + 127) & ~(size_t)127;
    long room = (long)kSmemMax - (long)kFixed - (long)prefix - 128;
    int s = room > 0 ? (int)(room / page_bytes) : 0;
    return s > 8 ? 8 : s;
}

int hy3a_launch_decode(hy3a_ctx *ctx, int layer, const float *q, size_t q_stride, float *out, size_t out_stride, float *partials) {
    decode_args a;
    a.q = q; a.q_stride = q_stride; a.out = out; a.out_stride = out_stride; a.user_partials = partials;
    a.scratch = ctx->d_partials; a.counters = ctx->d_counters; a.err = ctx->d_err; a.layer = layer;
    hy3a_cache_view cv = hy3a_view(ctx);
    hy3a_batch_view bv = hy3a_bview(ctx);
    cudaError_t e;
    switch (ctx->cfg.kv_dtype) {
        case 0: e = launch_decode_dt<0>(ctx, cv, bv, a); break;
        case 1: e = launch_decode_dt<1>(ctx, cv, bv, a); break;
        default: e = launch_decode_dt<2>(ctx, cv, bv, a); break;
    }
    ctx->launches++;
    if (e != cudaSuccess) return hy3a_fail(ctx, HY3A_ECUDA, "decode launch: %s", cudaGetErrorString(e));
    return HY3A_OK;
}

int hy3a_launch_merge(hy3a_ctx *ctx, const float *partials, int n_parts, int n_rows, int n_heads, float *out, size_t out_stride) {
    hy3a_merge_kernel<<<n_rows * n_heads, 32, 0, ctx->stream>>>(partials, n_parts, n_rows, n_heads, out, out_stride);
    ctx->launches++;
    HY3A_CUDA(ctx, cudaGetLastError());
    return HY3A_OK;
}
