/*
 * decode.cu -- split-KV GQA decode attention over the paged FP16 and INT4 caches (INT8 caches: decode_umma.cu),
 * the launch entry points of all three, and the merge kernel.
 *
 * Replaces attention_split_kv[_int4]_kernel + attention_reduce_kernel of the reference
 * (hy3_gpu.cu:183-247, :274-325).  The reference runs one warp per (query head, split),
 * so every KV byte is fetched once per query head of its group (8x) with 4-byte loads at
 * an 83 KB stride.  Here a warp processes 16 tokens of one KV head for ALL 8 query heads
 * of the group at once, on tensor cores, so each KV byte is read exactly once:
 *
 *   S[16 x 8]   = Q2[16 x 128] . K^T    rows 0-7 = the 8 heads, rows 8-15 = a residual of the
 *                                       same 8 queries (M=16 is the MMA minimum, so the second
 *                                       half of the tile buys near-fp32 queries for free).
 *                                       INT4 cache: integer MMA (m16n8k32.s8) directly on the
 *                                       stored nibbles -- Q is split into two int8 digits
 *                                       (q ~ sq*(hi + lo/254)), the products are exact, and no
 *                                       per-element conversion of K is needed at all.
 *                                       FP16 cache: m16n8k16.f16 with Q = fp16 + fp16 residual.
 *   O[16 x 128] += P[16 x 16] . V       m16n8k16.f16; INT4 codes become fp16 exactly with one lop3 +
 *                                       one fp16 subtract (or fma) per pair.
 *
 * The per-token scales are applied once per score (K) and once per probability (V), never
 * per element.  The contraction dimension of Q.K^T and the output dimension of P.V are
 * permuted so that every thread's MMA operands are exactly the 16-byte chunks it loads.
 *
 * Scheduling: unit = one 128-token page of one (batch row, KV head); units are laid out
 * row-major, head, page and cut into contiguous ranges, one per CTA, so one launch shape
 * serves every length (lengths come from device memory; nothing is baked into a captured
 * graph, cf. hy3_gpu.cu:774-789).  A producer warp streams the CTA's pages into a shared-
 * memory ring with bulk asynchronous copies (cp.async.bulk + mbarrier transaction counts);
 * the consumer warps take the 16-token granules of the pages round-robin.  The piece a CTA
 * computes for a (row, head) segment is folded in shared memory; if the segment spans
 * several CTAs each writes an {m, l, acc} record and the LAST CTA to arrive (atomic
 * counter) folds them -- the LSE-merge epilogue, no second launch.
 *
 * Roofline: HBM.  Algorithmic bytes per (token, KV head): 512 (FP16), 132 (INT4); per token and
 * layer x8.
 */
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>

#include "ctx.h"
#include "decode_common.cuh"
#include "rowops.cuh"

namespace {

constexpr int kWarps = HY3A_DECODE_WARPS;              /* consumer warps */
static_assert(kWarps >= 8, "the Q packing and the reductions use the first 8 consumer warps");
constexpr int kThreads = kWarps * 32;
constexpr int kFixedO = kWarps * 8 * HY3A_D * 4;
constexpr int kFixedML = ((kWarps * 8 * 2 * 4) + 127) / 128 * 128;
constexpr int kFixedQ = 8 * 32 * 16;
constexpr int kBarBytes = 256;      /* mbarriers of the page ring: empty[8], full[16] */
constexpr int kFixed = kFixedO + kFixedML + kFixedQ;   /* bytes of shared memory in front of the page-count prefix */
constexpr bool kPSplit = true;                         /* carry the fp16 residual of P in MMA rows 8-15 */
constexpr int kRecFloats = HY3A_REC_FLOATS;             /* floats per head record in the merge scratch (130 used) */
constexpr int kShardBatch = 5;                          /* ranks polled at once by the sharded epilogue */
static_assert(kShardBatch * 8 * (HY3A_PARTIAL_FLOATS / 2) * 16 <= kFixedO, "landing zone of the rank records exceeds the staging area");
constexpr float kRescaleThreshold = 8.f;               /* lazy rescale: the running max may lag by 2^8 */

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
__device__ __forceinline__ void mma16816(float c[4], const unsigned a[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

/* ---- exact integer-code -> fp16x2 conversions of V --------------------------------------
 * INT4 V codes are stored offset-binary (n+8; see append.cu), so that no sign fix-up is needed here. */
/* INT4: nibbles (i, i+4) become one fp16x2.  Low positions: (x & 0x000f000f) | 0x6400 =
 * 1024 + (n+8), minus 1032.  High positions: (x & 0x00f000f0) | 0x6400 = 1024 + 16(n+8);
 * times 1/16 minus 72 = n.                                                               */
__device__ __forceinline__ unsigned cvt_u4_lo(unsigned x) {
    unsigned v;
    asm("lop3.b32 %0, %1, 0x000f000f, 0x64006400, 0xea;" : "=r"(v) : "r"(x));
    return hsub2(v, 0x64086408u);
}
__device__ __forceinline__ unsigned cvt_u4_hi(unsigned x) {
    unsigned v;
    asm("lop3.b32 %0, %1, 0x00f000f0, 0x64006400, 0xea;" : "=r"(v) : "r"(x));
    return hfma2(v, 0x2c002c00u /* 1/16 */, 0xd480d480u /* -72 */);
}

/* ---- contraction-dimension maps of Q.K^T -------------------------------------------------
 * FP16 cache (m16n8k16): for k-step j (0..7) the four MMA k-slots (2tig, 2tig+1, 2tig+8,
 * 2tig+9) of thread-in-group tig carry head dims kdim16(j, tig, 0..3).
 * INT8/INT4 caches (m16n8k32): for k-step kk (0..3) the eight k-slots (4tig..4tig+3,
 * 16+4tig..16+4tig+3) carry head dims kdim32<DT>(kk, tig, 0..7).  In both cases these are
 * exactly the dims whose codes the thread gets out of its own 16-byte loads.              */
__device__ __forceinline__ int kdim16(int j, int tig, int s) { int c = tig + 4 * (j >> 1); return 8 * c + 4 * (j & 1) + s; }
/* ---- output-dimension map of P.V: n-block jn (0..15), column n (0..7) -> head dim. */
template <int DT> __device__ __forceinline__ int vdim(int jn, int n) {
    if (DT == 2) return 16 * n + jn;
    return 8 * n + 64 * (jn >> 3) + (jn & 7);
}

struct warp_state {
    float m;      /* reference max (base-2 logits), identical in the 4 lanes of a head; may lag the true max by 2^8 */
    float l;      /* this lane's share of the denominator */
    float o[16][4];
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

/* One 16-token granule of one warp: loads, S = Q.K^T, online softmax, O += P.V.
 * SM: operands come from a shared-memory copy of the page (32-bit shared addresses) instead
 * of global memory.  FULL: all 16 tokens are valid (no masking).  sq: shared address of this
 * lane's Q fragments; qf: score factor of this lane's head (integer-MMA path).             */
template <int DT, bool SM, bool FULL>
__device__ __forceinline__ void granule(warp_state &st, unsigned sq, float qf, const uint8_t *gpage, unsigned spage, const hy3a_geom &geom,
                                        const int (&k_off)[2][4], const int (&v_off)[8], const int (&sc_off)[2], int gi, int tig, int valid,
                                        float pscale) {
    static_assert(DT == 0 || DT == 2, "INT8 caches are served by decode_umma.cu");
    constexpr int NK = DT == 0 ? 4 : 1;
    constexpr int NV = DT == 0 ? 8 : 2;
    /* page-relative byte offsets of granule gi (16 tokens = 16 K rows = 8 V pair-rows) */
    const int gk = gi * 16 * geom.k_row, gv = geom.v_off + gi * (DT == 0 ? 16 : 8) * geom.v_prow, gs = gi * 32;
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

    /* ---- raw scores r[nb][e] of head g for tokens 16gi + 8nb + 2tig + e (before the K scale) */
    float r[2][2];
    if (DT == 0) {
        unsigned qa[8][4];
#pragma unroll
        for (int j = 0; j < 8; j++) { uint4 t = lds16(sq + j * 512); qa[j][0] = t.x; qa[j][1] = t.y; qa[j][2] = t.z; qa[j][3] = t.w; }
        float sc[2][4], sd[2][4];   /* even / odd k-steps accumulate separately: four independent MMA chains */
#pragma unroll
        for (int nb = 0; nb < 2; nb++) { sc[nb][0] = sc[nb][1] = sc[nb][2] = sc[nb][3] = 0.f; sd[nb][0] = sd[nb][1] = sd[nb][2] = sd[nb][3] = 0.f; }
#pragma unroll
        for (int i = 0; i < NK; i++) {
#pragma unroll
            for (int nb = 0; nb < 2; nb++) {
                mma16816(sc[nb], qa[2 * i], kr[nb][i].x, kr[nb][i].y);
                mma16816(sd[nb], qa[2 * i + 1], kr[nb][i].z, kr[nb][i].w);
            }
        }
#pragma unroll
        for (int nb = 0; nb < 2; nb++) { r[nb][0] = (sc[nb][0] + sd[nb][0]) + (sc[nb][2] + sd[nb][2]); r[nb][1] = (sc[nb][1] + sd[nb][1]) + (sc[nb][3] + sd[nb][3]); }
    } else {
        uint4 qa[4];
#pragma unroll
        for (int kk = 0; kk < 4; kk++) qa[kk] = lds16(sq + kk * 512);
        int ce[2][4], co[2][4];     /* even / odd k-steps: four independent integer-MMA chains */
#pragma unroll
        for (int nb = 0; nb < 2; nb++) { ce[nb][0] = ce[nb][1] = ce[nb][2] = ce[nb][3] = 0; co[nb][0] = co[nb][1] = co[nb][2] = co[nb][3] = 0; }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
#pragma unroll
            for (int nb = 0; nb < 2; nb++) {
                /* two's-complement nibbles: moving a nibble to the top of its byte gives 16 x code as int8 */
                const unsigned w = kk == 0 ? kr[nb][0].x : (kk == 1 ? kr[nb][0].y : (kk == 2 ? kr[nb][0].z : kr[nb][0].w));
                const unsigned b0 = (w << 4) & 0xF0F0F0F0u, b1 = w & 0xF0F0F0F0u;
                imma16832((kk & 1) ? co[nb] : ce[nb], qa[kk], b0, b1);
            }
        }
        /* rows 0-7 carry the high digit of q, rows 8-15 the low digit: q ~ sq*(hi + lo/254) */
#pragma unroll
        for (int nb = 0; nb < 2; nb++) {
            r[nb][0] = (float)((ce[nb][0] + co[nb][0]) * 254 + (ce[nb][2] + co[nb][2])) * qf;
            r[nb][1] = (float)((ce[nb][1] + co[nb][1]) * 254 + (ce[nb][3] + co[nb][3])) * qf;
        }
    }
    /* ---- logits (base 2) and V scales */
    float s[2][2], vs[2][2];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) {
        float2 kf = make_float2(1.f, 1.f), vf = make_float2(1.f, 1.f);
        if (DT != 0) { kf = unpack_h2(ksw[nb]); vf = unpack_h2(vsw[nb]); }
        const int t0 = 16 * gi + 8 * nb + 2 * tig;
        s[nb][0] = (FULL || t0 < valid) ? r[nb][0] * kf.x : -INFINITY;
        s[nb][1] = (FULL || t0 + 1 < valid) ? r[nb][1] * kf.y : -INFINITY;
        vs[nb][0] = (FULL || t0 < valid) ? vf.x * pscale : 0.f;
        vs[nb][1] = (FULL || t0 + 1 < valid) ? vf.y * pscale : 0.f;
    }
    /* ---- online softmax with a lazily updated reference max: O and l are only rescaled when
     * the granule's max exceeds the reference by more than 2^8; until then p <= 2^8, which the
     * fp16 range of P has room for (pscale leaves 2^8 of headroom).                           */
    float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));   /* finite: token 16gi of this granule is valid */
    const bool grow = mx > st.m + kRescaleThreshold;       /* also true while st.m == -inf */
    if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? mx : st.m;
        const float alpha = ex2(st.m - m_new);             /* 0 on the first granule (m = -inf), 1 if unchanged */
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
                const float pe = ex2(s[nb][e] - st.m); /* -inf -> 0 */
                st.l += pe;
                w[nb][e] = pe * vs[nb][e];
            }
        }
        pa[0] = pack_h2(w[0][0], w[0][1]);
        pa[2] = pack_h2(w[1][0], w[1][1]);
        if (kPSplit) {
            float2 h0 = unpack_h2(pa[0]), h1 = unpack_h2(pa[2]);
            pa[1] = pack_h2(w[0][0] - h0.x, w[0][1] - h0.y);
            pa[3] = pack_h2(w[1][0] - h1.x, w[1][1] - h1.y);
        } else {
            pa[1] = pa[3] = 0u;
        }
    }
    /* ---- O += P.V over 16 n-blocks of 8 output dims */
    if (DT == 2) {
        unsigned a4[4] = {vr[0].x, vr[0].y, vr[0].z, vr[0].w};
        unsigned b4[4] = {vr[1].x, vr[1].y, vr[1].z, vr[1].w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const unsigned xa = a4[k], xb = b4[k], xah = xa >> 8, xbh = xb >> 8;
            mma16816(st.o[4 * k + 0], pa, cvt_u4_lo(xa), cvt_u4_lo(xb));
            mma16816(st.o[4 * k + 1], pa, cvt_u4_hi(xa), cvt_u4_hi(xb));
            mma16816(st.o[4 * k + 2], pa, cvt_u4_lo(xah), cvt_u4_lo(xbh));
            mma16816(st.o[4 * k + 3], pa, cvt_u4_hi(xah), cvt_u4_hi(xbh));
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

/* DIRECT variant (STAGED=false): operands fetched straight from global memory with 128-bit
 * loads (no ring, no producer).  STAGED variant: kWarps consumer warps + 1 producer warp.
 * Same arithmetic, same results.                                                          */
/* SHARD: the sequence-sharded variant (exchange + final fold in the epilogue); a separate instantiation so that the
 * single-GPU kernel's register allocation is untouched by it. */
template <int DT, bool STAGED, bool SHARD = false>
__global__ void __launch_bounds__(kThreads + (STAGED ? 32 : 0), 1) hy3a_decode_kernel(hy3a_cache_view cache, hy3a_batch_view batch, decode_args a) {
    /* dynamic shared memory: [s_o | s_ml | s_q | page-count prefix | full[8] empty[8] | ring of pages] */
    extern __shared__ __align__(128) uint8_t s_dyn[];
    float (*s_o)[8][HY3A_D] = reinterpret_cast<float (*)[8][HY3A_D]>(s_dyn);                       /* per-warp unnormalised outputs */
    float (*s_ml)[8][2] = reinterpret_cast<float (*)[8][2]>(s_dyn + kFixedO);                      /* per-warp {m, l} */
    uint4 (*s_q)[32] = reinterpret_cast<uint4 (*)[32]>(s_dyn + kFixedO + kFixedML);                /* Q fragments: [k-step][lane] */
    __shared__ float s_qf[8];
    __shared__ unsigned s_vnew;
    __shared__ int s_flag;
    __shared__ int s_abort;

    const hy3a_geom geom = hy3a_make_geom(DT);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int n = batch.n, G = cache.kv_heads;
    const int cta = blockIdx.x;

    int *s_prefix = reinterpret_cast<int *>(s_dyn + kFixed);
    const unsigned bar_base = smem_u32(s_dyn + kFixed + a.prefix_bytes);
    const unsigned ring_base = bar_base + kBarBytes;

    /* ---- schedule: prefix of pages per row */
    for (int i = tid; i < n; i += blockDim.x) {
        int len = batch.slot[i] + 1;
        s_prefix[i + 1] = len > 0 ? (len + HY3A_PT - 1) / HY3A_PT : 0;
    }
    if (tid == 0) {
        s_prefix[0] = 0;
        s_abort = 0;
        if (STAGED) {
            for (int i = 0; i < a.stages; i++) mbar_init(bar_base + 8 * i, 256);          /* empty[stage]: every thread of the 8 warps that share a page */
            for (int i = 0; i < 2 * a.stages; i++) mbar_init(bar_base + 64 + 8 * i, 1);   /* full[page mod 2 stages]: the producer's expect_tx */
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    __syncthreads();
    if (warp == 0 && n > 1) {
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

    const long long U = (long long)G * s_prefix[n];
    bool idle = (U == 0);
    /* Two ways to cut the units into per-CTA ranges:
     *  - few segments (n*G < grid): every segment gets its own whole number of CTAs, roughly in
     *    proportion to its pages, so no CTA straddles two segments (a straddling CTA pays the
     *    query set-up and the fold twice and becomes the critical path of a small batch);
     *  - many segments: one contiguous, equally sized range per CTA over all units.
     * In both, never more CTAs than units, and the CTAs sharing a segment are contiguous.       */
    const bool aligned = (long long)n * G < (long long)gridDim.x && aligned_split_balanced(s_prefix, n, G, gridDim.x, lane);
    int C = (long long)gridDim.x < U ? (int)gridDim.x : (int)U;
    long long u_begin = 0, u_end = 0;
    int al_first = 0, al_pieces = 1;
    if (idle) {
    } else if (aligned) {
        int rows_ne = 0;
        for (int r = 0; r < n; r++) rows_ne += (s_prefix[r + 1] != s_prefix[r]);
        const long long spare = (long long)gridDim.x - (long long)rows_ne * G, P = s_prefix[n];
        int base = 0;
        bool found = false;
        u_begin = u_end = 0;
        for (int r = 0; r < n && !found; r++) {
            const int p = s_prefix[r + 1] - s_prefix[r];
            if (p == 0) continue;
            int c = 1 + (int)(spare * p / (P * G));
            c = c < p ? c : p;
            if (cta < base + G * c) {
                const int idx = cta - base, hl = idx / c, k = idx % c;
                const long long seg0 = (long long)G * s_prefix[r] + (long long)hl * p;
                u_begin = seg0 + (long long)k * p / c;
                u_end = seg0 + (long long)(k + 1) * p / c;
                al_first = base + hl * c;
                al_pieces = c;
                found = true;
            }
            base += G * c;
        }
        if (!found) idle = true;
    } else {
        if (cta >= C) idle = true;
        u_begin = (long long)cta * U / C;
        u_end = (long long)(cta + 1) * U / C;
        if (idle) u_begin = u_end = 0;
    }
    /* ---- fused step, still before the wait: what the query set-up needs besides the queries themselves
     * (norm weights, RoPE table, the row's position -> cos/sin) comes from the host, so warps 0-7 fetch
     * and compute it now, off the critical path.                                                       */
    const int rl_d0 = (lane >> 4) * 64 + (lane & 15) * 4;
    float4 pre_w = make_float4(1.f, 1.f, 1.f, 1.f);
    float pre_c[4] = {1.f, 1.f, 1.f, 1.f}, pre_s[4] = {0.f, 0.f, 0.f, 0.f};
    int pre_row = -1;
    if (a.fused && !idle && warp < 8) {
        pre_w = *reinterpret_cast<const float4 *>(a.norm_w + rl_d0);
        pre_row = locate(s_prefix, batch, n, G, u_begin, u_end).row;
        hy3a_rowops::rope_coeffs(pre_c, pre_s, a.rope, batch.pos[pre_row], lane);
    }
    /* Everything above reads only what the host wrote (batch descriptor).  From here on the kernel
     * touches memory that the preceding kernel in the stream may produce (queries, the newest KV
     * slot, scratch records), so wait for it -- except the producer lane, which first starts the
     * copies of pages that lie wholly below the newest slot (append-only cache: immutable).       */
    const bool is_producer = STAGED && warp == kWarps;
    if (!is_producer) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        /* Only now may the NEXT kernel in the stream start its prologue: it then knows that everything
         * older than this kernel is complete, so the only writes it can race with are this kernel's
         * (the newest slot of each row), which its early page fetches stay clear of.                  */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    /* rows with no keys on this rank: zero output / empty partial (hy3_gpu.cu:197-199) */
    for (int i = cta; i < n; i += gridDim.x) {
        if (s_prefix[i + 1] != s_prefix[i]) continue;
        if (SHARD) {
            /* sharded: the empty record {m = -inf, l = 0} of every head goes to every other rank now (one flagged line;
             * the fold skips it without reading acc); this rank's own fold of the row happens at the end of the kernel,
             * when the other ranks' records are due */
            if (is_producer) continue;
            for (int e = tid; e < G * 8; e += kThreads) {
                const unsigned flag = a.shard_round[i * G * 8 + e] + 1u;
                for (int r = 0; r < a.n_dest; r++)
                    if (r != a.my_rank) shard_store_line(a.dest[r] + ((size_t)i * G * 8 + e) * kShardLines, -INFINITY, 0.f, flag);
            }
            continue;
        }
        for (int e = tid; e < G * 8 * HY3A_D && !is_producer; e += kThreads) {
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

    if (idle && !SHARD) return;   /* sharded: idle CTAs may still own the fold of rows without local keys */


    if (STAGED && warp == kWarps) {
        /* ================= producer warp: one lane streams the CTA's pages into the ring */
        if (lane == 0) {
            unsigned it = 0;
            bool ok = true;
            bool waited = false;   /* griddepcontrol.wait executed yet? */
            const unsigned long long pol = l2_evict_first_policy();
            if (!a.early_prefetch) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
            for (long long u = u_begin; u < u_end && ok;) {
                segment sg = locate(s_prefix, batch, n, G, u, u_end);
                const int *bt = cache.block_table + (size_t)sg.seq * cache.max_blocks_per_seq;
                int block_next = bt[sg.p_begin];
                for (int p = sg.p_begin; p < sg.p_end && ok; p++, it++) {
                    const unsigned stage = it % (unsigned)a.stages, phase = (it / (unsigned)a.stages) & 1u;
                    const int block = block_next;
                    if (p + 1 < sg.p_end) block_next = bt[p + 1];   /* in flight while we wait for the stage */
                    /* before the preceding kernel is known to be complete only pages that lie wholly below
                     * the newest slot may be fetched, and only into stages that were never used            */
                    if (!waited && (it >= (unsigned)a.stages || (p + 1) * HY3A_PT > sg.len - 2)) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
                    ok = mbar_wait(bar_base + 8 * stage, phase ^ 1u, &s_abort, a.err, 1u);
                    if (!ok) break;
                    const uint8_t *page = cache.pool + hy3a_page_index(cache, block, a.layer, sg.hl) * (size_t)cache.page_bytes;
                    const unsigned full = bar_base + 64 + 8 * (it % (2u * (unsigned)a.stages));
                    mbar_expect_tx(full, (unsigned)geom.page_bytes);
                    bulk_g2s(ring_base + stage * (unsigned)geom.page_bytes, page, (unsigned)geom.page_bytes, full, pol);
                }
                u = sg.seg_u0 + sg.p_end;
            }
            if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
            if (!ok) {
                /* gave up: let the copies already issued land before the CTA's shared memory goes away */
                const unsigned first = it > (unsigned)a.stages ? it - (unsigned)a.stages : 0u;
                for (unsigned j = first; j < it; j++) {
                    const unsigned fb = j % (2u * (unsigned)a.stages), fphase = (j / (2u * (unsigned)a.stages)) & 1u;
                    for (unsigned spin = 0; spin < (1u << 20) && !mbar_test(bar_base + 64 + 8 * fb, fphase); spin++) __nanosleep(64);
                }
            }
        }
        return;
    }

    /* ================= consumer warps */
    int k_off[2][4];   /* [n-block][chunk], relative to the granule, loop invariant */
    int v_off[8];
    int sc_off[2];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) {
        int tok = 8 * nb + g;
        if (DT == 2) { k_off[nb][0] = hy3a_k_chunk_off<2>(tok, tig); k_off[nb][1] = k_off[nb][2] = k_off[nb][3] = 0; }
        else { for (int i = 0; i < 4; i++) k_off[nb][i] = hy3a_k_chunk_off<0>(tok, tig + 4 * i); }
        sc_off[nb] = 2 * (8 * nb + 2 * tig);
    }
    {
        int pr0 = tig, pr1 = pr0 + 4;
        if (DT == 2) {
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
    const unsigned sq = smem_u32(&s_q[0][lane]);

    unsigned it = 0; /* pages consumed by this CTA so far (ring position) */
    long long u = u_begin;
    while (u < u_end) {
        const segment sg = locate(s_prefix, batch, n, G, u, u_end);
        const int row = sg.row, hl = sg.hl, sidx = sg.sidx;
        const int head0 = (cache.kv_head_begin + hl) * 8;   /* first of the segment's 8 query heads */

        /* ---- Q operand fragments of the segment's 8 heads, pre-packed per (k-step, lane).
         * Warp w < 8 owns head w as a row of 4 values per lane (dims d0..d0+3); in the fused step it
         * first applies the per-head RMSNorm and RoPE (same code as the append kernel).  The softmax
         * scale 1/sqrt(128) (hy3_gpu.cu:193) and log2(e) are folded into the fragments.            */
        float qf = 1.f;
        float *s_qx = reinterpret_cast<float *>(s_dyn);                 /* FP16 cache: [8][128] fp32 staging */
        signed char *s_q8 = reinterpret_cast<signed char *>(s_dyn);     /* INT8/INT4: [2][8][128] int8 digits */
        if (warp < 8) {
            const int d0 = (lane >> 4) * 64 + (lane & 15) * 4;
            float x[4];
            if (a.fused) {
                const float4 xv = *reinterpret_cast<const float4 *>(a.q_in + (size_t)row * a.qi_stride + (size_t)(head0 + warp) * HY3A_D + d0);
                x[0] = xv.x; x[1] = xv.y; x[2] = xv.z; x[3] = xv.w;
                if (row != pre_row) { hy3a_rowops::rope_coeffs(pre_c, pre_s, a.rope, batch.pos[row], lane); pre_row = row; }
                hy3a_rowops::norm_rope_apply(x, pre_w, a.eps, pre_c, pre_s, lane);
                if (a.q_out && sg.p_begin == 0)
                    *reinterpret_cast<float4 *>(a.q_out + (size_t)row * a.q_out_stride + (size_t)(head0 + warp) * HY3A_D + d0) = make_float4(x[0], x[1], x[2], x[3]);
            } else {
                const float4 xv = *reinterpret_cast<const float4 *>(a.q + (size_t)row * a.q_stride + (size_t)(head0 + warp) * HY3A_D + d0);
                x[0] = xv.x; x[1] = xv.y; x[2] = xv.z; x[3] = xv.w;
            }
            if (DT == 0) {
                const float qs = 0.08838834764831845f * kLog2e;
                *reinterpret_cast<float4 *>(s_qx + warp * HY3A_D + d0) = make_float4(x[0] * qs, x[1] * qs, x[2] * qs, x[3] * qs);
            } else {
                /* two int8 digits per query element: q ~ sq*(hi + lo/254), |hi|,|lo| <= 127, so the
                 * quantisation step is absmax/32258 per head                                       */
                float m = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                const float sqv = m > 0.f ? m * (1.f / 127.f) : 1.f, inv = 1.f / sqv;
                unsigned hw = 0, lw = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float hi = fminf(127.f, fmaxf(-127.f, rintf(x[j] * inv)));
                    const float lo = fminf(127.f, fmaxf(-127.f, rintf((x[j] - hi * sqv) * (254.f * inv))));
                    hw |= ((unsigned)(int)hi & 0xFFu) << (8 * j);
                    lw |= ((unsigned)(int)lo & 0xFFu) << (8 * j);
                }
                *reinterpret_cast<unsigned *>(s_q8 + warp * HY3A_D + d0) = hw;
                *reinterpret_cast<unsigned *>(s_q8 + (8 + warp) * HY3A_D + d0) = lw;
                if (lane == 0) s_qf[warp] = sqv * (1.f / 254.f) * 0.08838834764831845f * kLog2e * (DT == 2 ? 0.0625f : 1.f);
            }
        } else if (warp == 8) {
            /* fused step: the scale the new V row will get (hy3_gpu.cu:260-262), so that every CTA of the
             * segment sizes its P scale for it as well                                                 */
            unsigned vb = 0;
            if (DT != 0 && a.fused && a.k_in) {
                const float4 xv = *reinterpret_cast<const float4 *>(a.v_in + (size_t)row * a.vi_stride + (size_t)(cache.kv_head_begin + hl) * HY3A_D + 4 * lane);
                float m = fmaxf(fmaxf(fabsf(xv.x), fabsf(xv.y)), fmaxf(fabsf(xv.z), fabsf(xv.w)));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                vb = (unsigned)__half_as_ushort(__float2half(__fadd_rn(__fdiv_rn(m, 7.f), 1e-8f)));
            }
            if (lane == 0) s_vnew = vb;
        }
        consumer_sync();
        if (DT == 0) {
            /* fp16 value in rows 0-7, fp16 residual in rows 8-15 */
            if (tid < 256) {
                const int j = tid >> 5;
                float xx[4], hi4[4], lo4[4];
#pragma unroll
                for (int s2 = 0; s2 < 4; s2++) xx[s2] = s_qx[g * HY3A_D + kdim16(j, tig, s2)];
#pragma unroll
                for (int s2 = 0; s2 < 4; s2++) { hi4[s2] = __half2float(__float2half_rn(xx[s2])); lo4[s2] = xx[s2] - hi4[s2]; }
                s_q[j][lane] = make_uint4(pack_h2(hi4[0], hi4[1]), pack_h2(lo4[0], lo4[1]), pack_h2(hi4[2], hi4[3]), pack_h2(lo4[2], lo4[3]));
            }
        } else {
            /* pack the digits into MMA A-fragments: rows 0-7 = hi, rows 8-15 = lo */
            if (tid < 128) {
                const int kk = tid >> 5;
                unsigned w[4] = {0, 0, 0, 0};
#pragma unroll
                for (int s2 = 0; s2 < 8; s2++) {
                    const int d = kdim32<DT>(kk, tig, s2);
                    w[2 * (s2 >> 2)] |= ((unsigned)(unsigned char)s_q8[g * HY3A_D + d]) << (8 * (s2 & 3));
                    w[2 * (s2 >> 2) + 1] |= ((unsigned)(unsigned char)s_q8[(8 + g) * HY3A_D + d]) << (8 * (s2 & 3));
                }
                s_q[kk][lane] = make_uint4(w[0], w[1], w[2], w[3]);
            }
            qf = s_qf[g];
        }
        const unsigned vnew = s_vnew;
        consumer_sync();
        /* P scale: w = p * vscale * 2^E with vs_max * 2^E <= 2^6 and p <= 2^8, so fp16 P never
         * overflows and its subnormal floor sits 2^-30 below the reference max.               */
        float pscale;
        {
            int E = 6;
            if (DT != 0) {
                unsigned vb = cache.vs_max[a.layer * G + hl];
                vb = vb > vnew ? vb : vnew;   /* positive fp16 bit patterns order like the numbers */
                __half_raw hr; hr.x = (unsigned short)vb;
                float vmax = __half2float(__half(hr));
                int ex;
                frexpf(fmaxf(vmax, 1e-30f), &ex); /* vmax < 2^ex */
                E = 6 - ex;
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
                const unsigned q2 = pit / (2u * (unsigned)a.stages), r2 = pit - q2 * 2u * (unsigned)a.stages;   /* ring round pair, position in it */
                const unsigned stage = r2 < (unsigned)a.stages ? r2 : r2 - (unsigned)a.stages;
                const unsigned spage = ring_base + stage * (unsigned)geom.page_bytes;
                /* the page's "full" barrier is one of 2 x stages: a warp holds granules in 8 of every 11 pages, so it may skip a
                 * use of a stage, and an mbarrier wait only knows the parity of a phase.  With one barrier per stage the warp's next
                 * wait on that stage could pass on the stale phase while the skipped page is still landing (seen with the two-stage
                 * ring of FP16 pages).  With two barriers per stage the phase a warp can miss is two ring rounds old: every page the
                 * warp has consumed since was filled after that one had been filled, consumed and its stage filled again. */
                mbar_wait(bar_base + 64 + 8 * r2, q2 & 1u, &s_abort, a.err, 2u);
                if (a.fused && a.k_in && p == ((sg.len - 1) >> 7) && gi == (((sg.len - 1) & 127) >> 4)) {
                    /* fused append: this warp holds the only granule that contains the newest slot.  It
                     * normalises, rotates and quantises the new K row and quantises the new V row exactly
                     * as the append kernel does, writes them to the page in HBM (for later steps) and into
                     * the shared-memory copy it is about to read.                                         */
                    const int d0 = (lane >> 4) * 64 + (lane & 15) * 4, tok = (sg.len - 1) & 127;
                    const int block = cache.block_table[(size_t)sg.seq * cache.max_blocks_per_seq + p];
                    uint8_t *gp = cache.pool + hy3a_page_index(cache, block, a.layer, hl) * (size_t)cache.page_bytes;
                    uint8_t *sp = s_dyn + kFixed + a.prefix_bytes + kBarBytes + (size_t)stage * geom.page_bytes;
                    const int kvh = cache.kv_head_begin + hl;
                    float4 kv4 = *reinterpret_cast<const float4 *>(a.k_in + (size_t)row * a.ki_stride + (size_t)kvh * HY3A_D + d0);
                    float y[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
                    hy3a_rowops::norm_rope_row(y, a.norm_w + HY3A_D, a.eps, a.rope, batch.pos[row], lane);
                    hy3a_rowops::store_row<DT>(gp, geom, tok, false, y, d0, lane);
                    hy3a_rowops::store_row<DT>(sp, geom, tok, false, y, d0, lane);
                    kv4 = *reinterpret_cast<const float4 *>(a.v_in + (size_t)row * a.vi_stride + (size_t)kvh * HY3A_D + d0);
                    y[0] = kv4.x; y[1] = kv4.y; y[2] = kv4.z; y[3] = kv4.w;
                    const unsigned sb = hy3a_rowops::store_row<DT>(gp, geom, tok, true, y, d0, lane);
                    hy3a_rowops::store_row<DT>(sp, geom, tok, true, y, d0, lane);
                    if (DT != 0 && lane == 0) atomicMax(cache.vs_max + a.layer * G + hl, sb);
                    __syncwarp();
                }
                if (16 * gi + 16 <= valid) granule<DT, true, true>(st, sq, qf, nullptr, spage, geom, k_off, v_off, sc_off, gi, tig, valid, pscale);
                else if (16 * gi < valid) granule<DT, true, false>(st, sq, qf, nullptr, spage, geom, k_off, v_off, sc_off, gi, tig, valid, pscale);
                mbar_arrive(bar_base + 8 * stage); /* every thread of the 8 warps that share a page releases it */
            } else {
                if (16 * gi >= valid) continue; /* warp-uniform */
                const int block = cache.block_table[(size_t)sg.seq * cache.max_blocks_per_seq + p];
                const uint8_t *page = cache.pool + hy3a_page_index(cache, block, a.layer, hl) * (size_t)cache.page_bytes;
                granule<DT, false, false>(st, sq, qf, page, 0u, geom, k_off, v_off, sc_off, gi, tig, valid, pscale);
            }
        }
        it = it_end;

        /* ---- fold the consumer warps of this CTA (shared memory) */
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
        consumer_sync(); /* s_o / s_ml free again */

        /* ---- how many CTAs share this segment? */
        const int c_first = aligned ? al_first : (int)(((sg.seg_u0 + 1) * C + U - 1) / U) - 1;
        const int npieces = aligned ? al_pieces : (int)((sg.seg_u1 * C + U - 1) / U) - 1 - c_first + 1;
        const int rec_base = aligned ? 0 : sidx;   /* record index = CTA (+ segment when CTAs may hold several pieces) */
        const size_t head_q = (size_t)(cache.kv_head_begin + hl) * 8 + h; /* global query head */
        u = sg.seg_u0 + sg.p_end;

        /* Which of the 8 heads this CTA finishes (writes out / exchanges): all of them, unless the fold of a
         * segment is spread over several of its CTAs (below). */
        int h_lo = 0, h_hi = 8;
        if (npieces > 1) {
            if (red) {
                float *rec = a.scratch + ((size_t)(cta + rec_base) * 8 + h) * kRecFloats;
                if (d4 == 0) { rec[0] = M; rec[1] = L; }
                rec[2 + d4] = acc[0]; rec[3 + d4] = acc[1]; rec[4 + d4] = acc[2]; rec[5 + d4] = acc[3];
            }
            consumer_sync();   /* the record is complete in CTA scope; the release below publishes it */
            if (STAGED && aligned && a.spread) {
                /* ---- CTA-aligned segments (small batches): the fold is SPREAD.  Every CTA announces its record on
                 * the segment's arrival counter; the first F pieces then each fold 8/F of the heads over all pieces
                 * (one warp per head: 33 16-byte asynchronous copies per record and lane 0 one more, all records in
                 * flight at once, landing in the idle page ring), instead of one CTA pulling every head of every
                 * piece while the others have left.  The remaining pieces leave at once.                          */
                const int Fmax = a.spread, F = npieces >= Fmax ? Fmax : (npieces >= 4 && Fmax >= 4 ? 4 : (npieces >= 2 && Fmax >= 2 ? 2 : 1)), hpf = 8 / F, piece = cta - c_first;
                if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.counters + sidx) : "memory");
                if (piece >= F) continue;   /* CTA-uniform */
                if (tid == 0) {
                    /* bounded wait for the other pieces (they are resident: one CTA per SM at most) */
                    unsigned seen = 0;
                    unsigned long long t0 = 0;
                    bool ok = false;
                    for (unsigned i = 0; i < (1u << 24); i++) {
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(a.counters + sidx) : "memory");
                        if (seen >= (unsigned)npieces) { ok = true; break; }
                        if ((i & 255u) == 255u) {
                            unsigned long long t1;
                            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                            if (t0 == 0) t0 = t1;
                            if (s_abort || (i >= (1u << 14) && t1 - t0 > 500000000ull)) break;
                        }
                    }
                    if (!ok) { s_abort = 1; if (atomicCAS(a.err, 0u, 4u) == 0u) { a.err[1] = 50u; a.err[2] = blockIdx.x; a.err[3] = seen; } }
                    s_flag = ok;
                }
                consumer_sync();
                h_lo = piece * hpf; h_hi = h_lo + hpf;
                const bool mine = red && h >= h_lo && h < h_hi;
                M = -INFINITY; L = 0.f; acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                if (s_flag && mine) {
                    /* landing zone of head h: npieces x 528 bytes in the ring (idle: this CTA's pages are consumed) */
                    const unsigned zone = (unsigned)((h - h_lo) * npieces) * (unsigned)(kRecFloats * 4);
                    const uint8_t *src = reinterpret_cast<const uint8_t *>(a.scratch + ((size_t)c_first * 8 + h) * kRecFloats);
                    for (int c = 0; c < npieces; c++) {
                        const unsigned dst = ring_base + zone + (unsigned)c * (unsigned)(kRecFloats * 4);
                        const uint8_t *g = src + (size_t)c * 8 * kRecFloats * 4;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * (unsigned)lane), "l"(g + 16 * lane) : "memory");
                        if (lane == 0) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 512u), "l"(g + 512) : "memory");
                    }
                    asm volatile("cp.async.wait_all;" ::: "memory");
                    __syncwarp();
                    const float *zf = reinterpret_cast<const float *>(s_dyn + kFixed + a.prefix_bytes + kBarBytes + zone);
                    for (int c = 0; c < npieces; c++) {
                        const float *pr = zf + (size_t)c * kRecFloats;
                        const float pm = pr[0], pl = pr[1];
                        if (!(pl > 0.f)) continue;
                        const float2 v01 = *reinterpret_cast<const float2 *>(pr + 2 + d4), v23 = *reinterpret_cast<const float2 *>(pr + 4 + d4);
                        const float nm = fmaxf(M, pm), os = ex2(M - nm), rs = ex2(pm - nm);
                        L = L * os + pl * rs;
                        acc[0] = acc[0] * os + v01.x * rs; acc[1] = acc[1] * os + v01.y * rs;
                        acc[2] = acc[2] * os + v23.x * rs; acc[3] = acc[3] * os + v23.y * rs;
                        M = nm;
                    }
                }
                consumer_sync();   /* every landing zone is read (the sharded exchange lands its lines in the ring too) */
                if (tid == 0) {
                    /* the last of the F folders puts both counters back to zero for the next launch */
                    const unsigned old = atomicAdd(a.counters + a.n_counters + sidx, 1u);
                    if (old == (unsigned)(F - 1)) { a.counters[sidx] = 0u; a.counters[a.n_counters + sidx] = 0u; }
                }
            } else {
                /* ---- a CTA may hold pieces of several segments (large batches): the LAST CTA to arrive folds, nobody waits */
                if (tid == 0) {
                    unsigned old;
                    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(a.counters + sidx) : "memory");
                    s_flag = (old == (unsigned)(npieces - 1));
                }
                consumer_sync();
                if (!s_flag) continue;   /* CTA-uniform */
                /* fold all pieces with the rule of hy3_gpu.cu:233-247.  The pieces' records (contiguous) are fetched
                 * into the merge buffer with 16-byte asynchronous copies issued by all threads at once and folded
                 * from there; larger segments go through it in several rounds.                                    */
                const unsigned land = smem_u32(s_dyn);
                const float *land_g = reinterpret_cast<const float *>(s_dyn);
                const int land_cap = kFixedO / (8 * kRecFloats * 4);
                M = -INFINITY; L = 0.f; acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                for (int c0 = 0; c0 < npieces; c0 += land_cap) {
                    const int nc = min(land_cap, npieces - c0);
                    const uint8_t *src = reinterpret_cast<const uint8_t *>(a.scratch + (size_t)(c_first + c0 + rec_base) * 8 * kRecFloats);
                    for (int i = tid; i < nc * (8 * kRecFloats / 4); i += kThreads)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(land + 16u * (unsigned)i), "l"(src + 16 * (size_t)i) : "memory");
                    asm volatile("cp.async.wait_all;" ::: "memory");
                    consumer_sync();
                    if (red) {
                        for (int c = 0; c < nc; c++) {
                            const float *pr = land_g + ((size_t)c * 8 + h) * kRecFloats;
                            const float pm = pr[0], pl = pr[1];
                            if (!(pl > 0.f)) continue;
                            const float2 v01 = *reinterpret_cast<const float2 *>(pr + 2 + d4), v23 = *reinterpret_cast<const float2 *>(pr + 4 + d4);
                            const float nm = fmaxf(M, pm), os = ex2(M - nm), rs = ex2(pm - nm);
                            L = L * os + pl * rs;
                            acc[0] = acc[0] * os + v01.x * rs; acc[1] = acc[1] * os + v01.y * rs;
                            acc[2] = acc[2] * os + v23.x * rs; acc[3] = acc[3] * os + v23.y * rs;
                            M = nm;
                        }
                    }
                    if (c0 + land_cap < npieces) consumer_sync();   /* landing zone is reused */
                }
                if (tid == 0) a.counters[sidx] = 0u; /* self-reset for the next launch */
                consumer_sync();   /* the landing zone is read; the next segment may reuse the buffer */
            }
        }
        const bool fin = red && h >= h_lo && h < h_hi;   /* this thread finishes its (head, 4 dims) of the segment */
        if (SHARD) {
            /* sequence sharding: this rank's records of the segment go into every other rank's gather buffer as
             * flagged lines (no fence, no separate flag: a line is valid when both of its flag words carry this
             * use's number), then the same threads collect the other ranks' lines and finish the segment */
            const int seg = row * G + hl;
            if (fin) {
                const unsigned flag = a.shard_round[seg * 8 + h] + 1u;   /* use count of this (slot, segment, head) */
                const float m_nat = M * kLn2;
                const size_t ro = ((size_t)seg * 8 + h) * kShardLines;
                for (int r = 0; r < a.n_dest; r++) {
                    if (r == a.my_rank) continue;
                    uint4 *rec = a.dest[r] + ro;
                    if (d4 == 0) shard_store_line(rec, m_nat, L, flag);
                    shard_store_line(rec + 1 + (d4 >> 1), acc[0], acc[1], flag);
                    shard_store_line(rec + 2 + (d4 >> 1), acc[2], acc[3], flag);
                }
                shard_fold_args fa;
                fa.rec0 = a.gathered + ro; fa.rank_stride = (size_t)n * G * 8 * kShardLines; fa.err = a.err;
                fa.out = a.out + (size_t)row * a.out_stride + ((size_t)(cache.kv_head_begin + hl) * 8 + h) * HY3A_D + d4;
                fa.n_ranks = a.n_dest; fa.my_rank = a.my_rank; fa.line_a = 1 + (d4 >> 1); fa.flag = flag; fa.stage = reinterpret_cast<const uint4 *>(s_dyn); fa.h = h; fa.lane = lane;
                fa.own_m = m_nat; fa.own_l = L; fa.own_acc[0] = acc[0]; fa.own_acc[1] = acc[1]; fa.own_acc[2] = acc[2]; fa.own_acc[3] = acc[3];
                if (STAGED && aligned && (size_t)a.stages * geom.page_bytes >= (size_t)8 * 8 * kShardLines * 16) {
                    /* CTA-aligned segments: the page ring is idle by now and holds all 8 ranks' records at once, so
                     * every rank is polled in the same round */
                    fa.stage = reinterpret_cast<const uint4 *>(s_dyn + kFixed + a.prefix_bytes + kBarBytes);
                    shard_fold<8>(fa);
                } else {
                    shard_fold<kShardBatch>(fa);
                }
                __syncwarp();                /* every lane of the head's warp has read the use count */
                if (d4 == 0) a.shard_round[seg * 8 + h] = flag;
            }
            consumer_sync();                 /* the landing zones may be reused by the next segment */
            continue;
        }
        if (!fin) continue;
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
    /* sharded: rows without keys on this rank were announced at the top; the other ranks' records are folded here */
    if (SHARD)
        for (int i = cta; i < n; i += gridDim.x) {
            if (s_prefix[i + 1] != s_prefix[i]) continue;
            for (int hl = 0; hl < G; hl++) {
                const int seg = i * G + hl;
                if (tid < 256) {
                    const int h = (tid >> 5) & 7, d4 = (tid & 31) * 4;
                    shard_fold_args fa;
                    fa.rec0 = a.gathered + ((size_t)seg * 8 + h) * kShardLines; fa.rank_stride = (size_t)n * G * 8 * kShardLines; fa.err = a.err;
                    fa.out = a.out + (size_t)i * a.out_stride + ((size_t)(cache.kv_head_begin + hl) * 8 + h) * HY3A_D + d4;
                    fa.n_ranks = a.n_dest; fa.my_rank = a.my_rank; fa.line_a = 1 + (d4 >> 1); fa.flag = a.shard_round[seg * 8 + h] + 1u; fa.stage = reinterpret_cast<const uint4 *>(s_dyn); fa.h = h; fa.lane = lane;
                    fa.own_m = -INFINITY; fa.own_l = 0.f; fa.own_acc[0] = fa.own_acc[1] = fa.own_acc[2] = fa.own_acc[3] = 0.f;
                    shard_fold<kShardBatch>(fa);
                    __syncwarp();
                    if (d4 == 0) a.shard_round[seg * 8 + h] = fa.flag;
                }
                consumer_sync();
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
    static bool attr_dev[64][3][3];   /* function attributes are per device: [device ordinal][cache type][variant] */
    bool (*attr_set)[3] = attr_dev[ctx->device & 63];
    a.prefix_bytes = (int)prefix;
    if (ctx->decode_stages >= 2) {
        a.stages = ctx->decode_stages;
        const size_t smem = kFixed + prefix + kBarBytes + (size_t)a.stages * ctx->geom.page_bytes;
        const bool shard = a.n_dest > 0;
        if (!attr_set[DT][shard ? 2 : 1]) {
            cudaError_t e = shard ? cudaFuncSetAttribute(hy3a_decode_kernel<DT, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax)
                                  : cudaFuncSetAttribute(hy3a_decode_kernel<DT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
            if (e != cudaSuccess) return e;
            attr_set[DT][shard ? 2 : 1] = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid; cfg.blockDim = dim3(kThreads + 32); cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = ctx->use_pdl ? 1 : 0;
        if (shard) return cudaLaunchKernelEx(&cfg, hy3a_decode_kernel<DT, true, true>, cv, bv, a);
        return cudaLaunchKernelEx(&cfg, hy3a_decode_kernel<DT, true>, cv, bv, a);
    } else {
        a.stages = 0;
        if (!attr_set[DT][0]) {
            cudaError_t e = cudaFuncSetAttribute(hy3a_decode_kernel<DT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
            if (e != cudaSuccess) return e;
            attr_set[DT][0] = true;
        }
        hy3a_decode_kernel<DT, false><<<grid, kThreads, kFixed + prefix + kBarBytes, ctx->stream>>>(cv, bv, a);
    }
    return cudaGetLastError();
}

/* Pages that fit in the ring for a given page size and batch capacity. */
int hy3a_decode_ring_capacity(int page_bytes, int max_batch) {
    const size_t prefix = ((size_t)(max_batch + 1) * sizeof(int) + 127) & ~(size_t)127;
    long room = (long)kSmemMax - (long)kFixed - (long)prefix - kBarBytes;
    int s = room > 0 ? (int)(room / page_bytes) : 0;
    return s > 8 ? 8 : s;
}
/* Largest grid the last-arrival merge can stage in the merge buffer. */
int hy3a_decode_max_ctas(void) { return kFixedO / 64; }
static_assert(kRecFloats >= HY3A_PARTIAL_FLOATS && (kRecFloats * 4) % 16 == 0, "a head's record must start on a 16-byte boundary");

int hy3a_launch_decode(hy3a_ctx *ctx, int layer, const float *q, size_t q_stride, float *out, size_t out_stride, float *partials,
                       const hy3a_step_inputs *step) {
    decode_args a;
    memset(&a, 0, sizeof(a));
    a.q = q; a.q_stride = q_stride; a.out = out; a.out_stride = out_stride; a.user_partials = partials;
    a.scratch = ctx->d_partials; a.counters = ctx->d_counters; a.n_counters = ctx->cfg.max_batch * ctx->cfg.kv_head_count; a.err = ctx->d_err; a.layer = layer;
    /* the spread fold pays off where the epilogue is the cross-GPU exchange (8 CTAs store to the peers instead of one); on one
     * GPU the folders only hold their SMs longer, which delays the next launch's CTAs there.  Its folders wait for the other
     * pieces, so every CTA of the grid must be resident */
    a.spread = (ctx->shard_slot >= 0 && ctx->decode_ctas <= ctx->sm_count) ? 4 : 0;   /* folders per segment: 4 measured best on 8 GPUs (8: 28.8, 4: 27.8, 2: 27.8, 1: 29.2 us per layer) */
    a.early_prefetch = ctx->use_pdl && !ctx->bulk_write_pending;
    if (ctx->shard_slot >= 0) {   /* set by hy3a_decode_step_sharded around this call */
        const int W = ctx->shard_world, slot = ctx->shard_slot;
        const size_t n_seg = (size_t)ctx->shard_rows * ctx->cfg.kv_head_count;
        const size_t slice = n_seg * 8 * (HY3A_PARTIAL_FLOATS / 2);    /* 16-byte lines per rank and slot */
        a.n_dest = W; a.my_rank = ctx->shard_rank;
        for (int r = 0; r < W; r++) a.dest[r] = reinterpret_cast<uint4 *>(ctx->shard_peer[r]) + ((size_t)slot * W + ctx->shard_rank) * slice;
        a.gathered = reinterpret_cast<const uint4 *>(ctx->shard_local) + (size_t)slot * W * slice;
        a.shard_round = reinterpret_cast<unsigned *>(ctx->shard_local + ctx->shard_state_off) + (size_t)slot * n_seg * 8;
    }
    if (step) {
        a.fused = 1;
        a.q_in = step->q_in; a.k_in = step->k_in; a.v_in = step->v_in;
        a.qi_stride = step->q_stride; a.ki_stride = step->k_stride; a.vi_stride = step->v_stride;
        a.q_out = step->q_out; a.q_out_stride = step->q_out_stride;
        a.norm_w = ctx->d_norm_w + (size_t)layer * 2 * HY3A_D; a.eps = ctx->cfg.rms_eps; a.rope = ctx->rope;
    }
    hy3a_cache_view cv = hy3a_view(ctx);
    hy3a_batch_view bv = hy3a_bview(ctx);
    cudaError_t e;
    switch (ctx->geom.dtype) {
        case 0: e = launch_decode_dt<0>(ctx, cv, bv, a); break;
        case 1: e = hy3a_launch_decode_umma(ctx, cv, bv, a); break;
        default: e = launch_decode_dt<2>(ctx, cv, bv, a); break;
    }
    ctx->launches++;
    ctx->bulk_write_pending = 0;   /* the kernel after this one only has this one to stay clear of */
    if (e != cudaSuccess) return hy3a_fail(ctx, HY3A_ECUDA, "decode launch: %s", cudaGetErrorString(e));
    return HY3A_OK;
}

/* ---- decode without any allocation ---------------------------------------------------------
 * Scratch for hy3a_decode_noalloc: the records and arrival counters of the cross-CTA merge live in
 * this file-scope device array instead of buffers the context allocated.  Every GPU that loads the
 * library holds these 2.4 MB until the process exits.  Layout: [kNoAllocRecords][8][132] floats of
 * records, then two counters (arrivals, finished folds) per segment.                                               */
constexpr int kNoAllocRows = 64;                                   /* most (batch row, KV head) segments per call */
constexpr int kNoAllocRecords = 512 + kNoAllocRows;                /* one per CTA of the largest grid + one per segment */
constexpr size_t kNoAllocRecordBytes = (size_t)kNoAllocRecords * 8 * kRecFloats * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocRecordBytes + 2 * kNoAllocRows * sizeof(unsigned)];
static unsigned char *g_noalloc_ptr[64];                           /* device address of the array, per device ordinal */

extern "C" int hy3a_decode_noalloc(hy3a_ctx *ctx, int layer, const float *q, size_t q_stride, float *out, size_t out_stride) {
    if (!ctx) return HY3A_EINVAL;
    if (layer < 0 || layer >= ctx->cfg.n_layers) return hy3a_fail(ctx, HY3A_EINVAL, "decode_noalloc: layer %d out of range", layer);
    if (ctx->batch_n < 1) return hy3a_fail(ctx, HY3A_ESTATE, "decode_noalloc: no batch set (call hy3a_batch_set first)");
    if (!q || !out || (((uintptr_t)q | (uintptr_t)out) & 15) || ((q_stride | out_stride) & 3))
        return hy3a_fail(ctx, HY3A_EINVAL, "decode_noalloc: q and out must be non-NULL, 16-byte aligned, strides multiples of 4");
    if (ctx->batch_n * ctx->cfg.kv_head_count > kNoAllocRows)
        return hy3a_fail(ctx, HY3A_EINVAL, "decode_noalloc: %d batch rows x %d KV heads exceed the built-in scratch (%d segments); use hy3a_decode",
                         ctx->batch_n, ctx->cfg.kv_head_count, kNoAllocRows);
    if (ctx->decode_ctas > 512) return hy3a_fail(ctx, HY3A_EINVAL, "decode_noalloc: grid of %d CTAs exceeds the built-in scratch", ctx->decode_ctas);
    if (ctx->device < 0 || ctx->device >= 64) return hy3a_fail(ctx, HY3A_EINVAL, "decode_noalloc: device ordinal %d not supported", ctx->device);
    {   /* the launch below goes to the current device: it must be the context's */
        int cur = -1;
        HY3A_CUDA(ctx, cudaGetDevice(&cur));
        if (cur != ctx->device)
            return hy3a_fail(ctx, HY3A_ESTATE, "decode_noalloc: the context lives on device %d but device %d is current (cudaSetDevice first)", ctx->device, cur);
    }
    if (!g_noalloc_ptr[ctx->device]) {
        /* one-time set-up on this device (it is current): in host code the array's name is only a handle, the
         * kernel needs the device address                                                                  */
        void *p = NULL;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) return hy3a_fail(ctx, HY3A_ECUDA, "decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_noalloc_ptr[ctx->device] = (unsigned char *)p;
    }
    unsigned char *scratch = g_noalloc_ptr[ctx->device];
    /* the arrival counters must start at zero; a call that was cut short may have left some behind */
    HY3A_CUDA(ctx, cudaMemsetAsync(scratch + kNoAllocRecordBytes, 0, 2 * kNoAllocRows * sizeof(unsigned), ctx->stream));
    decode_args a;
    memset(&a, 0, sizeof(a));
    a.q = q; a.q_stride = q_stride; a.out = out; a.out_stride = out_stride;
    a.scratch = reinterpret_cast<float *>(scratch);
    a.counters = reinterpret_cast<unsigned *>(scratch + kNoAllocRecordBytes);
    a.n_counters = kNoAllocRows;
    a.err = ctx->d_err; a.layer = layer;
    a.early_prefetch = 0;
    hy3a_cache_view cv = hy3a_view(ctx);
    hy3a_batch_view bv = hy3a_bview(ctx);
    cudaError_t e;
    switch (ctx->geom.dtype) {
        case 0: e = launch_decode_dt<0>(ctx, cv, bv, a); break;
        case 1: e = hy3a_launch_decode_umma(ctx, cv, bv, a); break;
        default: e = launch_decode_dt<2>(ctx, cv, bv, a); break;
    }
    ctx->launches++;
    ctx->bulk_write_pending = 0;
    if (e != cudaSuccess) return hy3a_fail(ctx, HY3A_ECUDA, "decode_noalloc launch: %s", cudaGetErrorString(e));
    return HY3A_OK;
}


int hy3a_launch_merge(hy3a_ctx *ctx, const float *partials, int n_parts, int n_rows, int n_heads, float *out, size_t out_stride) {
    hy3a_merge_kernel<<<n_rows * n_heads, 32, 0, ctx->stream>>>(partials, n_parts, n_rows, n_heads, out, out_stride);
    ctx->launches++;
    HY3A_CUDA(ctx, cudaGetLastError());
    return HY3A_OK;
}
