/*
 * decode_umma.cu -- split-KV GQA decode attention for INT8 caches: scores on mma.sync, P.V on tcgen05 / TMEM.
 *
 * Same job, schedule, records and merge as decode.cu (replaces attention_split_kv_kernel + attention_reduce_kernel,
 * hy3_gpu.cu:183-247); what changes is who multiplies by V.  In decode.cu every warp converts the V codes of its 16
 * tokens to fp16 and keeps a 16 x 128 output tile in registers: 64 conversions + 16 MMAs per 16 tokens, 64 accumulator
 * registers per lane, a shared-memory fold of all warps at the end -- the CUDA cores, not HBM, set the pace of a page.
 * Here the V area of a page is stored TRANSPOSED (row = head dim, 128 token bytes, 128-byte swizzle: layout.h), so the
 * copy that lands in shared memory IS a tensor-core operand, and the head dims, not the heads, are the M dimension:
 *
 *   S[16 x 32]        = Qd . K^T         mma.sync m16n8k32.s8 on the stored codes, as in decode.cu: rows 0-7 = high int8
 *                                        digit of the 8 queries, rows 8-15 = low digit (q ~ sq (hi + lo / 254))
 *   O^T[128 dim x 16] = V^T . Pd^T       tcgen05.mma kind::i8, M = 128, N = 16, K = 32 tokens: the 16 columns are the
 *                                        8 heads x {high, low} int8 digit of w = p * vscale(token) / wb, wb = the largest
 *                                        V scale of the 32 tokens; products and sums are exact integers
 *
 * Roles (19 warps, coupled by mbarriers only):
 *   warps 0-7   accumulators: thread = (head dim = TMEM lane, 4 of the 8 heads).  Per page they read the four groups' integer
 *               results from TMEM (tcgen05.ld) and add them, scaled, to 4 fp32 registers.  Before the stream starts they
 *               also run the fused append (one warp per new row).
 *   warp 8      page producer (one lane): bulk copies (cp.async.bulk + mbarrier transaction counts, evict-first in L2) into a
 *               ring of pages; the first ring fill runs before the preceding kernel is known to be complete (pages below
 *               the newest slot are immutable), and once the queries are loaded it asks L2 for the pages beyond the ring.
 *   warp 9      MMA issuer (one lane): when the four groups' digits of a page are in shared memory it issues the four
 *               tcgen05.mma back to back, one tcgen05.commit for the accumulators and one that frees the ring stage.  It
 *               does nothing else: scalar code between two MMAs of a lane costs more than the MMA.
 *   warp 10     bookkeeper (lane = (group, head)): the online-softmax bookkeeping of the page -- running max, rescale factor,
 *               denominator, the factor of every (group, head) -- once for all accumulators, while the tensor core works.
 *   warps 11-18 score warps: a warp takes a 32-token group: 16 integer MMAs, scales, the group's own max (2 shuffles),
 *               8 exponentials per lane, digits, 8 two-byte stores into the P^T tile, {max, sum, wb} for the bookkeeper.
 *               No output accumulators, no conversion of V: about 250 instructions per 32 tokens instead of 860.
 *               The same warps run the query set-up and the epilogue (records, merge, exchange).
 *   Every waiter of an mbarrier waits for every phase of it, in order (a wait only knows a phase's parity).
 *
 * Every wait is bounded; a wait that runs out raises a CTA-wide abort flag and records a code in the context's error
 * word, every later wait returns at once, all roles keep their control flow to the end and TMEM is released.
 *
 * Roofline: HBM; algorithmic bytes per (token, KV head) = 260.
 */
#include <cuda_fp16.h>
#include <math.h>
#include <stddef.h>
#include <string.h>

#include "ctx.h"
#include "decode_common.cuh"
#include "rowops.cuh"

namespace {

constexpr int kAccWarps = 8, kProdWarp = 8, kIssWarp = 9, kBkWarp = 10, kQkWarp0 = 11, kQkWarps = 8;
constexpr int kAccThreads = kAccWarps * 32;
constexpr int kQkThreads = kQkWarps * 32;
constexpr int kUThreads = (kQkWarp0 + kQkWarps) * 32;
constexpr int kSlots = 8;                        /* pages in flight between the score warps and the accumulators (8 x 64 TMEM columns) */
constexpr int kStages = HY3A_UMMA_STAGES;        /* pages in the ring */
constexpr int kStageBytes = 33792;               /* an INT8 page (33 280 B) rounded up to 1 KB: every V^T tile 1024-byte aligned */
constexpr int kVtOff = 16384, kKsOff = 32768, kVsOff = 33024;
constexpr int kRecFloats = HY3A_REC_FLOATS;
constexpr int kShardBatchU = 1;                  /* ranks polled at once by the sharded epilogue when the ring is not idle (8 320 B of landing zone each) */
constexpr float kDigits = 32258.f;               /* 127 * 254: the largest two-digit value */

struct u_misc {
    unsigned long long rfull[8], rempty[8], pfull[kSlots], ofull[kSlots], bk[kSlots], sfree[kSlots], qload;
    unsigned tmem;
    int abort_flag, flag, app_ready;         /* app_ready: the fused appends of this CTA are in HBM */
    float qf[8];
    float ml[8][2];                              /* {M, L} of the segment piece the accumulators just finished */
    float meta_m[kSlots][4][8], meta_l[kSlots][4][8], meta_wb[kSlots][4];
    /* read as float4 by the accumulators */
    __align__(16) float fa[kSlots][32];
    __align__(16) float rr[kSlots][8];
};
static_assert(offsetof(u_misc, fa) % 16 == 0 && offsetof(u_misc, rr) % 16 == 0 && offsetof(u_misc, rfull) % 8 == 0, "alignment of the vector-loaded members");
/* shared-memory map, bytes from a 1024-byte aligned base.  The P^T tiles double as the hand-over area of a finished piece
 * and as the landing zone of the epilogue: all three uses follow one another (the accumulators hand a piece over when every
 * MMA of it is done; the score warps copy it into registers, run the epilogue, and only then start the next piece's digits). */
constexpr int kOffPt = 0;                            /* kSlots x [16 rows][128 B]: P digits, transposed, 128-byte swizzle */
constexpr int kOffAcc = 0;                           /* [8 heads][128 dims] fp32: the finished piece, handed to the epilogue */
constexpr int kOffLand = 0;                          /* landing zone of records / exchange lines when the page ring is not idle */
constexpr int kLandBytes = kSlots * 2048;
constexpr unsigned kLate = 4, kLateCut = 2;      /* the last pieces of a single-row grid start late: they take fewer pages */
constexpr int kOffQ = kOffPt + kSlots * 2048;        /* Q fragments [4 k-steps][32 lanes] x 16 B */
constexpr int kOffQ8 = kOffQ + 2048;                 /* Q digits [2][8][128] int8 */
constexpr int kOffMisc = kOffQ8 + 2048;
constexpr int kOffPrefix = kOffMisc + ((sizeof(u_misc) + 127) / 128) * 128;
static_assert(kShardBatchU * 8 * (HY3A_PARTIAL_FLOATS / 2) * 16 <= kLandBytes, "landing zone too small for the exchange");
static_assert(8 * kRecFloats * 4 <= kLandBytes && 8 * HY3A_D * 4 <= kLandBytes, "landing zone too small for a record / the hand-over");
static_assert(kStages >= 2 && kStages <= 8, "ring depth");

/* descriptors: K-major, 128-byte swizzle, 8-row groups 1024 B apart (version 1, layout type 2) */
__device__ __forceinline__ unsigned long long make_desc(unsigned saddr) {
    return (unsigned long long)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
/* instruction descriptor, kind::i8: D = s32 (2 at bit 4), A = B = signed 8-bit (1 at bits 7 and 10), both K-major,
 * N = 16 (>> 3 at bit 17), M = 128 (>> 4 at bit 24) */
constexpr unsigned kIdescI8 = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
__device__ __forceinline__ void umma_i8(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, 0, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdescI8) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16_nowait(unsigned taddr, int *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld4_nowait(unsigned taddr, int *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void qk_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kQkThreads) : "memory"); }
/* hand-over of a finished piece: the accumulators arrive, the score warps wait */
__device__ __forceinline__ void epi_arrive() { asm volatile("bar.arrive 3, %0;" ::"n"(kAccThreads + kQkThreads) : "memory"); }
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 3, %0;" ::"n"(kAccThreads + kQkThreads) : "memory"); }
__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ void sts16(unsigned addr, unsigned v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory"); }
#define UBAR(field) smem_u32(&(field))
/* every wait of this kernel: blocking try_wait, bounded, a no-op once the CTA has given up */
#define UWAIT(field, parity, where) mbar_wait_blocking(UBAR(field), (parity), &mi.abort_flag, a.err, (where))

/* One 32-token group of one score warp: S = Qd . K^T, the group's max / sum, digits of w into the P^T tile.
 * FULL: all 32 tokens are valid.  spage: shared address of the page; pt: shared address of the slot's P^T tile. */
template <bool FULL>
__device__ __forceinline__ void score_group(u_misc &mi, int slot, unsigned sq, float qf, unsigned spage, unsigned pt, int k_off0, int k_off1, int gi, int g, int tig, int lane, int valid) {
    unsigned ksw[4], vsw[4];
#pragma unroll
    for (int nb = 0; nb < 4; nb++) {
        ksw[nb] = lds4(spage + kKsOff + gi * 64 + nb * 16 + 4 * tig);
        vsw[nb] = lds4(spage + kVsOff + gi * 64 + nb * 16 + 4 * tig);
    }
    int c[4][4];
#pragma unroll
    for (int nb = 0; nb < 4; nb++) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0;
    /* two 8-token blocks at a time: two independent chains of four dependent MMAs, 16 registers of K codes in flight */
#pragma unroll
    for (int half = 0; half < 2; half++) {
        uint4 kr[2][2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            kr[j][0] = lds16(spage + gi * 4096 + (2 * half + j) * 1024 + k_off0);
            kr[j][1] = lds16(spage + gi * 4096 + (2 * half + j) * 1024 + k_off1);
        }
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            const uint4 qa = lds16(sq + kk * 512);
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const unsigned b0 = kk == 0 ? kr[j][0].x : (kk == 1 ? kr[j][0].y : (kk == 2 ? kr[j][0].z : kr[j][0].w));
                const unsigned b1 = kk == 0 ? kr[j][1].x : (kk == 1 ? kr[j][1].y : (kk == 2 ? kr[j][1].z : kr[j][1].w));
                imma16832(c[2 * half + j], qa, b0, b1);
            }
        }
    }
    /* logits (base 2) of head g for tokens 32 gi + 8 nb + 2 tig + e, and the V scales of those tokens */
    float s[4][2], vs[4][2];
#pragma unroll
    for (int nb = 0; nb < 4; nb++) {
        const float2 kf = unpack_h2(ksw[nb]), vf = unpack_h2(vsw[nb]);
        const float r0 = (float)(c[nb][0] * 254 + c[nb][2]) * qf, r1 = (float)(c[nb][1] * 254 + c[nb][3]) * qf;
        const int t0 = 32 * gi + 8 * nb + 2 * tig;
        s[nb][0] = (FULL || t0 < valid) ? r0 * kf.x : -INFINITY;
        s[nb][1] = (FULL || t0 + 1 < valid) ? r1 * kf.y : -INFINITY;
        vs[nb][0] = (FULL || t0 < valid) ? vf.x : 0.f;
        vs[nb][1] = (FULL || t0 + 1 < valid) ? vf.y : 0.f;
    }
    float mx = fmaxf(fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1])), fmaxf(fmaxf(s[2][0], s[2][1]), fmaxf(s[3][0], s[3][1])));
    float wb = fmaxf(fmaxf(fmaxf(vs[0][0], vs[0][1]), fmaxf(vs[1][0], vs[1][1])), fmaxf(fmaxf(vs[2][0], vs[2][1]), fmaxf(vs[3][0], vs[3][1])));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    wb = fmaxf(wb, __shfl_xor_sync(0xffffffffu, wb, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    wb = fmaxf(wb, __shfl_xor_sync(0xffffffffu, wb, 2));
    const float msafe = mx == -INFINITY ? 0.f : mx;
    const float inv = wb > 0.f ? __fdividef(kDigits, wb) : 0.f;
    /* two int8 digits per w through the 1.5 * 2^23 trick: the low mantissa byte of (x + magic) is round(x) as int8 */
    const float magic = 12582912.f;
    float lsum = 0.f;
    const unsigned pt_row = pt + (unsigned)g * 128u;
#pragma unroll
    for (int nb = 0; nb < 4; nb++) {
        unsigned hb[2], lb[2];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const float p = ex2(s[nb][e] - msafe);               /* -inf -> 0 */
            lsum += p;
            const float d = p * vs[nb][e] * inv;                 /* 0 .. 32258 */
            const float t = fmaf(d, 1.f / 254.f, magic);
            const float hf = t - magic;
            const float u = fmaf(hf, -254.f, d + magic);
            hb[e] = __float_as_uint(t);
            lb[e] = __float_as_uint(u);
        }
        /* byte column 32 gi + 8 nb + 2 tig of rows g (high digit) and 8 + g (low digit); 16-byte chunk c of a row sits at
         * chunk c ^ (row & 7) = c ^ g */
        const unsigned col = (unsigned)(((2 * gi + (nb >> 1)) ^ g) << 4) + (unsigned)(8 * (nb & 1) + 2 * tig);
        sts16(pt_row + col, prmt(hb[0], hb[1], 0x0040u));
        sts16(pt_row + 1024u + col, prmt(lb[0], lb[1], 0x0040u));
    }
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
    lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
    if (tig == 0) { mi.meta_m[slot][gi][g] = mx; mi.meta_l[slot][gi][g] = lsum; }
    if (lane == 0) mi.meta_wb[slot][gi] = wb;
    /* the digits were written through the generic proxy; the tensor core reads through the async proxy */
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    mbar_arrive(UBAR(mi.pfull[slot]));
}

template <bool SHARD>
__global__ void __launch_bounds__(kUThreads, 1) hy3a_decode_umma_kernel(hy3a_cache_view cache, hy3a_batch_view batch, decode_args a) {
    extern __shared__ __align__(128) uint8_t s_raw[];
    uint8_t *s_dyn = s_raw + ((1024u - (smem_u32(s_raw) & 1023u)) & 1023u);   /* 1024-aligned in the shared window */
    const unsigned s_base = smem_u32(s_dyn);
    u_misc &mi = *reinterpret_cast<u_misc *>(s_dyn + kOffMisc);
    int *s_prefix = reinterpret_cast<int *>(s_dyn + kOffPrefix);
    const hy3a_geom geom = hy3a_make_geom(1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, tig = lane & 3;
    const int n = batch.n, G = cache.kv_heads;
    const int cta = blockIdx.x;
    int *s_pos = s_prefix + n + 1;                                   /* RoPE positions of the rows */
    const unsigned ring_off = (unsigned)((kOffPrefix + a.prefix_bytes + 1023) & ~1023);
    const unsigned ring_base = s_base + ring_off;
    const int qw = warp - kQkWarp0, qtid = tid - kQkWarp0 * 32;      /* score-warp numbering (negative for the other roles) */
    const bool is_qk = warp >= kQkWarp0;

    /* ---- prologue: everything here reads only what the host wrote.  The loads are issued together. */
    const int rl_d0 = (lane >> 4) * 64 + (lane & 15) * 4;
    float4 pre_w = make_float4(1.f, 1.f, 1.f, 1.f), pre_f = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.fused && is_qk && qw < 8) {
        pre_w = *reinterpret_cast<const float4 *>(a.norm_w + rl_d0);
        pre_f = *reinterpret_cast<const float4 *>(a.rope.inv_freq + (lane & 15) * 4);
    }
    if (warp == kIssWarp) {
        /* TMEM: kSlots pages x 4 groups x 16 columns (allocated by every CTA up front: the allocation takes about a microsecond) */
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&mi.tmem)), "n"(kSlots * 64) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < n; i += kUThreads) {
        const int len = batch.slot[i] + 1;
        s_prefix[i + 1] = len > 0 ? (len + HY3A_PT - 1) / HY3A_PT : 0;
        s_pos[i] = batch.pos[i];
    }
    if (tid == 0) {
        s_prefix[0] = 0;
        mi.abort_flag = 0;
        mi.app_ready = 0;
        for (int i = 0; i < kStages; i++) { mbar_init(UBAR(mi.rfull[i]), 1); mbar_init(UBAR(mi.rempty[i]), 1); }
        for (int i = 0; i < kSlots; i++) {
            mbar_init(UBAR(mi.pfull[i]), 128);      /* the four score warps of a page, every lane */
            mbar_init(UBAR(mi.ofull[i]), 1);
            mbar_init(UBAR(mi.bk[i]), 1);
            mbar_init(UBAR(mi.sfree[i]), kAccWarps);
        }
        mbar_init(UBAR(mi.qload), 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (n > 1) {
        if (warp == 0) {
            int carry = 0;
            for (int base = 0; base < n; base += 32) {
                const int i = base + lane;
                int v = i < n ? s_prefix[i + 1] : 0;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, v, o);
                    if (lane >= o) v += t;
                }
                if (i < n) s_prefix[i + 1] = v + carry;
                carry += __shfl_sync(0xffffffffu, v, 31);
            }
        }
        __syncthreads();
    }
    /* ---- schedule: the unit split of decode.cu, in 32-bit arithmetic where the counts allow it (a 64-bit division costs
     * hundreds of cycles, and a CTA that starts late has this code on the launch's critical path) */
    const unsigned Pn = (unsigned)s_prefix[n];
    const long long U = (long long)G * Pn;
    bool idle = (U == 0);
    const bool aligned = (long long)n * G < (long long)gridDim.x && aligned_split_balanced(s_prefix, n, G, gridDim.x, lane);
    const int C = (long long)gridDim.x < U ? (int)gridDim.x : (int)U;
    long long u_begin = 0, u_end = 0;
    int al_first = 0, al_pieces = 1;
    if (idle) {
    } else if (aligned && Pn < (1u << 23)) {
        int rows_ne = 0;
        for (int r = 0; r < n; r++) rows_ne += (s_prefix[r + 1] != s_prefix[r]);
        const unsigned spare = gridDim.x - (unsigned)(rows_ne * G), PG = Pn * (unsigned)G;   /* spare < 2^8, pages < 2^23 */
        int base = 0;
        bool found = false;
        for (int r = 0; r < n && !found; r++) {
            const unsigned p = (unsigned)(s_prefix[r + 1] - s_prefix[r]);
            if (p == 0) continue;
            unsigned c = 1u + spare * p / PG;
            c = c < p ? c : p;
            if (cta < base + G * (int)c) {
                const unsigned idx = (unsigned)(cta - base), hl = idx / c, k = idx - hl * c;
                const unsigned seg0 = (unsigned)G * (unsigned)s_prefix[r] + hl * p;
                u_begin = seg0 + k * p / c;
                u_end = seg0 + (k + 1u) * p / c;
                /* The CTAs with the highest indices are dispatched last, onto the SMs that the preceding launch's folding CTAs
                 * held longest: they start their ring fill late and would finish last (and then fold, and hold their SMs again).
                 * In a single-row grid the last kLate pieces therefore take kLateCut pages less each and the other pieces of that
                 * segment share them: 18.83 instead of 19.02 us per launch on the benchmark. */
                if (rows_ne == 1 && hl == (unsigned)G - 1u && c > 2u * kLate && p >= 8u * c) {
                    const unsigned pp = p + kLate * kLateCut, k1 = k + 1u;
                    u_begin = seg0 + k * pp / c - kLateCut * (k > c - kLate ? k - (c - kLate) : 0u);
                    u_end = seg0 + k1 * pp / c - kLateCut * (k1 > c - kLate ? k1 - (c - kLate) : 0u);
                }
                al_first = base + (int)(hl * c);
                al_pieces = (int)c;
                found = true;
            }
            base += G * (int)c;
        }
        if (!found) idle = true;
    } else if (aligned) {
        int rows_ne = 0;
        for (int r = 0; r < n; r++) rows_ne += (s_prefix[r + 1] != s_prefix[r]);
        const long long spare = (long long)gridDim.x - (long long)rows_ne * G, P = s_prefix[n];
        int base = 0;
        bool found = false;
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
    if (idle && !SHARD) {
        /* nothing to do: give the tensor memory back and leave (sharded: idle CTAs may still own the fold of rows without local keys) */
        fence_before();
        __syncthreads();
        if (warp == kIssWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(mi.tmem), "n"(kSlots * 64) : "memory");
        return;
    }
    segment sg0;                                                    /* the CTA's first piece */
    sg0.row = 0; sg0.hl = 0;
    if (!idle) sg0 = locate(s_prefix, batch, n, G, u_begin, u_end);

    /* fused step: cos / sin of the first segment's row (positions are in shared memory, the table in registers) */
    float pre_c[4] = {1.f, 1.f, 1.f, 1.f}, pre_s[4] = {0.f, 0.f, 0.f, 0.f};
    int pre_row = -1;
    auto rope_of_row = [&](int row) {
        const int ti = s_pos[row];
        const int pos = (ti + (ti >= a.rope.pos_jump_at ? a.rope.pos_jump : 0)) * a.rope.pos_stride;
        const float fr4[4] = {pre_f.x, pre_f.y, pre_f.z, pre_f.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float fr = (float)pos * fr4[j];
            pre_c[j] = cosf(fr) * a.rope.attn_factor;
            pre_s[j] = sinf(fr) * a.rope.attn_factor;
        }
        pre_row = row;
    };
    if (a.fused && !idle && is_qk && qw < 8) rope_of_row(sg0.row);
    /* The step's inputs may still be on their way from the preceding kernel, so they are read after the wait below; asking
     * L2 for their lines now is harmless (L2 is the point of coherence) and saves a trip to HBM when they are old. */
    if (!idle) {
        const int row0 = sg0.row, hl0 = sg0.hl;
        const int hd0 = (cache.kv_head_begin + hl0) * 8;
        if (is_qk && qw < 8 && (lane & 7) == 0) {
            const float *qp = (a.fused ? a.q_in + (size_t)row0 * a.qi_stride : a.q + (size_t)row0 * a.q_stride) + (size_t)(hd0 + qw) * HY3A_D + (lane >> 3) * 32;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(qp));
        }
        if (warp == 0 && a.fused && a.k_in && lane < 8) {
            const float *kp = (lane < 4 ? a.k_in + (size_t)row0 * a.ki_stride : a.v_in + (size_t)row0 * a.vi_stride) + (size_t)(cache.kv_head_begin + hl0) * HY3A_D + (lane & 3) * 32;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(kp));
        }
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = mi.tmem;

    /* From here on the kernel touches memory that the preceding kernel in the stream may produce (queries, the newest KV
     * slot, scratch records): wait for it -- except the producer lane, which first starts the copies of pages that lie
     * wholly below the newest slot (append-only cache: immutable). */
    const bool is_producer = warp == kProdWarp;
    if (!is_producer) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    /* rows with no keys on this rank: zero output / empty partial (hy3_gpu.cu:197-199) */
    if (is_qk)
        for (int i = cta; i < n; i += gridDim.x) {
            if (s_prefix[i + 1] != s_prefix[i]) continue;
            if (SHARD) {
                for (int e = qtid; e < G * 8; e += kQkThreads) {
                    const unsigned flag = a.shard_round[i * G * 8 + e] + 1u;
                    for (int r = 0; r < a.n_dest; r++)
                        if (r != a.my_rank) shard_store_line(a.dest[r] + ((size_t)i * G * 8 + e) * kShardLines, -INFINITY, 0.f, flag);
                }
                continue;
            }
            for (int e = qtid; e < G * 8 * HY3A_D; e += kQkThreads) {
                const int hq = e / HY3A_D, d = e % HY3A_D;
                if (a.user_partials) {
                    float *p = a.user_partials + ((size_t)i * G * 8 + hq) * HY3A_PARTIAL_FLOATS;
                    p[2 + d] = 0.f;
                    if (d == 0) { p[0] = -INFINITY; p[1] = 0.f; }
                } else {
                    a.out[(size_t)i * a.out_stride + (size_t)(cache.kv_head_begin * 8 + hq) * HY3A_D + d] = 0.f;
                }
            }
        }

    if (!idle && warp == kProdWarp) {
        /* ================= producer: one lane streams the CTA's pages into the ring */
        if (lane == 0) {
            unsigned it = 0;
            bool waited = false;   /* griddepcontrol.wait executed yet? */
            bool app_seen = false; /* the CTA's fused appends are known to be complete */
            const unsigned long long pol = l2_evict_first_policy();
            /* once the preceding kernel is complete: ask L2 for the pages that do not fit the ring, so that HBM works
             * while the queries are being prepared and the ring's own copies later hit L2 */
            auto prefetch_rest = [&]() {
                unsigned k = 0;
                for (long long u2 = u_begin; u2 < u_end;) {
                    const segment s2 = locate(s_prefix, batch, n, G, u2, u_end);
                    const int *bt2 = cache.block_table + (size_t)s2.seq * cache.max_blocks_per_seq;
                    for (int p2 = s2.p_begin; p2 < s2.p_end; p2++, k++) {
                        if (k < (unsigned)kStages) continue;
                        if (k >= (unsigned)kStages + 24u) return;    /* far enough ahead */
                        const uint8_t *pg = cache.pool + hy3a_page_index(cache, bt2[p2], a.layer, s2.hl) * (size_t)cache.page_bytes;
                        asm volatile("cp.async.bulk.prefetch.L2.global.L2::cache_hint [%0], %1, %2;" ::"l"(pg), "r"((unsigned)geom.page_bytes), "l"(pol) : "memory");
                    }
                    u2 = s2.seg_u0 + s2.p_end;
                }
            };
            if (!a.early_prefetch) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
            for (long long u = u_begin; u < u_end;) {
                const segment sg = locate(s_prefix, batch, n, G, u, u_end);
                const int *bt = cache.block_table + (size_t)sg.seq * cache.max_blocks_per_seq;
                int block_next = bt[sg.p_begin];
                for (int p = sg.p_begin; p < sg.p_end; p++, it++) {
                    const unsigned stage = it % (unsigned)kStages, phase = (it / (unsigned)kStages) & 1u;
                    const int block = block_next;
                    if (p + 1 < sg.p_end) block_next = bt[p + 1];   /* in flight while we wait for the stage */
                    /* before the preceding kernel is known to be complete only pages that lie wholly below the newest
                     * slot may be fetched, and only into stages that were never used */
                    if (!waited && (it >= (unsigned)kStages || (p + 1) * HY3A_PT > sg.len - 2)) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
                    if (it == (unsigned)kStages) {
                        /* the ring is full and nothing is consumed yet: once the score warps hold their queries (their loads are
                         * not to queue behind this burst), ask L2 for the rest */
                        UWAIT(mi.qload, 0u, 4u);
                        prefetch_rest();
                    }
                    if (!UWAIT(mi.rempty[stage], phase ^ 1u, 1u)) continue;      /* gave up: issue nothing more */
                    const uint8_t *page = cache.pool + hy3a_page_index(cache, block, a.layer, sg.hl) * (size_t)cache.page_bytes;
                    if (a.fused && a.k_in && p == ((sg.len - 1) >> 7) && !app_seen) {
                        /* the page that holds a newest slot: the accumulator warps append those rows at the start of the
                         * kernel; their stores must be in HBM / L2 before the copy reads the page */
                        volatile int *ready = &mi.app_ready;
                        unsigned long long t0 = 0;
                        for (unsigned i = 0; !*ready && i < (1u << 24); i++) {
                            if ((i & 255u) == 255u) {
                                unsigned long long t1;
                                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                                if (t0 == 0) t0 = t1;
                                if (mi.abort_flag || (i >= (1u << 14) && t1 - t0 > 500000000ull)) { mi.abort_flag = 1; if (atomicCAS(a.err, 0u, 5u) == 0u) a.err[1] = 60u; break; }
                            }
                        }
                        app_seen = true;
                    }
                    mbar_expect_tx(UBAR(mi.rfull[stage]), (unsigned)geom.page_bytes);
                    bulk_g2s(ring_base + stage * (unsigned)kStageBytes, page, (unsigned)geom.page_bytes, UBAR(mi.rfull[stage]), pol);
                }
                u = sg.seg_u0 + sg.p_end;
            }
            if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
        }
    } else if (!idle && warp == kIssWarp) {
        /* ================= MMA issuer: one lane; per page one wait, four MMAs back to back, one commit (the scalar code
         * between two tcgen05.mma of a thread costs more than the MMA itself, so this loop does nothing else) */
        if (lane == 0) {
            const unsigned n_pages = (unsigned)(u_end - u_begin);
            const unsigned long long dv0 = make_desc(ring_base + (unsigned)kVtOff), dp0 = make_desc(s_base + kOffPt);
            for (unsigned it = 0; it < n_pages; it++) {
                const unsigned stage = it % (unsigned)kStages, slot = it % (unsigned)kSlots, sph = (it / (unsigned)kSlots) & 1u;
                const unsigned long long dv = dv0 + (unsigned long long)(stage * (unsigned)(kStageBytes >> 4)), dp = dp0 + (unsigned long long)(slot * (2048u >> 4));
                const unsigned d = tmem + slot * 64u;
                UWAIT(mi.pfull[slot], sph, 20u);
                fence_after();
                /* a group's 32 tokens are bytes 32 gi .. 32 gi + 31 of every row of both tiles: + 32 B on the descriptors */
                umma_i8(d, dv, dp);
                umma_i8(d + 16u, dv + 2ull, dp + 2ull);
                umma_i8(d + 32u, dv + 4ull, dp + 4ull);
                umma_i8(d + 48u, dv + 6ull, dp + 6ull);
                umma_commit(UBAR(mi.ofull[slot]));
                umma_commit(UBAR(mi.rempty[stage]));    /* K was consumed by the scores, V^T by these MMAs: the stage can be refilled */
            }
        }
    } else if (!idle && warp == kBkWarp) {
        /* ================= bookkeeper: lane = (group, head).  Per page the online-softmax bookkeeping -- running max, rescale
         * factor, denominator, the factor of every (group, head) -- once for all accumulators, while the tensor core works. */
        const int bk_gi = lane >> 3, bk_h = lane & 7;
        float Mh = -INFINITY, Lh = 0.f;                 /* running max / denominator of head bk_h (replicated over the 4 group lanes) */
        unsigned it = 0;
        for (long long u = u_begin; u < u_end;) {
            const segment sg = locate(s_prefix, batch, n, G, u, u_end);
            Mh = -INFINITY; Lh = 0.f;
            for (int p = sg.p_begin; p < sg.p_end; p++, it++) {
                const unsigned slot = it % (unsigned)kSlots, sph = (it / (unsigned)kSlots) & 1u;
                UWAIT(mi.pfull[slot], sph, 25u);
                const float m = mi.meta_m[slot][bk_gi][bk_h], l = mi.meta_l[slot][bk_gi][bk_h], wbv = mi.meta_wb[slot][bk_gi];
                float mx = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float Mn = fmaxf(Mh, mx);
                const float r = Mn == -INFINITY ? 1.f : ex2(Mh - Mn);     /* 0 when Mh = -inf */
                const float f = m == -INFINITY ? 0.f : ex2(m - Mn);
                float ls = l * f;
                ls += __shfl_xor_sync(0xffffffffu, ls, 8);
                ls += __shfl_xor_sync(0xffffffffu, ls, 16);
                Lh = Lh * r + ls;
                Mh = Mn;
                mi.fa[slot][lane] = f * wbv * (1.f / kDigits);
                if (bk_gi == 0) {
                    mi.rr[slot][bk_h] = r;
                    if (p + 1 == sg.p_end) { mi.ml[bk_h][0] = Mh; mi.ml[bk_h][1] = Lh; }   /* the piece is complete */
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(UBAR(mi.bk[slot]));
            }
            u = sg.seg_u0 + sg.p_end;
        }
    } else if (!idle && warp < kAccWarps) {
        /* ================= accumulators: thread = (head dim = TMEM lane, 4 of the 8 heads) */
        const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
        const int hq0 = 4 * (warp >> 2), dim = (warp & 3) * 32 + lane;
        float acc[4];
        unsigned it = 0;
        if (a.fused && a.k_in) {
            /* ---- fused append, up front: the newest token of every segment whose last page lies in this CTA's range is
             * normalised, rotated, quantised and stored exactly as the append kernel does (hy3_gpu.cu:750-756), one warp
             * per row, while the score warps prepare the queries.  The page is copied into the ring afterwards (the
             * producer waits for app_ready), so the kernel attends over the new token from the same bytes later steps read. */
            int j = 0;
            for (long long u2 = u_begin; u2 < u_end;) {
                const segment sg = locate(s_prefix, batch, n, G, u2, u_end);
                const int last_page = (sg.len - 1) >> 7;
                if (last_page >= sg.p_begin && last_page < sg.p_end) {
                    if ((j & (kAccWarps - 1)) == warp) {
                        const int tok = (sg.len - 1) & 127, kvh = cache.kv_head_begin + sg.hl;
                        const int block = cache.block_table[(size_t)sg.seq * cache.max_blocks_per_seq + last_page];
                        uint8_t *gp = cache.pool + hy3a_page_index(cache, block, a.layer, sg.hl) * (size_t)cache.page_bytes;
                        float4 kv4 = *reinterpret_cast<const float4 *>(a.k_in + (size_t)sg.row * a.ki_stride + (size_t)kvh * HY3A_D + rl_d0);
                        const float4 vv4 = *reinterpret_cast<const float4 *>(a.v_in + (size_t)sg.row * a.vi_stride + (size_t)kvh * HY3A_D + rl_d0);
                        float y[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
                        float kc[4], ks[4];
                        hy3a_rowops::rope_coeffs(kc, ks, a.rope, s_pos[sg.row], lane);
                        hy3a_rowops::norm_rope_apply(y, *reinterpret_cast<const float4 *>(a.norm_w + HY3A_D + rl_d0), a.eps, kc, ks, lane);
                        hy3a_rowops::store_row<1>(gp, geom, tok, false, y, rl_d0, lane);
                        y[0] = vv4.x; y[1] = vv4.y; y[2] = vv4.z; y[3] = vv4.w;
                        const unsigned sb = hy3a_rowops::store_row<1>(gp, geom, tok, true, y, rl_d0, lane);
                        if (lane == 0) atomicMax(cache.vs_max + a.layer * G + sg.hl, sb);
                    }
                    j++;
                }
                u2 = sg.seg_u0 + sg.p_end;
            }
            /* the rows were stored through the generic proxy, the bulk copy reads through the async proxy */
            asm volatile("fence.proxy.async.global;" ::: "memory");
            asm volatile("bar.sync 2, %0;" ::"n"(kAccThreads) : "memory");
            if (tid == 0) { __threadfence_block(); *reinterpret_cast<volatile int *>(&mi.app_ready) = 1; }
        }
        for (long long u = u_begin; u < u_end;) {
            const segment sg = locate(s_prefix, batch, n, G, u, u_end);
            acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
            for (int p = sg.p_begin; p < sg.p_end; p++, it++) {
                const unsigned slot = it % (unsigned)kSlots, sph = (it / (unsigned)kSlots) & 1u;
                UWAIT(mi.ofull[slot], sph, 30u);
                fence_after();
                int c[4][8];   /* [group][high digits of the 4 heads | low digits] */
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    tmem_ld4_nowait(tmem + lane_base + slot * 64u + q * 16u + hq0, &c[q][0]);
                    tmem_ld4_nowait(tmem + lane_base + slot * 64u + q * 16u + 8u + hq0, &c[q][4]);
                }
                UWAIT(mi.bk[slot], sph, 31u);
                const float4 rv = *reinterpret_cast<const float4 *>(&mi.rr[slot][hq0]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                acc[0] *= rv.x; acc[1] *= rv.y; acc[2] *= rv.z; acc[3] *= rv.w;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float4 fv = *reinterpret_cast<const float4 *>(&mi.fa[slot][8 * q + hq0]);
                    acc[0] = fmaf((float)(c[q][0] * 254 + c[q][4]), fv.x, acc[0]);
                    acc[1] = fmaf((float)(c[q][1] * 254 + c[q][5]), fv.y, acc[1]);
                    acc[2] = fmaf((float)(c[q][2] * 254 + c[q][6]), fv.z, acc[2]);
                    acc[3] = fmaf((float)(c[q][3] * 254 + c[q][7]), fv.w, acc[3]);
                }
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(UBAR(mi.sfree[slot]));          /* TMEM slot, P^T tile, meta and factors of the slot are free */
            }
            /* hand the finished piece to the epilogue (score warps) */
            float *s_acc = reinterpret_cast<float *>(s_dyn + kOffAcc);
#pragma unroll
            for (int h = 0; h < 4; h++) s_acc[(hq0 + h) * HY3A_D + dim] = acc[h];
            epi_arrive();
            u = sg.seg_u0 + sg.p_end;
        }
    } else if (is_qk) {
        /* ================= score warps (+ query set-up, fused append, epilogue) */
        const int k_off0 = hy3a_k_chunk_off<1>(g, tig), k_off1 = hy3a_k_chunk_off<1>(g, tig + 4);
        const unsigned sq = s_base + kOffQ + 16u * (unsigned)lane;
        uint4 (*s_q)[32] = reinterpret_cast<uint4 (*)[32]>(s_dyn + kOffQ);
        signed char *s_q8 = reinterpret_cast<signed char *>(s_dyn + kOffQ8);
        unsigned it = 0;
        long long u = u_begin;
        while (u < u_end) {
            const segment sg = locate(s_prefix, batch, n, G, u, u_end);
            const int row = sg.row, hl = sg.hl, sidx = sg.sidx;
            const int head0 = (cache.kv_head_begin + hl) * 8;
            /* ---- Q digits of the segment's 8 heads, packed as MMA A fragments (as in decode.cu) */
            if (qw < 8) {
                float x[4];
                if (a.fused) {
                    const float4 xv = *reinterpret_cast<const float4 *>(a.q_in + (size_t)row * a.qi_stride + (size_t)(head0 + qw) * HY3A_D + rl_d0);
                    x[0] = xv.x; x[1] = xv.y; x[2] = xv.z; x[3] = xv.w;
                    if (row != pre_row) rope_of_row(row);
                    hy3a_rowops::norm_rope_apply(x, pre_w, a.eps, pre_c, pre_s, lane);
                    if (a.q_out && sg.p_begin == 0)
                        *reinterpret_cast<float4 *>(a.q_out + (size_t)row * a.q_out_stride + (size_t)(head0 + qw) * HY3A_D + rl_d0) = make_float4(x[0], x[1], x[2], x[3]);
                } else {
                    const float4 xv = *reinterpret_cast<const float4 *>(a.q + (size_t)row * a.q_stride + (size_t)(head0 + qw) * HY3A_D + rl_d0);
                    x[0] = xv.x; x[1] = xv.y; x[2] = xv.z; x[3] = xv.w;
                }
                float m = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
                if (u == u_begin && lane == 0) mbar_arrive(UBAR(mi.qload));   /* the first piece's queries have arrived */
                const float sqv = m > 0.f ? m * (1.f / 127.f) : 1.f, inv = 1.f / sqv;
                unsigned hw = 0, lw = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float hi = fminf(127.f, fmaxf(-127.f, rintf(x[j] * inv)));
                    const float lo = fminf(127.f, fmaxf(-127.f, rintf((x[j] - hi * sqv) * (254.f * inv))));
                    hw |= ((unsigned)(int)hi & 0xFFu) << (8 * j);
                    lw |= ((unsigned)(int)lo & 0xFFu) << (8 * j);
                }
                *reinterpret_cast<unsigned *>(s_q8 + qw * HY3A_D + rl_d0) = hw;
                *reinterpret_cast<unsigned *>(s_q8 + (8 + qw) * HY3A_D + rl_d0) = lw;
                if (lane == 0) mi.qf[qw] = sqv * (1.f / 254.f) * 0.08838834764831845f * kLog2e;
            }
            qk_sync();
            if (qtid < 128) {
                const int kk = qtid >> 5;
                unsigned w[4] = {0, 0, 0, 0};
#pragma unroll
                for (int s2 = 0; s2 < 8; s2++) {
                    const int d = kdim32<1>(kk, tig, s2);
                    w[2 * (s2 >> 2)] |= ((unsigned)(unsigned char)s_q8[g * HY3A_D + d]) << (8 * (s2 & 3));
                    w[2 * (s2 >> 2) + 1] |= ((unsigned)(unsigned char)s_q8[(8 + g) * HY3A_D + d]) << (8 * (s2 & 3));
                }
                s_q[kk][lane] = make_uint4(w[0], w[1], w[2], w[3]);
            }
            qk_sync();
            const float qf = mi.qf[g];

            /* group X = 4 * (ring position of the page) + group-in-page; warp w takes X = w (mod kQkWarps) */
            const unsigned it_end = it + (unsigned)(sg.p_end - sg.p_begin);
            for (unsigned X = it * 4u + ((unsigned)qw + kQkWarps - (it * 4u) % kQkWarps) % kQkWarps; X < it_end * 4u; X += kQkWarps) {
                const unsigned pit = X >> 2;
                const int gi = (int)(X & 3u), p = sg.p_begin + (int)(pit - it);
                const int valid = min(HY3A_PT, sg.len - p * HY3A_PT);
                const unsigned stage = pit % (unsigned)kStages, rph = (pit / (unsigned)kStages) & 1u;
                const unsigned slot = pit % (unsigned)kSlots, sph = (pit / (unsigned)kSlots) & 1u;
                const unsigned spage = ring_base + stage * (unsigned)kStageBytes;
                UWAIT(mi.rfull[stage], rph, 2u);
                UWAIT(mi.sfree[slot], sph ^ 1u, 3u);        /* the accumulators are through with the page that used this slot before */
                const unsigned pt = s_base + kOffPt + slot * 2048u;
                if (32 * gi + 32 <= valid) score_group<true>(mi, (int)slot, sq, qf, spage, pt, k_off0, k_off1, gi, g, tig, lane, valid);
                else score_group<false>(mi, (int)slot, sq, qf, spage, pt, k_off0, k_off1, gi, g, tig, lane, valid);
            }
            it = it_end;

            /* ---- the piece of this CTA, from the accumulators: thread -> (head, 4 dims) */
            epi_sync();
            const bool red = qtid < 256;
            const int h = (qtid >> 5) & 7, d4 = (qtid & 31) * 4;
            float M = mi.ml[h][0], L = mi.ml[h][1], acc[4];
            {
                const float4 o4 = *reinterpret_cast<const float4 *>(s_dyn + kOffAcc + (h * HY3A_D + d4) * 4);
                acc[0] = o4.x; acc[1] = o4.y; acc[2] = o4.z; acc[3] = o4.w;
            }
            qk_sync();   /* everybody holds its share: the accumulators may overwrite the hand-over area (next piece) */

            /* ---- how many CTAs share this segment? */
            const int c_first = aligned ? al_first : (int)(((sg.seg_u0 + 1) * C + U - 1) / U) - 1;
            const int npieces = aligned ? al_pieces : (int)((sg.seg_u1 * C + U - 1) / U) - 1 - c_first + 1;
            const int rec_base = aligned ? 0 : sidx;   /* record index = CTA (+ segment when CTAs may hold several pieces) */
            const size_t head_q = (size_t)(cache.kv_head_begin + hl) * 8 + h; /* global query head */
            u = sg.seg_u0 + sg.p_end;

            int h_lo = 0, h_hi = 8;
            if (npieces > 1) {
                if (red) {
                    float *rec = a.scratch + ((size_t)(cta + rec_base) * 8 + h) * kRecFloats;
                    if (d4 == 0) { rec[0] = M; rec[1] = L; }
                    rec[2 + d4] = acc[0]; rec[3 + d4] = acc[1]; rec[4 + d4] = acc[2]; rec[5 + d4] = acc[3];
                }
                qk_sync();   /* the record is complete in CTA scope; the release below publishes it */
                if (aligned && a.spread) {
                    /* CTA-aligned segments: the fold is spread over the first F pieces (see decode.cu) */
                    const int Fmax = a.spread, F = npieces >= Fmax ? Fmax : (npieces >= 4 && Fmax >= 4 ? 4 : (npieces >= 2 && Fmax >= 2 ? 2 : 1)), hpf = 8 / F, piece = cta - c_first;
                    if (qtid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(a.counters + sidx) : "memory");
                    if (piece >= F) continue;   /* CTA-uniform */
                    if (qtid == 0) {
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
                                if (mi.abort_flag || (i >= (1u << 14) && t1 - t0 > 500000000ull)) break;
                            }
                        }
                        if (!ok) { mi.abort_flag = 1; if (atomicCAS(a.err, 0u, 4u) == 0u) { a.err[1] = 50u; a.err[2] = blockIdx.x; a.err[3] = seen; } }
                        mi.flag = ok;
                    }
                    qk_sync();
                    h_lo = piece * hpf; h_hi = h_lo + hpf;
                    const bool mine = red && h >= h_lo && h < h_hi;
                    M = -INFINITY; L = 0.f; acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    if (mi.flag && mine) {
                        /* landing zone of head h: npieces x 528 bytes in the ring (idle: this CTA's pages are consumed) */
                        const unsigned zone = (unsigned)((h - h_lo) * npieces) * (unsigned)(kRecFloats * 4);
                        const uint8_t *src = reinterpret_cast<const uint8_t *>(a.scratch + ((size_t)c_first * 8 + h) * kRecFloats);
                        for (int c = 0; c < npieces; c++) {
                            const unsigned dst = ring_base + zone + (unsigned)c * (unsigned)(kRecFloats * 4);
                            const uint8_t *gsrc = src + (size_t)c * 8 * kRecFloats * 4;
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * (unsigned)lane), "l"(gsrc + 16 * lane) : "memory");
                            if (lane == 0) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 512u), "l"(gsrc + 512) : "memory");
                        }
                        asm volatile("cp.async.wait_all;" ::: "memory");
                        __syncwarp();
                        const float *zf = reinterpret_cast<const float *>(s_dyn + ring_off + zone);
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
                    qk_sync();   /* every landing zone is read (the sharded exchange lands its lines in the ring too) */
                    if (qtid == 0) {
                        const unsigned old = atomicAdd(a.counters + a.n_counters + sidx, 1u);
                        if (old == (unsigned)(F - 1)) { a.counters[sidx] = 0u; a.counters[a.n_counters + sidx] = 0u; }
                    }
                } else {
                    /* the LAST CTA to arrive folds, nobody waits */
                    if (qtid == 0) {
                        unsigned old;
                        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(a.counters + sidx) : "memory");
                        mi.flag = (old == (unsigned)(npieces - 1));
                    }
                    qk_sync();
                    if (!mi.flag) continue;   /* CTA-uniform */
                    /* fold all pieces with the rule of hy3_gpu.cu:233-247: the records are fetched with 16-byte asynchronous
                     * copies issued by all threads at once into the page ring when it is idle (CTA-aligned segments: this
                     * CTA's pages are consumed), else into the small landing zone, in rounds */
                    const unsigned land = aligned ? ring_base : s_base + kOffLand;
                    const float *land_g = reinterpret_cast<const float *>(aligned ? s_dyn + ring_off : s_dyn + kOffLand);
                    const int land_cap = (aligned ? kStages * kStageBytes : kLandBytes) / (8 * kRecFloats * 4);
                    M = -INFINITY; L = 0.f; acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    for (int c0 = 0; c0 < npieces; c0 += land_cap) {
                        const int nc = min(land_cap, npieces - c0);
                        const uint8_t *src = reinterpret_cast<const uint8_t *>(a.scratch + (size_t)(c_first + c0 + rec_base) * 8 * kRecFloats);
                        for (int i = qtid; i < nc * (8 * kRecFloats / 4); i += kQkThreads)
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(land + 16u * (unsigned)i), "l"(src + 16 * (size_t)i) : "memory");
                        asm volatile("cp.async.wait_all;" ::: "memory");
                        qk_sync();
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
                        if (c0 + land_cap < npieces) qk_sync();   /* landing zone is reused */
                    }
                    if (qtid == 0) a.counters[sidx] = 0u; /* self-reset for the next launch */
                    qk_sync();   /* the landing zone is read */
                }
            }
            const bool fin = red && h >= h_lo && h < h_hi;   /* this thread finishes its (head, 4 dims) of the segment */
            if (SHARD) {
                /* sequence sharding: this rank's records go into every other rank's gather buffer as flagged lines, then
                 * the same threads collect the other ranks' lines and finish the segment (see decode.cu) */
                const int seg = row * G + hl;
                if (fin) {
                    const unsigned flag = a.shard_round[seg * 8 + h] + 1u;
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
                    fa.n_ranks = a.n_dest; fa.my_rank = a.my_rank; fa.line_a = 1 + (d4 >> 1); fa.flag = flag; fa.h = h; fa.lane = lane;
                    fa.own_m = m_nat; fa.own_l = L; fa.own_acc[0] = acc[0]; fa.own_acc[1] = acc[1]; fa.own_acc[2] = acc[2]; fa.own_acc[3] = acc[3];
                    if (aligned) {
                        /* the page ring is idle by now and holds all 8 ranks' records at once: one round of polls */
                        fa.stage = reinterpret_cast<const uint4 *>(s_dyn + ring_off);
                        shard_fold<8>(fa);
                    } else {
                        fa.stage = reinterpret_cast<const uint4 *>(s_dyn + kOffLand);
                        shard_fold<kShardBatchU>(fa);
                    }
                    __syncwarp();
                    if (d4 == 0) a.shard_round[seg * 8 + h] = flag;
                }
                qk_sync();
                continue;
            }
            if (!fin) continue;
            if (a.user_partials) {
                float *rec = a.user_partials + ((size_t)row * G * 8 + (size_t)hl * 8 + h) * HY3A_PARTIAL_FLOATS;
                if (d4 == 0) { rec[0] = M * kLn2; rec[1] = L; } /* m in natural-log units like the reference record */
                rec[2 + d4] = acc[0]; rec[3 + d4] = acc[1]; rec[4 + d4] = acc[2]; rec[5 + d4] = acc[3];
            } else {
                const float inv = L > 0.f ? 1.f / L : 0.f;
                *reinterpret_cast<float4 *>(a.out + (size_t)row * a.out_stride + head_q * HY3A_D + d4) = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
            }
        }
        /* sharded: rows without keys on this rank were announced at the top; the other ranks' records are folded here */
        if (SHARD)
            for (int i = cta; i < n; i += gridDim.x) {
                if (s_prefix[i + 1] != s_prefix[i]) continue;
                for (int hl = 0; hl < G; hl++) {
                    const int seg = i * G + hl;
                    if (qtid < 256) {
                        const int h = (qtid >> 5) & 7, d4 = (qtid & 31) * 4;
                        shard_fold_args fa;
                        fa.rec0 = a.gathered + ((size_t)seg * 8 + h) * kShardLines; fa.rank_stride = (size_t)n * G * 8 * kShardLines; fa.err = a.err;
                        fa.out = a.out + (size_t)i * a.out_stride + ((size_t)(cache.kv_head_begin + hl) * 8 + h) * HY3A_D + d4;
                        fa.n_ranks = a.n_dest; fa.my_rank = a.my_rank; fa.line_a = 1 + (d4 >> 1); fa.flag = a.shard_round[seg * 8 + h] + 1u;
                        fa.stage = reinterpret_cast<const uint4 *>(s_dyn + kOffLand); fa.h = h; fa.lane = lane;
                        fa.own_m = -INFINITY; fa.own_l = 0.f; fa.own_acc[0] = fa.own_acc[1] = fa.own_acc[2] = fa.own_acc[3] = 0.f;
                        shard_fold<kShardBatchU>(fa);
                        __syncwarp();
                        if (d4 == 0) a.shard_round[seg * 8 + h] = fa.flag;
                    }
                    qk_sync();
                }
            }
    }
    /* ---- common exit: every role arrives here, also after a wait ran out */
    {
        if (warp == kProdWarp && lane == 0 && mi.abort_flag) {
            /* copies already issued must land before the shared memory goes away */
            for (int st = 0; st < kStages; st++)
                for (unsigned ph = 0; ph < 2; ph++)
                    for (unsigned spin = 0; spin < (1u << 14) && !mbar_test(UBAR(mi.rfull[st]), ph); spin++) __nanosleep(64);
        }
        fence_before();
        __syncthreads();
        if (warp == kIssWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kSlots * 64) : "memory");
    }
}

} /* namespace */

/* Bytes of dynamic shared memory for a batch capacity (prefix = page counts + positions of the rows). */
static size_t umma_prefix_bytes(int n) { return ((size_t)(2 * n + 2) * sizeof(int) + 127) & ~(size_t)127; }

int hy3a_decode_umma_fits(int max_batch) {
    return 1024 + ((kOffPrefix + umma_prefix_bytes(max_batch) + 1023) & ~(size_t)1023) + (size_t)kStages * kStageBytes <= (size_t)kSmemMax;
}

cudaError_t hy3a_launch_decode_umma(hy3a_ctx *ctx, const hy3a_cache_view &cv, const hy3a_batch_view &bv, hy3a_decode_args &a) {
    const size_t prefix = umma_prefix_bytes(ctx->batch_n);
    a.prefix_bytes = (int)prefix;
    a.stages = kStages;
    const size_t smem = 1024 + ((kOffPrefix + prefix + 1023) & ~(size_t)1023) + (size_t)kStages * kStageBytes;
    const bool shard = a.n_dest > 0;
    static bool attr_dev[64][2];   /* function attributes are per device */
    bool *attr_set = attr_dev[ctx->device & 63];
    if (!attr_set[shard ? 1 : 0]) {
        cudaError_t e = shard ? cudaFuncSetAttribute(hy3a_decode_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax)
                              : cudaFuncSetAttribute(hy3a_decode_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return e;
        attr_set[shard ? 1 : 0] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->decode_ctas); cfg.blockDim = dim3(kUThreads); cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    if (shard) return cudaLaunchKernelEx(&cfg, hy3a_decode_umma_kernel<true>, cv, bv, a);
    return cudaLaunchKernelEx(&cfg, hy3a_decode_umma_kernel<false>, cv, bv, a);
}
