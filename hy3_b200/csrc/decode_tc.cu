/*
 * decode_tc.cu -- split-KV GQA decode attention on the 5th-generation tensor cores (tcgen05 + TMEM)
 * for INT8 caches in the tensor-core page layout (layout 3, layout.h).
 *
 * Same job as decode.cu (replaces attention_split_kv_kernel + attention_reduce_kernel,
 * hy3_gpu.cu:183-247), same schedule, same records, same merge; what changes is who does the
 * arithmetic.  In decode.cu every warp builds mma.sync fragments from the page, converts V codes
 * to fp16 and runs softmax on 16-token granules: about 3 800 warp instructions per 128-token page
 * (INT4 more: that variant is compute-bound).  Here the page that the bulk copy lands in shared memory IS the
 * tensor-core operand (K tile: 128 tokens x 128 B; V^T tile: 128 dims x 128 B; both in the
 * K-major 128-byte-swizzle order) and the tokens, not the heads, are the M dimension:
 *
 *   S^T[128 tok x 16]  = K[128 x 128] . Qd^T     kind::i8, M=128 N=16 K=32 x4; the 16 columns are the
 *                                                8 query heads x {high, low} int8 digit of q
 *                                                (q ~ sq*(hi + lo/254)); products are exact
 *   O^T[128 dim x 16]  = V^T[128 x 128] . Pd^T   kind::i8; the 16 columns are the 8 heads x {high, low}
 *                                                digit of w = p * vscale(token) / vscale_max
 *
 * Accumulators live in TMEM (two S^T buffers per group, one O^T per group).  The CUDA cores only do the softmax: a
 * group of 256 threads owns a page; thread t of each 128-thread half owns token t of the page (one TMEM lane) for 4 of
 * the 8 query heads: 8 integers in, 4 scores, one page-wide max per head (warp redux + 4-warp exchange), 4
 * exponentials, 8 digit bytes out.  The same thread then owns output dim t of O^T: 8 integers added to 4 fp32
 * accumulators (rescaled every page by exp2(m_old - m_new): the state is small, no lazy threshold needed).  The P digits
 * are sized by the largest V scale of the page's valid tokens.  Two groups alternate pages.
 *
 * Warps: 0-7 softmax group 0, 8-15 group 1 (TMEM lane quadrant = warp % 4); 16 page producer; 17, 18 MMA issuers.
 *  - producer: two bulk copies per page into two rings (K tile: dead after Q.K^T; V^T + scales: live until P.V), and the
 *    fused append of the newest token (same arithmetic as the append kernel) into the landed copies and into HBM;
 *  - issuer of group g (one lane, blocking waits): Q.K^T of the group's next pages two ahead of its softmax, P.V as
 *    soon as the group's digits are written.  The scalar code around a tcgen05.mma costs more than the MMA (26 ns at
 *    N = 16 when issued back to back), so one issuer per group runs beside the softmax instead of inside it.
 * Every wait is bounded; a wait that runs out raises a CTA-wide abort flag, records a code in the context's error
 * word, every later wait returns at once and the kernel runs to its end; TMEM is always released.  All tcgen05.ld are
 * executed by whole warps under uniform control flow.  Events that one side can produce twice before the other side
 * looks (queries of the next segment ready, append done) are monotonic counters, not parity barriers.
 *
 * Roofline: HBM; algorithmic bytes per (token, KV head) = 260.
 *
 * Measured on B200 (INT8, 32 768 positions, batch 1): the stream phase runs at about 0.8 us per page and SM, the same
 * as decode.cu -- both are bound by HBM and ring depth there -- and the launch takes 22 us in both; what this kernel buys
 * is CUDA-core headroom (about 1/6 of the instructions).  It is the opt-in path (HY3A_INT8_TC=1) until the head and
 * tail of the launch, which the two kernels share, are shorter.
 */
#include <cuda_fp16.h>
#include <math.h>
#include <string.h>

#include "ctx.h"
#include "decode_common.cuh"
#include "rowops.cuh"

namespace {

#ifndef HY3A_TC_GROUPS
#define HY3A_TC_GROUPS 2
#endif
#ifdef HY3A_DECODE_TRACE
#define DBG(i, v) do { reinterpret_cast<volatile unsigned *>(mi.dbg)[i] = (unsigned)(v); } while (0)
#else
#define DBG(i, v) do { } while (0)
#endif
#ifndef HY3A_TC_HALVES
#define HY3A_TC_HALVES 2
#endif
constexpr int kGroups = HY3A_TC_GROUPS;         /* softmax groups; page j of a CTA belongs to group j % kGroups */
constexpr int kHalves = HY3A_TC_HALVES;         /* a group = kHalves x 128 threads; part k handles kHpt query heads of every token
                                                 * (and later of every output dim) of the page */
constexpr int kHpt = 8 / kHalves;               /* heads per thread */
constexpr int kGroupThreads = 128 * kHalves;
constexpr int kSmWarps = 4 * kHalves * kGroups;
static_assert(kSmWarps >= 8 && kSmWarps <= 30, "warps 0-7 prepare the queries; 1024 threads at most");
constexpr int kSmThreads = 32 * kSmWarps;       /* the softmax warps; warp kSmWarps = page producer, then one MMA issuer warp per group */
constexpr int kTcThreads = kSmThreads + 32 + 32 * kGroups;   /* + producer warp + one MMA issuer warp per group */
/* A page travels as two bulk copies into two rings: the K tile (first 16 KB) is dead as soon as Q.K^T has run, the rest
 * (V^T tile + K scales + V scales) lives until P.V has run -- about a softmax later.  Separate rings let the long-lived
 * parts be many without the short-lived ones taking room. */
constexpr int kKBytes = 16384, kKStages = 5;
constexpr int kVBytes = 16896, kVStride = 17408;   /* 17 KB stride keeps every V^T tile 1024-byte aligned */
constexpr int kVKsOff = 16384, kVVsOff = 16640;   /* scales inside a V stage */
/* shared-memory map, bytes from a 1024-byte aligned base */
constexpr int kOffQt = 0;                       /* Q digits^T: 16 rows x 128 B (rows 0-7 high digit of head r, rows 8-15 low digit) */
constexpr int kOffPt = 2048;                    /* P digits^T: kGroups x 16 rows x 128 B */
constexpr int kOffBar = kOffPt + 2048 * kGroups;   /* mbarriers (512 B) */
constexpr int kOffMisc = kOffBar + 512;         /* small exchange arrays (2 KB) */
constexpr int kOffFold = kOffMisc + 2048;       /* [kGroups][8 heads][128 dims] fp32; the same bytes later serve as ... */
constexpr int kOffLand = kOffFold;              /* ... the landing zone for records fetched from L2: 3 x 8 320 B */
constexpr int kLandPieces = 3;
constexpr int kFoldBytes = kGroups * 8 * HY3A_D * 4, kLandBytes = kLandPieces * 8 * HY3A_PARTIAL_FLOATS * 4;
constexpr int kOffPrefix = kOffLand + (kFoldBytes > kLandBytes ? kFoldBytes : kLandBytes);
enum { BAR_KFULL = 0, BAR_KEMPTY = 64, BAR_VFULL = 128, BAR_VEMPTY = 192, BAR_SFULL = 256, BAR_SFREE = 320, BAR_PFULL = 384, BAR_OFULL = 416, BAR_OFREE = 448, BAR_QREADY = 480, BAR_APPEND = 488 };
static_assert(kKStages <= 8 && 2 * kGroups <= 8, "barrier areas hold 8 entries each");
static_assert(kKStages >= 2 * kGroups + 1, "Q.K^T is issued two of a group's pages ahead: their K tiles must fit the K ring");
constexpr unsigned kColO = 32u * kGroups;       /* TMEM columns: S^T buffers (group g, page parity b: 16*(2g+b)), then O^T of group g at kColO + 16g */
constexpr unsigned kTmemCols = 256;
struct tc_misc {
    unsigned tmem;
    int abort_flag;
    int flag;
    unsigned dbg[16];           /* trace builds: progress marks of the roles, dumped when a wait ran out */
    unsigned q_ready;           /* segments whose query digits are in shared memory (monotonic, for the same reason as below) */
    unsigned appends_done;      /* fused appends completed by the producer warp so far (monotonic; a parity barrier would alias when the
                                 * producer runs two appends ahead of an issuer in a CTA that walks through many short segments) */
    float qf[8];
    int gmax[kGroups][2][kHalves][4][kHpt + 1];   /* [group][slot][part][warp][head of the part | V scale] */       /* [group][slot][warp][head | 8]: order-preserving ints of the per-warp page maxima of the
                                 * scores of each head and ([8]) of the V scales */
    float lpart[kGroups][kHalves][4][kHpt];
    float gm[kGroups][8];
};
static_assert(sizeof(tc_misc) <= kOffFold - kOffMisc, "misc area too small");

/* descriptors: K-major, 128-byte swizzle, 8-row groups 1024 B apart */
__device__ __forceinline__ unsigned long long make_desc(unsigned saddr) {
    return (unsigned long long)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
/* instruction descriptor, kind::i8: D = s32 (2 at bit 4), A = B = signed 8-bit (1 at bits 7 and 10), both K-major,
 * N = 16 (>>3 at bit 17), M = 128 (>>4 at bit 24) */
constexpr unsigned kIdescI8 = (2u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
__device__ __forceinline__ void umma_i8(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdescI8), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, int (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void sm_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kSmThreads) : "memory"); }
__device__ __forceinline__ void half_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(2 + id) : "memory"); }
/* the kHpt high-digit and kHpt low-digit columns of this thread's TMEM lane */
__device__ __forceinline__ void tmem_ld_pair(unsigned ta, unsigned tb, int (&x)[kHpt], int (&y)[kHpt]) {
    if constexpr (kHpt == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]) : "r"(ta) : "memory");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(y[0]), "=r"(y[1]), "=r"(y[2]), "=r"(y[3]) : "r"(tb) : "memory");
    } else {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(x[0]), "=r"(x[1]), "=r"(x[2]), "=r"(x[3]), "=r"(x[4]), "=r"(x[5]), "=r"(x[6]), "=r"(x[7]) : "r"(ta) : "memory");
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(y[0]), "=r"(y[1]), "=r"(y[2]), "=r"(y[3]), "=r"(y[4]), "=r"(y[5]), "=r"(y[6]), "=r"(y[7]) : "r"(tb) : "memory");
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
/* float -> int whose signed order is the float order (-inf included) */
__device__ __forceinline__ int ford(float x) { const int b = __float_as_int(x); return b >= 0 ? b : b ^ 0x7fffffff; }
__device__ __forceinline__ float funord(int b) { return __int_as_float(b >= 0 ? b : b ^ 0x7fffffff); }

template <bool SHARD>
__global__ void __launch_bounds__(kTcThreads, 1) hy3a_decode_tc_kernel(hy3a_cache_view cache, hy3a_batch_view batch, decode_args a) {
    extern __shared__ __align__(128) uint8_t s_raw[];
    uint8_t *s_dyn = s_raw + ((1024u - (smem_u32(s_raw) & 1023u)) & 1023u);   /* 1024-aligned in the shared window */
    const unsigned s_base = smem_u32(s_dyn);
    tc_misc &mi = *reinterpret_cast<tc_misc *>(s_dyn + kOffMisc);
    float (*s_fold)[8][HY3A_D] = reinterpret_cast<float (*)[8][HY3A_D]>(s_dyn + kOffFold);
    int *s_prefix = reinterpret_cast<int *>(s_dyn + kOffPrefix);
    const unsigned bar_base = s_base + kOffBar;
    const unsigned kring_off = (unsigned)((kOffPrefix + a.prefix_bytes + 1023) & ~1023), vring_off = kring_off + kKStages * kKBytes;
    const unsigned kring = s_base + kring_off, vring = s_base + vring_off;   /* a.stages = stages of the V ring */

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n = batch.n, G = cache.kv_heads;
    const int cta = blockIdx.x;
    if (warp == 0) TRACE(0);

    /* ---- schedule: prefix of pages per row (same unit split as decode.cu) */
    for (int i = tid; i < n; i += blockDim.x) {
        int len = batch.slot[i] + 1;
        s_prefix[i + 1] = len > 0 ? (len + HY3A_PT - 1) / HY3A_PT : 0;
    }
    if (tid == 0) {
        s_prefix[0] = 0;
        mi.abort_flag = 0;
        mi.appends_done = 0u;
        mi.q_ready = 0u;
        for (int i = 0; i < kKStages; i++) { mbar_init(bar_base + BAR_KFULL + 8 * i, 1); mbar_init(bar_base + BAR_KEMPTY + 8 * i, 1); }
        for (int i = 0; i < a.stages; i++) { mbar_init(bar_base + BAR_VFULL + 8 * i, 1); mbar_init(bar_base + BAR_VEMPTY + 8 * i, 1); }
        for (int b = 0; b < 2 * kGroups; b++) mbar_init(bar_base + BAR_SFULL + 8 * b, 1);
        for (int g2 = 0; g2 < kGroups; g2++) {
            mbar_init(bar_base + BAR_OFULL + 8 * g2, 1); mbar_init(bar_base + BAR_PFULL + 8 * g2, kGroupThreads);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
    const bool aligned = (long long)n * G < (long long)gridDim.x;
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
    if (idle && !SHARD) return;   /* sharded: idle CTAs may still own the fold of rows without local keys */

    /* ---- TMEM: two S^T buffers per group (so that Q.K^T runs ahead of the softmax) and one O^T per group */
    if (warp == kSmWarps && !idle) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&mi.tmem)), "n"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    /* fused step, still before the wait: norm weights and RoPE coefficients of the first segment's row come from the host */
    const int rl_d0 = (lane >> 4) * 64 + (lane & 15) * 4;
    float4 pre_w = make_float4(1.f, 1.f, 1.f, 1.f);
    float pre_c[4] = {1.f, 1.f, 1.f, 1.f}, pre_s[4] = {0.f, 0.f, 0.f, 0.f};
    int pre_row = -1;
    if (a.fused && !idle && warp < 8) {
        pre_w = *reinterpret_cast<const float4 *>(a.norm_w + rl_d0);
        pre_row = locate(s_prefix, batch, n, G, u_begin, u_end).row;
        hy3a_rowops::rope_coeffs(pre_c, pre_s, a.rope, batch.pos[pre_row], lane);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = mi.tmem;

    const bool is_producer = warp == kSmWarps;
    if (!is_producer) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    /* rows with no keys on this rank: zero output / empty partial (hy3_gpu.cu:197-199) */
    for (int i = cta; i < n; i += gridDim.x) {
        if (s_prefix[i + 1] != s_prefix[i] || warp >= kSmWarps) continue;
        if (SHARD) {
            for (int e = tid; e < G * 8; e += kSmThreads) {
                const unsigned flag = a.shard_round[i * G + (e >> 3)] + 1u;
                for (int r = 0; r < a.n_dest; r++)
                    if (r != a.my_rank) shard_store_line(a.dest[r] + ((size_t)i * G * 8 + e) * kShardLines, -INFINITY, 0.f, flag);
            }
            continue;
        }
        for (int e = tid; e < G * 8 * HY3A_D; e += kSmThreads) {
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
    if (warp == 0) TRACE(1);

    if (warp == kSmWarps) {
        /* ================= producer warp: lane 0 streams the CTA's pages into the ring; the whole warp performs the
         * fused append (new K / V row of the newest slot) into the landed page and into HBM */
        unsigned it = 0, appends = 0;
        bool ok = !idle;
        bool waited = false;   /* griddepcontrol.wait executed yet? */
        if (!a.early_prefetch) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
        for (long long u = u_begin; u < u_end && ok;) {
            const segment sg = locate(s_prefix, batch, n, G, u, u_end);
            const int *bt = cache.block_table + (size_t)sg.seq * cache.max_blocks_per_seq;
            const int last_page = (sg.len - 1) >> 7;
            for (int p = sg.p_begin; p < sg.p_end && ok; p++, it++) {
                const unsigned kst = it % (unsigned)kKStages, kph = (it / (unsigned)kKStages) & 1u;
                const unsigned vst = it % (unsigned)a.stages, vph = (it / (unsigned)a.stages) & 1u;
                /* before the preceding kernel is known to be complete only pages that lie wholly below the newest
                 * slot may be fetched, and only into stages that were never used */
                if (!waited && (it >= (unsigned)min(kKStages, a.stages) || (p + 1) * HY3A_PT > sg.len - 2)) { asm volatile("griddepcontrol.wait;" ::: "memory"); waited = true; }
                if (lane == 0) DBG(0, it);
                int okl = 1;
                uint8_t *page = cache.pool + hy3a_page_index(cache, bt[p], a.layer, sg.hl) * (size_t)cache.page_bytes;
                if (lane == 0) {
                    okl = mbar_wait_blocking(bar_base + BAR_KEMPTY + 8 * kst, kph ^ 1u, &mi.abort_flag, a.err, 1u) ? 1 : 0;
                    if (okl) {
                        mbar_expect_tx(bar_base + BAR_KFULL + 8 * kst, (unsigned)kKBytes);
                        bulk_g2s(kring + kst * (unsigned)kKBytes, page, (unsigned)kKBytes, bar_base + BAR_KFULL + 8 * kst);
                        DBG(1, it);
                        okl = mbar_wait_blocking(bar_base + BAR_VEMPTY + 8 * vst, vph ^ 1u, &mi.abort_flag, a.err, 2u) ? 1 : 0;
                        DBG(2, it);
                    }
                    if (okl) {
                        mbar_expect_tx(bar_base + BAR_VFULL + 8 * vst, (unsigned)kVBytes);
                        bulk_g2s(vring + vst * (unsigned)kVStride, page + kKBytes, (unsigned)kVBytes, bar_base + BAR_VFULL + 8 * vst);
                        TRACE(32 + it);
                    }
                }
                ok = __shfl_sync(0xffffffffu, okl, 0) != 0;
                if (!ok) break;
                if (a.fused && a.k_in && p == last_page) {
                    /* the newest token: normalise + rotate + quantise K, quantise V (same arithmetic as the append
                     * kernel), then patch the landed copies and the page in HBM */
                    const int tok = (sg.len - 1) & 127, kvh = cache.kv_head_begin + sg.hl;
                    const hy3a_geom geom = hy3a_make_geom(3);
                    float4 kv4 = *reinterpret_cast<const float4 *>(a.k_in + (size_t)sg.row * a.ki_stride + (size_t)kvh * HY3A_D + rl_d0);
                    float yk[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
                    hy3a_rowops::norm_rope_row(yk, a.norm_w + HY3A_D, a.eps, a.rope, batch.pos[sg.row], lane);
                    kv4 = *reinterpret_cast<const float4 *>(a.v_in + (size_t)sg.row * a.vi_stride + (size_t)kvh * HY3A_D + rl_d0);
                    const float yv[4] = {kv4.x, kv4.y, kv4.z, kv4.w};
                    mbar_wait_blocking(bar_base + BAR_KFULL + 8 * kst, kph, &mi.abort_flag, a.err, 3u);
                    mbar_wait_blocking(bar_base + BAR_VFULL + 8 * vst, vph, &mi.abort_flag, a.err, 4u);
                    /* shared-memory copy: K tile in the K ring; the bytes of the page from 16 384 on in the V stage */
                    uint8_t *sk = s_dyn + kring_off + (size_t)kst * kKBytes, *sv = s_dyn + vring_off + (size_t)vst * kVStride - kKBytes;
                    hy3a_rowops::store_row<3>(page, geom, tok, false, yk, rl_d0, lane);
                    hy3a_rowops::store_row<3>(sk, geom, tok, false, yk, rl_d0, lane, sv);
                    const unsigned sb = hy3a_rowops::store_row<3>(page, geom, tok, true, yv, rl_d0, lane);
                    hy3a_rowops::store_row<3>(sv, geom, tok, true, yv, rl_d0, lane);
                    if (lane == 0) atomicMax(cache.vs_max + a.layer * G + sg.hl, sb);
                    fence_async_smem();
                    __syncwarp();
                    appends++;
                    if (lane == 0) asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&mi.appends_done)), "r"(appends) : "memory");
                }
            }
            u = sg.seg_u0 + sg.p_end;
        }
        if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (!ok && !idle && lane == 0) {
            /* gave up: let the copies already issued land before the CTA's shared memory goes away */
            const unsigned depth = (unsigned)max(kKStages, a.stages), first = it > depth ? it - depth : 0u;
            for (unsigned j = first; j < it; j++) {
                if (j + (unsigned)kKStages >= it)
                    for (unsigned spin = 0; spin < (1u << 20) && !mbar_test(bar_base + BAR_KFULL + 8 * (j % (unsigned)kKStages), (j / (unsigned)kKStages) & 1u); spin++) __nanosleep(64);
                if (j + (unsigned)a.stages >= it)
                    for (unsigned spin = 0; spin < (1u << 20) && !mbar_test(bar_base + BAR_VFULL + 8 * (j % (unsigned)a.stages), (j / (unsigned)a.stages) & 1u); spin++) __nanosleep(64);
            }
        }
        (void)appends;
    } else if (warp > kSmWarps) {
        /* ================= MMA issuers: one warp (one lane) per softmax group.  It mirrors the group's walk over the
         * CTA's pages and issues, with blocking waits: Q.K^T of the group's first two pages of a segment; then, each time
         * the group has written the digits of page j (and has read S^T(j) and O^T of its previous page), P.V of page j and
         * Q.K^T of page j + 2 kGroups into the S^T buffer just read.  The scalar code around a tcgen05.mma costs far more
         * than the MMA itself (about 26 ns at N = 16), so issuing runs beside the softmax, not inside it. */
        const int group = warp - kSmWarps - 1;
        if (lane == 0 && !idle) {
            unsigned it = 0, cnt = 0, segs = 0, appends = 0;
            bool ok = true;
            /* wait (bounded, about half a second) until a monotonic counter in shared memory has passed `seen` */
            auto wait_counter = [&](unsigned *ctr, unsigned seen, unsigned where) {
                unsigned long long t0 = 0, t1;
                for (unsigned spin = 0;; spin++) {
                    unsigned done;
                    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(done) : "r"(smem_u32(ctr)) : "memory");
                    if (done > seen) return true;
                    if ((spin & 15u) == 15u) {
                        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                        if (t0 == 0) t0 = t1;
                        if (mi.abort_flag || t1 - t0 > 500000000ull) {
                            mi.abort_flag = 1;
                            if (atomicCAS(a.err, 0u, 1u) == 0u) a.err[1] = where;
                            return false;
                        }
                        __nanosleep(64);
                    }
                }
            };
            const unsigned long long dq = make_desc(s_base + kOffQt), dk0 = make_desc(kring), dv0 = make_desc(vring);
            const unsigned long long dp = make_desc(s_base + kOffPt + 2048u * (unsigned)group);
            for (long long u = u_begin; u < u_end && ok;) {
                const segment sg = locate(s_prefix, batch, n, G, u, u_end);
                const int npg = sg.p_end - sg.p_begin;
                const bool newest_here = a.fused && a.k_in && (sg.p_end - 1 == ((sg.len - 1) >> 7));
                const int j0 = (int)(((unsigned)group - it) % kGroups);
                auto issue_qk = [&](int jq, unsigned sbuf) {
                    const unsigned itq = it + (unsigned)jq, kst = itq % (unsigned)kKStages, kph = (itq / (unsigned)kKStages) & 1u;
                    DBG(4 + 3 * group, itq);
                    bool k2 = mbar_wait_blocking(bar_base + BAR_KFULL + 8 * kst, kph, &mi.abort_flag, a.err, 6u);
                    /* the producer warp has patched the newest token into this page when its counter has passed ours */
                    if (k2 && newest_here && jq == npg - 1) k2 = wait_counter(&mi.appends_done, appends, 7u);
                    if (!k2) return false;
                    fence_after();
                    const unsigned long long dk = dk0 + (unsigned long long)(kst * (unsigned)(kKBytes >> 4));
                    const unsigned d = tmem + 16u * sbuf;
                    umma_i8(d, dk, dq, 0u); umma_i8(d, dk + 2u, dq + 2u, 1u); umma_i8(d, dk + 4u, dq + 4u, 1u); umma_i8(d, dk + 6u, dq + 6u, 1u);
                    umma_commit(bar_base + BAR_SFULL + 8 * sbuf);
                    umma_commit(bar_base + BAR_KEMPTY + 8 * kst);   /* the K tile is consumed as soon as these MMAs have run */
                    if (itq < 8) TRACE(48 + itq);
                    return true;
                };
                ok = wait_counter(&mi.q_ready, segs, 5u);
                segs++;
                if (ok && j0 < npg) ok = issue_qk(j0, 2u * (unsigned)group + (cnt & 1u));
                if (ok && j0 + kGroups < npg) ok = issue_qk(j0 + kGroups, 2u * (unsigned)group + ((cnt + 1u) & 1u));
                for (int j = j0; j < npg && ok; j += kGroups) {
                    const unsigned itj = it + (unsigned)j, vst = itj % (unsigned)a.stages;
                    DBG(5 + 3 * group, itj);
                    ok = mbar_wait_blocking(bar_base + BAR_PFULL + 8 * group, cnt & 1u, &mi.abort_flag, a.err, 9u);
                    DBG(6 + 3 * group, itj);
                    if (!ok) break;
                    fence_after();
                    const unsigned long long dv = dv0 + (unsigned long long)(vst * (unsigned)(kVStride >> 4));
                    const unsigned d = tmem + kColO + 16u * (unsigned)group;
                    umma_i8(d, dv, dp, 0u); umma_i8(d, dv + 2u, dp + 2u, 1u); umma_i8(d, dv + 4u, dp + 4u, 1u); umma_i8(d, dv + 6u, dp + 6u, 1u);
                    umma_commit(bar_base + BAR_OFULL + 8 * group);
                    umma_commit(bar_base + BAR_VEMPTY + 8 * vst);   /* V^T and the scales are consumed: the producer may refill the stage */
                    if (itj < 8) TRACE(56 + itj);
                    if (j + 2 * kGroups < npg) ok = issue_qk(j + 2 * kGroups, 2u * (unsigned)group + (cnt & 1u));   /* the S^T buffer just read */
                    cnt++;
                }
                it += (unsigned)npg;
                if (newest_here) appends++;
                u = sg.seg_u0 + sg.p_end;
            }
        }
    } else {
        /* ================= softmax warps */
        const int group = warp / (4 * kHalves), half = (warp >> 2) % kHalves, wi = warp & 3, gt = tid & 127;
        const unsigned t_lane = (unsigned)(wi * 32) << 16;       /* TMEM lane quadrant of this warp */
        signed char *s_qt = reinterpret_cast<signed char *>(s_dyn + kOffQt);
        uint8_t *s_pt = s_dyn + kOffPt + 2048 * group;
        const bool qwarp = warp < 8;   /* warps 0-7 also prepare the queries (warp = head) and run the segment's tail */
        unsigned it = 0, cnt = 0, segs_done = 0;   /* ring position of the CTA; pages this group has processed; segments started */
        long long u = u_begin;
        while (u < u_end) {
            const segment sg = locate(s_prefix, batch, n, G, u, u_end);
            const int row = sg.row, hl = sg.hl, sidx = sg.sidx;
            const int head0 = (cache.kv_head_begin + hl) * 8;   /* first of the segment's 8 query heads */

            /* ---- Q digits of the segment's 8 heads: warp w owns head w as 4 values per lane (dims d0..d0+3); in the
             * fused step it first applies the per-head RMSNorm and RoPE (same code as the append kernel) */
            if (qwarp) {
                const int d0 = rl_d0;
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
                /* two int8 digits per query element: q ~ sq*(hi + lo/254), |hi|,|lo| <= 127 */
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
                *reinterpret_cast<unsigned *>(s_qt + hy3a_t_off(warp, d0)) = hw;
                *reinterpret_cast<unsigned *>(s_qt + hy3a_t_off(8 + warp, d0)) = lw;
                if (lane == 0) mi.qf[warp] = sqv * (1.f / 254.f) * 0.08838834764831845f * kLog2e;
                fence_async_smem();
            }
            sm_sync();
            if (tid == 0) asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&mi.q_ready)), "r"(segs_done + 1u) : "memory");
            segs_done++;
            float qf[kHpt];
#pragma unroll
            for (int h = 0; h < kHpt; h++) qf[h] = mi.qf[kHpt * half + h];
            float ostep = 0.f;   /* value of one unit of the O digits of the page whose P.V is in flight */
            if (warp == 0) TRACE(2);

            float m_ref[kHpt], l[kHpt], acc[kHpt];
#pragma unroll
            for (int h = 0; h < kHpt; h++) { m_ref[h] = -INFINITY; l[h] = 0.f; acc[h] = 0.f; }
            bool pending_o = false;
            const int npg = sg.p_end - sg.p_begin;
            const unsigned c_hi = (unsigned)(kHpt * half), c_lo = 8u + (unsigned)(kHpt * half);   /* this half's columns: high / low digits */
            const int j0 = (int)(((unsigned)group - it) % kGroups);
            for (int j = j0; j < npg; j += kGroups) {
                const unsigned itj = it + (unsigned)j, vst = itj % (unsigned)a.stages, vph = (itj / (unsigned)a.stages) & 1u;
                const int p = sg.p_begin + j;
                const uint8_t *sp = s_dyn + vring_off + (size_t)vst * kVStride;
                const unsigned sb = 2u * (unsigned)group + (cnt & 1u);   /* this page's S^T buffer */
                if ((tid % kGroupThreads) == 0) DBG(10 + 2 * group, itj);
                if (warp == 0 && cnt == 1) TRACE(23);
                mbar_wait_blocking(bar_base + BAR_SFULL + 8 * sb, (cnt >> 1) & 1u, &mi.abort_flag, a.err, 11u);
                mbar_wait_blocking(bar_base + BAR_VFULL + 8 * vst, vph, &mi.abort_flag, a.err, 12u);   /* orders the scale reads below */
                fence_after();
                int rh[kHpt], rl[kHpt];
                tmem_ld_pair(tmem + t_lane + 16u * sb + c_hi, tmem + t_lane + 16u * sb + c_lo, rh, rl);
                fence_before();
                if ((tid % kGroupThreads) == 0) DBG(11 + 2 * group, itj);
                if (warp == 0 && cnt == 1) TRACE(18);
                if (pending_o) {
                    /* O^T of this group's previous page (its digits are relative to the current m_ref) */
                    mbar_wait_blocking(bar_base + BAR_OFULL + 8 * group, (cnt - 1u) & 1u, &mi.abort_flag, a.err, 13u);
                    fence_after();
                    int oh[kHpt], ol[kHpt];
                    tmem_ld_pair(tmem + t_lane + kColO + 16u * (unsigned)group + c_hi, tmem + t_lane + kColO + 16u * (unsigned)group + c_lo, oh, ol);
                    fence_before();
#pragma unroll
                    for (int h = 0; h < kHpt; h++) acc[h] += (float)(oh[h] * 254 + ol[h]) * ostep;
                }
                if (warp == 0 && cnt == 1) TRACE(19);
                /* thread = token gt of the page, heads kHpt*half .. kHpt*half + kHpt-1 */
                const bool valid = p * HY3A_PT + gt < sg.len;
                const float ks = __half2float(*reinterpret_cast<const __half *>(sp + kVKsOff + 2 * gt));
                const float vs = __half2float(*reinterpret_cast<const __half *>(sp + kVVsOff + 2 * gt));
                float sc[kHpt];
                int *gmx = mi.gmax[group][cnt & 1u][half][wi];
#pragma unroll
                for (int h = 0; h < kHpt; h++) {
                    sc[h] = valid ? (float)(rh[h] * 254 + rl[h]) * (qf[h] * ks) : -INFINITY;
                    const int wm = __reduce_max_sync(0xffffffffu, ford(sc[h]));
                    if (lane == h) gmx[h] = wm;
                }
                {
                    const int wm = __reduce_max_sync(0xffffffffu, valid ? __float_as_int(vs) : 0);   /* scales are >= 0 */
                    if (lane == kHpt) gmx[kHpt] = wm;
                }
                if (warp == 0 && cnt == 1) TRACE(20);
                half_sync(kHalves * group + half);
                if (warp == 0 && cnt == 1) TRACE(21);
                /* P digits are sized by the largest V scale of this page's valid tokens: w = p * vs / vmax * 127 <= 127 */
                const int (*gm4)[kHpt + 1] = mi.gmax[group][cnt & 1u][half];
                const float vmax = fmaxf(__int_as_float(max(max(gm4[0][kHpt], gm4[1][kHpt]), max(gm4[2][kHpt], gm4[3][kHpt]))), 1e-30f);
                const float wv = valid ? vs * (127.f / vmax) : 0.f;
                ostep = vmax * (1.f / (127.f * 254.f));
#pragma unroll
                for (int h = 0; h < kHpt; h++) {
                    const float pm = funord(max(max(gm4[0][h], gm4[1][h]), max(gm4[2][h], gm4[3][h])));   /* finite: token 0 of the page is valid */
                    const float m_new = fmaxf(m_ref[h], pm);
                    const float alpha = ex2(m_ref[h] - m_new);      /* 0 on the first page (m_ref = -inf) */
                    const float pe = ex2(sc[h] - m_new);             /* -inf -> 0 */
                    acc[h] *= alpha;
                    l[h] = l[h] * alpha + pe;
                    m_ref[h] = m_new;
                    /* two int8 digits of w = p * vscale / vscale_max * 127 in [0, 127] */
                    const float X = pe * wv;
                    const float hi = rintf(X);
                    const float lo = rintf((X - hi) * 254.f);
                    s_pt[hy3a_t_off(kHpt * half + h, gt)] = (uint8_t)(int)hi;
                    s_pt[hy3a_t_off(8 + kHpt * half + h, gt)] = (uint8_t)(signed char)(int)lo;
                }
                if (warp == 0 && cnt == 1) TRACE(22);
                fence_async_smem();
                mbar_arrive(bar_base + BAR_PFULL + 8 * group);   /* digits written, S^T and O^T read: over to the group's issuer */
                pending_o = true;
                cnt++;
                if (warp == 0) TRACE(3 + j / kGroups);
            }
            if (pending_o) {
                mbar_wait_blocking(bar_base + BAR_OFULL + 8 * group, (cnt - 1u) & 1u, &mi.abort_flag, a.err, 14u);
                fence_after();
                int oh[kHpt], ol[kHpt];
                tmem_ld_pair(tmem + t_lane + kColO + 16u * (unsigned)group + c_hi, tmem + t_lane + kColO + 16u * (unsigned)group + c_lo, oh, ol);
                fence_before();
#pragma unroll
                for (int h = 0; h < kHpt; h++) acc[h] += (float)(oh[h] * 254 + ol[h]) * ostep;
            }
            it += (unsigned)npg;

            /* ---- fold the groups of this CTA (shared memory): thread = output dim gt of its group */
#pragma unroll
            for (int h = 0; h < kHpt; h++) {
                float lh = l[h];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) lh += __shfl_xor_sync(0xffffffffu, lh, o);
                if (lane == 0) mi.lpart[group][half][wi][h] = lh;
                s_fold[group][kHpt * half + h][gt] = acc[h];
                if (gt == h) mi.gm[group][kHpt * half + h] = m_ref[h];
            }
            sm_sync();
            const int h = (tid >> 5) & 7, d4 = (tid & 31) * 4;    /* thread -> (head, 4 dims); the first 256 threads carry the tail */
            float M = -INFINITY;
#pragma unroll
            for (int g2 = 0; g2 < kGroups; g2++) M = fmaxf(M, mi.gm[g2][h]);
            float L = 0.f, accv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int g2 = 0; g2 < kGroups; g2++) {
                const float mg = mi.gm[g2][h];
                if (mg == -INFINITY) continue;
                const float f = ex2(mg - M);
                const float (*lp)[kHpt] = mi.lpart[g2][h / kHpt];
                L += (lp[0][h % kHpt] + lp[1][h % kHpt] + lp[2][h % kHpt] + lp[3][h % kHpt]) * f;
                const float4 o4 = *reinterpret_cast<const float4 *>(&s_fold[g2][h][d4]);
                accv[0] += o4.x * f; accv[1] += o4.y * f; accv[2] += o4.z * f; accv[3] += o4.w * f;
            }
            sm_sync(); /* fold buffers free again */
            if (warp == 0) TRACE(24);

            /* ---- how many CTAs share this segment? (same record protocol as decode.cu) */
            const bool red = qwarp;
            const int c_first = aligned ? al_first : (int)(((sg.seg_u0 + 1) * C + U - 1) / U) - 1;
            const int npieces = aligned ? al_pieces : (int)((sg.seg_u1 * C + U - 1) / U) - 1 - c_first + 1;
            const int rec_base = aligned ? 0 : sidx;   /* record index = CTA (+ segment when CTAs may hold several pieces) */
            const size_t head_q = (size_t)(cache.kv_head_begin + hl) * 8 + h; /* global query head */
            u = sg.seg_u0 + sg.p_end;

            if (npieces > 1) {
                if (red) {
                    float *rec = a.scratch + ((size_t)(cta + rec_base) * 8 + h) * HY3A_PARTIAL_FLOATS;
                    if (d4 == 0) { rec[0] = M; rec[1] = L; }
                    rec[2 + d4] = accv[0]; rec[3 + d4] = accv[1]; rec[4 + d4] = accv[2]; rec[5 + d4] = accv[3];
                }
                __threadfence();   /* every writer orders its part of the record before the arrival below */
                sm_sync();
                if (tid == 0) {
                    unsigned old = atomicAdd(a.counters + sidx, 1u);
                    mi.flag = (old == (unsigned)(npieces - 1));
                }
                sm_sync();
                if (warp == 0) TRACE(25);
                if (!mi.flag) continue;   /* CTA-uniform among the softmax warps */
                __threadfence();
                /* last arrival: fold all pieces with the rule of hy3_gpu.cu:233-247; the records are fetched with 16-byte
                 * asynchronous copies into the idle page ring (CTA-aligned segments) or the small landing zone */
                const bool ring_idle = aligned;
                const unsigned land = ring_idle ? vring : s_base + kOffLand;
                const float *land_g = reinterpret_cast<const float *>(ring_idle ? s_dyn + vring_off : s_dyn + kOffLand);
                const int land_cap = ring_idle ? a.stages * kVStride / (8 * HY3A_PARTIAL_FLOATS * 4) : kLandPieces;
                M = -INFINITY; L = 0.f; accv[0] = accv[1] = accv[2] = accv[3] = 0.f;
                for (int c0 = 0; c0 < npieces; c0 += land_cap) {
                    const int nc = min(land_cap, npieces - c0);
                    const uint8_t *src = reinterpret_cast<const uint8_t *>(a.scratch + (size_t)(c_first + c0 + rec_base) * 8 * HY3A_PARTIAL_FLOATS);
                    for (int i = tid; i < nc * 260; i += kSmThreads)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(land + 16u * (unsigned)i), "l"(src + 16 * (size_t)i) : "memory");
                    asm volatile("cp.async.wait_all;" ::: "memory");
                    sm_sync();
                    for (int c = 0; c < nc && red; c++) {
                        const float *pr = land_g + ((size_t)c * 8 + h) * HY3A_PARTIAL_FLOATS;
                        const float pm = pr[0], pl = pr[1];
                        if (!(pl > 0.f)) continue;
                        const float2 v01 = *reinterpret_cast<const float2 *>(pr + 2 + d4), v23 = *reinterpret_cast<const float2 *>(pr + 4 + d4);
                        const float nm = fmaxf(M, pm), os = ex2(M - nm), rs = ex2(pm - nm);
                        L = L * os + pl * rs;
                        accv[0] = accv[0] * os + v01.x * rs; accv[1] = accv[1] * os + v01.y * rs;
                        accv[2] = accv[2] * os + v23.x * rs; accv[3] = accv[3] * os + v23.y * rs;
                        M = nm;
                    }
                    if (c0 + land_cap < npieces) sm_sync();   /* landing zone is reused */
                }
                if (tid == 0) a.counters[sidx] = 0u; /* self-reset for the next launch */
                sm_sync();   /* the landing zone is read; the next segment may reuse the buffer */
                if (warp == 0) TRACE(26);
            }
            if (SHARD) {
                /* sequence sharding: this rank's records of the segment go into every other rank's gather buffer as
                 * flagged lines, then the same threads collect the other ranks' lines and finish the segment */
                const int seg = row * G + hl;
                const unsigned flag = a.shard_round[seg] + 1u;
                const float m_nat = M * kLn2;
                const size_t ro = ((size_t)seg * 8 + h) * kShardLines;
                for (int r = 0; r < a.n_dest && red; r++) {
                    if (r == a.my_rank) continue;
                    uint4 *rec = a.dest[r] + ro;
                    if (d4 == 0) shard_store_line(rec, m_nat, L, flag);
                    shard_store_line(rec + 1 + (d4 >> 1), accv[0], accv[1], flag);
                    shard_store_line(rec + 2 + (d4 >> 1), accv[2], accv[3], flag);
                }
                if (warp == 0) TRACE(27);
                shard_fold_args fa;
                fa.rec0 = a.gathered + ro; fa.rank_stride = (size_t)n * G * 8 * kShardLines; fa.err = a.err;
                fa.out = a.out + (size_t)row * a.out_stride + ((size_t)(cache.kv_head_begin + hl) * 8 + h) * HY3A_D + d4;
                fa.n_ranks = a.n_dest; fa.my_rank = a.my_rank; fa.line_a = 1 + (d4 >> 1); fa.flag = flag;
                fa.stage = reinterpret_cast<const uint4 *>(s_dyn + kOffLand); fa.h = h; fa.lane = lane;
                fa.own_m = m_nat; fa.own_l = L; fa.own_acc[0] = accv[0]; fa.own_acc[1] = accv[1]; fa.own_acc[2] = accv[2]; fa.own_acc[3] = accv[3];
                if (red) {
                    if (aligned && (size_t)a.stages * kVStride >= (size_t)8 * 8 * kShardLines * 16) {
                        fa.stage = reinterpret_cast<const uint4 *>(s_dyn + vring_off);   /* the idle V ring holds all 8 ranks' records */
                        shard_fold<8>(fa);
                    } else {
                        shard_fold<kLandPieces>(fa);
                    }
                }
                if (warp == 0) TRACE(30);
                sm_sync();                 /* every thread has read the use count */
                if (tid == 0) a.shard_round[seg] += 1u;
                continue;
            }
            if (!red) continue;
            if (a.user_partials) {
                float *rec = a.user_partials + ((size_t)row * G * 8 + (size_t)hl * 8 + h) * HY3A_PARTIAL_FLOATS;
                if (d4 == 0) { rec[0] = M * kLn2; rec[1] = L; } /* m in natural-log units like the reference record */
                rec[2 + d4] = accv[0]; rec[3 + d4] = accv[1]; rec[4 + d4] = accv[2]; rec[5 + d4] = accv[3];
            } else {
                float inv = L > 0.f ? 1.f / L : 0.f;
                float4 o4 = make_float4(accv[0] * inv, accv[1] * inv, accv[2] * inv, accv[3] * inv);
                *reinterpret_cast<float4 *>(a.out + (size_t)row * a.out_stride + head_q * HY3A_D + d4) = o4;
            }
        }
        /* sharded: rows without keys on this rank were announced at the top; the other ranks' records are folded here */
        if (SHARD)
            for (int i = cta; i < n; i += gridDim.x) {
                if (s_prefix[i + 1] != s_prefix[i]) continue;
                for (int hl = 0; hl < G; hl++) {
                    const int seg = i * G + hl;
                    const int h = (tid >> 5) & 7, d4 = (tid & 31) * 4;
                    shard_fold_args fa;
                    fa.rec0 = a.gathered + ((size_t)seg * 8 + h) * kShardLines; fa.rank_stride = (size_t)n * G * 8 * kShardLines; fa.err = a.err;
                    fa.out = a.out + (size_t)i * a.out_stride + ((size_t)(cache.kv_head_begin + hl) * 8 + h) * HY3A_D + d4;
                    fa.n_ranks = a.n_dest; fa.my_rank = a.my_rank; fa.line_a = 1 + (d4 >> 1); fa.flag = a.shard_round[seg] + 1u;
                    fa.stage = reinterpret_cast<const uint4 *>(s_dyn + kOffLand); fa.h = h; fa.lane = lane;
                    fa.own_m = -INFINITY; fa.own_l = 0.f; fa.own_acc[0] = fa.own_acc[1] = fa.own_acc[2] = fa.own_acc[3] = 0.f;
                    if (qwarp) shard_fold<kLandPieces>(fa);
                    sm_sync();
                    if (tid == 0) a.shard_round[seg] += 1u;
                }
            }
    }

#ifdef HY3A_DECODE_TRACE
    __syncthreads();
    if (mi.abort_flag && tid < 16) a.trace[(size_t)blockIdx.x * 64 + 40 + tid] = 0x100000000ull | mi.dbg[tid];
#endif
    /* ---- everyone meets here; TMEM goes back */
    fence_before();
    __syncthreads();
    if (warp == kSmWarps && !idle) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(kTmemCols) : "memory");
    }
}

} /* namespace */

cudaError_t hy3a_launch_decode_tc(hy3a_ctx *ctx, const hy3a_cache_view &cv, const hy3a_batch_view &bv, hy3a_decode_args &a) {
    /* Known limitation of this opt-in kernel: when there are at least as many (row, KV head) segments as CTAs, a CTA walks
     * through pieces of several segments, and in that mode the pipeline has stalled intermittently on a B200 (the bounded
     * waits turn the stall into HY3A_ETIMEOUT; cause not found yet).  Such batches are refused here; the mma.sync kernel
     * (default layout) serves them at 0.88 of the HBM roofline. */
    if ((long long)ctx->batch_n * ctx->cfg.kv_head_count >= (long long)ctx->decode_ctas) return cudaErrorNotSupported;
    const size_t prefix = ((size_t)(ctx->batch_n + 1) * sizeof(int) + 127) & ~(size_t)127;
    a.prefix_bytes = (int)prefix;
    const size_t fixed = (((size_t)kOffPrefix + prefix + 1023) & ~(size_t)1023) + 1024;   /* + slack for the 1024-byte alignment */
    int stages = (int)(((size_t)kSmemMax - fixed - (size_t)kKStages * kKBytes) / kVStride);   /* V ring */
    if (stages > 8) stages = 8;
    if (ctx->decode_stages >= 2 && ctx->decode_stages < stages) stages = ctx->decode_stages;
    if (stages < 2) return cudaErrorInvalidConfiguration;
    a.stages = stages;
    const size_t smem = fixed + (size_t)kKStages * kKBytes + (size_t)stages * kVStride;
    static bool attr_dev[64][2];   /* function attributes are per device */
    bool *attr_set = attr_dev[ctx->device & 63];
    const bool shard = a.n_dest > 0;
    if (!attr_set[shard ? 1 : 0]) {
        cudaError_t e = shard ? cudaFuncSetAttribute(hy3a_decode_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax)
                              : cudaFuncSetAttribute(hy3a_decode_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return e;
        attr_set[shard ? 1 : 0] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctx->decode_ctas); cfg.blockDim = dim3(kTcThreads); cfg.dynamicSmemBytes = smem; cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    if (shard) return cudaLaunchKernelEx(&cfg, hy3a_decode_tc_kernel<true>, cv, bv, a);
    return cudaLaunchKernelEx(&cfg, hy3a_decode_tc_kernel<false>, cv, bv, a);
}
