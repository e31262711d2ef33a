/*
 * decode_common.cuh -- helpers of the decode kernel: the argument block, the unit schedule
 * (segment / locate), shared-memory, mbarrier and bulk-copy primitives with bounded waits, and the
 * receiving side of the sequence-shard exchange.  Everything lives in an unnamed namespace: each
 * translation unit gets its own copy.
 */
#ifndef HY3A_DECODE_COMMON_CUH
#define HY3A_DECODE_COMMON_CUH

#include <cuda_fp16.h>
#include <math.h>

#include "ctx.h"

/* Argument block of the decode kernels (filled by hy3a_launch_decode / hy3a_decode_noalloc in decode.cu). */
struct hy3a_decode_args {
    const float *q;
    size_t q_stride;
    float *out;
    size_t out_stride;
    float *user_partials; /* NULL or [n][8*kv_heads][130] */
    /* sequence sharding with the exchange inside the kernel (n_dest = world size > 0): the CTA that completes a
     * (row, KV head) segment stores its 8 records, as 16-byte lines {value, flag, value, flag}, into every other
     * rank's gather buffer (dest[r], already offset to this rank's slice there), then polls the lines the other
     * ranks store into its own buffer, folds all ranks' records in rank order and writes the final output.
     * flag = use count of the (slot, segment) + 1, kept in shard_round on every rank.                          */
    int n_dest, my_rank;
    uint4 *dest[8];
    const uint4 *gathered;        /* local: [n_dest][n*kv_heads*8][65] lines of the slot */
    unsigned *shard_round;        /* local: [n*kv_heads*8] uses of the slot so far, per head */
    float *scratch;       /* merge records: [(gridDim.x + n*kv_heads)][8][HY3A_REC_FLOATS] */
    unsigned int *counters; /* [2][n_counters]: arrivals per (row, KV head) segment, then finished folds */
    int n_counters;
    int spread;           /* > 0: CTA-aligned segments spread their fold over up to this many of their CTAs (the whole grid is resident) */
    unsigned int *err;
    int layer;
    /* fused step (fused != 0): the kernel itself normalises + rotates the queries read from q_in and
     * the CTA that streams the page of the newest slot quantises and appends the new K / V row   */
    int fused;
    int early_prefetch;   /* pages below the newest slots may be fetched before griddepcontrol.wait */
    const float *q_in, *k_in, *v_in;
    size_t qi_stride, ki_stride, vi_stride;
    float *q_out;         /* optional: normalised + rotated queries, fp32 [n][64][128] */
    size_t q_out_stride;
    const float *norm_w;  /* [2][128] of this layer */
    float eps;
    hy3a_rope_params rope;
    int stages;           /* staged variant: pages in the shared-memory ring (2..8) */
    int prefix_bytes;     /* bytes reserved for the page-count prefix */
};

/* the INT8 decode kernel (decode_umma.cu) */
cudaError_t hy3a_launch_decode_umma(hy3a_ctx *ctx, const hy3a_cache_view &cv, const hy3a_batch_view &bv, hy3a_decode_args &a);

namespace {

constexpr int kSmemMax = 232448 - 1024;                /* opt-in limit per block minus the driver's reserve */
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

typedef hy3a_decode_args decode_args;

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
    sg.hl = (int)((unsigned)(u - row_u0) / (unsigned)sg.pages);   /* both fit 32 bits: a 64-bit division costs hundreds of cycles */
    sg.seg_u0 = row_u0 + (long long)sg.hl * sg.pages;
    sg.seg_u1 = sg.seg_u0 + sg.pages;
    sg.p_begin = (int)(u - sg.seg_u0);
    sg.p_end = (int)((sg.seg_u1 < u_end ? sg.seg_u1 : u_end) - sg.seg_u0);
    sg.sidx = lo * G + sg.hl;
    sg.len = batch.slot[lo] + 1;
    sg.seq = batch.seq[lo];
    return sg;
}

/* The CTA-aligned split gives every (row, KV head) segment whole CTAs in proportion to its pages.  With few segments that is
 * balanced to a page; when the segments are about as many as the CTAs the rounding leaves some CTAs with far more pages than
 * the even share (64 rows of one KV head on 148 CTAs: up to 1.75 x), and the plain equal split over all units is the better
 * one.  Returns whether the aligned split stays within 5/4 of the even share.  Every lane takes rows lane, lane + 32, ...;
 * call with all lanes of the warp; the result is the same in every warp. */
__device__ __forceinline__ bool aligned_split_balanced(const int *s_prefix, int n, int G, unsigned grid, int lane) {
    if ((unsigned)(n * G) * 4u <= grid) return true;   /* at least four CTAs per segment */
    const unsigned long long P = (unsigned)s_prefix[n];
    int ne = 0;
    for (int r = lane; r < n; r += 32) ne += (s_prefix[r + 1] != s_prefix[r]);
    ne = __reduce_add_sync(0xffffffffu, ne);
    const unsigned long long spare = grid - (unsigned)(ne * G), PG = P * (unsigned)G;
    if (PG == 0) return true;
    unsigned worst = 0;
    for (int r = lane; r < n; r += 32) {
        const unsigned p = (unsigned)(s_prefix[r + 1] - s_prefix[r]);
        if (p == 0) continue;
        unsigned long long c = 1ull + spare * p / PG;
        if (c > p) c = p;
        const unsigned w = (unsigned)((p + c - 1ull) / c);
        worst = worst > w ? worst : w;
    }
    worst = __reduce_max_sync(0xffffffffu, worst);
    const unsigned long long even = (PG + grid - 1ull) / grid;
    return (unsigned long long)worst * 4ull <= even * 5ull + 4ull;
}

/* ---- shared-memory / mbarrier / bulk-copy primitives ---------------------------------- */
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
/* Blocking flavour of the wait: mbarrier.try_wait suspends the thread in hardware (up to the hinted time) instead of
 * spinning, so that waiting warps do not take issue slots from working ones.  Bounded in time (about half a second)
 * through the global timer; on expiry same protocol as mbar_wait below. */
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity, unsigned hint_ns) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_blocking(unsigned bar, unsigned parity, volatile int *abort_flag, unsigned *err, unsigned where) {
    if (mbar_try(bar, parity, 2000u)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (unsigned i = 0; i < (1u << 22); i++) {
        if (mbar_try(bar, parity, 20000u)) return true;
        if (*abort_flag) return false;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        /* both a real amount of waiting and the clock must agree: the global timer can step (it is re-synchronised with the
         * host clock), and a try_wait may return long before its hint */
        if (i >= (1u << 13) && t1 - t0 > 500000000ull) break;
    }
    *abort_flag = 1;
    if (atomicCAS(err, 0u, 1u) == 0u) { err[1] = where; err[2] = blockIdx.x; err[3] = bar; }
    return false;
}
/* The KV stream is read once per step: its lines are marked evict-first in L2, so that what is small and re-read by every
 * launch (queries, batch descriptor, block table, norm weights, merge records) stays resident beside 68 MB of pages per launch. */
__device__ __forceinline__ unsigned long long l2_evict_first_policy() {
    unsigned long long pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s(unsigned dst, const void *src, unsigned bytes, unsigned bar, unsigned long long policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy) : "memory");
}
/* Bounded wait: gives up after ~2^22 polls (far beyond any legitimate wait), records the
 * failure in the device error word and raises the CTA-wide abort flag; once the flag is up
 * every later wait returns at once, so all warps keep the same control flow and the kernel
 * runs to its end (with a meaningless result that the host discards on seeing the error). */
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int *abort_flag, unsigned *err, unsigned where) {
    if (mbar_test(bar, parity)) return true;
    for (unsigned i = 0; i < (1u << 22); i++) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 63u) == 63u) { if (*abort_flag) return false; __nanosleep(32); }
    }
    *abort_flag = 1;
    if (atomicCAS(err, 0u, 1u) == 0u) err[1] = where;
    return false;
}
/* ---- pieces both decode kernels use */
__device__ __forceinline__ void imma16832(int c[4], const uint4 &a, unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float2 unpack_h2(unsigned v) {
    __half2 h = *reinterpret_cast<__half2 *>(&v);
    return __half22float2(h);
}
/* INT8/INT4 caches, Q.K^T on m16n8k32: for k-step kk (0..3) the eight k-slots (4tig..4tig+3, 16+4tig..16+4tig+3) of
 * thread-in-group tig carry head dims kdim32<DT>(kk, tig, 0..7): exactly the dims whose codes the thread gets out of its own
 * 16-byte loads of a K row. */
template <int DT> __device__ __forceinline__ int kdim32(int kk, int tig, int s) {
    if (DT == 1) return 16 * (tig + 4 * (s >> 2)) + 4 * kk + (s & 3);   /* chunk tig / tig+4, word kk */
    return 32 * tig + 8 * kk + 2 * (s & 3) + (s >> 2);                   /* word kk: even nibbles, then odd nibbles */
}

/* Sequence sharding: lines of one head's record in a gather buffer: line 0 = {m, l}, line 1 + j = acc[2j], acc[2j+1]. */
constexpr int kShardLines = HY3A_PARTIAL_FLOATS / 2;   /* 65 */
__device__ __forceinline__ void shard_store_line(uint4 *p, float x, float y, unsigned flag) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(p), "r"(__float_as_uint(x)), "r"(flag), "r"(__float_as_uint(y)) : "memory");
}
__device__ __forceinline__ uint4 shard_load_line(const uint4 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

/* Sequence sharding, receiving side; run by the first 8 warps of one CTA for one (row, KV head) segment: thread
 * (h, d4) polls the three lines it needs of every other rank's record (all ranks' loads are issued before any is
 * checked, so the usual cost is one L2 round trip), takes its own rank's values from registers, folds in rank
 * order with the rule of hy3_gpu.cu:233-247 (same order on every rank: identical bits) and writes the normalised
 * output.  The wait is bounded in polls and in time (about a second); when it runs out a code goes into the
 * error word, later waits return at once and the kernel runs to its end.                                      */
struct shard_fold_args {
    const uint4 *rec0;     /* line 0 of rank 0's record of this thread's (segment, head) */
    size_t rank_stride;    /* lines between consecutive ranks' records */
    unsigned *err;
    float *out;            /* this thread's 4 output floats */
    const uint4 *stage;    /* shared memory, [kShardBatch][8 heads][65] lines: landing zone of the polls */
    int n_ranks, my_rank, line_a, h, lane;
    unsigned flag;
    float own_m, own_l, own_acc[4];
};

/* Run by the first 8 warps (all lanes) for one segment.  Polling costs no registers: every thread copies the three
 * lines it needs of each pending rank's record into shared memory with 16-byte asynchronous copies (L2 -> shared),
 * all ranks of a batch in flight at once, and checks the flags there; the usual cost is one L2 round trip per batch.
 * Own rank: values from registers.  Fold in rank order (hy3_gpu.cu:233-247): identical bits on every rank.
 * The wait is bounded in polls and in time (about a second); when it runs out a code goes into the error word, the
 * missing records count as empty, later waits return at once and the kernel runs to its end.                       */
template <int kShardBatch>   /* ranks polled at once: kShardBatch x 8 320 bytes of landing zone */
__device__ __forceinline__ void shard_fold(const shard_fold_args &a) {
    float ms = -INFINITY, ss = 0.f, ov[4] = {0.f, 0.f, 0.f, 0.f};
    const unsigned stage_u32 = smem_u32(a.stage);
#pragma unroll 1
    for (int base = 0; base < a.n_ranks; base += kShardBatch) {
        const int cnt = min(kShardBatch, a.n_ranks - base);
        unsigned pending = 0u;   /* bit j: rank base + j not complete yet (per thread) */
        for (int j = 0; j < cnt; j++) if (base + j != a.my_rank) pending |= 1u << j;
        unsigned long long t0 = 0;
        bool gave_up = false;
#pragma unroll 1
        for (unsigned i = 0; __any_sync(0xffffffffu, pending != 0u); i++) {
#pragma unroll 1
            for (int j = 0; j < cnt; j++)
                if (pending & (1u << j)) {
                    const uint4 *rec = a.rec0 + (size_t)(base + j) * a.rank_stride;
                    const unsigned dst = stage_u32 + (unsigned)((j * 8 + a.h) * kShardLines) * 16u;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * (unsigned)a.line_a), "l"(rec + a.line_a) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * (unsigned)(a.line_a + 1)), "l"(rec + a.line_a + 1) : "memory");
                    if (a.lane == 0) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(rec) : "memory");
                }
            asm volatile("cp.async.wait_all;" ::: "memory");
            __syncwarp();
#pragma unroll 1
            for (int j = 0; j < cnt; j++)
                if (pending & (1u << j)) {
                    const uint4 *st = a.stage + (j * 8 + a.h) * kShardLines;
                    const uint4 l0 = st[0];
                    if (l0.y != a.flag || l0.w != a.flag) continue;
                    if (__uint_as_float(l0.z) > 0.f) {
                        const uint4 la = st[a.line_a], lb = st[a.line_a + 1];
                        if (la.y != a.flag || la.w != a.flag || lb.y != a.flag || lb.w != a.flag) continue;
                    }
                    pending &= ~(1u << j);
                }
            __syncwarp();   /* lane 0 may overwrite line 0 in the next round */
            if ((i & 15u) == 15u) {
                bool stop = *reinterpret_cast<volatile unsigned *>(a.err) != 0u;
                if (!stop && pending) {
                    unsigned long long t1;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
                    if (t0 == 0) t0 = t1;
                    if (t1 - t0 > 1000000000ull || i > (1u << 24)) {
                        if (atomicCAS(a.err, 0u, 3u) == 0u) a.err[1] = 41u;
                        stop = true;
                    }
                }
                if (__any_sync(0xffffffffu, stop && pending)) { gave_up = true; break; }
                __nanosleep(32);
            }
        }
#pragma unroll 1
        for (int j = 0; j < cnt; j++) {
            float pm, pl, pv[4];
            if (base + j == a.my_rank) {
                pm = a.own_m; pl = a.own_l; pv[0] = a.own_acc[0]; pv[1] = a.own_acc[1]; pv[2] = a.own_acc[2]; pv[3] = a.own_acc[3];
                if (!(pl > 0.f)) continue;
            } else {
                if (gave_up && (pending & (1u << j))) continue;
                const uint4 *st = a.stage + (j * 8 + a.h) * kShardLines;
                const uint4 l0 = st[0];
                pm = __uint_as_float(l0.x); pl = __uint_as_float(l0.z);
                if (!(pl > 0.f)) continue;
                const uint4 la = st[a.line_a], lb = st[a.line_a + 1];
                pv[0] = __uint_as_float(la.x); pv[1] = __uint_as_float(la.z); pv[2] = __uint_as_float(lb.x); pv[3] = __uint_as_float(lb.z);
            }
            const float nm = fmaxf(ms, pm), os = __expf(ms - nm), rs = __expf(pm - nm);
            ss = ss * os + pl * rs;
            ov[0] = ov[0] * os + pv[0] * rs; ov[1] = ov[1] * os + pv[1] * rs; ov[2] = ov[2] * os + pv[2] * rs; ov[3] = ov[3] * os + pv[3] * rs;
            ms = nm;
        }
        __syncwarp();   /* the landing zone is reused by the next batch of ranks */
    }
    const float inv = ss > 0.f ? 1.f / ss : 0.f;
    *reinterpret_cast<float4 *>(a.out) = make_float4(ov[0] * inv, ov[1] * inv, ov[2] * inv, ov[3] * inv);
}

} /* namespace */
#endif
