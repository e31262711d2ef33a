/*
 * prefill.cu -- causal chunk attention on 5th-generation tensor cores (tcgen05 + TMEM + TMA).
 *
 * Replaces prefill_attn_int8/int4_kernel (hy3_gpu.cu:383-447), which walks the keys serially with
 * one warp per (query head, 16-query tile) on CUDA cores.  Semantics kept: query i of the chunk has
 * global index base+i and attends keys [0, base+i]; the chunk's own K/V were appended first, so
 * queries see the cache's (quantised) K/V also for their own chunk (hy3_gpu.cu:823-832).
 *
 * Two kernels per (layer, chunk):
 *   1. hy3a_kv_to_f16_kernel<DT>: converts the sequence's pages of this layer into dense fp16 operands,
 *      dequantising INT8/INT4 (value = code * fp16 scale, hy3_gpu.cu:206-215): K as [head][token][128]
 *      (d contiguous) and V TRANSPOSED as [head][128][token] (tokens contiguous), so that both are
 *      K-major operands for the tensor cores.  The operands of a layer are kept across chunks (the
 *      context's per-layer mirrors), so a chunk only converts the pages it appended.
 *   2. hy3a_prefill_kernel: one CTA per (32 query tokens x the 8 query heads of one KV head) = two
 *      128-row Q tiles (GQA packing: the 8 heads share every K/V tile).  Warp-specialised:
 *        TMA producer: Q once, then 64-key K / V tiles into 4-stage rings (cp.async.bulk.tensor,
 *                 128-byte swizzle, mbarrier transaction counts)
 *        MMA issuers (one warp per Q tile, one elected lane): S = Q.K^T (M=128, N=64, K=16) and
 *                 O += P.V (N=128) with tcgen05.mma.cta_group::1.kind::f16, accumulators in TMEM
 *                 (per Q tile two S buffers of 64 columns and O of 128); tcgen05.commit signals mbarriers
 *        softmax warps, one thread per row: tcgen05.ld the row of S, online softmax in base 2 with a
 *                 lazily updated reference max, P as packed fp16 over the S columns (tcgen05.st; P.V
 *                 reads its A operand from tensor memory), conditional rescale of O in TMEM;
 *                 epilogue O / l -> fp32 output.
 *      Causal masking only touches the tiles that cross the diagonal.
 *
 * Every wait is bounded; a wait that runs out raises a CTA-wide abort flag, records a code in the
 * context's error word, lets all warps fall through to the end, and TMEM is always released.
 *
 * Roofline: tensor (dense fp16).  Algorithmic FLOPs = 4 * 128 * 64 * sum over queries of (pos+1).
 */
#include <cuda.h>
#include <cuda_fp16.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "ctx.h"

namespace {

constexpr int kQTok = 16;            /* query tokens per CTA (x 8 heads = 128 rows) */
constexpr int kTileBytes = 128 * 128 * 2;   /* one 128x128 fp16 operand tile = two 16 KB swizzled sub-tiles */
constexpr float kScaleLog2 = 0.08838834764831845f * 1.4426950408889634f;   /* 1/sqrt(128) * log2(e) */
constexpr float kPfThreshold = 8.f;

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_arrive(unsigned bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
/* bounded wait, see the header comment: mbarrier.try_wait suspends the thread until the phase completes or the hint elapses,
 * so the waiter wakes within tens of ns of the arrival */
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
        if (i >= (1u << 13) && t1 - t0 > 500000000ull) break;   /* both many polls and half a second: the timer can step */
    }
    *abort_flag = 1;
    if (atomicCAS(err, 0u, 2u) == 0u) err[1] = where;
    return false;
}
__device__ __forceinline__ void tma_load_3d(unsigned dst, const CUtensorMap *map, unsigned bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
/* shared-memory matrix descriptor: K-major, 128-byte swizzle; 8-row groups 1024 B apart (SBO), LBO = 1 (unused
 * for swizzled K-major), descriptor version 1 (Blackwell), layout type 2 = SWIZZLE_128B                       */
__device__ __forceinline__ unsigned long long make_desc(unsigned saddr) {
    return (unsigned long long)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
/* instruction descriptor: D = f32 (bit 4), A = B = f16 (0), both K-major, N = 128 (>>3 at bit 17), M = 128 (>>4 at bit 24) */
constexpr unsigned kIdesc = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
/* the same load without the wait: several loads can be in flight before one tcgen05.wait::ld */
__device__ __forceinline__ void tmem_ld32_nowait(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
/* The MMA issuers run in uniform control flow (the operands are then computed in the uniform data path the instruction
 * reads them from) and one lane, elected once per walk, issues: `lead` is 1 in that lane. */
__device__ __forceinline__ unsigned elect_one() {
    unsigned p;
    asm volatile("{\n .reg .pred e;\n elect.sync _|e, 0xffffffff;\n selp.u32 %0, 1, 0, e;\n}" : "=r"(p));
    return p;
}
__device__ __forceinline__ void umma_f16_ta_lead(unsigned d_tmem, unsigned a_tmem, unsigned long long b_desc, unsigned accumulate, unsigned lead) {
    asm volatile("{\n .reg .pred p, e;\n setp.ne.b32 e, %5, 0;\n setp.ne.b32 p, %4, 0;\n @e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(kIdesc), "r"(accumulate), "r"(lead) : "memory");
}
__device__ __forceinline__ void umma_commit_lead(unsigned bar, unsigned lead) {
    asm volatile("{\n .reg .pred e;\n setp.ne.b32 e, %1, 0;\n @e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}" ::"r"(bar), "r"(lead) : "memory");
}
__device__ __forceinline__ float fmax3(float a, float b, float c) { float r; asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c)); return r; }
__device__ __forceinline__ float ex2f(float x) { float r; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x)); return r; }
__device__ __forceinline__ unsigned pack_h2(float lo, float hi) { unsigned r; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }

/* ---- pass 1: pages -> dense fp16 K [head][tok][128] and V^T [head][128][tok] ------------------- */
template <int DT>
__global__ void __launch_bounds__(256) hy3a_kv_to_f16_kernel(hy3a_cache_view cache, int layer, int seq, int pg0, int ntok, int tok_stride, __half *ws_k, __half *ws_vt) {
    const hy3a_geom g = hy3a_make_geom(DT);
    const int pg = pg0 + blockIdx.x, hl = blockIdx.y, tid = threadIdx.x;
    /* programmatic dependent launch: the appended rows must be complete; the attention kernel may set itself up */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int block = cache.block_table[(size_t)seq * cache.max_blocks_per_seq + pg];
    const uint8_t *page = cache.pool + hy3a_page_index(cache, block, layer, hl) * (size_t)cache.page_bytes;
    const __half *ks = reinterpret_cast<const __half *>(page + g.ks_off), *vs = reinterpret_cast<const __half *>(page + g.vs_off);
    /* one block converts 32 tokens of the page (blockIdx.z): short dependent chains and 4x the blocks, because a chunk only
     * brings a handful of new pages and the attention kernel waits for this one */
    const int tq = blockIdx.z * 32;
    /* K: 32 tokens x 16 groups of 8 dims */
#pragma unroll
    for (int idx = tid; idx < 32 * 16; idx += 256) {
        const int tok = tq + (idx >> 4), d = (idx & 15) * 8, t = pg * 128 + tok;
        uint4 o = make_uint4(0, 0, 0, 0);
        if (t < ntok) {
            if (DT == 0) {
                o = *reinterpret_cast<const uint4 *>(page + hy3a_k_dim_off<0>(tok, d));
            } else {
                const float s = __half2float(ks[tok]);
                float f[8];
                if (DT == 1) {
                    const uint2 w = *reinterpret_cast<const uint2 *>(page + hy3a_k_dim_off<1>(tok, d));
                    const unsigned ww[2] = {w.x, w.y};
#pragma unroll
                    for (int i = 0; i < 8; i++) f[i] = (float)(signed char)((ww[i >> 2] >> (8 * (i & 3))) & 0xFF) * s;
                } else {
                    const unsigned w = *reinterpret_cast<const unsigned *>(page + hy3a_k_dim_off<2>(tok, d));
#pragma unroll
                    for (int i = 0; i < 8; i++) { int n = (w >> (4 * i)) & 0xF; f[i] = (float)(n > 7 ? n - 16 : n) * s; }
                }
                __half2 h0 = __floats2half2_rn(f[0], f[1]), h1 = __floats2half2_rn(f[2], f[3]), h2 = __floats2half2_rn(f[4], f[5]), h3 = __floats2half2_rn(f[6], f[7]);
                o = make_uint4(*reinterpret_cast<unsigned *>(&h0), *reinterpret_cast<unsigned *>(&h1), *reinterpret_cast<unsigned *>(&h2), *reinterpret_cast<unsigned *>(&h3));
            }
        }
        *reinterpret_cast<uint4 *>(ws_k + ((size_t)hl * tok_stride + t) * HY3A_D + d) = o;
    }
    /* V^T: thread = (dim, 16 of the block's tokens); 8 consecutive tokens per 16-byte store */
    const int d = tid & 127, th = tid >> 7;
#pragma unroll
    for (int t8 = 0; t8 < 2; t8++) {
        __half hv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int tok = tq + th * 16 + t8 * 8 + i, t = pg * 128 + tok;
            float v = 0.f;
            if (t < ntok) {
                if (DT == 0) {
                    v = __half2float(*reinterpret_cast<const __half *>(page + g.v_off + hy3a_v16_dim_off(tok, d)));
                } else if (DT == 1) {
                    v = (float)(signed char)page[g.v_off + hy3a_vt_off(d, tok)] * __half2float(vs[tok]);
                } else {
                    const int b = page[g.v_off + hy3a_v_unit_off<2>(tok, d & ~3) + ((d & 3) >> 1)];
                    v = (float)(((b >> ((d & 1) * 4)) & 0xF) - 8) * __half2float(vs[tok]);
                }
            }
            hv[i] = __float2half_rn(v);
        }
        *reinterpret_cast<uint4 *>(ws_vt + ((size_t)hl * HY3A_D + d) * tok_stride + pg * 128 + tq + th * 16 + t8 * 8) = *reinterpret_cast<uint4 *>(hv);
    }
}

struct prefill_args {
    float *out;
    size_t out_stride;
    int base, nq, kv_head_begin;
    unsigned *err;
};

/* ---- pass 2: the attention kernel -------------------------------------------------------------------------------------
 * One CTA = 32 query tokens x the 8 query heads of one KV head = two 128-row Q tiles A and B that share every K/V tile
 * (GQA packing); P lives in tensor memory.  A K/V tile is 64 keys, so that each Q tile has TWO S buffers (2 x 64 TMEM columns) beside its O (128
 * columns): 2 x 256 = 512 columns.  S_x(j+2) is issued right behind P_x(j).V_j into the buffer P_x(j) lives in, i.e. the
 * scores of a step are computed while the softmax of the step before runs, and the loop
 *      S ready -> softmax -> P -> P.V -> next S
 * falls apart into a softmax chain (one thread per row, 64 columns
 * per step, no exchange between threads) and an MMA chain that only meet at the P and S barriers.  The softmax warps
 * wait for P.V only when a row's reference maximum moved (lazy rescale of O) and at the end.
 * Warps 0-3 / 4-7: softmax of tile A / B; warp 8: TMA producer (4-stage rings of 16 KB K and V tiles); warps 9 / 10:
 * MMA issuers of tile A / B, each in uniform control flow with one lane elected once (one thread issues an MMA every
 * ~26 ns at best, which a single issuer for both tiles would be bound by).                                       */
constexpr int kQTok2 = 32;                     /* query tokens per CTA = two tiles of kQTok */
constexpr int kKeys3 = 64;
constexpr int kK3Bytes = kKeys3 * 128 * 2;      /* one K tile = two sub-tiles [64 keys][64 dims]; one V^T tile = [128 dims][64 keys] */
constexpr int kSt3 = 4;                         /* ring stages */
constexpr int kPf3Threads = 352;
constexpr int kOff3Q = 0, kOff3K = kOff3Q + 2 * kTileBytes, kOff3V = kOff3K + kSt3 * kK3Bytes, kOff3Bar = kOff3V + kSt3 * kK3Bytes;
constexpr int kPf3Smem = kOff3Bar + 512 + 1024;
/* K0F, K0E [2]: the first two K tiles (loaded / consumed); DF, DE [4 stages]: step j's data = V_j and K_(j+2) (loaded /
 * consumed); SF, P [tile][buffer]; O [tile][last but one, last]: each completes once */
enum { B3_Q = 0, B3_K0F = 1, B3_K0E = 3, B3_DF = 5, B3_DE = 9, B3_SF = 13, B3_P = 17, B3_O = 21 };
constexpr unsigned kIdescN64 = (1u << 4) | ((64u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_f16_n64_lead(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc, unsigned accumulate, unsigned lead) {
    asm volatile("{\n .reg .pred p, e;\n setp.ne.b32 e, %5, 0;\n setp.ne.b32 p, %4, 0;\n @e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdescN64), "r"(accumulate), "r"(lead) : "memory");
}
__global__ void __launch_bounds__(kPf3Threads, 1)
hy3a_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, prefill_args a) {
    extern __shared__ uint8_t s_raw[];
    uint8_t *sm = s_raw + ((1024u - (smem_u32(s_raw) & 1023u)) & 1023u);
    const unsigned sbase = smem_u32(sm);
    const unsigned bar0 = sbase + kOff3Bar;
    volatile unsigned *s_tmem = reinterpret_cast<volatile unsigned *>(sm + kOff3Bar + 256);
    volatile int *s_abort = reinterpret_cast<volatile int *>(sm + kOff3Bar + 260);
#define BAR(i) (bar0 + 8u * (unsigned)(i))

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q0 = blockIdx.x * kQTok2, hl = blockIdx.y;
    const int kv_end = min(a.base + q0 + kQTok2, a.base + a.nq);   /* keys [0, kv_end) matter for this CTA */
    const int ntiles = (kv_end + kKeys3 - 1) / kKeys3;

    if (tid == 0) {
        *s_abort = 0;
        mbar_init(BAR(B3_Q), 1);
        for (int i = 0; i < 2; i++) { mbar_init(BAR(B3_K0F + i), 1); mbar_init(BAR(B3_K0E + i), 2); }
        for (int i = 0; i < kSt3; i++) { mbar_init(BAR(B3_DF + i), 1); mbar_init(BAR(B3_DE + i), 2); }   /* K0E, DE: one commit per issuer */
        for (int i = 0; i < 4; i++) { mbar_init(BAR(B3_SF + i), 1); mbar_init(BAR(B3_P + i), 4); }   /* P: one arrival per softmax warp of the tile */
        for (int i = 0; i < 4; i++) mbar_init(BAR(B3_O + i), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {   /* one warp allocates all 512 TMEM columns (1 CTA per SM) */
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + kOff3Bar + 256), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = *s_tmem;
    /* tile x: S buffers at columns 128x and 128x + 64 (P over the first 32 columns of its S), O at columns 256 + 128x */

    if (warp == 8) {
        /* ===================== TMA producer ===================== */
        if (lane == 0) {
            /* programmatic dependent launch: everything above ran beside the tail of the conversion kernel; the
             * operands are complete from here on (all global reads of this CTA follow this thread's copies) */
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            mbar_expect_tx(BAR(B3_Q), 2 * kTileBytes);
            for (int x = 0; x < 2; x++) {
                tma_load_3d(sbase + kOff3Q + x * kTileBytes, &tm_q, BAR(B3_Q), 0, (a.kv_head_begin + hl) * 8, q0 + x * kQTok);
                tma_load_3d(sbase + kOff3Q + x * kTileBytes + 16384, &tm_q, BAR(B3_Q), 64, (a.kv_head_begin + hl) * 8, q0 + x * kQTok);
            }
            /* the first two K tiles, then per step j one transaction: V_j and K_(j+2) (S_(j+2) is issued behind P_j.V_j,
             * so the issuers need both at the same time and wait for them once) */
            for (int j = 0; j < 2 && j < ntiles; j++) {
                mbar_expect_tx(BAR(B3_K0F + j), kK3Bytes);
                tma_load_3d(sbase + kOff3K + j * kK3Bytes, &tm_k, BAR(B3_K0F + j), 0, j * kKeys3, hl);
                tma_load_3d(sbase + kOff3K + j * kK3Bytes + 8192, &tm_k, BAR(B3_K0F + j), 64, j * kKeys3, hl);
            }
            for (int j = 0; j < ntiles; j++) {
                const int st = j & (kSt3 - 1), j2 = j + 2, st2 = j2 & (kSt3 - 1); const unsigned ph = (unsigned)(j / kSt3) & 1u;
                /* V slot st held V_(j-4), K slot st2 held K_(j-2): both were released by step j-4 -- except K_0 and K_1, which
                 * the issuers release on barriers of their own */
                if (!mbar_wait_blocking(BAR(B3_DE + st), ph ^ 1u, s_abort, a.err, 10u)) break;
                if ((j == 2 || j == 3) && j2 < ntiles && !mbar_wait_blocking(BAR(B3_K0E + j - 2), 0u, s_abort, a.err, 11u)) break;
                mbar_expect_tx(BAR(B3_DF + st), j2 < ntiles ? 2 * kK3Bytes : kK3Bytes);
                tma_load_3d(sbase + kOff3V + st * kK3Bytes, &tm_v, BAR(B3_DF + st), j * kKeys3, 0, hl);
                if (j2 < ntiles) {
                    tma_load_3d(sbase + kOff3K + st2 * kK3Bytes, &tm_k, BAR(B3_DF + st), 0, j2 * kKeys3, hl);
                    tma_load_3d(sbase + kOff3K + st2 * kK3Bytes + 8192, &tm_k, BAR(B3_DF + st), 64, j2 * kKeys3, hl);
                }
            }
        }
    } else if (warp >= 9) {
        /* ===================== MMA issuer of tile x (whole warp, one elected lane issues) =====================
         * order: S_x(0) S_x(1) | PV_x(0) S_x(2) | PV_x(1) S_x(3) | ...   tcgen05.commit covers what this thread issued, so
         * a K or V stage is released by one commit of each issuer */
        const int x = warp - 9;
        /* one election for the whole walk: `lead` is 1 in the issuing lane (an elect.sync in front of every MMA and commit
         * costs 1.7 % of the kernel) */
        const unsigned lead = elect_one();
        bool ok = mbar_wait_blocking(BAR(B3_Q), 0u, s_abort, a.err, 20u);
        const unsigned long long dQ = make_desc(sbase + kOff3Q + x * kTileBytes);
        const unsigned long long dK0 = make_desc(sbase + kOff3K), dV0 = make_desc(sbase + kOff3V);
        const unsigned tm_sx = tmem + 128u * x, tm_ox = tmem + 256u + 128u * x;
        auto issue_qk = [&](int j) {      /* S_x(j) = Q_x . K_j^T into buffer j & 1: 8 k-steps of 16 over d = 128 */
            const unsigned long long k = dK0 + (unsigned long long)((j & (kSt3 - 1)) * (kK3Bytes >> 4));
            const unsigned d = tm_sx + 64u * (j & 1);
#pragma unroll
            for (int kk = 0; kk < 8; kk++)      /* the second half of d lies one sub-tile further on: 16 KB for Q, 8 KB for K */
                umma_f16_n64_lead(d, dQ + (unsigned long long)((kk >> 2) * 1024 + (kk & 3) * 2), k + (unsigned long long)((kk >> 2) * 512 + (kk & 3) * 2), kk > 0, lead);
            umma_commit_lead(BAR(B3_SF + 2 * x + (j & 1)), lead);
        };
        /* tile B starts when the first softmax of tile A is through: half a period out of phase, the MMAs of one tile
         * run while the other tile's issuer is between two steps and its softmax warps have the SM's exponential
         * unit to themselves (nothing pulls the two loops apart by itself when they start together) */
        if (ok && x == 1) ok = mbar_wait_blocking(BAR(B3_P + 0), 0u, s_abort, a.err, 22u);
        for (int j = 0; j < 2 && j < ntiles && ok; j++) {
            ok = __all_sync(0xffffffffu, mbar_wait_blocking(BAR(B3_K0F + j), 0u, s_abort, a.err, 21u));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_qk(j);
            umma_commit_lead(BAR(B3_K0E + j), lead);
        }
        for (int j = 0; j < ntiles && ok; j++) {
            const int st = j & (kSt3 - 1), j2 = j + 2; const unsigned ph = (unsigned)(j / kSt3) & 1u;
            ok = mbar_wait_blocking(BAR(B3_DF + st), ph, s_abort, a.err, 23u);                                               /* V_j and K_(j+2) */
            if (ok) ok = mbar_wait_blocking(BAR(B3_P + 2 * x + (j & 1)), (unsigned)(j >> 1) & 1u, s_abort, a.err, 24u);   /* P_x(j) in tensor memory, O_x rescaled */
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            /* O_x += P_x(j) . V_j : 4 k-steps of 16 keys; A = 8 columns of packed fp16 pairs per step */
            {
                const unsigned long long v = dV0 + (unsigned long long)(st * (kK3Bytes >> 4));
                const unsigned pa = tm_sx + 64u * (j & 1);
                const unsigned acc0 = j > 0 ? 1u : 0u;
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ta_lead(tm_ox, pa + 8u * kk, v + (unsigned long long)(kk * 2), kk > 0 ? 1u : acc0, lead);
            }
            /* completion of P.V is only asked for directly at the end (last rescale, epilogue); before that the softmax
             * warps learn it from S_x(j+2), which this thread issues behind it */
            if (j + 2 >= ntiles) umma_commit_lead(BAR(B3_O + 2 * x + (j + 1 == ntiles ? 1 : 0)), lead);
            if (j2 < ntiles) issue_qk(j2);
            umma_commit_lead(BAR(B3_DE + st), lead);
        }
    } else {
        /* ===================== softmax warps: tile x = warp / 4; thread = one row of Q tile x ===================== */
        const int x = warp >> 2, r = tid & 127, t_local = r >> 3, h = r & 7;
        const int tq0 = q0 + x * kQTok;                          /* first query token of this tile */
        const int qpos = a.base + tq0 + t_local;                 /* global index of this row's query */
        const bool row_valid = (tq0 + t_local) < a.nq;
        const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16; /* this warp's quarter of the TMEM lanes */
        const unsigned tm_o = tmem + 256u + 128u * x + lane_base;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < ntiles && ok; j++) {
            const unsigned tm_s = tmem + 128u * x + 64u * (j & 1) + lane_base;
            ok = __all_sync(0xffffffffu, mbar_wait_blocking(BAR(B3_SF + 2 * x + (j & 1)), (unsigned)(j >> 1) & 1u, s_abort, a.err, 30u));   /* keep the warp together */
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int k0 = j * kKeys3;
            const bool masked = (k0 + kKeys3 - 1 > a.base + tq0);   /* the tile crosses the diagonal of some row */
            unsigned v0[32], v1[32];
            tmem_ld32_nowait(tm_s, v0);
            tmem_ld32_nowait(tm_s + 32u, v1);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (masked) {      /* only the tiles on the diagonal pay for the causal test */
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (k0 + i > qpos) v0[i] = 0xff800000u;
                    if (k0 + 32 + i > qpos) v1[i] = 0xff800000u;
                }
            }
            /* the maximum is taken over the raw scores (the scale is positive) and the scale is folded into the exponent's
             * argument: one FFMA per element.  Four independent chains keep the dependent-issue latency hidden. */
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 32; i++) mx4[i & 3] = fmax3(mx4[i & 3], __uint_as_float(v0[i]), __uint_as_float(v1[i]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * kScaleLog2;
            /* a tile that is masked for the whole row (its keys all lie behind the row's query; only in the last tiles of
             * the CTA) has mx = -inf: nothing moves and all its P are 0 */
            const bool grow = mx > m + kPfThreshold;              /* true while m == -inf (key 0 is never masked) */
            const float m_new = grow ? mx : m;
            const float neg_m = -m_new;
            unsigned pk[32];
            float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
                /* the denominator sums the unrounded values: the fp16 rounding of P is a zero-mean 2^-12 relative error per
                 * term, far below the tolerance */
                const float e0 = ex2f(fmaf(__uint_as_float(v0[i]), kScaleLog2, neg_m)), e1 = ex2f(fmaf(__uint_as_float(v0[i + 1]), kScaleLog2, neg_m));
                const float e2 = ex2f(fmaf(__uint_as_float(v1[i]), kScaleLog2, neg_m)), e3 = ex2f(fmaf(__uint_as_float(v1[i + 1]), kScaleLog2, neg_m));
                pk[i >> 1] = pack_h2(e0, e1); pk[16 + (i >> 1)] = pack_h2(e2, e3);
                ls[0] += e0; ls[1] += e1; ls[2] += e2; ls[3] += e3;
            }
            const float lsum = (ls[0] + ls[1]) + (ls[2] + ls[3]);
            /* tcgen05.ld / .st are warp-collective: the whole warp rescales its 32 rows as soon as one of them moved its
             * reference (the others multiply by exactly 1).  O_x is only ours when P_x(j-1).V_(j-1) has completed. */
            const float alpha = grow ? ex2f(m - m_new) : 1.f;     /* 0 on the first tile (m = -inf) */
            if (__any_sync(0xffffffffu, grow)) {
                if (j > 0) {
                    /* S_x(j+1) was issued behind P_x(j-1).V, and a commit covers everything its thread issued before */
                    ok = __all_sync(0xffffffffu, j + 1 < ntiles ? mbar_wait_blocking(BAR(B3_SF + 2 * x + ((j + 1) & 1)), (unsigned)((j + 1) >> 1) & 1u, s_abort, a.err, 31u)
                                                               : mbar_wait_blocking(BAR(B3_O + 2 * x), 0u, s_abort, a.err, 31u));
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (ok) {
#pragma unroll
                        for (int c = 0; c < 4; c++) {
                            unsigned v[32];
                            tmem_ld32(tm_o + 32u * c, v);
#pragma unroll
                            for (int i = 0; i < 32; i++) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                            tmem_st32(tm_o + 32u * c, v);
                        }
                    }
                }
                l *= alpha;
                m = m_new;
            }
            l += lsum;
            /* P over the first 32 columns of this S buffer (column c = keys 2c, 2c+1) */
            tmem_st32(tm_s, pk);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR(B3_P + 2 * x + (j & 1)));
        }
        /* epilogue: O / l.  The issuer commits P.V of the last two tiles on barriers of their own, which therefore complete
         * exactly once (a parity wait on a barrier that runs through many phases can only tell the last completed phase
         * from the one before it, and a waiter here could be two behind).  The last commit covers all earlier MMAs. */
        if (ok && ntiles > 0) ok = mbar_wait_blocking(BAR(B3_O + 2 * x + 1), 0u, s_abort, a.err, 32u);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (__all_sync(0xffffffffu, ok) && ntiles > 0) {      /* warp-uniform: tcgen05.ld is warp-collective */
            const float inv = l > 0.f ? 1.f / l : 0.f;
            float *orow = a.out + (size_t)(tq0 + t_local) * a.out_stride + (size_t)((a.kv_head_begin + hl) * 8 + h) * HY3A_D;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                unsigned v[32];
                tmem_ld32(tm_o + 32u * c, v);
                if (row_valid)
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4 *>(orow + 32 * c + i) = make_float4(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv,
                                                                                   __uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            }
        }
    }
    /* ---- common exit: everybody arrives here, also after a wait ran out; release TMEM */
    if (*s_abort && warp == 8 && lane == 0) {
        /* copies already issued must land before the shared memory goes away */
        for (int st = 0; st < kSt3; st++)
            for (unsigned ph = 0; ph < 2; ph++)
                for (unsigned spin = 0; spin < (1u << 12) && !mbar_test(BAR(B3_DF + st), ph); spin++) __nanosleep(64);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
#undef BAR
}


} /* namespace */

typedef CUresult (*hy3a_encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                         const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                         CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static hy3a_encode_tiled_fn get_encode_tiled(void) {
    static hy3a_encode_tiled_fn fn = NULL;
    if (!fn) {
        void *p = NULL;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = (hy3a_encode_tiled_fn)p;
    }
    return fn;
}

/* 3-D fp16 tensor map with a 128-byte swizzle; dims/box innermost first, strides in bytes for dims 1 and 2 */
static int make_map(hy3a_ctx *ctx, CUtensorMap *map, void *base, const cuuint64_t dims[3], const cuuint64_t strides[2], const cuuint32_t box[3]) {
    hy3a_encode_tiled_fn enc = get_encode_tiled();
    if (!enc) return hy3a_fail(ctx, HY3A_ECUDA, "prefill: cuTensorMapEncodeTiled is not available from the driver");
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return hy3a_fail(ctx, HY3A_ECUDA, "prefill: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return HY3A_OK;
}

int hy3a_launch_prefill(hy3a_ctx *ctx, int layer, int seq, int base_slot, int nq, const void *q16, float *out, size_t out_stride) {
    const int kvh = ctx->cfg.kv_head_count;
    const int ntok = base_slot + nq;
    const int pages = (ntok + HY3A_PT - 1) / HY3A_PT;
    int tok_stride = pages * HY3A_PT, pg0 = 0;
    void *ws_k = NULL, *ws_v = NULL;
    /* 1st choice: this layer's operand mirror -- only the pages written since the last chunk are converted */
    if (ctx->pf_mbudget) {
        if (ctx->pf_mseq != seq) { for (int l = 0; l < ctx->cfg.n_layers; l++) ctx->pf_mntok[l] = 0; ctx->pf_mseq = seq; }
        const int want = (tok_stride + 1023) / 1024 * 1024;
        if (want > ctx->pf_mcap[layer]) {
            const int seq_cap = (ctx->cfg.max_blocks_per_seq * HY3A_PT + 1023) / 1024 * 1024;
            int cap = 2 * ctx->pf_mcap[layer];
            if (cap > seq_cap) cap = seq_cap;
            if (cap < want) cap = want;
            const size_t old_b = 2 * (size_t)kvh * ctx->pf_mcap[layer] * HY3A_D * sizeof(__half), new_b = 2 * (size_t)kvh * cap * HY3A_D * sizeof(__half);
            if (ctx->pf_mbytes - old_b + new_b <= ctx->pf_mbudget) {
                HY3A_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
                cudaFree(ctx->pf_mk[layer]); cudaFree(ctx->pf_mv[layer]);
                ctx->pf_mk[layer] = ctx->pf_mv[layer] = NULL; ctx->pf_mcap[layer] = 0; ctx->pf_mntok[layer] = 0; ctx->pf_mbytes -= old_b;
                /* zeroed once: columns past a sequence's end are read by the last tile (and masked), so they must never
                 * hold a NaN or Inf pattern; afterwards only finite values are written */
                if (cudaMalloc(&ctx->pf_mk[layer], new_b / 2) == cudaSuccess && cudaMalloc(&ctx->pf_mv[layer], new_b / 2) == cudaSuccess &&
                    cudaMemsetAsync(ctx->pf_mk[layer], 0, new_b / 2, ctx->stream) == cudaSuccess && cudaMemsetAsync(ctx->pf_mv[layer], 0, new_b / 2, ctx->stream) == cudaSuccess) {
                    ctx->pf_mcap[layer] = cap; ctx->pf_mbytes += new_b;
                } else {
                    cudaGetLastError();
                    cudaFree(ctx->pf_mk[layer]); ctx->pf_mk[layer] = ctx->pf_mv[layer] = NULL;   /* fall through to the shared workspace */
                }
            }
        }
        if (want <= ctx->pf_mcap[layer]) {
            ws_k = ctx->pf_mk[layer]; ws_v = ctx->pf_mv[layer];
            tok_stride = ctx->pf_mcap[layer];
            /* a partly filled page is converted again; nothing is, when the append kernel wrote the rows through */
            pg0 = ctx->pf_mntok[layer] >= ntok ? pages : ctx->pf_mntok[layer] / HY3A_PT;
            if (ctx->pf_mntok[layer] < ntok) ctx->pf_mntok[layer] = ntok;
        }
    }
    /* 2nd choice: one workspace shared by all layers, rebuilt from the pages on every call (grow-only, in steps of
     * 1024 tokens) */
    if (!ws_k) {
        const size_t need = (size_t)kvh * (((size_t)tok_stride + 1023) / 1024 * 1024) * HY3A_D * sizeof(__half);
        if (need > ctx->pf_bytes) {
            HY3A_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            cudaFree(ctx->d_pf_k); cudaFree(ctx->d_pf_v);
            ctx->d_pf_k = ctx->d_pf_v = NULL; ctx->pf_bytes = 0;
            if (cudaMalloc(&ctx->d_pf_k, need) != cudaSuccess || cudaMalloc(&ctx->d_pf_v, need) != cudaSuccess) {
                cudaFree(ctx->d_pf_k); ctx->d_pf_k = NULL;
                return hy3a_fail(ctx, HY3A_ENOMEM, "prefill: cannot allocate 2 x %zu bytes of fp16 workspace", need);
            }
            ctx->pf_bytes = need;
        }
        ws_k = ctx->d_pf_k; ws_v = ctx->d_pf_v;
    }
    hy3a_cache_view cv = hy3a_view(ctx);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    if (pages > pg0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(pages - pg0, kvh, 4); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = ctx->stream;
        cfg.attrs = attr; cfg.numAttrs = ctx->use_pdl ? 1 : 0;
        __half *wk = (__half *)ws_k, *wv = (__half *)ws_v;
        cudaError_t e;
        switch (ctx->geom.dtype) {
            case 0: e = cudaLaunchKernelEx(&cfg, hy3a_kv_to_f16_kernel<0>, cv, layer, seq, pg0, ntok, tok_stride, wk, wv); break;
            case 1: e = cudaLaunchKernelEx(&cfg, hy3a_kv_to_f16_kernel<1>, cv, layer, seq, pg0, ntok, tok_stride, wk, wv); break;
            default: e = cudaLaunchKernelEx(&cfg, hy3a_kv_to_f16_kernel<2>, cv, layer, seq, pg0, ntok, tok_stride, wk, wv); break;
        }
        ctx->launches++;
        HY3A_CUDA(ctx, e);
    }

    const int keys = kKeys3;
    CUtensorMap tq, tk, tv;
    {
        const cuuint64_t dq[3] = {HY3A_D, HY3A_N_HEAD, (cuuint64_t)nq}, sq[2] = {HY3A_D * 2, HY3A_N_HEAD * HY3A_D * 2};
        const cuuint32_t bq[3] = {64, 8, kQTok};
        int rc = make_map(ctx, &tq, const_cast<void *>(q16), dq, sq, bq);
        if (rc) return rc;
        const cuuint64_t dk[3] = {HY3A_D, (cuuint64_t)tok_stride, (cuuint64_t)kvh}, sk[2] = {HY3A_D * 2, (cuuint64_t)tok_stride * HY3A_D * 2};
        const cuuint32_t bk[3] = {64, (cuuint32_t)keys, 1};
        rc = make_map(ctx, &tk, ws_k, dk, sk, bk);
        if (rc) return rc;
        const cuuint64_t dv[3] = {(cuuint64_t)tok_stride, HY3A_D, (cuuint64_t)kvh}, sv[2] = {(cuuint64_t)tok_stride * 2, (cuuint64_t)tok_stride * HY3A_D * 2};
        const cuuint32_t bv[3] = {64, HY3A_D, 1};
        rc = make_map(ctx, &tv, ws_v, dv, sv, bv);
        if (rc) return rc;
    }
    static bool attr_dev[64];   /* function attributes are per device */
    bool &attr_set = attr_dev[ctx->device & 63];
    if (!attr_set) {
        HY3A_CUDA(ctx, cudaFuncSetAttribute(hy3a_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPf3Smem));
        attr_set = true;
    }
    prefill_args a;
    a.out = out; a.out_stride = out_stride; a.base = base_slot; a.nq = nq; a.kv_head_begin = ctx->cfg.kv_head_begin; a.err = ctx->d_err;
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((nq + kQTok2 - 1) / kQTok2, kvh); cfg.stream = ctx->stream;
        cfg.blockDim = dim3(kPf3Threads); cfg.dynamicSmemBytes = kPf3Smem;
        cfg.attrs = attr; cfg.numAttrs = ctx->use_pdl ? 1 : 0;
        HY3A_CUDA(ctx, cudaLaunchKernelEx(&cfg, hy3a_prefill_kernel, tq, tk, tv, a));
    }
    ctx->launches++;
    ctx->bulk_write_pending = 1;
    HY3A_CUDA(ctx, cudaGetLastError());
    return HY3A_OK;
}
