/*
 * hy3_gpu_dropin.cu -- the reference engine's CUDA backend API on top of the B200 attention library.
 *
 * Defines the three symbols the engine binds (hy3.c:1367-1377 dispatches on m->gpu_ctx; hy3_cli.c:280 and
 * hy3_model_free call init / free):
 *      int  hy3_gpu_init(hy3_model *m, int n_gpu_layers);                                   hy3_gpu.cu:544-630
 *      void hy3_gpu_free(hy3_model *m);                                                     hy3_gpu.cu:632-642
 *      int  hy3_eval_gpu(hy3_model *m, const hy3_tokens *t, float *logits, int *pos);       hy3_gpu.cu:844-961
 * (plus hy3_gpu_eval, the name hy3_gpu.h:8 declares, as an alias).  It is compiled against the ENGINE's own
 * hy3.h -- the structs are not restated here -- and is linked into the engine in place of its hy3_cuda.o.
 *
 * What is kept of the contract: the context hangs off m->gpu_ctx; the layer count is clamped as there; the
 * switches HY3_KV_INT4, HY3_PREFILL_CHUNK, HY3_POS_STRIDE, HY3_POS_JUMP[_AT] are read once at init (new:
 * HY3_KV_FP16, HY3_KV_TOKENS); the RoPE table comes from hy3_rope_get_params; the init line names the cache
 * type ("INT8 KV" / "INT4 KV", which eval/hy3_needle.py:103 looks for); tokens are processed as positions
 * cache_len/80, cache_len/80 + 1, ... with cache_len owned -- and set back -- by the caller (hy3.c:1514, :960),
 * so the position is re-derived from it on every call; with HY3_PREFILL_CHUNK=N all tokens of a call but the
 * last go through chunks of <= N, the last one through the decode path (hy3_gpu.cu:857-866); logits of the last
 * token only; *pos = cache_len; layers beyond n_gpu_layers run on the host through forward_layer_dense / _moe
 * (hy3_gpu.cu:948).  Returns 0 / -1 and never exits: every CUDA, cuBLAS and attention-library call is checked.
 *
 * What is new: the attention of a layer is ONE launch of the attention library (hy3a_decode_step: norm + RoPE +
 * quantise/append + split-KV attention + merge; chunks: hy3a_append + hy3a_prefill on tcgen05), the KV cache is
 * its paged pool (no reallocation, no copy, no graph recapture when it grows), and the single-token step is
 * replayed as one CUDA graph whose launches read positions from device memory.
 *
 * Everything that is not attention (embedding, norms, projections, router, experts, logits) is plain code for
 * correctness: cuBLAS GEMMs for dense weights (fp32 weights stay fp32; F16 / Q8_0 / Q4_K dense weights become fp16
 * as in hy3_gpu.cu:523-540) and simple warp-per-row kernels for the routed experts, which stay in their file
 * format on the device (F32, F16 or Q4_K blocks).
 */
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

extern "C" {
#include "hy3.h"   /* the engine's header, found through the include path given at build time */
}
#include "../../include/hy3_attn.h"

namespace {

constexpr int E = HY3_N_EMBD, QS = HY3_N_HEAD * HY3_HEAD_DIM, KVD = HY3_N_KV_HEAD * HY3_HEAD_DIM, QKV = QS + 2 * KVD;
constexpr int NL = HY3_N_LAYER, NX = HY3_N_EXPERT, MI = HY3_MOE_INTERMED, DI = HY3_DENSE_INTERMED;
constexpr float kEps = 1e-5f;            /* HY3_RMS_EPS, hy3.c:25 */
constexpr float kRouterScale = 2.826f;   /* hy3.c:1284 */

enum { T_F32 = 0, T_F16 = 1, T_Q8_0 = 8, T_Q4_K = 12 };

struct dmat {            /* a dense weight on the device: fp32 or fp16, row-major [rows][cols] */
    void *w;
    int f16, rows, cols;
};
struct xmat {            /* a routed-expert weight in its file format */
    const uint8_t *w;
    int type;
};
struct layer_dev {
    float *attn_norm, *ffn_norm;
    dmat wq, wk, wv, wo;
    dmat gate, up, down;              /* dense FFN (layer 0) or shared expert */
    dmat router;
    float *bias;                      /* expert bias or NULL */
    xmat *xgate, *xup, *xdown;        /* device arrays [192] */
};

struct upload_entry { const void *host; void *dev; int kind; };

struct dropin_ctx {
    hy3a_ctx *attn;
    cublasHandle_t cublas;
    cudaStream_t stream;
    int n_gpu_layers, chunk, kv_dtype, max_tokens, vocab;
    void *embd; int embd_f16;
    float *out_norm;
    dmat out_w;
    layer_dev L[NL];
    /* activations for up to cap tokens */
    int cap;
    float *x, *s, *qkv, *ao, *o, *ff, *ff2, *logits_d, *router, *rw, *xg, *xu, *xd;
    __half *h16;
    int *ids, *tok_d, *tok_h;
    /* single-token graph */
    cudaGraphExec_t graph;
    int graph_ready, warmed, use_graph;
    /* uploads deduplicated by host pointer (models whose layers share tensors upload them once) */
    upload_entry *up; int n_up, cap_up;
    char err[512];
};

int fail(dropin_ctx *c, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    fprintf(stderr, "hy3_gpu: %s\n", buf);
    if (c) snprintf(c->err, sizeof c->err, "%s", buf);
    return -1;
}
#define CK(c, call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail((c), "%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); } while (0)
#define CKB(c, call) do { cublasStatus_t s_ = (call); if (s_ != CUBLAS_STATUS_SUCCESS) return fail((c), "%s: cuBLAS status %d (%s:%d)", #call, (int)s_, __FILE__, __LINE__); } while (0)
#define CKA(c, call) do { int r_ = (call); if (r_) return fail((c), "%s: %s", #call, hy3a_last_error((c)->attn)); } while (0)
#define CKL(c) CK(c, cudaGetLastError())

/* ---------------------------------------------------------------- kernels (correctness code, not tuned) */
__global__ void embed_kernel(float *x, const void *table, int f16, const int *tok, int n) {
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t o = (size_t)tok[t] * n + i;
    x[(size_t)t * n + i] = f16 ? __half2float(((const __half *)table)[o]) : ((const float *)table)[o];
}
/* out = rmsnorm(x (+ a)) * w per token; with a != NULL also x += a (residual add fused, hy3_gpu.cu:453) */
__global__ void rmsnorm_kernel(float *out, float *x, const float *a, const float *w, int n) {
    __shared__ float red[256];
    float *xr = x + (size_t)blockIdx.x * n;
    const float *ar = a ? a + (size_t)blockIdx.x * n : nullptr;
    float sum = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i];
        if (ar) { v += ar[i]; xr[i] = v; }
        sum += v * v;
    }
    red[threadIdx.x] = sum;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) { if ((int)threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s]; __syncthreads(); }
    const float r = rsqrtf(red[0] / (float)n + kEps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)blockIdx.x * n + i] = xr[i] * r * w[i];
}
__global__ void add_kernel(float *x, const float *a, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] += a[i];
}
/* g[t][i] = silu(g[t][i]) * u[t][i]; rows of g and u have their own strides */
__global__ void silu_mul_kernel(float *dst, size_t dst_stride, const float *g, const float *u, size_t src_stride, int n) {
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float a = g[(size_t)t * src_stride + i];
    dst[(size_t)t * dst_stride + i] = a / (1.f + expf(-a)) * u[(size_t)t * src_stride + i];
}
__global__ void f2h_kernel(__half *d, const float *s, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) d[i] = __float2half(s[i]);
}
/* sigmoid scores, optional bias for the selection only, top-k by repeated arg-max (lowest index wins ties,
 * as topk_select in hy3.c:654), weights = sigmoid / sum * 2.826 (hy3.c:1266-1287).  One block per token; ids and
 * weights are written as [token][k]. */
__global__ void router_kernel(const float *logits, const float *bias, int *ids, float *wts, int k) {
    __shared__ float sig[NX], sc[NX];
    const float *lg = logits + (size_t)blockIdx.x * NX;
    for (int i = threadIdx.x; i < NX; i += blockDim.x) {
        const float s = 1.0f / (1.0f + expf(-lg[i]));
        sig[i] = s;
        sc[i] = bias ? s + bias[i] : s;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.f;
        for (int j = 0; j < k; j++) {
            int best = -1;
            float bv = 0.f;
            for (int i = 0; i < NX; i++) if (sc[i] != -INFINITY && (best < 0 || sc[i] > bv)) { best = i; bv = sc[i]; }
            ids[blockIdx.x * k + j] = best;
            wts[blockIdx.x * k + j] = sig[best];
            sum += sig[best];
            sc[best] = -INFINITY;
        }
        const float inv = 1.0f / (sum + 1e-20f);
        for (int j = 0; j < k; j++) wts[blockIdx.x * k + j] = wts[blockIdx.x * k + j] * inv * kRouterScale;
    }
}
/* Q4_K: 256 values per 144-byte block = d, dmin (fp16), 12 bytes of 6-bit scales / mins, 128 bytes of nibbles; the
 * four 64-value chunks keep sub-block 2c in the low and 2c+1 in the high nibbles of their 32 bytes (hy3.c:1007-1041). */
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t *q, int &sc, int &mn) {
    if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
    else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}
__device__ __forceinline__ float row_dot(const uint8_t *w, int type, size_t row, const float *x, int n, int lane) {
    float acc = 0.f;
    if (type == T_F32) {
        const float *r = (const float *)w + row * n;
        for (int i = lane; i < n; i += 32) acc += r[i] * x[i];
    } else if (type == T_F16) {
        const __half *r = (const __half *)w + row * n;
        for (int i = lane; i < n; i += 32) acc += __half2float(r[i]) * x[i];
    } else {                                     /* Q4_K: lane = (chunk, 8 of its 32 bytes) per block */
        const int nb = n / 256;
        const uint8_t *r = w + row * (size_t)nb * 144;
        for (int b = 0; b < nb; b++) {
            const uint8_t *blk = r + (size_t)b * 144;
            const float d = __half2float(*(const __half *)blk), dm = __half2float(*(const __half *)(blk + 2));
            const int c = lane >> 3, l0 = (lane & 7) * 4;
            int s1, m1, s2, m2;
            q4k_scale_min(2 * c, blk + 4, s1, m1);
            q4k_scale_min(2 * c + 1, blk + 4, s2, m2);
            const uint8_t *q = blk + 16 + c * 32 + l0;
            const float *xl = x + b * 256 + c * 64 + l0, *xh = xl + 32;
            float a1 = 0.f, a2 = 0.f, x1 = 0.f, x2 = 0.f;
            for (int l = 0; l < 4; l++) { a1 += (float)(q[l] & 0xF) * xl[l]; x1 += xl[l]; a2 += (float)(q[l] >> 4) * xh[l]; x2 += xh[l]; }
            acc += d * (float)s1 * a1 - dm * (float)m1 * x1 + d * (float)s2 * a2 - dm * (float)m2 * x2;
        }
    }
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    return acc;
}
/* dst[slot][row] = W[ids[slot]][row] . x[slot / per][:]; warp per row, grid (ceil(m / 8), slots).
 * per = slots that share one input vector (k experts of a token read the same s; the down projection has its own) */
__global__ void expert_gemv_kernel(float *dst, const xmat *mats, const int *ids, const float *x, size_t x_stride, int per, int m, int n) {
    const int slot = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp;
    if (row >= m) return;
    const xmat mt = mats[ids[slot]];
    const float v = row_dot(mt.w, mt.type, (size_t)row, x + (size_t)(slot / per) * x_stride, n, lane);
    if (lane == 0) dst[(size_t)slot * m + row] = v;
}
/* x[t] += sum_j w[t][j] * down[t][j] (selection order, hy3.c:1316-1318) */
__global__ void combine_kernel(float *x, const float *down, const float *wts, int k, int n) {
    const int t = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int j = 0; j < k; j++) acc += wts[t * k + j] * down[((size_t)t * k + j) * n + i];
    x[(size_t)t * n + i] += acc;
}
/* file formats -> fp16 (dense weights that are not fp32) */
__global__ void q8_to_f16_kernel(__half *dst, const uint8_t *src, size_t nblk) {   /* 36-byte blocks: float d, 32 int8 (hy3_gpu.cu:513) */
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nblk * 32) return;
    const uint8_t *b = src + (i / 32) * 36;
    float d;
    memcpy(&d, b, 4);
    dst[i] = __float2half((float)((const int8_t *)(b + 4))[i % 32] * d);
}
__global__ void q4k_to_f16_kernel(__half *dst, const uint8_t *src, size_t nblk) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nblk * 256) return;
    const uint8_t *blk = src + (i / 256) * 144;
    const int j = (int)(i % 256), c = j / 64, r = j % 64;
    int sc, mn;
    q4k_scale_min(2 * c + (r >= 32), blk + 4, sc, mn);
    const uint8_t q = blk[16 + c * 32 + (r & 31)];
    const float v = __half2float(*(const __half *)blk) * (float)sc * (float)(r >= 32 ? q >> 4 : q & 0xF) - __half2float(*(const __half *)(blk + 2)) * (float)mn;
    dst[i] = __float2half(v);
}

/* ---------------------------------------------------------------- uploads */
size_t type_bytes(int type, uint64_t n) {
    switch (type) {
        case T_F32: return n * 4;
        case T_F16: return n * 2;
        case T_Q8_0: return n / 32 * 36;
        case T_Q4_K: return n / 256 * 144;
        default: return 0;
    }
}
/* raw bytes of a tensor on the device, one copy per distinct host pointer */
int upload_raw(dropin_ctx *c, const hy3_weight *w, void **out, int kind) {
    *out = NULL;
    if (!w || !w->data || !w->t || !w->t->elements) return 0;
    for (int i = 0; i < c->n_up; i++) if (c->up[i].host == w->data && c->up[i].kind == kind) { *out = c->up[i].dev; return 1; }
    const size_t bytes = type_bytes((int)w->t->ggml_type, w->t->elements);
    if (!bytes) return fail(c, "tensor type %u is not supported by this backend", w->t->ggml_type);
    void *d = NULL;
    CK(c, cudaMalloc(&d, bytes));
    CK(c, cudaMemcpy(d, w->data, bytes, cudaMemcpyHostToDevice));
    if (c->n_up == c->cap_up) {
        c->cap_up = c->cap_up ? 2 * c->cap_up : 256;
        c->up = (upload_entry *)realloc(c->up, (size_t)c->cap_up * sizeof(upload_entry));
        if (!c->up) return fail(c, "out of host memory");
    }
    c->up[c->n_up].host = w->data; c->up[c->n_up].dev = d; c->up[c->n_up].kind = kind; c->n_up++;
    *out = d;
    return 0;
}
int upload_f32(dropin_ctx *c, const hy3_weight *w, float **out) {
    *out = NULL;
    if (!w || !w->data || !w->t) return 0;
    if (w->t->ggml_type != T_F32) return fail(c, "norm / bias tensors must be F32 (got type %u)", w->t->ggml_type);
    void *d;
    int rc = upload_raw(c, w, &d, 0);
    if (rc < 0) return rc;
    *out = (float *)d;
    return 0;
}
/* dense weight for cuBLAS: fp32 stays, everything else becomes fp16 */
int upload_dense(dropin_ctx *c, const hy3_weight *w, dmat *out, int rows, int cols) {
    memset(out, 0, sizeof *out);
    if (!w || !w->data || !w->t) return 0;
    if ((uint64_t)rows * cols != w->t->elements) return fail(c, "weight has %llu elements, expected %d x %d", (unsigned long long)w->t->elements, rows, cols);
    out->rows = rows; out->cols = cols;
    const int type = (int)w->t->ggml_type;
    void *raw;
    int rc = upload_raw(c, w, &raw, type == T_F32 || type == T_F16 ? 0 : 1);
    if (rc < 0) return rc;
    if (type == T_F32 || type == T_F16) { out->w = raw; out->f16 = type == T_F16; return 0; }
    if (rc == 1) { out->w = raw; out->f16 = 1; return 0; }        /* already converted (kind 1 entries hold the fp16 image) */
    const uint64_t n = w->t->elements;
    __half *h = NULL;
    CK(c, cudaMalloc(&h, n * sizeof(__half)));
    const unsigned grid = (unsigned)((n + 255) / 256);
    if (type == T_Q8_0) q8_to_f16_kernel<<<grid, 256>>>(h, (const uint8_t *)raw, n / 32);
    else q4k_to_f16_kernel<<<grid, 256>>>(h, (const uint8_t *)raw, n / 256);
    CKL(c);
    CK(c, cudaDeviceSynchronize());
    cudaFree(raw);
    c->up[c->n_up - 1].dev = h;      /* the entry made by upload_raw now owns the fp16 image */
    out->w = h; out->f16 = 1;
    return 0;
}
int upload_experts(dropin_ctx *c, const hy3_weight *w, xmat **out) {
    xmat host[NX];
    for (int e = 0; e < NX; e++) {
        const int type = w[e].t ? (int)w[e].t->ggml_type : -1;
        if (type != T_F32 && type != T_F16 && type != T_Q4_K) return fail(c, "expert tensors must be F32, F16 or Q4_K (got type %d)", type);
        void *raw;
        if (upload_raw(c, &w[e], &raw, 0) < 0) return -1;
        host[e].w = (const uint8_t *)raw; host[e].type = type;
    }
    CK(c, cudaMalloc(out, sizeof host));
    CK(c, cudaMemcpy(*out, host, sizeof host, cudaMemcpyHostToDevice));
    return 0;
}

/* ---------------------------------------------------------------- building blocks on the stream */
/* dst[t][0..rows) = W . x[t][0..cols) for t < C (token-major, given row strides) */
int matmul(dropin_ctx *c, const dmat &w, const float *x, size_t x_stride, float *dst, size_t dst_stride, int C) {
    const float one = 1.f, zero = 0.f;
    if (!w.w) return fail(c, "a weight this step needs is missing from the model");
    if (!w.f16) {
        CKB(c, cublasSgemm(c->cublas, CUBLAS_OP_T, CUBLAS_OP_N, w.rows, C, w.cols, &one, (const float *)w.w, w.cols, x, (int)x_stride, &zero, dst, (int)dst_stride));
    } else {
        /* fp16 weights: the activations are rounded to fp16 as well (hy3_gpu.cu:647-655) */
        if (x_stride != (size_t)w.cols) return fail(c, "fp16 projection needs dense input rows");
        const size_t n = (size_t)C * w.cols;
        f2h_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(c->h16, x, n);
        CKL(c);
        CKB(c, cublasGemmEx(c->cublas, CUBLAS_OP_T, CUBLAS_OP_N, w.rows, C, w.cols, &one, w.w, CUDA_R_16F, w.cols, c->h16, CUDA_R_16F, w.cols, &zero,
                            dst, CUDA_R_32F, (int)dst_stride, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT));
    }
    return 0;
}

int ensure_cap(dropin_ctx *c, int C) {
    if (C <= c->cap) return 0;
    CK(c, cudaStreamSynchronize(c->stream));
    float **bufs[] = {&c->x, &c->s, &c->qkv, &c->ao, &c->o, &c->ff, &c->ff2, &c->router, &c->rw, &c->xg, &c->xu, &c->xd};
    for (float **b : bufs) { cudaFree(*b); *b = NULL; }
    cudaFree(c->h16); cudaFree(c->ids); cudaFree(c->tok_d);
    c->h16 = NULL; c->ids = NULL; c->tok_d = NULL;
    const size_t n = (size_t)C, big = DI > QS ? DI : QS;
    CK(c, cudaMalloc(&c->x, n * E * 4));
    CK(c, cudaMalloc(&c->s, n * E * 4));
    CK(c, cudaMalloc(&c->qkv, n * QKV * 4));
    CK(c, cudaMalloc(&c->ao, n * QS * 4));
    CK(c, cudaMalloc(&c->o, n * E * 4));
    CK(c, cudaMalloc(&c->ff, n * 2 * DI * 4));
    CK(c, cudaMalloc(&c->ff2, n * DI * 4));
    CK(c, cudaMalloc(&c->router, n * NX * 4));
    CK(c, cudaMalloc(&c->rw, n * HY3_N_EXPERT_USED * 4));
    CK(c, cudaMalloc(&c->xg, n * HY3_N_EXPERT_USED * MI * 4));
    CK(c, cudaMalloc(&c->xu, n * HY3_N_EXPERT_USED * MI * 4));
    CK(c, cudaMalloc(&c->xd, n * HY3_N_EXPERT_USED * E * 4));
    CK(c, cudaMalloc(&c->h16, n * big * sizeof(__half)));
    CK(c, cudaMalloc(&c->ids, n * HY3_N_EXPERT_USED * sizeof(int)));
    CK(c, cudaMalloc(&c->tok_d, n * sizeof(int)));
    c->cap = C;
    if (c->graph_ready) { cudaGraphExecDestroy(c->graph); c->graph_ready = 0; }   /* the graph holds the old pointers */
    return 0;
}

/* One layer for C tokens whose batch descriptor (positions t0 .. t0+C-1 of sequence 0) is already set. */
int layer_forward(dropin_ctx *c, hy3_model *m, int il, int t0, int C) {
    layer_dev &L = c->L[il];
    cudaStream_t st = c->stream;
    rmsnorm_kernel<<<C, 256, 0, st>>>(c->s, c->x, nullptr, L.attn_norm, E);
    CKL(c);
    if (matmul(c, L.wq, c->s, E, c->qkv, QKV, C) || matmul(c, L.wk, c->s, E, c->qkv + QS, QKV, C) || matmul(c, L.wv, c->s, E, c->qkv + QS + KVD, QKV, C)) return -1;
    if (C == 1) {
        /* decode path: norm + RoPE + quantise/append + attention + merge in one launch (hy3_gpu.cu:750-758) */
        CKA(c, hy3a_decode_step(c->attn, il, c->qkv, QKV, c->qkv + QS, QKV, c->qkv + QS + KVD, QKV, NULL, 0, c->ao, QS, NULL));
    } else {
        /* chunk path: the chunk's K/V go into the cache first, then causal attention over [0, t0 + i] (hy3_gpu.cu:823-832) */
        CKA(c, hy3a_append(c->attn, il, c->qkv, QKV, c->qkv + QS, QKV, c->qkv + QS + KVD, QKV, NULL, 0, c->h16));
        CKA(c, hy3a_prefill(c->attn, il, 0, t0, C, c->h16, c->ao, QS));
    }
    if (matmul(c, L.wo, c->ao, QS, c->o, E, C)) return -1;
    rmsnorm_kernel<<<C, 256, 0, st>>>(c->s, c->x, c->o, L.ffn_norm, E);      /* x += o; s = norm(x) */
    CKL(c);
    if (il < HY3_N_LAYER_DENSE) {
        if (matmul(c, L.gate, c->s, E, c->ff, 2 * DI, C) || matmul(c, L.up, c->s, E, c->ff + DI, 2 * DI, C)) return -1;
        silu_mul_kernel<<<dim3((DI + 255) / 256, C), 256, 0, st>>>(c->ff2, DI, c->ff, c->ff + DI, 2 * DI, DI);
        CKL(c);
        if (matmul(c, L.down, c->ff2, DI, c->o, E, C)) return -1;
        add_kernel<<<(unsigned)(((size_t)C * E + 255) / 256), 256, 0, st>>>(c->x, c->o, (size_t)C * E);
        CKL(c);
        return 0;
    }
    int k = m->n_expert_used;
    if (k < 1) k = 1;
    if (k > HY3_N_EXPERT_USED) k = HY3_N_EXPERT_USED;
    if (matmul(c, L.router, c->s, E, c->router, NX, C)) return -1;
    router_kernel<<<C, 256, 0, st>>>(c->router, L.bias, c->ids, c->rw, k);
    CKL(c);
    /* routed experts: slot = token * k + j; gate and up read the token's s, down reads the slot's own activation */
    expert_gemv_kernel<<<dim3((MI + 7) / 8, C * k), 256, 0, st>>>(c->xg, L.xgate, c->ids, c->s, E, k, MI, E);
    expert_gemv_kernel<<<dim3((MI + 7) / 8, C * k), 256, 0, st>>>(c->xu, L.xup, c->ids, c->s, E, k, MI, E);
    silu_mul_kernel<<<dim3((MI + 255) / 256, C * k), 256, 0, st>>>(c->xg, MI, c->xg, c->xu, MI, MI);
    expert_gemv_kernel<<<dim3((E + 7) / 8, C * k), 256, 0, st>>>(c->xd, L.xdown, c->ids, c->xg, MI, 1, E, MI);
    CKL(c);
    /* shared expert */
    if (matmul(c, L.gate, c->s, E, c->ff, 2 * MI, C) || matmul(c, L.up, c->s, E, c->ff + MI, 2 * MI, C)) return -1;
    silu_mul_kernel<<<dim3((MI + 255) / 256, C), 256, 0, st>>>(c->ff2, MI, c->ff, c->ff + MI, 2 * MI, MI);
    CKL(c);
    if (matmul(c, L.down, c->ff2, MI, c->o, E, C)) return -1;
    add_kernel<<<(unsigned)(((size_t)C * E + 255) / 256), 256, 0, st>>>(c->x, c->o, (size_t)C * E);
    combine_kernel<<<dim3((E + 255) / 256, C), 256, 0, st>>>(c->x, c->xd, c->rw, k, E);
    CKL(c);
    return 0;
}

int set_batch(dropin_ctx *c, int t0, int C) {
    int *seq = (int *)calloc((size_t)3 * C, sizeof(int));
    if (!seq) return fail(c, "out of host memory");
    int *slot = seq + C, *pos = seq + 2 * C;
    for (int i = 0; i < C; i++) { slot[i] = t0 + i; pos[i] = t0 + i; }
    const int rc = hy3a_batch_set(c->attn, C, seq, slot, pos);
    free(seq);
    if (rc) return fail(c, "KV cache: %s (HY3_KV_TOKENS sets the capacity, now %d tokens)", hy3a_last_error(c->attn), c->max_tokens);
    return 0;
}

int embed_tokens(dropin_ctx *c, const int *tok, int C) {
    for (int i = 0; i < C; i++) if (tok[i] < 0 || tok[i] >= HY3_N_VOCAB) return fail(c, "token id %d out of range", tok[i]);
    CK(c, cudaStreamSynchronize(c->stream));          /* the pinned staging buffer is free again */
    memcpy(c->tok_h, tok, (size_t)C * sizeof(int));
    CK(c, cudaMemcpyAsync(c->tok_d, c->tok_h, (size_t)C * sizeof(int), cudaMemcpyHostToDevice, c->stream));
    return 0;
}
int launch_embed(dropin_ctx *c, int C) {
    embed_kernel<<<dim3((E + 255) / 256, C), 256, 0, c->stream>>>(c->x, c->embd, c->embd_f16, c->tok_d, E);
    CKL(c);
    return 0;
}

double now_sec() { struct timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts); return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec; }

void free_ctx(dropin_ctx *c) {
    if (!c) return;
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->graph_ready) cudaGraphExecDestroy(c->graph);
    if (c->attn) hy3a_destroy(c->attn);
    for (int i = 0; i < c->n_up; i++) cudaFree(c->up[i].dev);
    free(c->up);
    for (int il = 0; il < NL; il++) { cudaFree(c->L[il].xgate); cudaFree(c->L[il].xup); cudaFree(c->L[il].xdown); }
    float *bufs[] = {c->x, c->s, c->qkv, c->ao, c->o, c->ff, c->ff2, c->logits_d, c->router, c->rw, c->xg, c->xu, c->xd};
    for (float *b : bufs) cudaFree(b);
    cudaFree(c->h16); cudaFree(c->ids); cudaFree(c->tok_d);
    if (c->tok_h) cudaFreeHost(c->tok_h);
    if (c->cublas) cublasDestroy(c->cublas);
    if (c->stream) cudaStreamDestroy(c->stream);
    free(c);
}

int env_int(const char *name, int dflt) { const char *e = getenv(name); return e ? atoi(e) : dflt; }

} /* namespace */

extern "C" {

int hy3_gpu_init(hy3_model *m, int n_gpu_layers) {
    if (!m) return -1;
    dropin_ctx *c = (dropin_ctx *)calloc(1, sizeof(dropin_ctx));
    if (!c) return -1;
#define INIT_FAIL() do { free_ctx(c); return -1; } while (0)
    if (cudaStreamCreate(&c->stream) != cudaSuccess || cublasCreate(&c->cublas) != CUBLAS_STATUS_SUCCESS || cublasSetStream(c->cublas, c->stream) != CUBLAS_STATUS_SUCCESS) {
        fail(c, "no usable CUDA device / cuBLAS (%s)", cudaGetErrorString(cudaGetLastError()));
        INIT_FAIL();
    }
    cublasSetMathMode(c->cublas, CUBLAS_PEDANTIC_MATH);      /* fp32 weights are multiplied in fp32 */
    if (n_gpu_layers <= 0 || n_gpu_layers > 81) n_gpu_layers = 81;      /* hy3_gpu.cu:555 */
    m->gpu_layers = n_gpu_layers;
    c->n_gpu_layers = n_gpu_layers > NL ? NL : n_gpu_layers;
    /* weights */
    {
        void *raw;
        const hy3_weight *te = &m->w.token_embd;
        if (!te->t || (te->t->ggml_type != T_F32 && te->t->ggml_type != T_F16)) { fail(c, "token_embd must be F32 or F16"); INIT_FAIL(); }
        if (upload_raw(c, te, &raw, 0) < 0) INIT_FAIL();
        c->embd = raw; c->embd_f16 = te->t->ggml_type == T_F16;
        if (upload_f32(c, &m->w.output_norm, &c->out_norm)) INIT_FAIL();
        c->vocab = m->w.output.t ? (int)m->w.output.t->dim[0] : 0;     /* hy3.c:1409 */
        if (c->vocab < 1 || c->vocab > HY3_N_VOCAB) c->vocab = HY3_N_VOCAB;
        if (upload_dense(c, &m->w.output, &c->out_w, c->vocab, E)) INIT_FAIL();
    }
    for (int il = 0; il < c->n_gpu_layers; il++) {
        hy3_layer_weights *l = &m->w.layers[il];
        layer_dev &L = c->L[il];
        if (upload_f32(c, &l->attn_norm, &L.attn_norm) || upload_f32(c, &l->ffn_norm, &L.ffn_norm)) INIT_FAIL();
        if (upload_dense(c, &l->attn_q, &L.wq, QS, E) || upload_dense(c, &l->attn_k, &L.wk, KVD, E) || upload_dense(c, &l->attn_v, &L.wv, KVD, E) ||
            upload_dense(c, &l->attn_output, &L.wo, E, QS)) INIT_FAIL();
        if (il < HY3_N_LAYER_DENSE) {
            if (upload_dense(c, &l->ffn_gate, &L.gate, DI, E) || upload_dense(c, &l->ffn_up, &L.up, DI, E) || upload_dense(c, &l->ffn_down, &L.down, E, DI)) INIT_FAIL();
        } else {
            if (upload_dense(c, &l->ffn_gate_shexp, &L.gate, MI, E) || upload_dense(c, &l->ffn_up_shexp, &L.up, MI, E) || upload_dense(c, &l->ffn_down_shexp, &L.down, E, MI) ||
                upload_dense(c, &l->ffn_gate_inp, &L.router, NX, E)) INIT_FAIL();
            if (L.router.f16) { fail(c, "the router projection must be F32 (hy3_gpu.cu:659)"); INIT_FAIL(); }
            if (l->has_expert_bias) {
                if (cudaMalloc(&L.bias, NX * sizeof(float)) != cudaSuccess || cudaMemcpy(L.bias, l->expert_bias, NX * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) { fail(c, "expert bias upload failed"); INIT_FAIL(); }
                /* owned through the upload table so that free_ctx releases it */
                if (c->n_up == c->cap_up) { c->cap_up = c->cap_up ? 2 * c->cap_up : 256; c->up = (upload_entry *)realloc(c->up, (size_t)c->cap_up * sizeof(upload_entry)); }
                c->up[c->n_up].host = NULL; c->up[c->n_up].dev = L.bias; c->up[c->n_up].kind = 2; c->n_up++;
            }
            if (upload_experts(c, l->ffn_gate_exps, &L.xgate) || upload_experts(c, l->ffn_up_exps, &L.xup) || upload_experts(c, l->ffn_down_exps, &L.xdown)) INIT_FAIL();
        }
    }
    /* switches, read once (hy3_gpu.cu:598-606) */
    c->kv_dtype = env_int("HY3_KV_INT4", 0) ? HY3A_KV_INT4 : (env_int("HY3_KV_FP16", 0) ? HY3A_KV_FP16 : HY3A_KV_INT8);
    c->chunk = env_int("HY3_PREFILL_CHUNK", 0) > 0 ? env_int("HY3_PREFILL_CHUNK", 0) : 0;
    if (c->chunk > 0) fprintf(stderr, "hy3_gpu: chunked prefill enabled (chunk=%d tokens)\n", c->chunk);
    const int pos_jump = env_int("HY3_POS_JUMP", 0), pos_jump_at = env_int("HY3_POS_JUMP_AT", 0);
    int pos_stride = env_int("HY3_POS_STRIDE", 1);
    if (pos_stride < 1) pos_stride = 1;
    if (pos_jump > 0) fprintf(stderr, "hy3_gpu: RoPE pos jump=+%d for token idx>=%d\n", pos_jump, pos_jump_at);
    if (pos_stride > 1) fprintf(stderr, "hy3_gpu: RoPE position stride=%d\n", pos_stride);
    c->use_graph = !env_int("HY3_NO_GRAPH", 0);
    /* KV pool: HY3_KV_TOKENS, else what 80 % of the free memory holds, at most 131072 tokens; the pool is paged, so this
     * is a capacity, not a reallocation step (hy3_gpu.cu:607, :692-698) */
    hy3a_config cfg;
    hy3a_default_config(&cfg);
    cfg.kv_dtype = c->kv_dtype;
    cfg.n_layers = NL;
    cfg.max_batch = c->chunk > 1 ? c->chunk : 1;
    {
        const size_t per_block = hy3a_block_bytes(&cfg);
        size_t fr = 0, tot = 0;
        cudaMemGetInfo(&fr, &tot);
        long long tokens = env_int("HY3_KV_TOKENS", 0);
        if (tokens <= 0) { tokens = (long long)(fr / 10 * 8 / per_block) * HY3A_PAGE_TOKENS; if (tokens > 131072) tokens = 131072; }
        if (tokens < HY3A_PAGE_TOKENS) tokens = HY3A_PAGE_TOKENS;
        cfg.max_blocks = cfg.max_blocks_per_seq = (int)((tokens + HY3A_PAGE_TOKENS - 1) / HY3A_PAGE_TOKENS);
        c->max_tokens = cfg.max_blocks * HY3A_PAGE_TOKENS;
    }
    cfg.rms_eps = kEps;
    if (hy3a_create(&cfg, &c->attn)) { fail(c, "attention context: %s", hy3a_last_error(NULL)); INIT_FAIL(); }
    if (hy3a_set_stream(c->attn, c->stream)) INIT_FAIL();
    {
        float inv[HY3_HEAD_DIM / 2], af = 1.f;
        hy3_rope_get_params(m, inv, &af);                     /* hy3_gpu.cu:625 */
        if (hy3a_set_rope(c->attn, inv, af, pos_stride, pos_jump, pos_jump_at)) { fail(c, "%s", hy3a_last_error(c->attn)); INIT_FAIL(); }
    }
    for (int il = 0; il < c->n_gpu_layers; il++) {
        const hy3_layer_weights *l = &m->w.layers[il];
        /* a layer without QK-norm tensors skips the norm on the host (hy3.c:1238); unit weights still normalise, so
         * such a model is refused rather than run differently */
        if (!l->attn_q_norm.data || !l->attn_k_norm.data) { fail(c, "layer %d has no attn_q_norm / attn_k_norm", il); INIT_FAIL(); }
        if (hy3a_set_norm_weights(c->attn, il, (const float *)l->attn_q_norm.data, (const float *)l->attn_k_norm.data)) { fail(c, "%s", hy3a_last_error(c->attn)); INIT_FAIL(); }
    }
    if (cudaMalloc(&c->logits_d, (size_t)HY3_N_VOCAB * sizeof(float)) != cudaSuccess || cudaHostAlloc((void **)&c->tok_h, (size_t)(c->chunk > 1 ? c->chunk : 1) * sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
        fail(c, "out of device memory"); INIT_FAIL();
    }
    if (ensure_cap(c, c->chunk > 1 ? c->chunk : 1)) INIT_FAIL();
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) { fail(c, "device error during init: %s", cudaGetErrorString(cudaGetLastError())); INIT_FAIL(); }
    m->gpu_ctx = c;
    fprintf(stderr, "hy3_gpu: initialized (%d layers, %s KV, online attn)\n", n_gpu_layers,
            c->kv_dtype == HY3A_KV_INT4 ? "INT4" : (c->kv_dtype == HY3A_KV_FP16 ? "FP16" : "INT8"));
    return 0;
#undef INIT_FAIL
}

void hy3_gpu_free(hy3_model *m) {
    if (!m || !m->gpu_ctx) return;
    free_ctx((dropin_ctx *)m->gpu_ctx);
    m->gpu_ctx = NULL;
}

int hy3_eval_gpu(hy3_model *m, const hy3_tokens *tokens, float *logits, int *pos) {
    dropin_ctx *c = m ? (dropin_ctx *)m->gpu_ctx : NULL;
    if (!c) return -1;
    if (!tokens || tokens->len < 1 || !logits || !pos) return fail(c, "hy3_eval_gpu: bad argument");
    if (m->cache_len % NL) return fail(c, "cache_len %d is not a multiple of %d", m->cache_len, NL);
    const int ng = c->n_gpu_layers, full = ng >= NL;
    int i_start = 0;
    /* ---- chunked prefill of all tokens but the last (hy3_gpu.cu:857-866) */
    if (full && c->chunk > 0 && tokens->len > 1) {
        const int npre = tokens->len - 1;
        const double t_begin = now_sec();
        double t_last = t_begin;
        for (int off = 0; off < npre;) {
            const int n = c->chunk < npre - off ? c->chunk : npre - off;
            const int t0 = m->cache_len / NL;
            if (ensure_cap(c, n) || set_batch(c, t0, n) || embed_tokens(c, tokens->v + off, n) || launch_embed(c, n)) return -1;
            for (int il = 0; il < NL; il++) if (layer_forward(c, m, il, t0, n)) return -1;
            if (hy3a_sync(c->attn)) return fail(c, "%s", hy3a_last_error(c->attn));
            m->cache_len = (t0 + n) * NL;
            off += n;
            const double now = now_sec(), dt = now - t_last;
            t_last = now;
            fprintf(stderr, "hy3_gpu: prefill %d/%d tok (%.1f%%) | chunk %d in %.1fs (%.1f tok/s) | elapsed %.0fs\n", off, npre, 100.0 * off / npre, n, dt, n / (dt + 1e-9), now - t_begin);
        }
        i_start = npre;
    }
    /* ---- token by token */
    for (int i = i_start; i < tokens->len; i++) {
        const int cb = m->cache_len, t = cb / NL;
        if (set_batch(c, t, 1) || embed_tokens(c, tokens->v + i, 1)) return -1;
        if (full && tokens->len == 1 && c->use_graph && c->warmed) {
            /* the single-token step as one graph: every launch reads its position from the batch descriptor in device
             * memory and the cache never moves, so it is captured once (cf. the recapture rules of hy3_gpu.cu:774-789) */
            if (!c->graph_ready) {
                cudaGraph_t g;
                CK(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
                int rc = launch_embed(c, 1);
                for (int il = 0; il < NL && !rc; il++) rc = layer_forward(c, m, il, t, 1);
                cudaError_t e = cudaStreamEndCapture(c->stream, &g);
                if (rc || e != cudaSuccess) return fail(c, "graph capture failed (%s)", cudaGetErrorString(e));
                e = cudaGraphInstantiate(&c->graph, g, 0);
                cudaGraphDestroy(g);
                if (e != cudaSuccess) return fail(c, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
                c->graph_ready = 1;
            }
            CK(c, cudaGraphLaunch(c->graph, c->stream));
        } else {
            if (launch_embed(c, 1)) return -1;
            for (int il = 0; il < ng; il++) if (layer_forward(c, m, il, t, 1)) return -1;
            if (full) c->warmed = 1;
        }
        if (!full) {
            /* layers beyond n_gpu_layers on the host (hy3_gpu.cu:945-950): their K/V live in the model's own fp32 cache */
            const int need = cb + NL;
            if (!m->cache_k || need > m->ctx_size) {
                const size_t cap = (size_t)need + 1024;
                float *nk = (float *)realloc(m->cache_k, cap * KVD * sizeof(float)), *nv = (float *)realloc(m->cache_v, cap * KVD * sizeof(float));
                if (nk) m->cache_k = nk;
                if (nv) m->cache_v = nv;
                if (!nk || !nv) return fail(c, "out of host memory for the CPU layers' cache");
                m->ctx_size = (int)cap;
            }
            CK(c, cudaMemcpyAsync(m->embed, c->x, E * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
            CK(c, cudaStreamSynchronize(c->stream));
            for (int il = ng; il < NL; il++) {
                m->cache_len = cb + il;
                if (il < HY3_N_LAYER_DENSE) forward_layer_dense(m, il, t); else forward_layer_moe(m, il, t);
            }
            CK(c, cudaMemcpyAsync(c->x, m->embed, E * sizeof(float), cudaMemcpyHostToDevice, c->stream));
        }
        m->cache_len = cb + NL;
    }
    /* ---- logits of the last token (hy3_gpu.cu:952-956) */
    if (c->out_norm) { rmsnorm_kernel<<<1, 256, 0, c->stream>>>(c->x, c->x, nullptr, c->out_norm, E); CKL(c); }
    if (matmul(c, c->out_w, c->x, E, c->logits_d, c->vocab, 1)) return -1;
    CK(c, cudaMemcpyAsync(logits, c->logits_d, (size_t)c->vocab * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    if (hy3a_sync(c->attn)) return fail(c, "%s", hy3a_last_error(c->attn));
    *pos = m->cache_len;
    return 0;
}

/* hy3_gpu.h:8 declares this name; the engine calls hy3_eval_gpu (hy3.c:1370). */
int hy3_gpu_eval(hy3_model *m, const hy3_tokens *tokens, float *logits, int *pos) { return hy3_eval_gpu(m, tokens, logits, pos); }

const char *hy3_gpu_last_error(const hy3_model *m) { return m && m->gpu_ctx ? ((const dropin_ctx *)m->gpu_ctx)->err : ""; }

} /* extern "C" */
