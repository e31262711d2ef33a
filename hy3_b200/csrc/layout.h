/*
 * layout.h -- geometry of the paged KV cache in HBM (shared by host and device code).
 *
 * The reference keeps one slot per (token, layer) holding all 8 KV heads
 * ([8 x fp16 scale][8 x 128 codes], slot = token*80 + layer; hy3_gpu.cu:26-35, :205-209),
 * so one layer's keys of one head are 128-byte fragments at an 83 200-byte stride.
 * Here the unit is a PAGE: 128 consecutive tokens of ONE (layer, KV head), contiguous:
 *
 *      [ K codes : 128 rows ][ V codes : 64 pair-rows (128 rows for FP16) ][ K scales fp16[128] ][ V scales fp16[128] ]
 *
 *   INT8  33 280 B   K row 128 B,  V area = the TRANSPOSED tile: 128 rows (head dims) x 128 token bytes
 *   INT4  16 896 B   K row  64 B,  V pair-row 128 B
 *   FP16  65 536 B   K row 256 B,  V row      256 B, no scales
 *
 * A BLOCK is the set of pages of all layers and all owned KV heads for the same 128
 * tokens; page address = pool + ((block*n_layers + layer)*kv_heads + head) * page_bytes.
 * Sequences map token/128 -> block through a block table, so growth, rollback and
 * ragged batches never move data.
 *
 * INT8 V area: row = head dim, column = token, two's complement, in the tensor core's K-major 128-byte-swizzle order
 * (16-byte chunk c of row r sits at chunk c ^ (r & 7)), so that the page copied verbatim into 1024-byte-aligned shared
 * memory is a tcgen05.mma operand with the head dims as M and the tokens as K (decode_umma.cu).
 *
 * V "pair layout" (INT4): tokens 2i and 2i+1 share a pair-row in which 16-bit units
 * alternate between the two tokens (unit u of token 2i+e sits at 16-bit index 2u+e).  A
 * 32-bit word then holds the same dims of two consecutive tokens, which is exactly the
 * operand pairing the P.V tensor-core fragment wants, so the int->fp16 conversion and the
 * pairing are one byte-permute.  Rows are additionally XOR-swizzled at 16-byte chunk
 * granularity so the decode kernel's fragment loads from a shared-memory copy of a page
 * are bank-conflict free.  Only codes and scales match the reference, not addresses.
 */
#ifndef HY3A_LAYOUT_H
#define HY3A_LAYOUT_H

#include <stdint.h>

#if defined(__CUDACC__)
#define HY3A_HD __host__ __device__ __forceinline__
#else
#define HY3A_HD static inline
#endif

#define HY3A_D 128
#define HY3A_PT 128 /* tokens per page */

struct hy3a_geom {
    int dtype;      /* 0 fp16, 1 int8, 2 int4 */
    int k_row;      /* bytes per K row */
    int v_off;      /* byte offset of the V area */
    int v_prow;     /* bytes per V pair-row (INT8/INT4) or V row (FP16) */
    int ks_off;     /* byte offset of K scales (0 = none) */
    int vs_off;     /* byte offset of V scales */
    int page_bytes;
};

HY3A_HD hy3a_geom hy3a_make_geom(int dtype) {
    hy3a_geom g;
    g.dtype = dtype;
    if (dtype == 1) { g.k_row = 128; g.v_off = 16384; g.v_prow = 256; g.ks_off = 32768; g.vs_off = 33024; g.page_bytes = 33280; }
    else if (dtype == 2) { g.k_row = 64; g.v_off = 8192; g.v_prow = 128; g.ks_off = 16384; g.vs_off = 16640; g.page_bytes = 16896; }
    else { g.k_row = 256; g.v_off = 32768; g.v_prow = 256; g.ks_off = 0; g.vs_off = 0; g.page_bytes = 65536; }
    return g;
}

/* ---- K: byte offset (inside the page) of 16-byte chunk `chunk` of token row `tok`. */
template <int DT> HY3A_HD int hy3a_k_chunk_off(int tok, int chunk) {
    if (DT == 2) return tok * 64 + chunk * 16;                          /* 4 chunks, no swizzle needed */
    const int row = (DT == 1) ? 128 : 256;
    return tok * row + ((chunk ^ ((tok & 1) << 2)) << 4);
}
/* byte offset of the K element group starting at dim d (d % 4 == 0) of token tok */
template <int DT> HY3A_HD int hy3a_k_dim_off(int tok, int d) {
    if (DT == 1) return hy3a_k_chunk_off<1>(tok, d >> 4) + (d & 15);          /* 1 B / dim */
    if (DT == 2) return hy3a_k_chunk_off<2>(tok, d >> 5) + ((d & 31) >> 1);   /* 1/2 B / dim */
    return hy3a_k_chunk_off<0>(tok, d >> 3) + ((d & 7) << 1);                 /* 2 B / dim */
}

/* ---- V, INT8: byte offset relative to the V area of (head dim d, token tok) in the transposed, swizzled tile. */
HY3A_HD int hy3a_vt_off(int d, int tok) { return d * 128 + ((((tok >> 4) ^ (d & 7))) << 4) + (tok & 15); }

/* ---- V (INT4 pair layout; DT = 1 is the geometry the fp16-converting decode path of INT8 used and is kept for the
 * template's sake): offset relative to the V area of chunk `chunk` of pair-row pr. */
template <int DT> HY3A_HD int hy3a_v_chunk_off(int pr, int chunk) {
    const int prow = (DT == 1) ? 256 : 128;
    return pr * prow + ((chunk ^ ((pr & 3) << 1)) << 4);
}
/* offset (relative to the V area) of the 16-bit unit that holds dims [d, d+2) (INT8, d%2==0)
 * or [d, d+4) (INT4, d%4==0) of token tok.                                              */
template <int DT> HY3A_HD int hy3a_v_unit_off(int tok, int d) {
    const int u = (DT == 1) ? (d >> 1) : (d >> 2);
    const int pos = ((u << 1) + (tok & 1)) << 1; /* byte position in the unswizzled pair-row */
    return hy3a_v_chunk_off<DT>(tok >> 1, pos >> 4) + (pos & 15);
}
/* ---- V (FP16 plain rows): offset relative to the V area of chunk `chunk` (8 halfs) of token tok. */
HY3A_HD int hy3a_v16_chunk_off(int tok, int chunk) { return tok * 256 + ((chunk ^ (((tok >> 1) & 3) << 1)) << 4); }
HY3A_HD int hy3a_v16_dim_off(int tok, int d) { return hy3a_v16_chunk_off(tok, d >> 3) + ((d & 7) << 1); }

#endif /* HY3A_LAYOUT_H */
