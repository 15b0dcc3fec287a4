/*
 * kvarn_oracle.c -- CPU restatement of the KVarN G128 K4V4 quantized paged KV-cache path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the parity tests,
 * the smoke check and the CPU-baseline leg of the benchmark call it.  Nothing in the product
 * path (the CUDA library and its host bindings) links, imports or executes it.
 *
 * Parity status: the codec half (fp16 conversion, per-row 4-bit quantisation, Sinkhorn
 * balancing, record layout, dequantisation) is PINNED -- it is checked byte-for-byte against
 * the reference's own CPU oracle compiled from its sources and against the reference's GVK2
 * golden records.  The P1 plane slot map is pinned against the reference's slot-map table.
 * The attention half has no counterpart in the reference (its attention kernels are not in the
 * tree): it is plain softmax attention over the de-quantised cache, "parity unpinned".
 *
 * Each function cites the reference file:line it follows (paths relative to the reference
 * repository root):
 *   ORACLE  kvarn-evidence/oracle/bee_oracle.cpp
 *   LAYOUT  kvarn-port/engine/src/ops/kv_cache/kvarn_layout.h
 *   CODEC   kvarn-port/engine/src/ops/kv_cache/append/kvarn128_codec.cuh
 *   LAUNCH  kvarn-port/engine/src/ops/kv_cache/append/kvarn128_launch.cu
 *   CPUREF  kvarn-evidence/decode-g128/kvarn128_cpu_reference.h
 *   HAD     kvarn-evidence/wht-gate/ninfer_hadamard_d256_verbatim.h
 *
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared -pthread (see oracle/Makefile).  Contraction of
 * a*b+c into a fused multiply-add must stay off: the reference gates compare bytes and are built
 * without FMA contraction.
 */
#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KVO_TILE 128  /* tokens per tile                LAYOUT:34 */
#define KVO_PAGE 64   /* tokens per page                LAYOUT:35 */
#define KVO_SLICE 128 /* dims per quantisation record   LAYOUT:38 */

/* ------------------------------------------------------------------------------------------
 * fp16 / bf16 conversion.  ORACLE:49-100 (round-to-nearest-even, subnormals, inf/nan).
 * ------------------------------------------------------------------------------------------ */
uint16_t kvo_f32_to_f16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    const uint32_t sign = (u >> 16) & 0x8000u;
    const uint32_t exp = (u >> 23) & 0xFFu;
    const uint32_t man = u & 0x7FFFFFu;
    if (exp == 0xFFu) return (uint16_t)(sign | (man ? 0x7E00u : 0x7C00u));
    const int32_t e = (int32_t)exp - 127;
    if (e > 15) return (uint16_t)(sign | 0x7C00u);
    if (e >= -14) {
        uint32_t half = sign | ((uint32_t)(e + 15) << 10) | (man >> 13);
        const uint32_t rest = man & 0x1FFFu;
        if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) half += 1u;
        return (uint16_t)half;
    }
    if (e < -25) return (uint16_t)sign;
    const uint32_t sig = man | 0x800000u;
    const int shift = -(e + 1); /* 14..24 */
    uint32_t q = sig >> shift;
    const uint32_t rem = sig & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
    return (uint16_t)(sign | q);
}

float kvo_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) {
            u = sign;
        } else {
            int32_t ee = 127 - 15 + 1;
            while (!(m & 0x400u)) {
                m <<= 1;
                --ee;
            }
            u = sign | ((uint32_t)ee << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 0x1Fu) {
        u = sign | 0x7F800000u | (m << 13);
    } else {
        u = sign | ((e + 127 - 15) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static float bf16_to_f32(uint16_t h) {
    const uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* input element -> fp32; dtype 0 = fp16, 1 = bf16 (LAUNCH:107-114 reads bf16; the codec is the
 * same for fp16 input because both are widened to fp32 before the rotation). */
static float in_to_f32(const uint16_t* p, int dtype) { return dtype ? bf16_to_f32(*p) : kvo_f16_to_f32(*p); }

/* ------------------------------------------------------------------------------------------
 * Rotation: normalised Sylvester-Hadamard over one head row, butterflies in increasing stride,
 * low = a+b, high = a-b, one final scale.  HAD:16-71 (D=256, scale exactly 2^-4), CPUREF:117-128.
 * D=128 uses the 128-point constant 0.08838834764831845f (kvarn-evidence/oracle/make_tiles.py:32),
 * applied once after the last stage.  Every butterfly of a stage is independent, so the result
 * does not depend on how lanes/registers hold the row.
 * ------------------------------------------------------------------------------------------ */
void kvo_hadamard(float* v, int dim) {
    for (int s = 1; s < dim; s <<= 1)
        for (int i = 0; i < dim; i += 2 * s)
            for (int j = i; j < i + s; ++j) {
                const float a = v[j], b = v[j + s];
                v[j] = a + b;
                v[j + s] = a - b;
            }
    const float norm = dim == 256 ? 0.0625f : 0.08838834764831845f;
    for (int i = 0; i < dim; ++i) v[i] = v[i] * norm;
}

/* ------------------------------------------------------------------------------------------
 * Geometry.  LAYOUT:61-131 generalised from D=256 (S=2) to S = head_dim/128 in {1,2}:
 * code row = head_dim/2 bytes; dim-axis entries fill the 64 page rows c = head_dim/64 per row.
 * ------------------------------------------------------------------------------------------ */
static int code_leading(int head_dim) { return head_dim / 2; }
static int k_scale_leading(int head_dim) { return 5 * (head_dim / KVO_SLICE); }
static int v_scale_leading(int head_dim) { return 4 * (head_dim / KVO_SLICE); }

/* LAYOUT:90-97 */
int64_t kvo_plane_offset(int leading, int heads, int page, int head, int page_off, int slot) {
    return (int64_t)leading * KVO_PAGE * ((int64_t)head + (int64_t)heads * page) + (int64_t)leading * page_off + slot;
}

/* Slot of one axis entry inside a scale page, as (row, col).  LAYOUT:99-131, CPUREF:70-86.
 * item: 0 = scale_axis, 1 = zp_axis, 2 = other_axis.  index = global dim for a dim-axis entry,
 * page-local token for a token-axis entry (slice selects the column then). */
void kvo_scale_slot(int head_dim, int is_value, int item, int slice, int index, int* row, int* col) {
    const int S = head_dim / KVO_SLICE, c = 2 * S;
    if (!is_value) {
        if (item == 0) { *row = index / c; *col = index % c; }
        else if (item == 1) { *row = index / c; *col = c + index % c; }
        else { *row = index; *col = 2 * c + slice; }
    } else {
        if (item == 2) { *row = index / c; *col = index % c; }
        else if (item == 0) { *row = index; *col = c + slice; }
        else { *row = index; *col = c + S + slice; }
    }
}

/* ------------------------------------------------------------------------------------------
 * Sinkhorn variance balancing in the GPU order.  ORACLE:193-255 == CODEC:104-186.
 * ------------------------------------------------------------------------------------------ */
static float std_col(const float* t, int R, int C, const float* sc, const float* sr, int col) {
    float sum = 0.0f, sq = 0.0f;
    for (int r = 0; r < R; ++r) {
        const float v = t[r * C + col] / (sc[col] * sr[r]);
        sum += v;
        sq += v * v;
    }
    const float mean = sum / (float)R;
    return sqrtf(fmaxf((sq - (float)R * mean * mean) / (float)(R - 1), 0.0f));
}
static float std_row(const float* t, int R, int C, const float* sc, const float* sr, int row) {
    (void)R;
    float sum = 0.0f, sq = 0.0f;
    for (int c = 0; c < C; ++c) {
        const float v = t[row * C + c] / (sc[c] * sr[row]);
        sum += v;
        sq += v * v;
    }
    const float mean = sum / (float)C;
    return sqrtf(fmaxf((sq - (float)C * mean * mean) / (float)(C - 1), 0.0f));
}

void kvo_sinkhorn(const float* tile, int R, int C, int iters, float* best_col, float* best_row, float* best_imbalance,
                  int* best_iter) {
    float *log_c = calloc(C, 4), *log_r = calloc(R, 4), *sc = malloc(C * 4), *sr = malloc(R * 4);
    float *cs = malloc(C * 4), *rs = malloc(R * 4);
    for (int i = 0; i < C; ++i) sc[i] = best_col[i] = 1.0f;
    for (int i = 0; i < R; ++i) sr[i] = best_row[i] = 1.0f;
    float best = FLT_MAX;
    int bi = -1;
    for (int c = 0; c < C; ++c) cs[c] = std_col(tile, R, C, sc, sr, c);
    for (int r = 0; r < R; ++r) rs[r] = std_row(tile, R, C, sc, sr, r);
    for (int iter = -1; iter < iters; ++iter) {
        if (iter >= 0) {
            for (int c = 0; c < C; ++c) {
                const float v = fminf(fmaxf(cs[c], 1e-3f), 1e3f);
                log_c[c] = fminf(fmaxf(log_c[c] + logf(v), -0.3f), 10.0f);
                sc[c] = expf(log_c[c]);
            }
            for (int r = 0; r < R; ++r) rs[r] = std_row(tile, R, C, sc, sr, r);
            for (int r = 0; r < R; ++r) {
                const float v = fminf(fmaxf(rs[r], 1e-3f), 1e3f);
                log_r[r] = fminf(fmaxf(log_r[r] + logf(v), -0.3f), 10.0f);
                sr[r] = expf(log_r[r]);
            }
            for (int r = 0; r < R; ++r) rs[r] = std_row(tile, R, C, sc, sr, r);
            for (int c = 0; c < C; ++c) cs[c] = std_col(tile, R, C, sc, sr, c);
        }
        float cmin = FLT_MAX, cmax = 0.0f, rmin = FLT_MAX, rmax = 0.0f;
        for (int c = 0; c < C; ++c) { cmin = fminf(cmin, cs[c]); cmax = fmaxf(cmax, cs[c]); }
        for (int r = 0; r < R; ++r) { rmin = fminf(rmin, rs[r]); rmax = fmaxf(rmax, rs[r]); }
        const float imb = cmax / fmaxf(cmin, 1e-8f) + rmax / fmaxf(rmin, 1e-8f);
        if (imb <= best) { /* "<=": a later tie wins, ORACLE:221 */
            best = imb;
            bi = iter;
            memcpy(best_col, sc, C * 4);
            memcpy(best_row, sr, R * 4);
        }
    }
    if (best_imbalance) *best_imbalance = best;
    if (best_iter) *best_iter = bi;
    free(log_c); free(log_r); free(sc); free(sr); free(cs); free(rs);
}

/* ------------------------------------------------------------------------------------------
 * Quantise one rows x cols fp32 matrix to a record = payload || scale_axis[rows] || zp_axis[rows]
 * || other_axis[cols] (fp16).  ORACLE:309-357; payload is an LSB-first bit string, ORACLE:152-163.
 * q_out (optional) receives the unpacked codes.
 * ------------------------------------------------------------------------------------------ */
size_t kvo_record_bytes(int rows, int cols, int bits) { return ((size_t)rows * cols * bits + 7) / 8 + (size_t)(2 * rows + cols) * 2; }

void kvo_quantize_tile(const float* tile, int rows, int cols, int bits, int iters, uint8_t* record, uint8_t* q_out,
                       float* best_col_out, float* best_row_out) {
    float *bc = malloc(cols * 4), *br = malloc(rows * 4);
    kvo_sinkhorn(tile, rows, cols, iters, bc, br, NULL, NULL);
    const int qmax = (1 << bits) - 1;
    const size_t payload = ((size_t)rows * cols * bits + 7) / 8;
    memset(record, 0, payload);
    uint16_t* axes = (uint16_t*)(record + payload);
    for (int r = 0; r < rows; ++r) {
        float lo = FLT_MAX, hi = -FLT_MAX;
        for (int c = 0; c < cols; ++c) {
            const float x = tile[(size_t)r * cols + c] / (bc[c] * br[r]);
            lo = fminf(lo, x);
            hi = fmaxf(hi, x);
        }
        const float scale = fmaxf((hi - lo) / (float)qmax, 1e-10f);
        for (int c = 0; c < cols; ++c) {
            const float x = tile[(size_t)r * cols + c] / (bc[c] * br[r]);
            const uint8_t q = (uint8_t)fminf(fmaxf(roundf((x - lo) / scale), 0.0f), (float)qmax);
            if (q_out) q_out[(size_t)r * cols + c] = q;
            const size_t bit0 = ((size_t)r * cols + c) * bits;
            for (int b = 0; b < bits; ++b) record[(bit0 + b) / 8] |= (uint8_t)(((q >> b) & 1u) << ((bit0 + b) % 8));
        }
        axes[r] = kvo_f32_to_f16(br[r] * scale);
        axes[rows + r] = kvo_f32_to_f16(br[r] * lo);
    }
    for (int c = 0; c < cols; ++c) axes[2 * rows + c] = kvo_f32_to_f16(bc[c]);
    if (best_col_out) memcpy(best_col_out, bc, cols * 4);
    if (best_row_out) memcpy(best_row_out, br, rows * 4);
    free(bc);
    free(br);
}

/* ORACLE:359-374: x[r][c] = (q*scale_axis[r] + zp_axis[r]) * other_axis[c], each step rounded. */
void kvo_dequant_tile(const uint8_t* record, int rows, int cols, int bits, float* tile) {
    const size_t payload = ((size_t)rows * cols * bits + 7) / 8;
    const uint16_t* axes = (const uint16_t*)(record + payload);
    for (int r = 0; r < rows; ++r) {
        const float sa = kvo_f16_to_f32(axes[r]), zp = kvo_f16_to_f32(axes[rows + r]);
        for (int c = 0; c < cols; ++c) {
            const float oa = kvo_f16_to_f32(axes[2 * rows + c]);
            const size_t bit0 = ((size_t)r * cols + c) * bits;
            unsigned q = 0;
            for (int b = 0; b < bits; ++b) q |= ((record[(bit0 + b) / 8] >> ((bit0 + b) % 8)) & 1u) << b;
            const float qs = (float)q * sa;
            const float qz = qs + zp;
            tile[(size_t)r * cols + c] = qz * oa;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Cache state of one layer (all caller-owned, like the CUDA library):
 *   k_code/v_code  u8   {head_dim/2, 64, H, pages}
 *   k_scale        f16  {5S, 64, H, pages}      v_scale f16 {4S, 64, H, pages}
 *   stage          f16  [which K|V][slot = tile%2][H][128][head_dim]   LAUNCH:84-120,262-322
 *   table          i32  logical page -> physical page                  CPUREF / LAUNCH:143-145
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    uint8_t* k_code;
    uint16_t* k_scale;
    uint8_t* v_code;
    uint16_t* v_scale;
    uint16_t* stage;
    const int32_t* table;
    int head_dim, kv_heads, iters;
} kvo_layer;

static uint16_t* stage_row(const kvo_layer* L, int which, int slot, int head, int tok) {
    const int64_t plane = (int64_t)2 * L->kv_heads * KVO_TILE * L->head_dim;
    return L->stage + which * plane + (((int64_t)slot * L->kv_heads + head) * KVO_TILE + tok) * L->head_dim;
}

/* Seal one tile of one head: quantise K and V slices from the fp16 stage and write the P1 planes
 * of the tile's two pages.  CODEC:357-409 (+ :233-306 for the plane writes). */
static void seal_tile(const kvo_layer* L, int tile, int head) {
    const int D = L->head_dim, S = D / KVO_SLICE, H = L->kv_heads, slot = tile & 1;
    const int32_t page[2] = {L->table[2 * tile], L->table[2 * tile + 1]};
    float* m = malloc(sizeof(float) * KVO_SLICE * KVO_TILE);
    uint8_t* q = malloc(KVO_SLICE * KVO_TILE);
    uint8_t* rec = malloc(kvo_record_bytes(128, 128, 4));
    const uint16_t* ax = (const uint16_t*)(rec + 128 * 128 / 2);
    for (int which = 0; which < 2; ++which) {
        uint8_t* code = which ? L->v_code : L->k_code;
        uint16_t* sc = which ? L->v_scale : L->k_scale;
        const int cl = code_leading(D), sl = which ? v_scale_leading(D) : k_scale_leading(D);
        for (int s = 0; s < S; ++s) {
            /* K: row = dim, col = token.  V: row = token, col = dim.  CODEC:366-379 */
            for (int r = 0; r < 128; ++r)
                for (int c = 0; c < 128; ++c) {
                    const int tok = which ? r : c, dim = which ? c : r;
                    m[r * 128 + c] = kvo_f16_to_f32(stage_row(L, which, slot, head, tok)[s * KVO_SLICE + dim]);
                }
            kvo_quantize_tile(m, 128, 128, 4, L->iters, rec, q, NULL, NULL);
            for (int tok = 0; tok < KVO_TILE; ++tok) {
                const int pg = page[tok / KVO_PAGE], off = tok % KVO_PAGE;
                /* codes: byte b of a token row holds dims 2b (low nibble) and 2b+1.  CODEC:227-266 */
                for (int dl = 0; dl < KVO_SLICE; dl += 2) {
                    const int q0 = which ? q[tok * 128 + dl] : q[dl * 128 + tok];
                    const int q1 = which ? q[tok * 128 + dl + 1] : q[(dl + 1) * 128 + tok];
                    code[kvo_plane_offset(cl, H, pg, head, off, (s * KVO_SLICE + dl) / 2)] = (uint8_t)(q0 | (q1 << 4));
                }
                /* token-axis entries.  CODEC:284-303 */
                int row, col;
                if (!which) {
                    kvo_scale_slot(D, 0, 2, s, off, &row, &col);
                    sc[kvo_plane_offset(sl, H, pg, head, row, col)] = ax[256 + tok]; /* other_axis[col=token] */
                } else {
                    kvo_scale_slot(D, 1, 0, s, off, &row, &col);
                    sc[kvo_plane_offset(sl, H, pg, head, row, col)] = ax[tok]; /* scale_axis[row=token] */
                    kvo_scale_slot(D, 1, 1, s, off, &row, &col);
                    sc[kvo_plane_offset(sl, H, pg, head, row, col)] = ax[128 + tok];
                }
            }
            /* dim-axis entries, duplicated in both pages of the tile (page-self-sufficient P1). */
            for (int p = 0; p < 2; ++p)
                for (int dl = 0; dl < KVO_SLICE; ++dl) {
                    const int d = s * KVO_SLICE + dl;
                    int row, col;
                    if (!which) {
                        kvo_scale_slot(D, 0, 0, s, d, &row, &col);
                        sc[kvo_plane_offset(sl, H, page[p], head, row, col)] = ax[dl];
                        kvo_scale_slot(D, 0, 1, s, d, &row, &col);
                        sc[kvo_plane_offset(sl, H, page[p], head, row, col)] = ax[128 + dl];
                    } else {
                        kvo_scale_slot(D, 1, 2, s, d, &row, &col);
                        sc[kvo_plane_offset(sl, H, page[p], head, row, col)] = ax[256 + dl];
                    }
                }
        }
    }
    free(m);
    free(q);
    free(rec);
}

/* Seal tile `tile` of head `head` from whatever the stage slot tile % 2 holds (what a roll-back followed by a
 * re-seal does, LAUNCH:262-273): lets a test place already-rotated rows in the stage and obtain the planes. */
void kvo_seal_tile(uint8_t* k_code, uint16_t* k_scale, uint8_t* v_code, uint16_t* v_scale, uint16_t* stage,
                   const int32_t* table, int head_dim, int kv_heads, int iters, int tile) {
    kvo_layer L = {k_code, k_scale, v_code, v_scale, stage, table, head_dim, kv_heads, iters};
    for (int h = 0; h < kv_heads; ++h) seal_tile(&L, tile, h);
}

/* Append `tokens` contiguous positions pos0.. of one sequence.  k/v: [tok][head][dim] 16-bit,
 * dtype 0 fp16 / 1 bf16.  Tile by tile: rotate the new rows into stage[tile%2], then seal the
 * tile if the append fills it.  LAUNCH:53-77 (tile geometry), :84-120 (rotate), :1066-1092 (loop). */
void kvo_append(uint8_t* k_code, uint16_t* k_scale, uint8_t* v_code, uint16_t* v_scale, uint16_t* stage,
                const int32_t* table, int head_dim, int kv_heads, int iters, const uint16_t* k, const uint16_t* v,
                int dtype, int pos0, int tokens) {
    if (tokens <= 0) return;
    kvo_layer L = {k_code, k_scale, v_code, v_scale, stage, table, head_dim, kv_heads, iters};
    const int last = pos0 + tokens - 1, D = head_dim;
    float row[256];
    for (int tile = pos0 / KVO_TILE; tile <= last / KVO_TILE; ++tile) {
        const int base = tile * KVO_TILE;
        const int b = pos0 > base ? pos0 - base : 0;
        const int e = last + 1 < base + KVO_TILE ? last + 1 - base : KVO_TILE;
        for (int tt = b; tt < e; ++tt)
            for (int h = 0; h < kv_heads; ++h)
                for (int which = 0; which < 2; ++which) {
                    const uint16_t* src = (which ? v : k) + ((int64_t)(base + tt - pos0) * kv_heads + h) * D;
                    for (int d = 0; d < D; ++d) row[d] = in_to_f32(src + d, dtype);
                    kvo_hadamard(row, D);
                    uint16_t* dst = stage_row(&L, which, tile & 1, h, tt);
                    for (int d = 0; d < D; ++d) dst[d] = kvo_f32_to_f16(row[d]);
                }
        if (base + KVO_TILE <= last + 1)
            for (int h = 0; h < kv_heads; ++h) seal_tile(&L, tile, h);
    }
}

/* De-quantise one token row of one head from the planes into fp32 (rotated domain).
 * CODEC:314-350, CPUREF:89-105: val = (q*scale_axis + zp_axis) * other_axis, no contraction. */
static void decode_row(const kvo_layer* L, int is_value, int page, int head, int off, float* out) {
    const int D = L->head_dim, H = L->kv_heads, cl = code_leading(D);
    const int sl = is_value ? v_scale_leading(D) : k_scale_leading(D);
    const uint8_t* code = is_value ? L->v_code : L->k_code;
    const uint16_t* sc = is_value ? L->v_scale : L->k_scale;
    for (int d = 0; d < D; ++d) {
        const int s = d / KVO_SLICE;
        const int by = code[kvo_plane_offset(cl, H, page, head, off, d / 2)];
        const float q = (float)((by >> ((d & 1) * 4)) & 15);
        int row, col;
        kvo_scale_slot(D, is_value, 0, s, is_value ? off : d, &row, &col);
        const float sa = kvo_f16_to_f32(sc[kvo_plane_offset(sl, H, page, head, row, col)]);
        kvo_scale_slot(D, is_value, 1, s, is_value ? off : d, &row, &col);
        const float zp = kvo_f16_to_f32(sc[kvo_plane_offset(sl, H, page, head, row, col)]);
        kvo_scale_slot(D, is_value, 2, s, is_value ? d : off, &row, &col);
        const float oa = kvo_f16_to_f32(sc[kvo_plane_offset(sl, H, page, head, row, col)]);
        const float qs = q * sa;
        const float qz = qs + zp;
        out[d] = qz * oa;
    }
}

/* One tile of one head -> rotated-domain fp16 [128][head_dim] for K and V.  LAUNCH:1099-1115. */
void kvo_decode_tile(const uint8_t* k_code, const uint16_t* k_scale, const uint8_t* v_code, const uint16_t* v_scale,
                     const int32_t* table, int head_dim, int kv_heads, int tile, int head, uint16_t* out_k,
                     uint16_t* out_v) {
    kvo_layer L = {(uint8_t*)k_code, (uint16_t*)k_scale, (uint8_t*)v_code, (uint16_t*)v_scale, NULL, table, head_dim, kv_heads, 0};
    float row[256];
    for (int tok = 0; tok < KVO_TILE; ++tok) {
        const int page = table[2 * tile + tok / KVO_PAGE], off = tok % KVO_PAGE;
        decode_row(&L, 0, page, head, off, row);
        for (int d = 0; d < head_dim; ++d) out_k[tok * head_dim + d] = kvo_f32_to_f16(row[d]);
        decode_row(&L, 1, page, head, off, row);
        for (int d = 0; d < head_dim; ++d) out_v[tok * head_dim + d] = kvo_f32_to_f16(row[d]);
    }
}

/* ------------------------------------------------------------------------------------------
 * Attention over the cache.  No counterpart in the reference tree; the semantics follow the
 * reference's consumer window (LAUNCH:194-229): a tile whose 128 tokens are all appended
 * ((tile+1)*128 <= kv_total) is read de-quantised from its pages, the open tile un-quantised from
 * stage[tile%2]; everything in the rotated domain.  logit_j = scale * <H q, K_j>, out = H(sum_j
 * softmax_j V_j).  Row (t, qh) sees keys at positions <= q_pos[t].
 *
 * Work is cut into (kv head, key chunk) jobs run by `threads` pthreads; each job produces an
 * un-normalised partial (m, l, o_rot) per query row and the partials are merged by
 * log-sum-exp -- the same merge the split-K kernels and the multi-GPU combine use.
 * Accumulation is in double so that the oracle is strictly more accurate than any fp32 path.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    const kvo_layer* L;
    const float* qrot; /* [T][QH][D] rotated, fp32 */
    const int32_t* q_pos;
    int T, QH, kv_total, key_begin, key_end, head;
    float scale;
    double *m, *l, *o; /* per (t, g): m, l, o[D] for this job */
} attn_job;

static void run_attn_job(attn_job* J) {
    const kvo_layer* L = J->L;
    const int D = L->head_dim, G = J->QH / L->kv_heads, h = J->head;
    float kr[256], vr[256];
    for (int i = 0; i < J->T * G; ++i) {
        J->m[i] = -INFINITY;
        J->l[i] = 0.0;
        memset(J->o + (size_t)i * D, 0, sizeof(double) * D);
    }
    for (int pos = J->key_begin; pos < J->key_end; ++pos) {
        const int tile = pos / KVO_TILE, tt = pos % KVO_TILE;
        if ((tile + 1) * KVO_TILE <= J->kv_total) {
            const int page = L->table[pos / KVO_PAGE];
            decode_row(L, 0, page, h, pos % KVO_PAGE, kr);
            decode_row(L, 1, page, h, pos % KVO_PAGE, vr);
        } else {
            const uint16_t* ks = stage_row(L, 0, tile & 1, h, tt);
            const uint16_t* vs = stage_row(L, 1, tile & 1, h, tt);
            for (int d = 0; d < D; ++d) {
                kr[d] = kvo_f16_to_f32(ks[d]);
                vr[d] = kvo_f16_to_f32(vs[d]);
            }
        }
        for (int t = 0; t < J->T; ++t) {
            if (pos > J->q_pos[t]) continue;
            for (int g = 0; g < G; ++g) {
                const float* q = J->qrot + ((size_t)t * J->QH + h * G + g) * D;
                double dot = 0.0;
                for (int d = 0; d < D; ++d) dot += (double)q[d] * (double)kr[d];
                const double s = dot * (double)J->scale;
                const int i = t * G + g;
                double* o = J->o + (size_t)i * D;
                if (s > J->m[i]) {
                    const double a = exp(J->m[i] - s);
                    J->l[i] *= a;
                    for (int d = 0; d < D; ++d) o[d] *= a;
                    J->m[i] = s;
                }
                const double p = exp(s - J->m[i]);
                J->l[i] += p;
                for (int d = 0; d < D; ++d) o[d] += p * (double)vr[d];
            }
        }
    }
}

typedef struct {
    attn_job* jobs;
    int n, next;
    pthread_mutex_t mu;
} job_queue;

static void* worker(void* arg) {
    job_queue* Q = arg;
    for (;;) {
        pthread_mutex_lock(&Q->mu);
        const int i = Q->next < Q->n ? Q->next++ : -1;
        pthread_mutex_unlock(&Q->mu);
        if (i < 0) return NULL;
        run_attn_job(&Q->jobs[i]);
    }
}

/* q: [T][QH][D] 16-bit (dtype as in kvo_append); q_pos: [T]; out: fp32 [T][QH][D] (un-rotated).
 * If part_m/part_l/part_o are non-NULL the merged, un-normalised rotated-domain partials
 * (m, l, o_rot) per (t, qh) are stored there too (what one GPU contributes to a combine). */
void kvo_attention(const uint8_t* k_code, const uint16_t* k_scale, const uint8_t* v_code, const uint16_t* v_scale,
                   const uint16_t* stage, const int32_t* table, int head_dim, int kv_heads, int q_heads,
                   const uint16_t* q, int dtype, const int32_t* q_pos, int T, int kv_total, int key_begin, int key_end,
                   float scale, int threads, float* out, float* part_m, float* part_l, float* part_o) {
    kvo_layer L = {(uint8_t*)k_code, (uint16_t*)k_scale, (uint8_t*)v_code, (uint16_t*)v_scale, (uint16_t*)stage, table, head_dim, kv_heads, 0};
    const int D = head_dim, G = q_heads / kv_heads;
    if (key_end > kv_total) key_end = kv_total;
    if (key_begin < 0) key_begin = 0;
    float* qrot = malloc(sizeof(float) * (size_t)T * q_heads * D);
    for (int i = 0; i < T * q_heads; ++i) {
        for (int d = 0; d < D; ++d) qrot[(size_t)i * D + d] = in_to_f32(q + (size_t)i * D + d, dtype);
        kvo_hadamard(qrot + (size_t)i * D, D);
    }
    if (threads < 1) threads = 1;
    const int span = key_end > key_begin ? key_end - key_begin : 0;
    int chunks = threads * 2 / kv_heads + 1;
    if (chunks > span / KVO_TILE + 1) chunks = span / KVO_TILE + 1;
    const int njobs = chunks * kv_heads, rows = T * G;
    attn_job* jobs = calloc(njobs, sizeof(attn_job));
    for (int h = 0; h < kv_heads; ++h)
        for (int c = 0; c < chunks; ++c) {
            attn_job* J = &jobs[h * chunks + c];
            J->L = &L; J->qrot = qrot; J->q_pos = q_pos; J->T = T; J->QH = q_heads; J->kv_total = kv_total;
            J->key_begin = key_begin + (int)((int64_t)span * c / chunks);
            J->key_end = key_begin + (int)((int64_t)span * (c + 1) / chunks);
            J->head = h; J->scale = scale;
            J->m = malloc(sizeof(double) * rows);
            J->l = malloc(sizeof(double) * rows);
            J->o = malloc(sizeof(double) * (size_t)rows * D);
        }
    job_queue Q = {jobs, njobs, 0, PTHREAD_MUTEX_INITIALIZER};
    pthread_t* th = malloc(sizeof(pthread_t) * threads);
    for (int i = 1; i < threads; ++i) pthread_create(&th[i], NULL, worker, &Q);
    worker(&Q);
    for (int i = 1; i < threads; ++i) pthread_join(th[i], NULL);
    /* log-sum-exp merge over the chunks of each head, then normalise and rotate back. */
    double* acc = malloc(sizeof(double) * D);
    float* orow = malloc(sizeof(float) * D);
    for (int h = 0; h < kv_heads; ++h)
        for (int i = 0; i < rows; ++i) {
            double m = -INFINITY, l = 0.0;
            for (int c = 0; c < chunks; ++c) m = fmax(m, jobs[h * chunks + c].m[i]);
            memset(acc, 0, sizeof(double) * D);
            for (int c = 0; c < chunks; ++c) {
                const attn_job* J = &jobs[h * chunks + c];
                if (J->m[i] == -INFINITY) continue;
                const double w = exp(J->m[i] - m);
                l += w * J->l[i];
                for (int d = 0; d < D; ++d) acc[d] += w * J->o[(size_t)i * D + d];
            }
            const int t = i / G, g = i % G;
            const size_t at = (size_t)t * q_heads + h * G + g;
            if (part_m) {
                part_m[at] = (float)m;
                part_l[at] = (float)l;
                for (int d = 0; d < D; ++d) part_o[at * D + d] = (float)acc[d];
            }
            for (int d = 0; d < D; ++d) orow[d] = l > 0.0 ? (float)(acc[d] / l) : 0.0f;
            kvo_hadamard(orow, D);
            memcpy(out + at * D, orow, sizeof(float) * D);
        }
    for (int j = 0; j < njobs; ++j) { free(jobs[j].m); free(jobs[j].l); free(jobs[j].o); }
    free(jobs); free(th); free(acc); free(orow); free(qrot);
}

/* Merge R partial sets (m, l, o_rot) per row by log-sum-exp, normalise, rotate back.
 * parts_*: [R][rows] / [R][rows][D]; out fp32 [rows][D]. */
void kvo_merge_partials(const float* parts_m, const float* parts_l, const float* parts_o, int R, int rows, int head_dim,
                        float* out) {
    const int D = head_dim;
    double* acc = malloc(sizeof(double) * D);
    for (int i = 0; i < rows; ++i) {
        double m = -INFINITY, l = 0.0;
        for (int r = 0; r < R; ++r) m = fmax(m, (double)parts_m[(size_t)r * rows + i]);
        memset(acc, 0, sizeof(double) * D);
        for (int r = 0; r < R; ++r) {
            const double mr = parts_m[(size_t)r * rows + i];
            if (mr == -INFINITY) continue;
            const double w = exp(mr - m);
            l += w * parts_l[(size_t)r * rows + i];
            for (int d = 0; d < D; ++d) acc[d] += w * parts_o[((size_t)r * rows + i) * D + d];
        }
        float* o = out + (size_t)i * D;
        for (int d = 0; d < D; ++d) o[d] = l > 0.0 ? (float)(acc[d] / l) : 0.0f;
        kvo_hadamard(o, D);
    }
    free(acc);
}
