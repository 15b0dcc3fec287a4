// kvb_attn.cu -- paged split-K attention over the quantised cache for 1..8 query tokens (decode, MTP
// verify), de-quantisation fused into the QK and PV loops.  head_dim 128.
//
// Grid (splits, kv heads, row blocks).  A CTA owns one KV head, one contiguous range of sealed pages and a block
// of up to 16 GQA-merged query rows (row = token * G + q head within the KV head); the last split of a head also
// reads the open tile, whose rows are still un-quantised fp16 in the stage.  Inside a CTA each of the 12 warps
// streams its own sub-range of pages through a private ring of three 4 KB slots in shared memory filled by bulk
// async copies (one mbarrier per slot) and never synchronises with another warp until the final merge.  A page
// arrives as two chunks: its K codes together with a small header (the page's V scale rows; its K scale rows when
// it is the first page of a tile the warp sees), then its V codes as four 1 KB sub-blocks, each shifted 16 bytes
// further, which makes the transposing ldmatrix reads of the V codes free of bank conflicts.  A slot is refilled
// as soon as its chunk has been consumed, so two thirds of a warp's ring are in flight at any time.
//
// Math per page (quantised-domain identities, no per-element de-quantisation), all on the int8 tensor path:
//   logit[r][j] = sum_d (q'[r][d] * scale_K[d]) * code_K[j][d]  +  sum_d q'[r][d] * zp_K[d]
//   o[r][d]    += sum_j (p[r][j] * scale_V[j]) * code_V[j][d]   +  sum_j p[r][j] * zp_V[j]
// with q' = H q * softmax_scale * log2(e).  Both contractions are mma.sync m16n8k32 (u8 x s8/u8 -> s32) with
// the KEYS (QK) and the DIMS (PV) on the 16-wide M side and the GQA-merged query rows on the 8-wide N side:
//   * QK: q' * scale_K is quantised per query row to 16 bits = a signed high and an unsigned low byte; the
//     packed code bytes feed the MMA as they lie in the page (byte & 0x0F = even dim, byte & 0xF0 = 16 x odd
//     dim), the four integer partial sums recombine exactly in int32.
//   * PV: p (relative to the row maximum of THIS page, so p <= 1) times scale_V is quantised to 16 bits = two
//     unsigned bytes; V codes are transposed to "four keys of one dim per register" by ldmatrix.trans plus one
//     byte permute and one AND per register; the integer sums of the page are converted once per page and
//     enter the running fp32 accumulators with the weight exp2(page max - running max).
// The page-local reference keeps 16 significant bits below each page's own maximum, whatever the global one is.
#include <algorithm>
#include <climits>
#include <cstddef>
#include <cstdlib>

#include "kvb_common.cuh"
#include "kvb_ptx.cuh"

namespace kvb {
namespace {

constexpr int D = 128;
constexpr int kWarpsDecode = 16;    // warps per CTA for up to 8 merged query rows (one N block per warp): 128 registers per thread
constexpr int kWarpsWide = 8;       // ... for 9..16 merged rows (two N blocks per warp: twice the accumulators): 255 registers
constexpr int kRows = 16;           // query rows per CTA: one or two 8-row N blocks
constexpr int kChunkBytes = kPage * (D / 2);  // 4096: the K or the V codes of one page
#ifndef KVB_V_SHIFT
#define KVB_V_SHIFT 16
#endif
constexpr int kVShift = KVB_V_SHIFT;  // 16: V codes lie as four sub-blocks of 16 keys, each shifted 16 bytes further (conflict-free ldmatrix, four copies); 0: one copy
constexpr int kVSub = 1024 + kVShift;  // sub-block a at a * kVSub: key k at k * 64 + kVShift * (k / 16)
constexpr int kSlotBytes = 4224;    // 4096 + 48 bytes of sub-block shifts, rounded up to 128
#ifndef KVB_SLOTS
#define KVB_SLOTS 2
#endif
constexpr int kSlots = KVB_SLOTS;   // ring slots per warp: the chunk in work and the next one(s) in flight
constexpr int kHdrs = KVB_SLOTS;            // header buffers per warp (a header lives from the issue of its page's K chunk to the end of the page)
constexpr int kHdrV = 512, kHdrK = 640, kHdrBytes = kHdrV + kHdrK;  // V scale rows of the page, then (first page of a tile) the K scale rows
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kMagic = 12582912.0f;   // 1.5 * 2^23: x + kMagic has round(x) in its low mantissa bits (|x| < 2^22)
constexpr float kPMax = 65000.0f;       // largest 16-bit weight (a margin below 65535 absorbs the rounding of the factor)
constexpr int kTabPad = 4;          // the per-dim tables are padded by 4 floats per 32 dims: the four 32-dim chunks a warp reads at once fall in different banks

struct AttnParams {
    LayerView L;
    const uint16_t* q;   // [T][q_heads][D]
    const int32_t* pos;  // [T] absolute positions of the query tokens (device)
    const int32_t* total_pos;  // position of the newest token in the cache (kv_total = *total_pos + 1)
    int T;
    float scale_log2;    // softmax scale * log2(e)
    int nsplit;          // CTAs over the sealed tiles of a head; the last one also reads the open tile
    int block_rows;      // GQA-merged query rows per row block (grid z): 8 (one 8-row block per warp) or 16 (two)
    int key_begin, key_end;
    float* ws_m;         // [H][Z][nsplit][16]
    float* ws_l;
    float* ws_o;         // [H][Z][nsplit][16][D]
};

struct __align__(128) WarpRing {
    uint8_t slots[kSlots][kSlotBytes];
    uint8_t hdr[kHdrs][kHdrBytes];
    float scale_k[D + 4 * kTabPad], zp_k[D + 4 * kTabPad];  // per-dim scale / zero point of K for the tile in work: dim d at d + kTabPad * (d / 32)
    uint64_t bars[kSlots];      // completes when the copies of the chunk in the slot have landed
};

template <int W> struct __align__(128) AttnSmem {
    WarpRing ring[W];
    float4 qfrag[2][8][32];  // q' in per-lane fragment order: [row half][j][lane] = dims 32t+4j..+3 of row g(+8)
    int row_pos[kRows];
};

// Per-thread state of the running softmax.  Lane (g, t) owns query rows 8 nb + 2t, 2t+1 of n-block nb and dims
// 32 db + 4g + i (db, i < 4):  o[nb][db][xy][c] is dim 32 db + 4g + xy + 2 (c >> 1), row 8 nb + 2t + (c & 1) -- the
// accumulator layout of the two MMAs per 32-dim block (xy = 0: even dims, 1: odd dims).  l and z are partial over the
// lane's keys; everything is relative to the running maximum m (log2 units).
template <int NB> struct Acc {
    float o[NB][4][2][4];
    float m[NB][2], l[NB][2], z[NB][2];
};

// B fragments of (q')^T per n-block and k-block (b0, b1), high and low fp16 parts: the open tile's rows are fp16.
template <int NB> struct QFrag {
    uint32_t hi[NB][8][2];
    uint32_t lo[NB][8][2];
};

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(p)));
}
// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8 | u8, col)
__device__ __forceinline__ void imma_us(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void imma_uu(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same with a zero accumulator: starts a sum without a register clear.
__device__ __forceinline__ void imma_us0(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_uu0(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Q-side fragments for the open tile from q' (shared memory, fragment order).  Lane (g, t) prepares row 8 nb + g, dims
// 32t .. 32t+31 in natural pairs (2e, 2e+1), split into an fp16 high and low part so the product keeps fp32 accuracy.
template <int NB, typename Smem>
__device__ __forceinline__ void build_qfrag(const Smem& sm, int lane, QFrag<NB>& f) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 qv = sm.qfrag[nb][j][lane];
            const float x[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int h = 0; h < 2; ++h) {  // dims 4j + 2h, +1 of the lane's 32: B register h of 16-dim k-block j
                const uint32_t hi = pack_half2(x[2 * h], x[2 * h + 1]);
                const float2 hf = unpack_half2(hi);
                f.hi[nb][j][h] = hi;
                f.lo[nb][j][h] = pack_half2(x[2 * h] - hf.x, x[2 * h + 1] - hf.y);
            }
        }
    }
}

// Integer form of (q' * scale_K)^T for the quantised pages: each row is scaled to 16-bit integers
// (row scale f = max|.| / 32639), Qi = 256 hi + lo with hi = Qi >> 8 signed and lo = Qi & 255 unsigned, so that the
// key side can feed its packed code bytes to the int8 tensor path without unpacking nibbles: with L = byte & 0x0F
// (even dim) and H = byte & 0xF0 (16 x odd dim),   sum_d Qi[d] code[d] = sum_b Qi[2b] L_b + (1/16) sum_b Qi[2b+1] H_b.
// b[nb][kb][part][digit] holds the B fragments (b0, b1) of 32-byte k-block kb: part 0 = even dims, 1 = odd dims;
// digit 0 = high (s8), 1 = low (u8).  The two bytes are read straight out of the float kMagic + Qi.
template <int NB> struct QInt {
    uint32_t b[NB][2][2][2][2];
    float f[NB][2];   // row scale / 16 of the lane's rows 2t, 2t+1
    float qz[NB][2];  // sum_d q'[row][d] * zp_K[d]
};

template <int NB, typename Smem>
__device__ __forceinline__ void build_qint(const Smem& sm, const WarpRing& R, int lane, QInt<NB>& f) {
    const int t = lane & 3;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        float qs[32];
        float qz = 0.0f, amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 qv = sm.qfrag[nb][j][lane];
            const float4 ks = *reinterpret_cast<const float4*>(&R.scale_k[(32 + kTabPad) * t + 4 * j]);
            const float4 kz = *reinterpret_cast<const float4*>(&R.zp_k[(32 + kTabPad) * t + 4 * j]);
            qs[4 * j + 0] = qv.x * ks.x; qs[4 * j + 1] = qv.y * ks.y;
            qs[4 * j + 2] = qv.z * ks.z; qs[4 * j + 3] = qv.w * ks.w;
            qz = fmaf(qv.x, kz.x, qz); qz = fmaf(qv.y, kz.y, qz);
            qz = fmaf(qv.z, kz.z, qz); qz = fmaf(qv.w, kz.w, qz);
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(qs[4 * j]), fabsf(qs[4 * j + 1]))), fmaxf(fabsf(qs[4 * j + 2]), fabsf(qs[4 * j + 3])));
        }
        qz += __shfl_xor_sync(0xffffffffu, qz, 1);
        qz += __shfl_xor_sync(0xffffffffu, qz, 2);  // every lane of group g now holds qz of row 8 nb + g
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float fr = amax > 0.0f ? amax * (1.0f / 32639.0f) : 1.0f, inv = amax > 0.0f ? 32639.0f / amax : 0.0f;
        f.qz[nb][0] = __shfl_sync(0xffffffffu, qz, 8 * t);      // row 2t   lives in lanes 4 * (2t) ..
        f.qz[nb][1] = __shfl_sync(0xffffffffu, qz, 8 * t + 4);  // row 2t+1 lives in lanes 4 * (2t+1) ..
        f.f[nb][0] = __shfl_sync(0xffffffffu, fr, 8 * t) * 0.0625f;
        f.f[nb][1] = __shfl_sync(0xffffffffu, fr, 8 * t + 4) * 0.0625f;
        uint32_t x[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) x[i] = __float_as_uint(fmaf(qs[i], inv, kMagic));  // low 16 bits: Qi (two's complement)
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
            for (int part = 0; part < 2; ++part)
#pragma unroll
                for (int r = 0; r < 2; ++r) {  // b0: local dims 16 kb + 2j + part, b1: +8
                    const int i0 = 16 * kb + 8 * r + part;
                    const uint32_t t01 = prmt(x[i0], x[i0 + 2], 0x5140), t23 = prmt(x[i0 + 4], x[i0 + 6], 0x5140);  // [lo lo hi hi]
                    f.b[nb][kb][part][1][r] = prmt(t01, t23, 0x5410);
                    f.b[nb][kb][part][0][r] = prmt(t01, t23, 0x7632);
                }
    }
}

// Scale rows of K -> per-dim tables in natural dim order, fp32.  A page row is 5 halves
// [scale(2r) scale(2r+1) zp(2r) zp(2r+1) other(r)]; lane l converts rows 2l and 2l+1 (20 bytes): dims 4l .. 4l+3.
__device__ __forceinline__ void transpose_k_scale(const uint8_t* kscale_rows, WarpRing& R, int lane) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(kscale_rows + 20 * lane);
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = w[4];
    // halves: w0 = s(4l) s(4l+1) | w1 = z(4l) z(4l+1) | w2 = o(2l) s(4l+2) | w3 = s(4l+3) z(4l+2) | w4 = z(4l+3) o(2l+1)
    const float2 s01 = unpack_half2(w0), s23 = unpack_half2(prmt(w2, w3, 0x5432));
    const float2 z01 = unpack_half2(w1), z23 = unpack_half2(prmt(w3, w4, 0x5432));
    *reinterpret_cast<float4*>(&R.scale_k[4 * lane + kTabPad * (lane >> 3)]) = make_float4(s01.x, s01.y, s23.x, s23.y);
    *reinterpret_cast<float4*>(&R.zp_k[4 * lane + kTabPad * (lane >> 3)]) = make_float4(z01.x, z01.y, z23.x, z23.y);
}

// Running maximum moves to mnew: rescale the accumulators of one row pair.  alpha = exp2(m_old - m_new).
template <int NB>
__device__ __forceinline__ void rescale(Acc<NB>& acc, const float (&alpha)[NB][2]) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int db = 0; db < 4; ++db)
#pragma unroll
            for (int xy = 0; xy < 2; ++xy)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc.o[nb][db][xy][c] *= alpha[nb][c & 1];
        acc.l[nb][0] *= alpha[nb][0]; acc.z[nb][0] *= alpha[nb][0];
        acc.l[nb][1] *= alpha[nb][1]; acc.z[nb][1] *= alpha[nb][1];
    }
}

// 16 keys of the open tile, read un-quantised (fp16, rotated) straight from the stage.
// krow/vrow point at the first of the 16 stage rows of this head (row stride D halves).
template <int NB>
__device__ __forceinline__ void process_stage_group(const __half* krow, const __half* vrow, const QFrag<NB>& qf,
                                                    Acc<NB>& acc, int lane, int first_pos, int kv_total,
                                                    const int (&row_lim)[NB][2], int key_begin, int key_end) {
    const int g = lane >> 2, t = lane & 3;
    float s[NB][4];
    {
        const __half* ka = krow + g * D + 32 * t;
        const __half* kb = krow + (8 + g) * D + 32 * t;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 a = *reinterpret_cast<const uint4*>(ka + 8 * i), b = *reinterpret_cast<const uint4*>(kb + 8 * i);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                mma16816(s[nb], a.x, b.x, a.y, b.y, qf.hi[nb][2 * i][0], qf.hi[nb][2 * i][1]);
                mma16816(s[nb], a.z, b.z, a.w, b.w, qf.hi[nb][2 * i + 1][0], qf.hi[nb][2 * i + 1][1]);
                mma16816(s[nb], a.x, b.x, a.y, b.y, qf.lo[nb][2 * i][0], qf.lo[nb][2 * i][1]);
                mma16816(s[nb], a.z, b.z, a.w, b.w, qf.lo[nb][2 * i + 1][0], qf.lo[nb][2 * i + 1][1]);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int p = first_pos + g + (e >> 1) * 8;
            const bool out = p >= kv_total || p < key_begin || p >= key_end;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
                if (out || p > row_lim[nb][e & 1]) s[nb][e] = -INFINITY;
        }
    }
    // online softmax over these 16 keys
    float alpha[NB][2], muse[NB][2];
    bool moved = false;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float mx = fmaxf(s[nb][j], s[nb][2 + j]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float mnew = fmaxf(acc.m[nb][j], mx);
            moved |= mnew > acc.m[nb][j];
            muse[nb][j] = mnew == -INFINITY ? 0.0f : mnew;
            alpha[nb][j] = fast_exp2(acc.m[nb][j] - muse[nb][j]);
            acc.m[nb][j] = mnew;
        }
    }
    if (__any_sync(0xffffffffu, moved)) rescale<NB>(acc, alpha);
    uint32_t b0[NB], b1[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            s[nb][e] = fast_exp2(s[nb][e] - muse[nb][e & 1]);
            acc.l[nb][e & 1] += s[nb][e];
        }
        b0[nb] = movmatrix_trans(pack_half2(s[nb][0], s[nb][1]));  // -> (row g; keys 2t, 2t+1)
        b1[nb] = movmatrix_trans(pack_half2(s[nb][2], s[nb][3]));  // -> (row g; keys 2t+8, 2t+9)
    }
    // A = V^T: the lane supplies dims 32 db + 4g .. +3 of keys 2t, 2t+1, 2t+8, 2t+9.  Keys at or beyond kv_total hold
    // stale rows: their p is exactly 0; zero V there so 0 * inf cannot appear.
#pragma unroll
    for (int db = 0; db < 4; ++db) {
        uint2 v[4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            const int key = 2 * t + (kk & 1) + (kk >> 1) * 8;
            const bool live = first_pos + key < kv_total;
            v[kk] = live ? *reinterpret_cast<const uint2*>(vrow + key * D + 32 * db + 4 * g) : make_uint2(0u, 0u);
        }
        const uint32_t x0 = prmt(v[0].x, v[1].x, 0x5410), x1 = prmt(v[0].y, v[1].y, 0x5410);  // dims 4g, 4g+2 of keys 2t, 2t+1
        const uint32_t x2 = prmt(v[2].x, v[3].x, 0x5410), x3 = prmt(v[2].y, v[3].y, 0x5410);  // ... of keys 2t+8, 2t+9
        const uint32_t y0 = prmt(v[0].x, v[1].x, 0x7632), y1 = prmt(v[0].y, v[1].y, 0x7632);  // dims 4g+1, 4g+3
        const uint32_t y2 = prmt(v[2].x, v[3].x, 0x7632), y3 = prmt(v[2].y, v[3].y, 0x7632);
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            mma16816(acc.o[nb][db][0], x0, x1, x2, x3, b0[nb], b1[nb]);
            mma16816(acc.o[nb][db][1], y0, y1, y2, y3, b0[nb], b1[nb]);
        }
    }
}

// The work of one CTA: split `split` of KV head `head`, row block `zb`; its partial goes to rows pidx .. pidx + 15 of
// the workspace.  NB = 8-row blocks of query rows per warp.  A pass = one page: its 64 logits per row are held at
// once.  Within a page the keys are taken in a fixed permutation (see key_lo below) that lets the QK accumulators
// feed the PV operands of the shifted V sub-blocks without any re-ordering.
// kOther: the cache was written with variance balancing (Sinkhorn iterations > 0): every key carries a factor other_K on
// its logits and every dim of a tile a factor other_V on its output (reference kvarn128_codec.cuh:331-347); both are 1
// otherwise and the arithmetic for them is compiled out.
template <int NB, int W, bool kOther = false>
__device__ __forceinline__ void attn_cta(const AttnParams& P, int split, int head, int zb, int64_t pidx) {
    constexpr int kWarps = W, kThreads = W * 32;
    constexpr int kGroups = kPage / 16;            // 16-key groups of a page
    constexpr int kDimSweeps = 4;                  // the V chunk of a page is swept one 32-dim block at a time: a quarter of the integer accumulators live (measured 1.6 % faster than two halves)
    constexpr int kORow = D + 4, kWarpFloats = 3 * kRows + kRows * kORow;  // merge buffer of a warp: m, l, z per row, then o
    static_assert(kWarps * kWarpFloats * 4 <= static_cast<int>(sizeof(WarpRing)) * kWarps, "merge buffer exceeds the rings");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    AttnSmem<W>& sm = *reinterpret_cast<AttnSmem<W>*>(smem_raw);
    const LayerView& L = P.L;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = L.q_heads / L.kv_heads;
    WarpRing& R = sm.ring[warp];
    // ---- order of the first memory requests: the few bytes everything waits for (positions, q rows, page table
    //      entries) go out first, then the first chunk of every warp, then -- after the rotation of q -- the rest of
    //      the ring.
    constexpr int kQIter = (8 * NB + W - 1) / W;  // warp w prepares rows w, w + W, ... of the block
    uint16_t qraw[kQIter][4];
    int qpos[kQIter];
#pragma unroll
    for (int i = 0; i < kQIter; ++i) {
        qraw[i][0] = qraw[i][1] = qraw[i][2] = qraw[i][3] = 0;
        qpos[i] = -1;
        const int r = warp + W * i;
        if (r < 8 * NB) {
            const int Rr = zb * P.block_rows + r, tq = Rr / G, gq = Rr % G;
            if (tq < P.T) {
                const uint16_t* qrow = P.q + (static_cast<int64_t>(tq) * L.q_heads + head * G + gq) * D;
#pragma unroll
                for (int j = 0; j < 4; ++j) qraw[i][j] = qrow[lane + 32 * j];
                qpos[i] = P.pos[tq];
            }
        }
    }
    const int kv_total = *P.total_pos + 1;
    const int key_end = min(P.key_end, kv_total), key_begin = max(P.key_begin, 0);
    const int sealed_pages = 2 * (kv_total / kTile);

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kSlots; ++s) mbar_init(&R.bars[s], 1);
        mbar_fence_init();
    }
    __syncwarp();
    // pages of this CTA, then of this warp
    int w0, w1;
    {
        const int pb = min(key_begin / kPage, sealed_pages), pe = min((key_end + kPage - 1) / kPage, sealed_pages);
        const int n = max(pe - pb, 0);
        const int c0 = pb + static_cast<int>(static_cast<int64_t>(n) * split / P.nsplit);
        const int c1 = pb + static_cast<int>(static_cast<int64_t>(n) * (split + 1) / P.nsplit);
        w0 = c0 + (c1 - c0) * warp / kWarps;
        w1 = c0 + (c1 - c0) * (warp + 1) / kWarps;
    }
    const int npages = w1 - w0, nchunks = 2 * npages;
    // ---- the refill side of the ring.  Chunk n of this warp is page w0 + n / 2: even n = K codes + header, odd n = V
    //      codes.  Page table entries are read 32 at a time, one per lane, a batch ahead of the chunk being issued (the
    //      only place page ids are needed): lane l of `ids` knows logical page ids_base + l, `ids_next` the 32 after.
    //      A page whose table entry is bad (-1) gets no copies and its pass is skipped; the error word says why.
    const int32_t* tbl = L.table();
    auto load_ids = [&](int base) -> int32_t { return base + lane < w1 ? L.page_of(tbl, base + lane) : -1; };
    int ids_base = w0;
    int32_t ids = npages > 0 ? load_ids(ids_base) : -1, ids_next = npages > 0 ? load_ids(ids_base + 32) : -1;
    // byte offsets of this head inside a page of each plane, and the planes' page strides
    const uint32_t code_stride = static_cast<uint32_t>(L.kv_heads) * kChunkBytes;
    const uint8_t* const kc = L.k_code + static_cast<size_t>(head) * kChunkBytes;
    const uint8_t* const vc = L.v_code + static_cast<size_t>(head) * kChunkBytes;
    const uint8_t* const ksr = reinterpret_cast<const uint8_t*>(L.k_scale) + static_cast<size_t>(head) * kHdrK;
    const uint8_t* const vsr = reinterpret_cast<const uint8_t*>(L.v_scale) + static_cast<size_t>(head) * kHdrV;
    uint32_t live = 0;       // bit s: a copy is in flight into / has landed in slot s
    int32_t issue_pid = -1;  // page id of the page whose K chunk was issued last (its V chunk comes next)
    int n_issued = 0;
    auto issue_next = [&](int slot) {  // whole warp; chunk n_issued goes into `slot`
        const int n = n_issued++;
        if ((n & 1) == 0) {
            const int lp = w0 + (n >> 1);
            if (lp - ids_base == 32) {
                ids = ids_next;
                ids_base += 32;
                ids_next = load_ids(ids_base + 32);
            }
            issue_pid = __shfl_sync(0xffffffffu, ids, lp - ids_base);
        }
        const int32_t pid = issue_pid;
        if (pid < 0) { live &= ~(1u << slot); return; }
        live |= 1u << slot;
        if (lane == 0) {
            uint8_t* dst = R.slots[slot];
            if (n & 1) {
                const uint8_t* src = vc + static_cast<size_t>(pid) * code_stride;
                mbar_expect_tx(&R.bars[slot], kChunkBytes);
                if constexpr (kVShift == 0) {
                    bulk_g2s(dst, src, kChunkBytes, &R.bars[slot]);
                } else {
#pragma unroll
                    for (int a = 0; a < 4; ++a) bulk_g2s(dst + a * kVSub, src + a * 1024, 1024, &R.bars[slot]);
                }
            } else {
                const int lp = w0 + (n >> 1);
                const bool with_k = kOther || (lp & 1) == 0 || lp == w0;  // K scale rows: with the first page of a tile this warp reads (their fifth column is other_K of the page's own keys: always, when it is not 1)
                uint8_t* hdr = R.hdr[(n >> 1) % kHdrs];
                mbar_expect_tx(&R.bars[slot], kChunkBytes + kHdrV + (with_k ? kHdrK : 0));
                bulk_g2s(dst, kc + static_cast<size_t>(pid) * code_stride, kChunkBytes, &R.bars[slot]);
                bulk_g2s(hdr, vsr + static_cast<size_t>(pid) * (static_cast<uint32_t>(L.kv_heads) * kHdrV), kHdrV, &R.bars[slot]);
                if (with_k) bulk_g2s(hdr + kHdrV, ksr + static_cast<size_t>(pid) * (static_cast<uint32_t>(L.kv_heads) * kHdrK), kHdrK, &R.bars[slot]);
            }
        }
    };
    if (nchunks > 0) issue_next(0);

    // ---- q' = H q * scale * log2(e) for the rows of this block, stored in fragment order
#pragma unroll
    for (int i = 0; i < kQIter; ++i) {
        const int r = warp + W * i;
        if (r < 8 * NB) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = L.dtype == KVB_DTYPE_BF16 ? in_to_f32<true>(qraw[i][j]) : in_to_f32<false>(qraw[i][j]);
            hadamard_warp<D>(v, lane);  // rows beyond T are zeros and stay zeros
            if (lane == 0) sm.row_pos[r] = qpos[i];
            float* dst = reinterpret_cast<float*>(sm.qfrag);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int d = lane + 32 * j;  // -> lane' = (r%8)*4 + d/32, slot j' = (d%32)/4, component d%4
                dst[(((r >> 3) * 8 + ((d & 31) >> 2)) * 32 + (r & 7) * 4 + (d >> 5)) * 4 + (d & 3)] = v[j] * P.scale_log2;
            }
        }
    }
    while (n_issued < kSlots && n_issued < nchunks) issue_next(n_issued);
    launch_dependents();  // the reduce kernel may take its place on the SMs; it waits for this grid's completion
    __syncthreads();

    const int g = lane >> 2, t = lane & 3;
    int row_lim[NB][2];
    int min_lim = INT_MAX;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        row_lim[nb][0] = sm.row_pos[8 * nb + 2 * t];
        row_lim[nb][1] = sm.row_pos[8 * nb + 2 * t + 1];
    }
    for (int r = 0; r < 8 * NB; ++r)
        if (sm.row_pos[r] >= 0) min_lim = min(min_lim, sm.row_pos[r]);

    Acc<NB> acc;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int db = 0; db < 4; ++db)
#pragma unroll
            for (int xy = 0; xy < 2; ++xy)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc.o[nb][db][xy][c] = 0.0f;
        acc.m[nb][0] = acc.m[nb][1] = -INFINITY;
        acc.l[nb][0] = acc.l[nb][1] = acc.z[nb][0] = acc.z[nb][1] = 0.0f;
    }

    // ---- open tile (last split of the head): its eight 16-key groups are dealt to the consumer warps, un-quantised,
    //      from the stage; the loads are in flight together with the first chunks of the ring
    if (split == P.nsplit - 1) {
        const int tile = kv_total / kTile, base = tile * kTile;
        for (int grp = warp; grp < 8; grp += W) {
            const int first = base + 16 * grp;
            if (first < key_end && first + 16 > key_begin && first < kv_total) {
                QFrag<NB> qf;
                build_qfrag<NB>(sm, lane, qf);
                process_stage_group<NB>(L.stage_row(0, tile & 1, head, 16 * grp), L.stage_row(1, tile & 1, head, 16 * grp), qf,
                                        acc, lane, first, kv_total, row_lim, key_begin, key_end);
            }
        }
    }

    // ---- sealed pages
    bool timed_out = false;
    int slot = 0;          // slot of the oldest chunk not yet released
    uint32_t phases = 0;   // bit s: parity the next wait on slot s expects
    // Wait for the chunk in slot s (bounded).  The first probe usually succeeds; a lane that has to keep probing finds
    // the barrier complete as soon as any lane has, so the verdict is the same in every lane without a vote.
    auto wait_slot = [&](int s) {
        if (timed_out) return;
        if (!mbar_try_wait(&R.bars[s], (phases >> s) & 1u) && !mbar_wait_lane_bounded(&R.bars[s], (phases >> s) & 1u)) timed_out = true;
    };
    auto release_chunk = [&](bool was_live) {  // the chunk in `slot` has been read by every lane: refill the slot, advance
        if (was_live) phases ^= 1u << slot;
        live &= ~(1u << slot);
        __syncwarp();
        if (n_issued < nchunks) {
            if (lane == 0) fence_proxy_async();  // generic-proxy reads of the slot are ordered before the refill
            issue_next(slot);
        }
        slot = slot + 1 == kSlots ? 0 : slot + 1;
    };
    // Key order inside a page: m-row i of 16-key group grp (lane g holds rows g and g + 8) is key
    //   16 ((i & 7) >> 1) + 8 (grp >> 1) + 4 (grp & 1) + 2 (i >> 3) + (i & 1)
    // so that, after the accumulator -> operand transposition, the weights of a group line up with the keys ldmatrix
    // gathers from the four shifted sub-blocks of the V chunk.
    const int key_lo = 16 * (g >> 1) + (g & 1);  // + 8 (grp >> 1) + 4 (grp & 1): key of m-row g; m-row g + 8 is 2 keys further

    QInt<NB> qi;
    float ov[4][2][2];  // kOther: other_V of dims 32 db + 4g + xy + 2h of the current tile
    int cur_tile = -1;
    for (int pi = 0; pi < npages; ++pi) {
        const int lp = w0 + pi;
        timed_out = __any_sync(0xffffffffu, timed_out);  // one verdict for the warp before anything branches on it
        if (timed_out) break;
        if (!((live >> slot) & 1u)) {  // a page that could not be addressed: nothing was copied, nothing is read
            release_chunk(false);
            release_chunk(false);
            continue;
        }
        // ---- K chunk + header
        wait_slot(slot);
        const uint8_t* hdr = R.hdr[pi % kHdrs];
        if ((lp >> 1) != cur_tile) {  // per-dim scale / zero point of K belong to the tile
            cur_tile = lp >> 1;
            __syncwarp();
            transpose_k_scale(hdr + kHdrV, R, lane);
            __syncwarp();
            build_qint<NB>(sm, R, lane, qi);
            if constexpr (kOther) {  // other_V of the lane's 16 dims: V scale row d / 2 starts with (other(d even), other(d odd))
#pragma unroll
                for (int db = 0; db < 4; ++db)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float2 o2 = unpack_half2(*reinterpret_cast<const uint32_t*>(hdr + (16 * db + 2 * g + h) * 8));
                        ov[db][0][h] = o2.x;
                        ov[db][1][h] = o2.y;
                    }
            }
        }
        const int first = lp * kPage;
        const bool need_mask = first + kPage - 1 > min_lim || first < key_begin || first + kPage > key_end;
        // ---- QK: integer logits of the page
        int tot[NB][kGroups][4];
        {
            const uint8_t* ch = R.slots[slot] + key_lo * 64 + 16 * t;
#pragma unroll
            for (int grp = 0; grp < kGroups; ++grp) {
                const int koff = (8 * (grp >> 1) + 4 * (grp & 1)) * 64;
                const uint4 ka = *reinterpret_cast<const uint4*>(ch + koff);
                const uint4 kb8 = *reinterpret_cast<const uint4*>(ch + koff + 2 * 64);
                const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w}, wb[4] = {kb8.x, kb8.y, kb8.z, kb8.w};
                int ceh[NB][4], cel[NB][4], coh[NB][4], col[NB][4];
#pragma unroll
                for (int kb = 0; kb < 2; ++kb) {
                    const uint32_t l0 = wa[2 * kb] & 0x0F0F0F0Fu, l1 = wb[2 * kb] & 0x0F0F0F0Fu, l2 = wa[2 * kb + 1] & 0x0F0F0F0Fu,
                                   l3 = wb[2 * kb + 1] & 0x0F0F0F0Fu;
                    const uint32_t h0 = wa[2 * kb] & 0xF0F0F0F0u, h1 = wb[2 * kb] & 0xF0F0F0F0u, h2 = wa[2 * kb + 1] & 0xF0F0F0F0u,
                                   h3 = wb[2 * kb + 1] & 0xF0F0F0F0u;
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        if (kb == 0) {
                            imma_us0(ceh[nb], l0, l1, l2, l3, qi.b[nb][kb][0][0][0], qi.b[nb][kb][0][0][1]);
                            imma_uu0(cel[nb], l0, l1, l2, l3, qi.b[nb][kb][0][1][0], qi.b[nb][kb][0][1][1]);
                            imma_us0(coh[nb], h0, h1, h2, h3, qi.b[nb][kb][1][0][0], qi.b[nb][kb][1][0][1]);
                            imma_uu0(col[nb], h0, h1, h2, h3, qi.b[nb][kb][1][1][0], qi.b[nb][kb][1][1][1]);
                        } else {
                            imma_us(ceh[nb], l0, l1, l2, l3, qi.b[nb][kb][0][0][0], qi.b[nb][kb][0][0][1]);
                            imma_uu(cel[nb], l0, l1, l2, l3, qi.b[nb][kb][0][1][0], qi.b[nb][kb][0][1][1]);
                            imma_us(coh[nb], h0, h1, h2, h3, qi.b[nb][kb][1][0][0], qi.b[nb][kb][1][0][1]);
                            imma_uu(col[nb], h0, h1, h2, h3, qi.b[nb][kb][1][1][0], qi.b[nb][kb][1][1][1]);
                        }
                    }
                }
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; ++e)  // 16 * sum = 256 (16 even_hi + odd_hi) + (16 even_lo + odd_lo); |.| < 2^31
                        tot[nb][grp][e] = ((ceh[nb][e] * 16 + coh[nb][e]) << 8) + (cel[nb][e] * 16 + col[nb][e]);
            }
        }
        release_chunk(true);
        if (need_mask) {  // keys a row may not see (causal limit, key range) leave the row maximum ...
#pragma unroll
            for (int grp = 0; grp < kGroups; ++grp)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int p = first + key_lo + 8 * (grp >> 1) + 4 * (grp & 1) + 2 * (e >> 1);
                    const bool out = p < key_begin || p >= key_end;
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb)
                        if (out || p > row_lim[nb][e & 1]) tot[nb][grp][e] = INT_MIN;
                }
        }
        // ---- softmax of the page relative to its own row maxima; weights of the page against the running state
        float wq[NB][2];     // weight of the integer sums of this page in the running accumulators
        float zfull[NB][2];  // kOther: sum over the page's keys of p * zp_V, weighted like the integer sums
        uint32_t bh[NB][kGroups], bl[NB][kGroups];  // 16-bit weights as B fragments: high and low bytes
        {
            // per-key scale of V: the largest of the page bounds p * scale_V; one factor for all rows
            float svmax = fmaxf(fabsf(__half2float(*reinterpret_cast<const __half*>(hdr + lane * 8 + 4))),
                                fabsf(__half2float(*reinterpret_cast<const __half*>(hdr + (lane + 32) * 8 + 4))));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) svmax = fmaxf(svmax, __shfl_xor_sync(0xffffffffu, svmax, o));
            const float F = svmax > 0.0f ? kPMax / svmax : 0.0f, invF = svmax * (1.0f / kPMax);
            float alpha[NB][2], wpass[NB][2], cst[NB][2];
            bool moved = false;
            float sl[NB][kGroups][4];  // logits relative to the page maximum (log2 units)
            if constexpr (kOther) {
                // logits = other_K(key) * (f * integer sum + qz): the page maximum is taken on the floats
                float ok[kGroups][2];
#pragma unroll
                for (int grp = 0; grp < kGroups; ++grp)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        ok[grp][h] = __half2float(*reinterpret_cast<const __half*>(hdr + kHdrV + (key_lo + 8 * (grp >> 1) + 4 * (grp & 1) + 2 * h) * 10 + 8));
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int grp = 0; grp < kGroups; ++grp)
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            sl[nb][grp][e] = tot[nb][grp][e] == INT_MIN ? -INFINITY
                                                                         : fmaf(static_cast<float>(tot[nb][grp][e]), qi.f[nb][e & 1], qi.qz[nb][e & 1]) * ok[grp][e >> 1];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        float mpass = -INFINITY;
#pragma unroll
                        for (int grp = 0; grp < kGroups; ++grp) mpass = fmaxf(mpass, fmaxf(sl[nb][grp][j], sl[nb][grp][2 + j]));
                        mpass = fmaxf(mpass, __shfl_xor_sync(0xffffffffu, mpass, 4));
                        mpass = fmaxf(mpass, __shfl_xor_sync(0xffffffffu, mpass, 8));
                        mpass = fmaxf(mpass, __shfl_xor_sync(0xffffffffu, mpass, 16));
                        const float mnew = fmaxf(acc.m[nb][j], mpass);
                        moved |= mnew > acc.m[nb][j];
                        const float muse = mnew == -INFINITY ? 0.0f : mnew;
                        alpha[nb][j] = fast_exp2(acc.m[nb][j] - muse);
                        wpass[nb][j] = fast_exp2(mpass - muse);
                        cst[nb][j] = mpass == -INFINITY ? 0.0f : mpass;
                        acc.m[nb][j] = mnew;
                        wq[nb][j] = wpass[nb][j] * invF;
                    }
                }
                if (__any_sync(0xffffffffu, moved)) rescale<NB>(acc, alpha);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int grp = 0; grp < kGroups; ++grp)
#pragma unroll
                        for (int e = 0; e < 4; ++e) sl[nb][grp][e] -= cst[nb][e & 1];  // masked keys stay at -inf
            } else {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    int mx = INT_MIN;
#pragma unroll
                    for (int grp = 0; grp < kGroups; ++grp) mx = max(mx, max(tot[nb][grp][j], tot[nb][grp][2 + j]));
                    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    const float mpass = mx == INT_MIN ? -INFINITY : fmaf(static_cast<float>(mx), qi.f[nb][j], qi.qz[nb][j]);
                    const float mnew = fmaxf(acc.m[nb][j], mpass);
                    moved |= mnew > acc.m[nb][j];
                    const float muse = mnew == -INFINITY ? 0.0f : mnew;
                    alpha[nb][j] = fast_exp2(acc.m[nb][j] - muse);
                    wpass[nb][j] = fast_exp2(mpass - muse);
                    cst[nb][j] = qi.qz[nb][j] - (mpass == -INFINITY ? 0.0f : mpass);
                    acc.m[nb][j] = mnew;
                    wq[nb][j] = wpass[nb][j] * invF;
                }
            }
            if (__any_sync(0xffffffffu, moved)) rescale<NB>(acc, alpha);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int grp = 0; grp < kGroups; ++grp)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sl[nb][grp][e] = fmaf(static_cast<float>(tot[nb][grp][e]), qi.f[nb][e & 1], cst[nb][e & 1]);
            if (need_mask) {  // ... and get weight exactly zero
#pragma unroll
                for (int grp = 0; grp < kGroups; ++grp)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int p = first + key_lo + 8 * (grp >> 1) + 4 * (grp & 1) + 2 * (e >> 1);
                        const bool out = p < key_begin || p >= key_end;
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb)
                            if (out || p > row_lim[nb][e & 1]) sl[nb][grp][e] = -INFINITY;
                    }
            }
            }
            float lp_[NB][2], zp_[NB][2];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) lp_[nb][0] = lp_[nb][1] = zp_[nb][0] = zp_[nb][1] = 0.0f;
            const uint8_t* vs = hdr + key_lo * 8 + 4;  // V scale rows are [other other scale zp] per key
#pragma unroll
            for (int grp = 0; grp < kGroups; ++grp) {
                const int koff = (8 * (grp >> 1) + 4 * (grp & 1)) * 8;
                const float2 sz0 = unpack_half2(*reinterpret_cast<const uint32_t*>(vs + koff));           // (scale, zp) of the key of m-row g
                const float2 sz1 = unpack_half2(*reinterpret_cast<const uint32_t*>(vs + koff + 2 * 8));   // ... of m-row g + 8
                const float sf0 = sz0.x * F, sf1 = sz1.x * F;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    float p[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        p[e] = fast_exp2(sl[nb][grp][e]);
                        lp_[nb][e & 1] += p[e];
                    }
                    zp_[nb][0] += p[0] * sz0.y + p[2] * sz1.y;
                    zp_[nb][1] += p[1] * sz0.y + p[3] * sz1.y;
                    // accumulator layout (m-row g; rows 2t, 2t+1) -> operand layout (row g; m-rows 2t, 2t+1 | 2t+8, 2t+9)
                    const uint32_t y0 = movmatrix_trans(prmt(__float_as_uint(fmaf(p[0], sf0, kMagic)), __float_as_uint(fmaf(p[1], sf0, kMagic)), 0x5410));
                    const uint32_t y1 = movmatrix_trans(prmt(__float_as_uint(fmaf(p[2], sf1, kMagic)), __float_as_uint(fmaf(p[3], sf1, kMagic)), 0x5410));
                    bl[nb][grp] = prmt(y0, y1, 0x6420);
                    bh[nb][grp] = prmt(y0, y1, 0x7531);
                }
            }
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    acc.l[nb][j] = fmaf(lp_[nb][j], wpass[nb][j], acc.l[nb][j]);
                    if constexpr (kOther) {  // the zero-point term takes other_V of the tile per dim: it enters the accumulators with the page
                        float zs = zp_[nb][j];
                        zs += __shfl_xor_sync(0xffffffffu, zs, 4);
                        zs += __shfl_xor_sync(0xffffffffu, zs, 8);
                        zs += __shfl_xor_sync(0xffffffffu, zs, 16);
                        zfull[nb][j] = zs * wpass[nb][j];
                    } else {
                        acc.z[nb][j] = fmaf(zp_[nb][j], wpass[nb][j], acc.z[nb][j]);
                    }
                }
        }
        // ---- PV on the int8 path.  Matrix i' of the page (8 rows) gathers keys 2i', 2i'+1 of each of the four sub-blocks:
        //      eight distinct 16-byte bank groups.  ldmatrix.trans hands lane (g, t) the code bytes of dims 32 db + 4g .. +3
        //      of keys 16t + 2i', +1; one byte permute gathers keys 16t + 8c + {0..3} (then + {4..7}) of a dim pair, one AND
        //      isolates the even dim (x) or 16 x the odd dim (y): the k slots of MMA c, matching groups 2c and 2c + 1.
        wait_slot(slot);
        {
            // lane L addresses row L & 7 of matrix L >> 3: key 16 ((L & 7) >> 1) + 2 (L >> 3) + (L & 1) (+ 8c), shifted with its sub-block
            const int vkey = 16 * ((lane & 7) >> 1) + 2 * (lane >> 3) + (lane & 1);
            const uint8_t* ch = R.slots[slot] + vkey * 64 + kVShift * (vkey >> 4);
#pragma unroll
            for (int sweep = 0; sweep < kDimSweeps; ++sweep) {
                constexpr int kDb = 4 / kDimSweeps;
                int ix[NB][kDb][2][2][4];  // [nb][db][xy][digit][c]
#pragma unroll
                for (int c = 0; c < 2; ++c) {  // 32-key halves of the page: keys 16t + 8c + {0..7}
#pragma unroll
                    for (int d = 0; d < kDb; ++d) {
                        const int db = sweep * kDb + d;
                        uint32_t r[4];
                        ldsm_x4_trans(r, ch + c * 8 * 64 + 16 * db);
                        const uint32_t u0 = prmt(r[0], r[1], 0x6420), v0 = prmt(r[0], r[1], 0x7531);
                        const uint32_t u1 = prmt(r[2], r[3], 0x6420), v1 = prmt(r[2], r[3], 0x7531);
                        const uint32_t ax0 = u0 & 0x0F0F0F0Fu, ax1 = v0 & 0x0F0F0F0Fu, ax2 = u1 & 0x0F0F0F0Fu, ax3 = v1 & 0x0F0F0F0Fu;
                        const uint32_t ay0 = u0 & 0xF0F0F0F0u, ay1 = v0 & 0xF0F0F0F0u, ay2 = u1 & 0xF0F0F0F0u, ay3 = v1 & 0xF0F0F0F0u;
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            if (c == 0) {
                                imma_uu0(ix[nb][d][0][0], ax0, ax1, ax2, ax3, bh[nb][0], bh[nb][1]);
                                imma_uu0(ix[nb][d][0][1], ax0, ax1, ax2, ax3, bl[nb][0], bl[nb][1]);
                                imma_uu0(ix[nb][d][1][0], ay0, ay1, ay2, ay3, bh[nb][0], bh[nb][1]);
                                imma_uu0(ix[nb][d][1][1], ay0, ay1, ay2, ay3, bl[nb][0], bl[nb][1]);
                            } else {
                                imma_uu(ix[nb][d][0][0], ax0, ax1, ax2, ax3, bh[nb][2], bh[nb][3]);
                                imma_uu(ix[nb][d][0][1], ax0, ax1, ax2, ax3, bl[nb][2], bl[nb][3]);
                                imma_uu(ix[nb][d][1][0], ay0, ay1, ay2, ay3, bh[nb][2], bh[nb][3]);
                                imma_uu(ix[nb][d][1][1], ay0, ay1, ay2, ay3, bl[nb][2], bl[nb][3]);
                            }
                        }
                    }
                }
                // ---- integer sums of the page -> running fp32 accumulators
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int d = 0; d < kDb; ++d)
#pragma unroll
                        for (int xy = 0; xy < 2; ++xy)
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const float v = static_cast<float>((ix[nb][d][xy][0][c] << 8) + ix[nb][d][xy][1][c]);
                                if constexpr (kOther) {  // (sum p code scale_V + sum p zp_V) * other_V(dim)
                                    const float tv = fmaf(v, xy ? wq[nb][c & 1] * 0.0625f : wq[nb][c & 1], zfull[nb][c & 1]);
                                    acc.o[nb][sweep * kDb + d][xy][c] = fmaf(tv, ov[sweep * kDb + d][xy][c >> 1], acc.o[nb][sweep * kDb + d][xy][c]);
                                } else {
                                    acc.o[nb][sweep * kDb + d][xy][c] = fmaf(v, xy ? wq[nb][c & 1] * 0.0625f : wq[nb][c & 1], acc.o[nb][sweep * kDb + d][xy][c]);
                                }
                            }
            }
        }
        release_chunk(true);
    }
    if (__any_sync(0xffffffffu, timed_out)) {
        if (lane == 0) L.flag(KVB_ERR_WAIT_TIMEOUT);
        // copies already issued must land before the CTA's shared memory is released: one more bounded wait each
        for (int s2 = 0; s2 < kSlots; ++s2)
            if ((live >> s2) & 1u) mbar_wait_lane_bounded(&R.bars[s2], (phases >> s2) & 1u);
    }

    // ---- merge the warps of the CTA (log-sum-exp) and store one partial per row; every slot has been consumed: the
    //      ring memory becomes the merge buffer
    __syncthreads();
    float* mbuf = reinterpret_cast<float*>(sm.ring) + warp * kWarpFloats;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                acc.l[nb][j] += __shfl_xor_sync(0xffffffffu, acc.l[nb][j], o);
                acc.z[nb][j] += __shfl_xor_sync(0xffffffffu, acc.z[nb][j], o);
            }
            if (g == 0) {
                const int row = 8 * nb + 2 * t + j;
                mbuf[row] = acc.m[nb][j];
                mbuf[kRows + row] = acc.l[nb][j];
                mbuf[2 * kRows + row] = acc.z[nb][j];
            }
        }
#pragma unroll
        for (int db = 0; db < 4; ++db)
#pragma unroll
            for (int j = 0; j < 2; ++j) {  // row 8 nb + 2t + j, dims 32 db + 4g .. +3
                float* dst = mbuf + 3 * kRows + (8 * nb + 2 * t + j) * kORow + 32 * db + 4 * g;
                *reinterpret_cast<float4*>(dst) = make_float4(acc.o[nb][db][0][j], acc.o[nb][db][1][j], acc.o[nb][db][0][2 + j], acc.o[nb][db][1][2 + j]);
            }
    }
    __syncthreads();
    const float* all = reinterpret_cast<const float*>(sm.ring);
    for (int e = threadIdx.x; e < 8 * NB * (D / 4); e += kThreads) {  // one thread: four dims of one row
        const int row = e / (D / 4), d = 4 * (e % (D / 4));
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) m = fmaxf(m, all[w * kWarpFloats + row]);
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        float l = 0.0f;
        if (m != -INFINITY) {
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const float* wb = all + w * kWarpFloats;
                const float wt = fast_exp2(wb[row] - m);  // exp2(-inf) = 0 for a warp that saw no key
                const float4 v = *reinterpret_cast<const float4*>(wb + 3 * kRows + row * kORow + d);
                const float z = wb[2 * kRows + row];
                l += wt * wb[kRows + row];
                o.x += wt * (v.x + z); o.y += wt * (v.y + z); o.z += wt * (v.z + z); o.w += wt * (v.w + z);
            }
        }
        *reinterpret_cast<float4*>(P.ws_o + (pidx + row) * D + d) = o;
        if (d == 0) { P.ws_m[pidx + row] = m; P.ws_l[pidx + row] = l; }
    }
}

template <int NB, int W, bool kOther = false>
__global__ void __launch_bounds__(W * 32, 1) attn_kernel(const AttnParams P) {
    grid_dependency_wait();  // q, the positions and the cache come from the kernels before this one
    const int head = blockIdx.y, zb = blockIdx.z, split = blockIdx.x;
    attn_cta<NB, W, kOther>(P, split, head, zb, ((static_cast<int64_t>(head) * gridDim.z + zb) * P.nsplit + split) * kRows);
}

// Batched decode: `n` independent sequences (their caches described by device-resident kvb_layer structs, same
// geometry) in one launch.  Sequence b owns parts prefix[b] .. prefix[b + 1] - 1 of the grid's x axis: its splits
// over sealed pages, then its open tile; the number of splits follows the host's bound of its length, so long and
// short sequences give CTAs of similar size.
constexpr int kBatchMax = 64;
struct BatchPlan {
    int n;                      // sequences; 0 = not a batched call
    int prefix[kBatchMax + 1];  // parts before sequence b
};
struct BatchParams {
    const LayerView* layers;  // [n], device memory (layout of kvb_layer)
    const uint16_t* q;        // [n][q_heads][D]
    const int32_t* pos;       // [n] position of the newest token of each sequence
    float scale_log2;
    int kv_heads, q_heads, dtype;  // geometry of the call: every entry must agree with it
    float* ws_m;              // [H][total parts][16]
    float* ws_l;
    float* ws_o;
    BatchPlan plan;
};

__device__ __forceinline__ int batch_entry_of(const BatchPlan& plan, int part) {  // largest b with prefix[b] <= part
    int lo = 0, hi = plan.n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (plan.prefix[mid] <= part) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

template <int NB, int W>
__global__ void __launch_bounds__(W * 32, 1) attn_batch_kernel(const BatchParams B) {
    constexpr int kThreads = W * 32;
    grid_dependency_wait();
    const int part = blockIdx.x, head = blockIdx.y;
    const int b = batch_entry_of(B.plan, part);
    AttnParams P;
    P.L = B.layers[b];
    const int64_t pidx = (static_cast<int64_t>(head) * gridDim.x + part) * kRows;
    if (P.L.head_dim != D || P.L.iters != 0 || P.L.kv_heads != B.kv_heads || P.L.q_heads != B.q_heads || P.L.dtype != B.dtype) {
        // an entry that disagrees with the call's geometry is flagged and contributes nothing: its partial reads as
        // "no key seen", so the merge writes zeros for that sequence and no plane is indexed with foreign strides
        if (threadIdx.x == 0) P.L.flag(KVB_ERR_GEOMETRY);
        for (int e = threadIdx.x; e < kRows * D; e += kThreads) B.ws_o[pidx * D + e] = 0.0f;
        if (threadIdx.x < kRows) { B.ws_m[pidx + threadIdx.x] = -INFINITY; B.ws_l[pidx + threadIdx.x] = 0.0f; }
        return;
    }
    P.q = B.q + static_cast<int64_t>(b) * B.q_heads * D;
    P.pos = B.pos + b;
    P.total_pos = B.pos + b;
    P.T = 1;
    P.scale_log2 = B.scale_log2;
    P.nsplit = B.plan.prefix[b + 1] - B.plan.prefix[b];
    P.block_rows = kRows;
    P.key_begin = 0;
    P.key_end = INT_MAX;
    P.ws_m = B.ws_m;
    P.ws_l = B.ws_l;
    P.ws_o = B.ws_o;
    attn_cta<NB, W>(P, part - B.plan.prefix[b], head, 0, pidx);
}

// Merge the partials of all splits of one query row, normalise, rotate back (H is its own inverse) and
// store in the output dtype -- or, for a sharded decode, export the merged partial (m in natural-log
// units, l, o in the rotated domain).  One CTA of 8 warps per (token, q head): warp w takes parts
// w, w+8, ... and issues all its loads before using any (the kernel is pure load latency), lane l owns
// dims 4l..4l+3; the eight warp sums meet in shared memory and warp 0 finishes the row.
constexpr int kReduceWarps = 8, kMaxPartsPerWarp = 8;  // up to 64 parts
// Where a sharded decode sends its partial: the ring buffers of all ranks (peer memory over NVLink; this rank's
// own buffer included), see kvb_peer_ring in the header.  A ring buffer holds [slot = call & 1][sender] blocks of
// {m, l}[rows] | o[rows][D]; every fp32 value travels in one aligned 8-byte word together with the number of the
// call that produced it (value in the low half, call number in the high half).  An 8-byte word arrives whole, so
// a reader that sees the expected call number in a word also sees its value: no fences, no separate flags, the
// latency of the exchange is one store across NVLink.  Words move in pairs (16-byte accesses, each half carrying
// its own call number).
constexpr int kRingMaxWorld = 16, kRingGroup = 8;
struct PushTarget {
    unsigned long long* peers[kRingMaxWorld];  // ring buffer of every rank, in rank order (kernel parameter space)
    uint32_t* state;                           // local words: [0] calls completed, [2] CTAs of this call that are done
    const unsigned long long* local_buf;       // this rank's own ring buffer (what the peers write)
    uint32_t max_spins;                        // bound of the wait for the peers' words
    uint32_t* error_word;
    int rank, world;                           // world 0: no push
};
// One 16-byte access = two 64-bit elements, each {value (low half), call number (high half)}: the element type of
// the vector access is 64 bits, so value and call number of a word are one access in the memory model, not two.
__device__ __forceinline__ void ring_store2(unsigned long long* p, float a, float b, uint32_t call) {
    const unsigned long long wa = static_cast<unsigned long long>(__float_as_uint(a)) | (static_cast<unsigned long long>(call) << 32);
    const unsigned long long wb = static_cast<unsigned long long>(__float_as_uint(b)) | (static_cast<unsigned long long>(call) << 32);
    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(p), "l"(wa), "l"(wb) : "memory");
}
__device__ __forceinline__ uint4 ring_load2(const unsigned long long* p) {
    unsigned long long wa, wb;
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(wa), "=l"(wb) : "l"(p) : "memory");
    return make_uint4(static_cast<uint32_t>(wa), static_cast<uint32_t>(wa >> 32), static_cast<uint32_t>(wb), static_cast<uint32_t>(wb >> 32));
}
__device__ __forceinline__ bool ring_arrived(const uint4& w, uint32_t call) { return w.y == call && w.w == call; }

__global__ void __launch_bounds__(kReduceWarps * 32) reduce_kernel(const float* __restrict__ ws_m, const float* __restrict__ ws_l,
                                                                  const float* __restrict__ ws_o, int parts, int T, int q_heads,
                                                                  int kv_heads, int zblocks, int block_rows, int dtype, uint16_t* __restrict__ out,
                                                                  float* __restrict__ part_m, float* __restrict__ part_l,
                                                                  float* __restrict__ part_o, const PushTarget push,
                                                                  const BatchPlan plan) {
    __shared__ float4 so[kReduceWarps][32];
    __shared__ float sl[kReduceWarps];
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = q_heads / kv_heads, tq = row / q_heads, qh = row % q_heads, head = qh / G, gq = qh % G;
    int64_t base;
    if (plan.n > 0) {  // batched decode: row = (sequence tq, q head); the sequence's parts are plan.prefix[tq] ..
        parts = plan.prefix[tq + 1] - plan.prefix[tq];
        base = (static_cast<int64_t>(head) * plan.prefix[plan.n] + plan.prefix[tq]) * kRows + gq;
    } else {
        const int R = tq * G + gq, zb = R / block_rows, r = R % block_rows;
        base = (static_cast<int64_t>(head) * zblocks + zb) * parts * kRows + r;
    }
    grid_dependency_wait();  // launched while the attention kernel still runs: its partials are complete from here on
    launch_dependents();
    // the number of this call on the ring (read early: its latency hides behind the partial loads)
    const uint32_t call = push.world > 0 && warp == 0 ? *reinterpret_cast<volatile uint32_t*>(push.state) + 1u : 0u;
    // every warp finds the global maximum (parts <= 64: two loads per lane)
    float m = lane < parts ? ws_m[base + static_cast<int64_t>(lane) * kRows] : -INFINITY;
    if (lane + 32 < parts) m = fmaxf(m, ws_m[base + static_cast<int64_t>(lane + 32) * kRows]);
    float4 v[kMaxPartsPerWarp];
    float pm[kMaxPartsPerWarp], pl[kMaxPartsPerWarp];
#pragma unroll
    for (int i = 0; i < kMaxPartsPerWarp; ++i) {
        const int p = warp + kReduceWarps * i;
        const bool on = p < parts;
        const int64_t idx = base + static_cast<int64_t>(on ? p : 0) * kRows;
        pm[i] = on ? ws_m[idx] : -INFINITY;
        pl[i] = on ? ws_l[idx] : 0.0f;
        v[i] = on ? *reinterpret_cast<const float4*>(ws_o + idx * D + 4 * lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));  // after the loads are in flight
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float l = 0.0f;
    if (m != -INFINITY) {
#pragma unroll
        for (int i = 0; i < kMaxPartsPerWarp; ++i) {
            const float w = fast_exp2(pm[i] - m);
            l += w * pl[i];
            acc.x += w * v[i].x; acc.y += w * v[i].y; acc.z += w * v[i].z; acc.w += w * v[i].w;
        }
    }
    so[warp][lane] = acc;
    if (lane == 0) sl[warp] = l;
    __syncthreads();
    if (warp != 0) return;
    acc = so[0][lane];
    l = sl[0];
#pragma unroll
    for (int w = 1; w < kReduceWarps; ++w) {
        const float4 x = so[w][lane];
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
        l += sl[w];
    }
    if (push.world > 0) {
        // Sharded decode: this CTA owns one query row on every rank.  It stores its partial of the row straight into
        // every peer's ring buffer, waits (bounded) for the peers' partials of the same row in its own ring buffer,
        // merges all of them in rank order (every rank computes the same bits), normalises, rotates back and
        // stores -- send, receive and merge in one kernel.  All loads of a polling round are issued before any is
        // examined, so a round costs one memory latency whatever the number of ranks.
        const uint32_t slot = call & 1u;
        const int rows = T * q_heads;
        const int64_t block = static_cast<int64_t>(rows) * (D + 2);
        const int64_t ml_off = 2 * static_cast<int64_t>(row), o_off = 2 * static_cast<int64_t>(rows) + static_cast<int64_t>(row) * D + 4 * lane;
        const float mine = m * kLn2;  // natural-log units, like every exported partial
        const int64_t my_block = (static_cast<int64_t>(slot) * push.world + push.rank) * block;
#pragma unroll
        for (int p = 0; p < kRingMaxWorld; ++p) {
            if (p >= push.world || p == push.rank) continue;
            unsigned long long* dst = push.peers[p] + my_block;
            ring_store2(dst + o_off, acc.x, acc.y, call);
            ring_store2(dst + o_off + 2, acc.z, acc.w, call);
            if (lane == 0) ring_store2(dst + ml_off, mine, l, call);
        }
        const unsigned long long* in = push.local_buf + static_cast<int64_t>(slot) * push.world * block;
        const uint32_t everyone = (push.world >= 32 ? 0xffffffffu : (1u << push.world) - 1u) & ~(1u << push.rank);
        uint32_t spins = 0;
        // (m, l) of every rank and, in the same polling rounds, the o words of the first kRingGroup ranks (all of them up
        // to eight GPUs): one memory latency after the last word has landed, not one per kind of word
        float rm[kRingMaxWorld], rl[kRingMaxWorld];
        uint4 a0[kRingGroup], b0[kRingGroup];
        uint32_t pending = everyone, pending_o = everyone & ((1u << kRingGroup) - 1u);
        while ((pending | pending_o) != 0u && spins < push.max_spins) {
            uint4 w[kRingMaxWorld];
#pragma unroll
            for (int p = 0; p < kRingMaxWorld; ++p)
                if (pending >> p & 1u) w[p] = ring_load2(in + p * block + ml_off);
#pragma unroll
            for (int i = 0; i < kRingGroup; ++i)
                if (pending_o >> i & 1u) {
                    a0[i] = ring_load2(in + i * block + o_off);
                    b0[i] = ring_load2(in + i * block + o_off + 2);
                }
#pragma unroll
            for (int p = 0; p < kRingMaxWorld; ++p)
                if ((pending >> p & 1u) && ring_arrived(w[p], call)) {
                    rm[p] = __uint_as_float(w[p].x);
                    rl[p] = __uint_as_float(w[p].z);
                    pending &= ~(1u << p);
                }
#pragma unroll
            for (int i = 0; i < kRingGroup; ++i)
                if ((pending_o >> i & 1u) && ring_arrived(a0[i], call) && ring_arrived(b0[i], call)) pending_o &= ~(1u << i);
            if ((pending | pending_o) != 0u) { ++spins; __nanosleep(32); }
        }
        bool ok = (pending | pending_o) == 0u;
        float gm = mine;
#pragma unroll
        for (int p = 0; p < kRingMaxWorld; ++p)
            if (everyone >> p & 1u) gm = fmaxf(gm, ok ? rm[p] : mine);
        float gl = 0.0f;
        float4 go = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int g = 0; g < kRingMaxWorld; g += kRingGroup) {
            if (g >= push.world || !ok) continue;
            uint4 a[kRingGroup], b[kRingGroup];
            pending = g == 0 ? 0u : everyone >> g & ((1u << kRingGroup) - 1u);  // the first group is already here
            if (g == 0) {
#pragma unroll
                for (int i = 0; i < kRingGroup; ++i) { a[i] = a0[i]; b[i] = b0[i]; }
            }
            while (pending != 0u && spins < push.max_spins) {
#pragma unroll
                for (int i = 0; i < kRingGroup; ++i)
                    if (pending >> i & 1u) {
                        a[i] = ring_load2(in + (g + i) * block + o_off);
                        b[i] = ring_load2(in + (g + i) * block + o_off + 2);
                    }
                uint32_t still = 0u;
#pragma unroll
                for (int i = 0; i < kRingGroup; ++i)
                    if ((pending >> i & 1u) && !(ring_arrived(a[i], call) && ring_arrived(b[i], call))) still |= 1u << i;
                pending = still;
                if (pending != 0u) { ++spins; __nanosleep(32); }
            }
            ok = pending == 0u;
#pragma unroll
            for (int i = 0; i < kRingGroup; ++i) {
                const int p = g + i;
                if (p >= push.world || !ok) continue;
                if (p == push.rank) {
                    const float w = gm == -INFINITY ? 0.0f : __expf(mine - gm);
                    gl += w * l;
                    go.x += w * acc.x; go.y += w * acc.y; go.z += w * acc.z; go.w += w * acc.w;
                } else {
                    const float w = gm == -INFINITY ? 0.0f : __expf(rm[p] - gm);
                    gl += w * rl[p];
                    go.x += w * __uint_as_float(a[i].x); go.y += w * __uint_as_float(a[i].z);
                    go.z += w * __uint_as_float(b[i].x); go.w += w * __uint_as_float(b[i].z);
                }
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok && lane == 0 && push.error_word != nullptr) atomicOr(push.error_word, KVB_ERR_WAIT_TIMEOUT);
        const float ginv = ok && gl > 0.0f ? 1.0f / gl : 0.0f;  // a wait that ran out: zeros, not a half-merged row
        so[0][lane] = make_float4(go.x * ginv, go.y * ginv, go.z * ginv, go.w * ginv);
        __syncwarp();
        const float* gflat = reinterpret_cast<const float*>(so[0]);
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = gflat[lane + 32 * j];
        hadamard_warp<D>(o, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            out[static_cast<int64_t>(row) * D + lane + 32 * j] = dtype == KVB_DTYPE_BF16 ? f32_to_out<true>(o[j]) : f32_to_out<false>(o[j]);
        if (lane == 0 && atomicAdd(&push.state[2], 1u) == gridDim.x - 1) {  // every CTA of this call has read the call number
            push.state[2] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(push.state) = call;
        }
        return;
    }
    if (part_m != nullptr) {
        if (lane == 0) { part_m[row] = m * kLn2; part_l[row] = l; }
        *reinterpret_cast<float4*>(part_o + static_cast<int64_t>(row) * D + 4 * lane) = acc;
        return;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    // the rotation wants lane l to hold dims l + 32 j: re-distribute through shared memory
    so[0][lane] = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
    __syncwarp();
    const float* flat = reinterpret_cast<const float*>(so[0]);
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = flat[lane + 32 * j];
    hadamard_warp<D>(o, lane);
#pragma unroll
    for (int j = 0; j < 4; ++j)
        out[static_cast<int64_t>(row) * D + lane + 32 * j] = dtype == KVB_DTYPE_BF16 ? f32_to_out<true>(o[j]) : f32_to_out<false>(o[j]);
}

// Cross-GPU (or cross-range) merge of exported partials: parts_m in natural-log units.
// Part p keeps its m and l at [p * ml_stride + row] and its o at [p * o_stride + row * D].
template <int DD>
__global__ void __launch_bounds__(128) merge_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                                                    const float* __restrict__ po, int parts, int rows, int64_t ml_stride,
                                                    int64_t o_stride, int dtype, uint16_t* __restrict__ out) {
    constexpr int R = DD / 32;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    float m = -INFINITY;
    for (int p = 0; p < parts; ++p) m = fmaxf(m, pm[p * ml_stride + row]);
    float l = 0.0f, o[R];
#pragma unroll
    for (int j = 0; j < R; ++j) o[j] = 0.0f;
    if (m != -INFINITY) {
        for (int p = 0; p < parts; ++p) {
            const int64_t i = p * ml_stride + row;
            const float w = __expf(pm[i] - m);
            l += w * pl[i];
#pragma unroll
            for (int j = 0; j < R; ++j) o[j] += w * po[p * o_stride + static_cast<int64_t>(row) * DD + lane + 32 * j];
        }
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int j = 0; j < R; ++j) o[j] *= inv;
    hadamard_warp<DD>(o, lane);
#pragma unroll
    for (int j = 0; j < R; ++j)
        out[static_cast<int64_t>(row) * DD + lane + 32 * j] = dtype == KVB_DTYPE_BF16 ? f32_to_out<true>(o[j]) : f32_to_out<false>(o[j]);
}

int sm_count() { return device_sm_count(); }

int zblocks_of(int q_heads, int kv_heads, int rows, int block_rows) { return (rows * (q_heads / kv_heads) + block_rows - 1) / block_rows; }

// Splits over the sealed tiles of a head: one CTA per SM in total, no more splits than tiles.
int split_count(int kv_len_max, int kv_heads, int zblocks) {
    const int tiles = kv_len_max / kTile;
    const int per = kv_heads * zblocks;
    int n = sm_count() / per;
    if (n > tiles) n = tiles;
    if (n > kReduceWarps * kMaxPartsPerWarp) n = kReduceWarps * kMaxPartsPerWarp;  // reduce_kernel holds 64 parts
    return n < 1 ? 1 : n;
}

}  // namespace
}  // namespace kvb

namespace kvb {
namespace {

}  // namespace
// kvb_attn_general.cu: head_dim 256 and caches written with Sinkhorn iterations > 0
size_t general_workspace_bytes(int kv_len_max, int q_heads, int head_dim, int rows);
int launch_general_attention(const kvb_layer* layer, const void* q, const int32_t* pos_dev, const int32_t* total_pos_dev, int T,
                             float scale, int kv_len_max, int key_begin, int key_end, void* workspace, void* out, float* part_m,
                             float* part_l, float* part_o, cudaStream_t stream);
namespace {

// One attention launch with W warps per CTA (the opt-in to large dynamic shared memory is made once per device and W).
template <int NB, int W, bool kOther = false>
cudaError_t launch_attn(dim3 grid, cudaStream_t stream, const AttnParams& P) {
    constexpr int smem = static_cast<int>(sizeof(AttnSmem<W>));
    static unsigned long long opted = 0;
    if (first_call_on_device(opted)) {
        const cudaError_t e = cudaFuncSetAttribute(attn_kernel<NB, W, kOther>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
    }
    return launch_early(attn_kernel<NB, W, kOther>, grid, dim3(W * 32), smem, stream, P);
}

// Warps per CTA for a decode call: 8, 12 or 16 (whole warp quartets: an SM hands registers and issue slots out per
// quartet; 10 or 14 warps measured no faster per warp than 12 or 16).  A warp works on whole pages, so a CTA with n
// pages needs ceil(n / W) rounds; a round and the fixed part (set-up, merge of the warps) take longer the more warps
// share the SM.  Times in microseconds, fitted to sweeps over 32K .. 379K tokens on B200: with 8 warps the SM is
// not yet saturated (a round of 8 pages takes 2.5 us, one of 16 pages 3.9 us).
int decode_warps(int kv_len_max, int nsplit, float* cost_us = nullptr) {
    static const int forced = [] { const char* e = std::getenv("KVB_DECODE_WARPS"); return e ? std::atoi(e) : 0; }();
    static const struct { int warps; float fixed_us, round_us; } kChoice[3] = {{16, 8.8f, 3.93f}, {12, 7.3f, 2.98f}, {8, 6.1f, 2.52f}};
    const int pages = 2 * (kv_len_max / kTile), per_cta = (pages + nsplit - 1) / nsplit;
    int best = 16;
    float best_cost = 1e30f;
    for (const auto& c : kChoice) {
        if ((forced == 8 || forced == 12 || forced == 16) && c.warps != forced) continue;
        const float cost = c.fixed_us + static_cast<float>((per_cta + c.warps - 1) / c.warps) * c.round_us;
        if (cost < best_cost - 1e-3f) { best_cost = cost; best = c.warps; }
    }
    if (cost_us != nullptr) *cost_us = best_cost;
    return best;
}

// How a call with `T` query tokens is cut into row blocks (grid z).  Up to 8 merged rows: one block.  More: either
// blocks of 16 rows on the two-block kernel (8 warps of 255 registers: about 4.4 us per round of 8 pages, measured at
// 131,072 tokens) or blocks of 8 rows on the one-block kernel with its 8 / 12 / 16 warps (more CTAs per head, so fewer
// key splits and more pages per CTA, but up to twice the warps): whichever the cost model puts first.  Balanced
// caches have the one-block kernel with 8 warps only, and take the 16-row blocks.
struct RowPlan {
    int nb, warps, block_rows, zblocks, nsplit;
};
RowPlan plan_rows(int kv_len_max, int kv_heads, int q_heads, int T, bool balanced) {
    const int merged = T * (q_heads / kv_heads);
    RowPlan one{1, 16, 8, zblocks_of(q_heads, kv_heads, T, 8), 0};
    one.nsplit = split_count(kv_len_max, kv_heads, one.zblocks);
    float cost_one = 0.0f;
    one.warps = decode_warps(kv_len_max, one.nsplit, &cost_one);
    if (balanced) one.warps = 8;
    if (merged <= 8) return one;
    RowPlan two{2, kWarpsWide, 16, zblocks_of(q_heads, kv_heads, T, 16), 0};
    two.nsplit = split_count(kv_len_max, kv_heads, two.zblocks);
    const int pages = 2 * (kv_len_max / kTile), per_cta = (pages + two.nsplit - 1) / two.nsplit;
    const float cost_two = 6.1f + static_cast<float>((per_cta + kWarpsWide - 1) / kWarpsWide) * 4.4f;
    return balanced || cost_two <= cost_one ? two : one;
}

int launch_attention(const kvb_layer* layer, const void* q, const int32_t* pos_dev, const int32_t* total_pos_dev, int T,
                     float scale, int kv_len_max,
                     int key_begin, int key_end, void* workspace, void* out, float* part_m, float* part_l,
                     float* part_o, cudaStream_t stream, const char* who, const PushTarget* push = nullptr) {
    if (int st = check_layer(layer, who)) return st;
    if (q == nullptr || pos_dev == nullptr || workspace == nullptr) return fail(KVB_EINVAL, "%s: null q / positions / workspace", who);
    if (out == nullptr && part_m == nullptr && push == nullptr) return fail(KVB_EINVAL, "%s: null output", who);
    if (T < 1 || T > 8) return fail(KVB_ERANGE, "%s: %d query tokens (1..8 supported)", who, T);
    if (kv_len_max < 1) return fail(KVB_EINVAL, "%s: kv_len_max %d", who, kv_len_max);
    if (layer->stage == nullptr) return fail(KVB_EINVAL, "%s: layer has no stage buffer", who);
    if (layer->head_dim != 128 && push != nullptr) return fail(KVB_ERANGE, "%s: the sharded decode covers head_dim 128", who);
    if (layer->head_dim != 128)  // two slices per key: general kernel, same semantics
        return launch_general_attention(layer, q, pos_dev, total_pos_dev, T, scale, kv_len_max, key_begin, key_end, workspace, out,
                                        part_m, part_l, part_o, stream);
    const RowPlan plan = plan_rows(kv_len_max, layer->kv_heads, layer->q_heads, T, layer->sinkhorn_iters != 0);
    const int Z = plan.zblocks, nsplit = plan.nsplit;
    const int parts = nsplit;
    AttnParams P;
    P.L = make_view(*layer);
    P.q = static_cast<const uint16_t*>(q);
    P.pos = pos_dev;
    P.total_pos = total_pos_dev;
    P.T = T;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.nsplit = nsplit;
    P.block_rows = plan.block_rows;
    P.key_begin = key_begin;
    P.key_end = key_end;
    const size_t rows = static_cast<size_t>(layer->kv_heads) * Z * parts * kRows;
    P.ws_m = static_cast<float*>(workspace);
    P.ws_l = P.ws_m + rows;
    P.ws_o = P.ws_l + rows;
    const bool upper = plan.nb == 2;
    const dim3 grid(parts, layer->kv_heads, Z);
    if (layer->sinkhorn_iters != 0) {  // balanced caches: other_K per key, other_V per dim (more registers: 8 warps)
        if (upper) {
            KVB_CUDA_OK((launch_attn<2, kWarpsWide, true>(grid, stream, P)));
        } else {
            KVB_CUDA_OK((launch_attn<1, 8, true>(grid, stream, P)));
        }
    } else if (upper) {
        KVB_CUDA_OK((launch_attn<2, kWarpsWide>(grid, stream, P)));
    } else {
        switch (plan.warps) {
            case 8: KVB_CUDA_OK((launch_attn<1, 8>(grid, stream, P))); break;
            case 12: KVB_CUDA_OK((launch_attn<1, 12>(grid, stream, P))); break;
            default: KVB_CUDA_OK((launch_attn<1, 16>(grid, stream, P))); break;
        }
    }
    const int total_rows = T * layer->q_heads;
    KVB_CUDA_OK(launch_early(reduce_kernel, dim3(total_rows), dim3(kReduceWarps * 32), 0, stream, P.ws_m, P.ws_l, P.ws_o, parts, T,
                             layer->q_heads, layer->kv_heads, Z, plan.block_rows, layer->dtype, static_cast<uint16_t*>(out), part_m, part_l, part_o,
                             push != nullptr ? *push : PushTarget{}, BatchPlan{}));
    return KVB_OK;
}

}  // namespace
}  // namespace kvb

// From this many GQA-merged query rows per KV head on, the tcgen05 kernel wins (measured at 131,072 tokens: widths 4-5 of a
// 24/4-head model are faster on the warp-level kernel, widths 6-8 on this one).
static constexpr int kDenseRows = 32;
extern "C" int kvb_split_capacity(int kv_len_max, int kv_heads, int q_heads, int rows, int batch) {
    (void)batch;
    if (kv_heads < 1 || q_heads < kv_heads || rows < 1) return 0;
    return kvb::plan_rows(kv_len_max, kv_heads, q_heads, rows > 8 ? 8 : rows, false).nsplit;
}

// Bytes one call with `r` query tokens needs (the split count, hence the size, is not monotonic in r).
static size_t workspace_bytes_for_rows(int kv_len_max, int kv_heads, int q_heads, int head_dim, int r) {
    size_t bytes = 0;
    for (int block_rows = 8; block_rows <= 16; block_rows += 8) {  // either cut of the rows into blocks (plan_rows)
        const int Z = kvb::zblocks_of(q_heads, kv_heads, r, block_rows);
        const size_t parts = kvb::split_count(kv_len_max, kv_heads, Z);
        bytes = std::max(bytes, static_cast<size_t>(kv_heads) * Z * parts * kvb::kRows * (head_dim + 2) * sizeof(float));
    }
    const size_t general = kvb::general_workspace_bytes(kv_len_max, q_heads, head_dim, r);
    if (general > bytes) bytes = general;
    if (r * (q_heads / kv_heads) >= kDenseRows) {  // verify steps this wide run on the chunk-attention kernel
        const size_t dense = kvb_prefill_workspace_bytes(kv_len_max, kv_heads, q_heads, head_dim, r);
        if (dense > bytes) bytes = dense;
    }
    return bytes;
}

// A workspace of this size serves every call with 1..rows query tokens: the maximum over the widths, since a narrower
// step can be cut into more splits than a wider one.
extern "C" size_t kvb_workspace_bytes(int kv_len_max, int kv_heads, int q_heads, int head_dim, int rows, int batch) {
    if (kv_heads < 1 || q_heads < kv_heads || rows < 1 || batch < 1) return 0;
    size_t bytes = 0;
    for (int r = 1; r <= rows && r <= 8; ++r) bytes = std::max(bytes, workspace_bytes_for_rows(kv_len_max, kv_heads, q_heads, head_dim, r));
    if (rows > 8) bytes = std::max(bytes, workspace_bytes_for_rows(kv_len_max, kv_heads, q_heads, head_dim, rows));
    return static_cast<size_t>(batch) * bytes;
}

extern "C" int kvb_attn_decode(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale, int kv_len_max,
                               void* workspace, void* out, void* stream) {
    return kvb::launch_attention(layer, q, pos_dev, pos_dev, 1, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr, nullptr,
                                 static_cast<cudaStream_t>(stream), "kvb_attn_decode");
}

extern "C" int kvb_attn_decode_partial(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale,
                                       int kv_len_max, int key_begin, int key_end, void* workspace, float* part_m,
                                       float* part_l, float* part_o, void* stream) {
    if (part_m == nullptr || part_l == nullptr || part_o == nullptr)
        return kvb::fail(KVB_EINVAL, "kvb_attn_decode_partial: null partial output");
    return kvb::launch_attention(layer, q, pos_dev, pos_dev, 1, scale, kv_len_max, key_begin, key_end, workspace, nullptr, part_m, part_l,
                                 part_o, static_cast<cudaStream_t>(stream), "kvb_attn_decode_partial");
}

extern "C" int kvb_merge_partials(const float* parts_m, const float* parts_l, const float* parts_o, int parts, int q_heads,
                                  int head_dim, int dtype, void* out, void* stream) {
    using namespace kvb;
    if (parts_m == nullptr || parts_l == nullptr || parts_o == nullptr || out == nullptr)
        return fail(KVB_EINVAL, "kvb_merge_partials: null argument");
    if (parts < 1 || q_heads < 1) return fail(KVB_EINVAL, "kvb_merge_partials: parts %d / q_heads %d", parts, q_heads);
    if (head_dim != 128 && head_dim != 256) return fail(KVB_ERANGE, "kvb_merge_partials: head_dim %d (128 or 256)", head_dim);
    const dim3 grid((q_heads + 3) / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (head_dim == 128)
        merge_kernel<128><<<grid, 128, 0, st>>>(parts_m, parts_l, parts_o, parts, q_heads, q_heads, static_cast<int64_t>(q_heads) * 128, dtype,
                                                static_cast<uint16_t*>(out));
    else
        merge_kernel<256><<<grid, 128, 0, st>>>(parts_m, parts_l, parts_o, parts, q_heads, q_heads, static_cast<int64_t>(q_heads) * 256, dtype,
                                                static_cast<uint16_t*>(out));
    KVB_CUDA_OK(cudaGetLastError());
    return KVB_OK;
}

extern "C" int kvb_merge_partials_packed(const float* packed, int parts, int q_heads, int head_dim, int dtype, void* out,
                                         void* stream) {
    using namespace kvb;
    if (packed == nullptr || out == nullptr) return fail(KVB_EINVAL, "kvb_merge_partials_packed: null argument");
    if (parts < 1 || q_heads < 1) return fail(KVB_EINVAL, "kvb_merge_partials_packed: parts %d / q_heads %d", parts, q_heads);
    if (head_dim != 128 && head_dim != 256) return fail(KVB_ERANGE, "kvb_merge_partials_packed: head_dim %d (128 or 256)", head_dim);
    const int64_t block = static_cast<int64_t>(q_heads) * (head_dim + 2);
    const dim3 grid((q_heads + 3) / 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (head_dim == 128)
        merge_kernel<128><<<grid, 128, 0, st>>>(packed, packed + q_heads, packed + 2 * q_heads, parts, q_heads, block, block, dtype,
                                                static_cast<uint16_t*>(out));
    else
        merge_kernel<256><<<grid, 128, 0, st>>>(packed, packed + q_heads, packed + 2 * q_heads, parts, q_heads, block, block, dtype,
                                                static_cast<uint16_t*>(out));
    KVB_CUDA_OK(cudaGetLastError());
    return KVB_OK;
}

extern "C" size_t kvb_peer_ring_bytes(int world, int q_heads, int head_dim) {
    if (world < 1 || world > kvb::kRingMaxWorld || q_heads < 1) return 0;
    return static_cast<size_t>(2) * world * q_heads * (head_dim + 2) * sizeof(unsigned long long);  // two slots, 8 bytes per value
}

namespace kvb {
// Checks a ring descriptor and turns it into the kernel's form.
static int make_push_target(const kvb_layer* layer, const kvb_peer_ring* ring, const void* out, const char* who, PushTarget& push,
                            int tokens = 1) {
    if (ring == nullptr || ring->peer_bufs == nullptr || ring->local_buf == nullptr || ring->state == nullptr || out == nullptr)
        return fail(KVB_EINVAL, "%s: null ring / buffers / out", who);
    if (layer != nullptr && static_cast<uint32_t>(tokens * layer->q_heads) > (ring->rows ? ring->rows : static_cast<uint32_t>(layer->q_heads)))
        return fail(KVB_ERANGE, "%s: %d query rows, the ring buffers hold %u", who, tokens * layer->q_heads,
                    ring->rows ? ring->rows : static_cast<uint32_t>(layer->q_heads));
    if (ring->world < 1 || ring->world > kRingMaxWorld || ring->rank < 0 || ring->rank >= ring->world)
        return fail(KVB_EINVAL, "%s: rank %d of world %d (1..%d ranks)", who, ring->rank, ring->world, kRingMaxWorld);
    push = PushTarget{};
    for (int p = 0; p < ring->world; ++p) {
        if (ring->peer_bufs[p] == nullptr || (reinterpret_cast<uintptr_t>(ring->peer_bufs[p]) & 15u) != 0)
            return fail(KVB_EINVAL, "%s: ring buffer of rank %d is null or not 16-byte aligned", who, p);
        push.peers[p] = static_cast<unsigned long long*>(ring->peer_bufs[p]);
    }
    if ((reinterpret_cast<uintptr_t>(ring->local_buf) & 15u) != 0) return fail(KVB_EINVAL, "%s: local ring buffer is not 16-byte aligned", who);
    push.state = ring->state;
    push.local_buf = static_cast<const unsigned long long*>(ring->local_buf);
    push.max_spins = ring->max_spins ? ring->max_spins : (1u << 20);
    push.error_word = layer != nullptr ? layer->error_word : nullptr;
    push.rank = ring->rank;
    push.world = ring->world;
    return KVB_OK;
}
}  // namespace kvb

extern "C" int kvb_attn_decode_sharded(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale, int kv_len_max,
                                       void* workspace, const kvb_peer_ring* ring, void* out, void* stream) {
    using namespace kvb;
    PushTarget push{};
    if (int st = make_push_target(layer, ring, out, "kvb_attn_decode_sharded", push)) return st;
    return launch_attention(layer, q, pos_dev, pos_dev, 1, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), "kvb_attn_decode_sharded", &push);
}

extern "C" int kvb_attn_rows_sharded(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int rows, float scale,
                                     int kv_len_max, void* workspace, const kvb_peer_ring* ring, void* out, void* stream) {
    using namespace kvb;
    if (rows < 1 || rows > 8) return fail(KVB_ERANGE, "kvb_attn_rows_sharded: %d query tokens (1..8)", rows);
    if (positions_dev == nullptr) return fail(KVB_EINVAL, "kvb_attn_rows_sharded: null positions");
    PushTarget push{};
    if (int st = make_push_target(layer, ring, out, "kvb_attn_rows_sharded", push, rows)) return st;
    return launch_attention(layer, q, positions_dev, positions_dev + (rows - 1), rows, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr,
                            nullptr, nullptr, static_cast<cudaStream_t>(stream), "kvb_attn_rows_sharded", &push);
}

// One decode step of a sequence in one call: append the newest token, then attend (kvb_append followed by
// kvb_attn_decode, or kvb_attn_decode_sharded when a ring is given, on the same stream).
extern "C" int kvb_append_decode(const kvb_layer* layer, const void* q, const void* k, const void* v, const int32_t* pos_dev, float scale,
                                 int kv_len_max, void* workspace, const kvb_peer_ring* ring, void* out, void* stream) {
    using namespace kvb;
    if (int st = kvb_append(layer, k, v, pos_dev, 1, stream)) return st;
    if (ring == nullptr)
        return launch_attention(layer, q, pos_dev, pos_dev, 1, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr, nullptr,
                                static_cast<cudaStream_t>(stream), "kvb_append_decode");
    PushTarget push{};
    if (int st = make_push_target(layer, ring, out, "kvb_append_decode", push)) return st;
    return launch_attention(layer, q, pos_dev, pos_dev, 1, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), "kvb_append_decode", &push);
}

// ---------------------------------------------------------------------------------------------------------
// Batched decode of independent sequences.
namespace kvb {
namespace {

static_assert(sizeof(LayerView) == sizeof(kvb_layer) && offsetof(LayerView, error_word) == offsetof(kvb_layer, error_word) &&
                  offsetof(LayerView, table_stride) == offsetof(kvb_layer, table_stride) &&
                  offsetof(LayerView, iters) == offsetof(kvb_layer, sinkhorn_iters),
              "the device reads kvb_layer structs as LayerView");

// Parts (splits over the sealed tiles; the last one also reads the open tile) of every sequence from the host's
// bounds of their lengths: chunks of at least 8 tiles, at most 64 splits per sequence.  The chunk size trades the fixed
// part of a CTA (about 8.8 us with 16 warps: set-up, first fetch, merge) against the balance of the SMs: the candidates
// are 2 .. 12 CTAs per SM in total, costed as (CTAs x time of a CTA) / SMs + half a CTA for the ragged end, a CTA taking
// 8.8 us + 3.93 us per round of 16 pages (the same figures as the single-sequence decode).
int plan_batch(const int32_t* kv_len_max, int batch, int kv_heads, BatchPlan& plan) {
    int64_t total_tiles = 0;
    for (int b = 0; b < batch; ++b) total_tiles += kv_len_max[b] / kTile;
    const int sms = sm_count();
    int64_t chunk = 8;
    float best = 1e30f;
    static const int kPerSm[] = {2, 3, 4, 6, 8, 12};
    for (int per_sm : kPerSm) {
        const int64_t want = std::max<int64_t>(batch, static_cast<int64_t>(per_sm) * sms / kv_heads);
        const int64_t c = std::max<int64_t>(8, (total_tiles + want - 1) / want);
        int64_t ctas = 0;
        for (int b = 0; b < batch; ++b)
            ctas += std::min<int64_t>(std::max<int64_t>((kv_len_max[b] / kTile + c - 1) / c, 1), kReduceWarps * kMaxPartsPerWarp);
        ctas *= kv_heads;
        const float one = 8.8f + 3.93f * static_cast<float>((2 * c + kWarpsDecode - 1) / kWarpsDecode);
        const float cost = static_cast<float>(ctas) * one / static_cast<float>(sms) + 0.5f * one;
        if (cost < best) { best = cost; chunk = c; }
    }
    plan.n = batch;
    plan.prefix[0] = 0;
    for (int b = 0; b < batch; ++b) {
        const int64_t tiles = kv_len_max[b] / kTile;
        int nsplit = static_cast<int>((tiles + chunk - 1) / chunk);
        nsplit = std::min(std::max(nsplit, 1), kReduceWarps * kMaxPartsPerWarp);
        plan.prefix[b + 1] = plan.prefix[b] + nsplit;
    }
    return plan.prefix[batch];
}

}  // namespace
}  // namespace kvb

extern "C" size_t kvb_batch_workspace_bytes(const int32_t* kv_len_max, int batch, int kv_heads, int q_heads, int head_dim) {
    using namespace kvb;
    if (kv_len_max == nullptr || batch < 1 || batch > kBatchMax || kv_heads < 1 || q_heads < kv_heads || head_dim != 128) return 0;
    for (int b = 0; b < batch; ++b)
        if (kv_len_max[b] < 1) return 0;
    BatchPlan plan;
    const size_t rows = static_cast<size_t>(kv_heads) * plan_batch(kv_len_max, batch, kv_heads, plan) * kRows;
    return rows * (2 + head_dim) * sizeof(float);
}

extern "C" int kvb_attn_decode_batch(const kvb_layer* layers_dev, int batch, int kv_heads, int q_heads, int head_dim, int dtype,
                                     const void* q, const int32_t* pos_dev, float scale, const int32_t* kv_len_max, void* workspace,
                                     void* out, void* stream) {
    using namespace kvb;
    if (layers_dev == nullptr || q == nullptr || pos_dev == nullptr || kv_len_max == nullptr || workspace == nullptr || out == nullptr)
        return fail(KVB_EINVAL, "kvb_attn_decode_batch: null argument");
    if (batch < 1 || batch > kBatchMax) return fail(KVB_ERANGE, "kvb_attn_decode_batch: %d sequences (1..%d per call)", batch, kBatchMax);
    if (head_dim != 128) return fail(KVB_ERANGE, "kvb_attn_decode_batch: head_dim %d (128 supported; other shapes: one kvb_attn_decode per sequence)", head_dim);
    if (kv_heads < 1 || kv_heads > 8 || q_heads < kv_heads || q_heads % kv_heads != 0 || q_heads / kv_heads > kRows)
        return fail(KVB_EINVAL, "kvb_attn_decode_batch: %d q heads over %d kv heads", q_heads, kv_heads);
    if (dtype != KVB_DTYPE_F16 && dtype != KVB_DTYPE_BF16) return fail(KVB_EINVAL, "kvb_attn_decode_batch: dtype %d", dtype);
    for (int b = 0; b < batch; ++b)
        if (kv_len_max[b] < 1) return fail(KVB_EINVAL, "kvb_attn_decode_batch: kv_len_max[%d] = %d", b, kv_len_max[b]);
    BatchParams B;
    const int total = plan_batch(kv_len_max, batch, kv_heads, B.plan);
    const size_t rows = static_cast<size_t>(kv_heads) * total * kRows;
    B.layers = reinterpret_cast<const LayerView*>(layers_dev);
    B.q = static_cast<const uint16_t*>(q);
    B.pos = pos_dev;
    B.scale_log2 = scale * 1.4426950408889634f;
    B.kv_heads = kv_heads;
    B.q_heads = q_heads;
    B.dtype = dtype;
    B.ws_m = static_cast<float*>(workspace);
    B.ws_l = B.ws_m + rows;
    B.ws_o = B.ws_l + rows;
    constexpr int smem1 = static_cast<int>(sizeof(AttnSmem<kWarpsDecode>)), smem2 = static_cast<int>(sizeof(AttnSmem<kWarpsWide>));
    static unsigned long long opted = 0;
    if (first_call_on_device(opted)) {
        KVB_CUDA_OK(cudaFuncSetAttribute(attn_batch_kernel<1, kWarpsDecode>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1));
        KVB_CUDA_OK(cudaFuncSetAttribute(attn_batch_kernel<2, kWarpsWide>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (q_heads / kv_heads > 8) KVB_CUDA_OK(launch_early(attn_batch_kernel<2, kWarpsWide>, dim3(total, kv_heads, 1), dim3(kWarpsWide * 32), smem2, st, B));
    else KVB_CUDA_OK(launch_early(attn_batch_kernel<1, kWarpsDecode>, dim3(total, kv_heads, 1), dim3(kWarpsDecode * 32), smem1, st, B));
    KVB_CUDA_OK(launch_early(reduce_kernel, dim3(batch * q_heads), dim3(kReduceWarps * 32), 0, st, B.ws_m, B.ws_l, B.ws_o, 0, batch, q_heads,
                             kv_heads, 1, kRows, dtype, static_cast<uint16_t*>(out), static_cast<float*>(nullptr), static_cast<float*>(nullptr),
                             static_cast<float*>(nullptr), PushTarget{}, B.plan));
    return KVB_OK;
}

namespace kvb {
int launch_chunk_attention(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int tokens, float scale,
                           int kv_len_max, void* workspace, void* out, cudaStream_t s, float* part_m, float* part_l,
                           float* part_o, const int32_t* total_pos_dev);  // kvb_prefill.cu
}

extern "C" int kvb_attn_verify(const kvb_layer* layer, const void* q, const void* k, const void* v,
                               const int32_t* positions_dev, int width, float scale, int kv_len_max, void* workspace,
                               void* out, void* stream) {
    if (width < 1 || width > 8) return kvb::fail(KVB_ERANGE, "kvb_attn_verify: width %d (1..8; the reference rejects more, too)", width);
    if (int st = kvb::check_layer(layer, "kvb_attn_verify")) return st;
    if (int st = kvb_append(layer, k, v, positions_dev, width, stream)) return st;
    if (width * (layer->q_heads / layer->kv_heads) >= kDenseRows && layer->head_dim == 128) {
        if (q == nullptr || workspace == nullptr || out == nullptr) return kvb::fail(KVB_EINVAL, "kvb_attn_verify: null q / workspace / out");
        return kvb::launch_chunk_attention(layer, q, positions_dev, width, scale, kv_len_max, workspace, out, static_cast<cudaStream_t>(stream),
                                           nullptr, nullptr, nullptr, nullptr);
    }
    return kvb::launch_attention(layer, q, positions_dev, positions_dev + (width - 1), width, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr,
                                 nullptr, static_cast<cudaStream_t>(stream), "kvb_attn_verify");
}

// Causal attention of `tokens` already-appended (or foreign) query rows over THIS cache alone, exported as log-sum-exp
// partials: the building block of verify steps and prefill chunks over a sequence whose tile ranges live on several
// GPUs.  The rows' positions are in this cache's own coordinates; a cache that holds an earlier range of the sequence
// passes its last position for every row (every key visible).
extern "C" int kvb_attn_chunk_partial(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int tokens, float scale,
                                      int kv_len_max, void* workspace, float* part_m, float* part_l, float* part_o, void* stream) {
    using namespace kvb;
    if (int st = check_layer(layer, "kvb_attn_chunk_partial")) return st;
    if (tokens < 1 || tokens > 65535) return fail(KVB_ERANGE, "kvb_attn_chunk_partial: %d tokens (1..65535)", tokens);
    if (q == nullptr || positions_dev == nullptr || workspace == nullptr || part_m == nullptr || part_l == nullptr || part_o == nullptr)
        return fail(KVB_EINVAL, "kvb_attn_chunk_partial: null argument");
    if (layer->stage == nullptr) return fail(KVB_EINVAL, "kvb_attn_chunk_partial: layer has no stage buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (layer->head_dim != 128)
        return launch_general_attention(layer, q, positions_dev, positions_dev + (tokens - 1), tokens, scale, kv_len_max, 0, INT_MAX, workspace,
                                        nullptr, part_m, part_l, part_o, st);
    if (tokens <= 8 && tokens * (layer->q_heads / layer->kv_heads) < kDenseRows)
        return launch_attention(layer, q, positions_dev, positions_dev + (tokens - 1), tokens, scale, kv_len_max, 0, INT_MAX, workspace, nullptr,
                                part_m, part_l, part_o, st, "kvb_attn_chunk_partial");
    return launch_chunk_attention(layer, q, positions_dev, tokens, scale, kv_len_max, workspace, nullptr, st, part_m, part_l, part_o, nullptr);
}

// Causal attention of 1..8 query rows whose K/V rows are already in the cache -- a verify step without its append, for
// callers that append a wide step once and attend it in column blocks.
extern "C" int kvb_attn_rows(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int rows, const int32_t* total_pos_dev,
                             float scale, int kv_len_max, void* workspace, void* out, void* stream) {
    using namespace kvb;
    if (rows < 1 || rows > 8) return fail(KVB_ERANGE, "kvb_attn_rows: %d rows (1..8)", rows);
    if (int st = check_layer(layer, "kvb_attn_rows")) return st;
    if (total_pos_dev == nullptr) return fail(KVB_EINVAL, "kvb_attn_rows: null total_pos_dev");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows * (layer->q_heads / layer->kv_heads) >= kDenseRows && layer->head_dim == 128) {
        if (q == nullptr || positions_dev == nullptr || workspace == nullptr || out == nullptr)
            return fail(KVB_EINVAL, "kvb_attn_rows: null q / positions / workspace / out");
        return launch_chunk_attention(layer, q, positions_dev, rows, scale, kv_len_max, workspace, out, st, nullptr, nullptr, nullptr, total_pos_dev);
    }
    return launch_attention(layer, q, positions_dev, total_pos_dev, rows, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr, nullptr,
                            st, "kvb_attn_rows");
}

// ---------------------------------------------------------------------------------------------------------
// Decode attention for callers that cannot provide a workspace.
//
// Some hosts of this library have no way to obtain device memory once they are running: an inference engine
// that sized its KV pool to fill the GPU at start-up has nothing left to allocate from, and a serving thread
// may be forbidden to touch the allocator at all.  For them the split-K partials of kvb_attn_decode live in
// the fixed array below instead of a caller-supplied buffer.  The array is part of the library image: every
// GPU that loads the library holds these 2 MiB until the process exits, whether or not the entry point is
// ever called.
//
// `g_static_scratch` is a device symbol.  In host code its name is only a stand-in and must never be handed
// to a kernel; the device address is obtained once per device with cudaGetSymbolAddress (below) and that
// pointer is what the kernels receive.
constexpr size_t kStaticScratchBytes = 2u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace kvb {
namespace {
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device ordinal

// First use on the current device: look the symbol up (no allocation happens here or anywhere below).
int static_scratch_for_current_device(void** out) {
    int dev = -1;
    KVB_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(KVB_ERANGE, "kvb_attn_decode_static: device ordinal %d (0..%d supported)", dev, kMaxDevices - 1);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        KVB_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scratch));
        if (p == nullptr) return fail(KVB_ECUDA, "kvb_attn_decode_static: cudaGetSymbolAddress returned a null address");
        g_static_scratch_ptr[dev] = p;
    }
    *out = g_static_scratch_ptr[dev];
    return KVB_OK;
}
}  // namespace
}  // namespace kvb

extern "C" size_t kvb_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int kvb_attn_decode_static(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale, int kv_len_max,
                                      void* out, void* stream) {
    using namespace kvb;
    if (int st = check_layer(layer, "kvb_attn_decode_static")) return st;
    const size_t need = kvb_workspace_bytes(kv_len_max, layer->kv_heads, layer->q_heads, layer->head_dim, 1, 1);
    if (need == 0 || need > kStaticScratchBytes)
        return fail(KVB_ERANGE,
                    "kvb_attn_decode_static: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu; "
                    "use kvb_attn_decode with a caller-owned workspace",
                    need, kStaticScratchBytes);
    void* scratch = nullptr;
    if (int st = static_scratch_for_current_device(&scratch)) return st;
    // Nothing in the scratch has to start at zero: every partial the merge reads is written earlier in the same call.
    return launch_attention(layer, q, pos_dev, pos_dev, 1, scale, kv_len_max, 0, INT_MAX, scratch, out, nullptr, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), "kvb_attn_decode_static");
}
