// kvb_attn.cu -- paged split-K attention over the quantised cache for 1..8 query tokens (decode, MTP
// verify), de-quantisation fused into the QK and PV loops.  head_dim 128.
//
// Grid (splits + 1, kv heads, row blocks).  A CTA owns one KV head, one contiguous range of sealed pages
// and a block of up to 16 GQA-merged query rows (row = token * G + q head within the KV head); the extra
// CTA in x handles the open tile, whose rows are still un-quantised fp16 in the stage.  Inside a CTA each
// of the 8 warps streams its own sub-range of pages through a private two-slot shared-memory ring filled
// by bulk async copies (one mbarrier per slot, four contiguous runs per page: K codes, V codes, K scales,
// V scales), so warps never synchronise with each other until the final merge.
//
// Math per page (quantised-domain identities, no per-element de-quantisation):
//   logit[r][j] = other_K[j] * ( sum_d (q'[r][d] * scale_K[d]) * code_K[j][d]  +  sum_d q'[r][d] * zp_K[d] )
//   o[r][d]    += other_V[d] * ( sum_j (p[r][j] * scale_V[j]) * code_V[j][d]  +  sum_j p[r][j] * zp_V[j] )
// with q' = H q * softmax_scale * log2(e).  The two contractions run on the warp-level tensor cores
// (m16n8k16, fp16 operands, fp32 accumulate) with the KEYS (QK) and the DIMS (PV) on the 16-wide M side and
// the GQA-merged query rows on the 8-wide N side, so six query heads waste a quarter of a tile, not five
// eighths: S^T[key][row] = K_codes . (q' scale_K)^T and O^T[dim][row] = V_codes^T . (p scale_V)^T.
// 4-bit codes are exact in fp16, q' * scale_K is split into an fp16 high and low part so the product keeps
// fp32 accuracy, and p * scale_V is rounded to fp16 once.  Codes are unpacked with one logic op per pair
// (see unpack8); V pairs are formed across two keys with a byte permute and the probabilities change from
// accumulator to operand layout with one movmatrix per 8 keys, so nothing is transposed through memory.
#include <algorithm>
#include <climits>
#include <cstddef>

#include "kvb_common.cuh"
#include "kvb_ptx.cuh"

namespace kvb {
namespace {

constexpr int D = 128;
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRows = 16;  // query rows per CTA: one or two 8-row N blocks
constexpr int kKCodeOff = 0, kVCodeOff = 4096, kKScaleOff = 8192, kVScaleOff = 8832, kPageBytes = 9344;
constexpr int kSlots = 2;
constexpr int kScratchBytes = 256 + 256 + 128;  // per warp: scale_K[128], zp_K[128], other_K[64] as fp16
constexpr float kLn2 = 0.6931471805599453f;

struct AttnParams {
    LayerView L;
    const uint16_t* q;   // [T][q_heads][D]
    const int32_t* pos;  // [T] absolute positions of the query tokens (device)
    const int32_t* total_pos;  // position of the newest token in the cache (kv_total = *total_pos + 1)
    int T;
    float scale_log2;    // softmax scale * log2(e)
    int nsplit;          // CTAs over sealed pages; blockIdx.x == nsplit is the open-tile CTA
    int key_begin, key_end;
    float* ws_m;         // [H][Z][nsplit+1][16]
    float* ws_l;
    float* ws_o;         // [H][Z][nsplit+1][16][D]
};

struct __align__(16) AttnSmem {
    uint8_t slots[kWarps][kSlots][kPageBytes];
    uint8_t scratch[kWarps][kScratchBytes];
    float4 qfrag[2][8][32];  // q' in per-lane fragment order: [row half][j][lane] = dims 32t+4j..+3 of row g(+8)
    uint64_t bars[kWarps][kSlots];
    int row_pos[kRows];
};

// Per-thread state of the running softmax.  Lane (g, t) owns query rows 8 nb + 2t, 2t+1 of n-block nb and,
// in the PV accumulators, dims 16g .. 16g+15: o[nb][mb] = {(dim 16g+mb, row 2t), (dim 16g+mb, row 2t+1),
// (dim 16g+8+mb, row 2t), (dim 16g+8+mb, row 2t+1)}.  l and z are partial over the lane's keys.
template <int NB> struct Acc {
    float o[NB][8][4];
    float m[NB][2], l[NB][2], z[NB][2];
};

// B fragments of (q' * scale_K)^T per n-block and k-block (b0, b1), high and low fp16 parts, and
// qz = sum_d q'[row][d] * zp_K[d] for the lane's two rows.
template <int NB> struct QFrag {
    uint32_t hi[NB][8][2];
    uint32_t lo[NB][8][2];
    float qz[NB][2];
};

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(x));
    return r;
}

// Build the Q-side fragments for one tile from q' (shared memory, fragment order) and the tile's per-dim
// scale / zero point (warp scratch, natural dim order).  Lane (g, t) prepares row 8 nb + g, dims
// 32t .. 32t+31.  k-slot pairing follows unpack8: word i of the 32-dim chunk feeds k-blocks 2i (dims
// +0,+4 | +1,+5) and 2i+1 (dims +2,+6 | +3,+7); un-quantised stage rows use natural pairs (2e, 2e+1).
template <bool kScaled, int NB>
__device__ __forceinline__ void build_qfrag(const AttnSmem& sm, const uint8_t* scratch, int lane, QFrag<NB>& f) {
    const int t = lane & 3;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        float qs[32];
        float qz = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 qv = sm.qfrag[nb][j][lane];
            if constexpr (kScaled) {
                const uint2 ks = *reinterpret_cast<const uint2*>(scratch + (32 * t + 4 * j) * 2);
                const uint2 kz = *reinterpret_cast<const uint2*>(scratch + 256 + (32 * t + 4 * j) * 2);
                const float2 s01 = unpack_half2(ks.x), s23 = unpack_half2(ks.y);
                const float2 z01 = unpack_half2(kz.x), z23 = unpack_half2(kz.y);
                qs[4 * j + 0] = qv.x * s01.x; qs[4 * j + 1] = qv.y * s01.y;
                qs[4 * j + 2] = qv.z * s23.x; qs[4 * j + 3] = qv.w * s23.y;
                qz = fmaf(qv.x, z01.x, qz); qz = fmaf(qv.y, z01.y, qz);
                qz = fmaf(qv.z, z23.x, qz); qz = fmaf(qv.w, z23.y, qz);
            } else {
                qs[4 * j + 0] = qv.x; qs[4 * j + 1] = qv.y; qs[4 * j + 2] = qv.z; qs[4 * j + 3] = qv.w;
            }
        }
        qz += __shfl_xor_sync(0xffffffffu, qz, 1);
        qz += __shfl_xor_sync(0xffffffffu, qz, 2);  // every lane of group g now holds qz of row 8 nb + g
        f.qz[nb][0] = __shfl_sync(0xffffffffu, qz, 8 * t);      // row 2t   lives in lanes 4 * (2t) ..
        f.qz[nb][1] = __shfl_sync(0xffffffffu, qz, 8 * t + 4);  // row 2t+1 lives in lanes 4 * (2t+1) ..
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float x0 = kScaled ? qs[8 * i + e] : qs[8 * i + 2 * e];
                const float x1 = kScaled ? qs[8 * i + e + 4] : qs[8 * i + 2 * e + 1];
                const uint32_t h = pack_half2(x0, x1);
                const float2 hf32 = unpack_half2(h);
                f.hi[nb][2 * i + (e >> 1)][e & 1] = h;
                f.lo[nb][2 * i + (e >> 1)][e & 1] = pack_half2(x0 - hf32.x, x1 - hf32.y);
            }
        }
    }
}

// Integer form of (q' * scale_K)^T for the quantised pages: each row is scaled to 16-bit integers
// (row scale f = max|.| / 32639) and split into two signed 8-bit digits, Qi = 256 hi + lo, so that the key side
// can feed its packed code bytes to the int8 tensor path without unpacking nibbles: with L = byte & 0x0F (even
// dim) and H = byte & 0xF0 (16 x odd dim),   sum_d Qi[d] code[d] = sum_b Qi[2b] L_b + (1/16) sum_b Qi[2b+1] H_b.
// b[nb][kb][part][digit] holds the B fragments (b0, b1) of 32-byte k-block kb: part 0 = even dims, 1 = odd dims.
template <int NB> struct QInt {
    uint32_t b[NB][2][2][2][2];
    float f[NB][2];   // row scale / 16 of the lane's rows 2t, 2t+1
    float qz[NB][2];  // sum_d q'[row][d] * zp_K[d]
};

__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NB>
__device__ __forceinline__ void build_qint(const AttnSmem& sm, const uint8_t* scratch, int lane, QInt<NB>& f) {
    const int t = lane & 3;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        float qs[32];
        float qz = 0.0f, amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 qv = sm.qfrag[nb][j][lane];
            const uint2 ks = *reinterpret_cast<const uint2*>(scratch + (32 * t + 4 * j) * 2);
            const uint2 kz = *reinterpret_cast<const uint2*>(scratch + 256 + (32 * t + 4 * j) * 2);
            const float2 s01 = unpack_half2(ks.x), s23 = unpack_half2(ks.y);
            const float2 z01 = unpack_half2(kz.x), z23 = unpack_half2(kz.y);
            qs[4 * j + 0] = qv.x * s01.x; qs[4 * j + 1] = qv.y * s01.y;
            qs[4 * j + 2] = qv.z * s23.x; qs[4 * j + 3] = qv.w * s23.y;
            qz = fmaf(qv.x, z01.x, qz); qz = fmaf(qv.y, z01.y, qz);
            qz = fmaf(qv.z, z23.x, qz); qz = fmaf(qv.w, z23.y, qz);
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(qs[4 * j]), fabsf(qs[4 * j + 1]))), fmaxf(fabsf(qs[4 * j + 2]), fabsf(qs[4 * j + 3])));
        }
        qz += __shfl_xor_sync(0xffffffffu, qz, 1);
        qz += __shfl_xor_sync(0xffffffffu, qz, 2);  // every lane of group g now holds qz of row 8 nb + g
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float fr = amax > 0.0f ? amax * (1.0f / 32639.0f) : 1.0f, inv = amax > 0.0f ? 32639.0f / amax : 0.0f;  // 32639 keeps the high digit within [-127, 127]
        f.qz[nb][0] = __shfl_sync(0xffffffffu, qz, 8 * t);      // row 2t   lives in lanes 4 * (2t) ..
        f.qz[nb][1] = __shfl_sync(0xffffffffu, qz, 8 * t + 4);  // row 2t+1 lives in lanes 4 * (2t+1) ..
        f.f[nb][0] = __shfl_sync(0xffffffffu, fr, 8 * t) * 0.0625f;
        f.f[nb][1] = __shfl_sync(0xffffffffu, fr, 8 * t + 4) * 0.0625f;
        int hi[32], lo[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int qi = __float2int_rn(qs[i] * inv);
            hi[i] = (qi + 128) >> 8;
            lo[i] = qi - (hi[i] << 8);
        }
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
            for (int part = 0; part < 2; ++part)
#pragma unroll
                for (int r = 0; r < 2; ++r) {  // b0: local dims 16 kb + 2j + part, b1: +8
                    const int i0 = 16 * kb + 8 * r + part;  // low bytes of four digits -> one word: three byte permutes
                    f.b[nb][kb][part][0][r] = prmt(prmt(hi[i0], hi[i0 + 2], 0x0040), prmt(hi[i0 + 4], hi[i0 + 6], 0x0040), 0x5410);
                    f.b[nb][kb][part][1][r] = prmt(prmt(lo[i0], lo[i0 + 2], 0x0040), prmt(lo[i0 + 4], lo[i0 + 6], 0x0040), 0x5410);
                }
    }
}

// Scale page of K -> warp scratch in natural dim order.  A page row is 5 halves
// [scale(2r) scale(2r+1) zp(2r) zp(2r+1) other(r)]; lane l re-packs rows 2l and 2l+1 (20 bytes).
__device__ __forceinline__ void transpose_k_scale(const uint8_t* kscale_page, uint8_t* scratch, int lane) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(kscale_page + 20 * lane);
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = w[4];
    // halves: w0 = s(4l) s(4l+1) | w1 = z(4l) z(4l+1) | w2 = o(2l) s(4l+2) | w3 = s(4l+3) z(4l+2) | w4 = z(4l+3) o(2l+1)
    *reinterpret_cast<uint2*>(scratch + 8 * lane) = make_uint2(w0, prmt(w2, w3, 0x5432));
    *reinterpret_cast<uint2*>(scratch + 256 + 8 * lane) = make_uint2(w1, prmt(w3, w4, 0x5432));
    *reinterpret_cast<uint32_t*>(scratch + 512 + 4 * lane) = prmt(w2, w4, 0x7610);
}

// Online-softmax update of NG groups of 16 keys whose logits (log2 units) sit in s[nb][grp][4]:
// {(key g, row 2t), (key g, row 2t+1), (key g+8, row 2t), (key g+8, row 2t+1)} of group grp.
// On return s holds p = exp2(logit - m_new); acc is rescaled if a row maximum moved.
template <int NB, int NG>
__device__ __forceinline__ void softmax_block(float (&s)[NB][NG][4], Acc<NB>& acc) {
    float muse[NB][2], alpha[NB][2];
    bool moved = false;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float mx = -INFINITY;
#pragma unroll
            for (int grp = 0; grp < NG; ++grp) mx = fmaxf(mx, fmaxf(s[nb][grp][j], s[nb][grp][2 + j]));
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
    if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
            for (int mb = 0; mb < 8; ++mb) {
                acc.o[nb][mb][0] *= alpha[nb][0]; acc.o[nb][mb][1] *= alpha[nb][1];
                acc.o[nb][mb][2] *= alpha[nb][0]; acc.o[nb][mb][3] *= alpha[nb][1];
            }
            acc.l[nb][0] *= alpha[nb][0]; acc.z[nb][0] *= alpha[nb][0];
            acc.l[nb][1] *= alpha[nb][1]; acc.z[nb][1] *= alpha[nb][1];
        }
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int grp = 0; grp < NG; ++grp) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[nb][grp][e] = fast_exp2(s[nb][grp][e] - muse[nb][e & 1]);
                acc.l[nb][e & 1] += s[nb][grp][e];
            }
        }
    }
}

// One sealed page (64 keys) of one KV head, staged in shared memory at `pg`: qk_page fills s with the masked
// logits (log2 units), softmax_block turns them into p, pv_page accumulates p V.  (Computing the logits of the
// next page between the softmax and the P V of this one was measured slower: more registers, no more overlap.)
template <int NB, bool kOther>
__device__ __forceinline__ void qk_page(const uint8_t* pg, const uint8_t* scratch, const QInt<NB>& qf, float (&s)[NB][4][4],
                                        int lane, bool need_mask, int first_pos, const int (&row_lim)[NB][2], int key_begin,
                                        int key_end) {
    const int g = lane >> 2, t = lane & 3;
    // ---- QK on the int8 tensor path: A = packed code bytes of keys (g, g+8) masked to their low / high nibbles,
    //      B = 8-bit digits of (q' scale_K)^T; exact 32-bit accumulation
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
        const uint4 ka = *reinterpret_cast<const uint4*>(pg + kKCodeOff + (grp * 16 + g) * 64 + 16 * t);
        const uint4 kb8 = *reinterpret_cast<const uint4*>(pg + kKCodeOff + (grp * 16 + 8 + g) * 64 + 16 * t);
        const uint32_t wa[4] = {ka.x, ka.y, ka.z, ka.w}, wb[4] = {kb8.x, kb8.y, kb8.z, kb8.w};
        int ceh[NB][4], cel[NB][4], coh[NB][4], col[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) ceh[nb][e] = cel[nb][e] = coh[nb][e] = col[nb][e] = 0;
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
            const uint32_t l0 = wa[2 * kb] & 0x0F0F0F0Fu, l1 = wb[2 * kb] & 0x0F0F0F0Fu, l2 = wa[2 * kb + 1] & 0x0F0F0F0Fu,
                           l3 = wb[2 * kb + 1] & 0x0F0F0F0Fu;
            const uint32_t h0 = wa[2 * kb] & 0xF0F0F0F0u, h1 = wb[2 * kb] & 0xF0F0F0F0u, h2 = wa[2 * kb + 1] & 0xF0F0F0F0u,
                           h3 = wb[2 * kb + 1] & 0xF0F0F0F0u;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                imma16832(ceh[nb], l0, l1, l2, l3, qf.b[nb][kb][0][0][0], qf.b[nb][kb][0][0][1]);
                imma16832(cel[nb], l0, l1, l2, l3, qf.b[nb][kb][0][1][0], qf.b[nb][kb][0][1][1]);
                imma16832(coh[nb], h0, h1, h2, h3, qf.b[nb][kb][1][0][0], qf.b[nb][kb][1][0][1]);
                imma16832(col[nb], h0, h1, h2, h3, qf.b[nb][kb][1][1][0], qf.b[nb][kb][1][1][1]);
            }
        }
        float o0 = 1.0f, o1 = 1.0f;  // other_K of keys g and g+8 of the group
        if constexpr (kOther) {
            o0 = __half2float(*reinterpret_cast<const __half*>(scratch + 512 + (grp * 16 + g) * 2));
            o1 = __half2float(*reinterpret_cast<const __half*>(scratch + 512 + (grp * 16 + 8 + g) * 2));
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // 16 * sum = 256 (16 even_hi + odd_hi) + (16 even_lo + odd_lo); |.| < 2^31 for 64 code bytes per row
                const int tot = ((ceh[nb][e] * 16 + coh[nb][e]) << 8) + (cel[nb][e] * 16 + col[nb][e]);
                s[nb][grp][e] = fmaf(static_cast<float>(tot), qf.f[nb][e & 1], qf.qz[nb][e & 1]) * (e < 2 ? o0 : o1);
            }
        }
    }
    if (need_mask) {
#pragma unroll
        for (int grp = 0; grp < 4; ++grp) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int p = first_pos + grp * 16 + g + (e >> 1) * 8;
                const bool out = p < key_begin || p >= key_end;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
                    if (out || p > row_lim[nb][e & 1]) s[nb][grp][e] = -INFINITY;
            }
        }
    }
}

template <int NB>
__device__ __forceinline__ void pv_page(const uint8_t* pg, const float (&s)[NB][4][4], Acc<NB>& acc, int lane) {
    const int g = lane >> 2, t = lane & 3;
    // ---- PV: A = V codes^T (dims x keys), B = (p scale_V)^T.  V scale page rows: [other other scale zp] per key
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
        const float2 sz0 = unpack_half2(*reinterpret_cast<const uint32_t*>(pg + kVScaleOff + (grp * 16 + g) * 8 + 4));
        const float2 sz1 = unpack_half2(*reinterpret_cast<const uint32_t*>(pg + kVScaleOff + (grp * 16 + 8 + g) * 8 + 4));
        uint32_t b0[NB], b1[NB];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const float(&p)[4] = s[nb][grp];
            acc.z[nb][0] += p[0] * sz0.y + p[2] * sz1.y;
            acc.z[nb][1] += p[1] * sz0.y + p[3] * sz1.y;
            b0[nb] = movmatrix_trans(pack_half2(p[0] * sz0.x, p[1] * sz0.x));  // -> (row g; keys 2t, 2t+1)
            b1[nb] = movmatrix_trans(pack_half2(p[2] * sz1.x, p[3] * sz1.x));  // -> (row g; keys 2t+8, 2t+9)
        }
        // lane (g, t): 16 dims 16g.. of keys 2t, 2t+1 (pa) and 2t+8, 2t+9 (pb), one half2 per dim
        const uint8_t* vb = pg + kVCodeOff + (grp * 16 + 2 * t) * 64 + 8 * g;
        const uint2 vA = *reinterpret_cast<const uint2*>(vb), vB = *reinterpret_cast<const uint2*>(vb + 64);
        const uint2 vC = *reinterpret_cast<const uint2*>(vb + 512), vD = *reinterpret_cast<const uint2*>(vb + 576);
        const uint32_t wa[2] = {vA.x, vA.y}, wb[2] = {vB.x, vB.y}, wc[2] = {vC.x, vC.y}, wd[2] = {vD.x, vD.y};
        uint32_t pa[16], pb[16];
#pragma unroll
        for (int wi = 0; wi < 2; ++wi) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const uint32_t sel = hh ? 0x7632u : 0x5410u;  // low / high 16 bits of both keys' words
                const uint32_t x0 = prmt(wa[wi], wb[wi], sel), x1 = prmt(wc[wi], wd[wi], sel);
                const uint32_t y0 = x0 >> 8, y1 = x1 >> 8;
                const int d = 8 * wi + 4 * hh;
                pa[d + 0] = hsub2_u32(lop3_and_or(x0, 0x000F000Fu, 0x64006400u), 0x64006400u);
                pa[d + 1] = hsub2_u32(lop3_and_or(x0, 0x00F000F0u, 0x54005400u), 0x54005400u);
                pa[d + 2] = hsub2_u32(lop3_and_or(y0, 0x000F000Fu, 0x64006400u), 0x64006400u);
                pa[d + 3] = hsub2_u32(lop3_and_or(y0, 0x00F000F0u, 0x54005400u), 0x54005400u);
                pb[d + 0] = hsub2_u32(lop3_and_or(x1, 0x000F000Fu, 0x64006400u), 0x64006400u);
                pb[d + 1] = hsub2_u32(lop3_and_or(x1, 0x00F000F0u, 0x54005400u), 0x54005400u);
                pb[d + 2] = hsub2_u32(lop3_and_or(y1, 0x000F000Fu, 0x64006400u), 0x64006400u);
                pb[d + 3] = hsub2_u32(lop3_and_or(y1, 0x00F000F0u, 0x54005400u), 0x54005400u);
            }
        }
#pragma unroll
        for (int mb = 0; mb < 8; ++mb) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) mma16816(acc.o[nb][mb], pa[mb], pa[8 + mb], pb[mb], pb[8 + mb], b0[nb], b1[nb]);
        }
    }
}

// 16 keys of the open tile, read un-quantised (fp16, rotated) straight from the stage.
// krow/vrow point at the first of the 16 stage rows of this head (row stride D halves).
template <int NB>
__device__ __forceinline__ void process_stage_group(const __half* krow, const __half* vrow, const QFrag<NB>& qf,
                                                    Acc<NB>& acc, int lane, int first_pos, int kv_total,
                                                    const int (&row_lim)[NB][2], int key_begin, int key_end) {
    const int g = lane >> 2, t = lane & 3;
    float s[NB][1][4];
    {
        const __half* ka = krow + g * D + 32 * t;
        const __half* kb = krow + (8 + g) * D + 32 * t;
        float c[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 a = *reinterpret_cast<const uint4*>(ka + 8 * i), b = *reinterpret_cast<const uint4*>(kb + 8 * i);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                mma16816(c[nb], a.x, b.x, a.y, b.y, qf.hi[nb][2 * i][0], qf.hi[nb][2 * i][1]);
                mma16816(c[nb], a.z, b.z, a.w, b.w, qf.hi[nb][2 * i + 1][0], qf.hi[nb][2 * i + 1][1]);
                mma16816(c[nb], a.x, b.x, a.y, b.y, qf.lo[nb][2 * i][0], qf.lo[nb][2 * i][1]);
                mma16816(c[nb], a.z, b.z, a.w, b.w, qf.lo[nb][2 * i + 1][0], qf.lo[nb][2 * i + 1][1]);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int p = first_pos + g + (e >> 1) * 8;
            const bool out = p >= kv_total || p < key_begin || p >= key_end;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) s[nb][0][e] = (out || p > row_lim[nb][e & 1]) ? -INFINITY : c[nb][e];
        }
    }
    softmax_block<NB, 1>(s, acc);
    uint32_t b0[NB], b1[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        b0[nb] = movmatrix_trans(pack_half2(s[nb][0][0], s[nb][0][1]));
        b1[nb] = movmatrix_trans(pack_half2(s[nb][0][2], s[nb][0][3]));
    }
    // keys at or beyond kv_total hold stale rows: their p is exactly 0; zero V there so 0 * inf cannot appear
    const __half* vb = vrow + (2 * t) * D + 16 * g;
    uint4 v[4][2];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        const int key = 2 * t + (kk & 1) + (kk >> 1) * 8;
        const bool live = first_pos + key < kv_total;
        const uint4* src = reinterpret_cast<const uint4*>(vb + ((kk & 1) + (kk >> 1) * 8) * D);
        v[kk][0] = live ? src[0] : make_uint4(0, 0, 0, 0);
        v[kk][1] = live ? src[1] : make_uint4(0, 0, 0, 0);
    }
    uint32_t pa[16], pb[16];
#pragma unroll
    for (int h8 = 0; h8 < 2; ++h8) {
        const uint32_t wa[4] = {v[0][h8].x, v[0][h8].y, v[0][h8].z, v[0][h8].w};
        const uint32_t wb[4] = {v[1][h8].x, v[1][h8].y, v[1][h8].z, v[1][h8].w};
        const uint32_t wc[4] = {v[2][h8].x, v[2][h8].y, v[2][h8].z, v[2][h8].w};
        const uint32_t wd[4] = {v[3][h8].x, v[3][h8].y, v[3][h8].z, v[3][h8].w};
#pragma unroll
        for (int r = 0; r < 4; ++r) {  // register r holds dims 8 h8 + 2r, +1 of one key
            pa[8 * h8 + 2 * r] = prmt(wa[r], wb[r], 0x5410); pa[8 * h8 + 2 * r + 1] = prmt(wa[r], wb[r], 0x7632);
            pb[8 * h8 + 2 * r] = prmt(wc[r], wd[r], 0x5410); pb[8 * h8 + 2 * r + 1] = prmt(wc[r], wd[r], 0x7632);
        }
    }
#pragma unroll
    for (int mb = 0; mb < 8; ++mb) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma16816(acc.o[nb][mb], pa[mb], pa[8 + mb], pb[mb], pb[8 + mb], b0[nb], b1[nb]);
    }
}

// The work of one CTA: split `split` (P.nsplit = the open tile) of KV head `head`, row block `zb`; its partial goes
// to rows pidx .. pidx + 15 of the workspace.
template <int NB, bool kOther>
__device__ __forceinline__ void attn_cta(const AttnParams& P, int split, int head, int zb, int64_t pidx) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(smem_raw);
    const LayerView& L = P.L;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = L.q_heads / L.kv_heads;
    // ---- order of the first memory requests: the few bytes everything waits for (positions, q rows, page table
    //      entries) go out first, then the first page of every warp, then -- after the rotation of q, about a
    //      microsecond later -- the second page.  At short contexts the whole cache is requested in this first burst:
    //      requested in this order the small loads do not queue behind it and all first pages land before any second.
    uint16_t qraw[NB][4];
    int qpos[NB];
#pragma unroll
    for (int i = 0; i < NB; ++i) {  // warp w prepares rows w and w + 8 of the block
        const int R = zb * kRows + warp + kWarps * i, tq = R / G, gq = R % G;
        qpos[i] = -1;
        qraw[i][0] = qraw[i][1] = qraw[i][2] = qraw[i][3] = 0;
        if (tq < P.T) {
            const uint16_t* qrow = P.q + (static_cast<int64_t>(tq) * L.q_heads + head * G + gq) * D;
#pragma unroll
            for (int j = 0; j < 4; ++j) qraw[i][j] = qrow[lane + 32 * j];
            qpos[i] = P.pos[tq];
        }
    }
    const int kv_total = *P.total_pos + 1;
    const int key_end = min(P.key_end, kv_total), key_begin = max(P.key_begin, 0);
    const int sealed_pages = 2 * (kv_total / kTile);

    uint64_t* bars = sm.bars[warp];
    if (lane == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        mbar_fence_init();
    }
    const int32_t* tbl = L.table();
    auto issue = [&](int32_t page, int slot) {  // lane 0: four bulk copies of one page into a slot
        uint8_t* dst = sm.slots[warp][slot];
        mbar_expect_tx(&bars[slot], kPageBytes);
        bulk_g2s(dst + kKCodeOff, L.k_code + page_head_offset(64, L.kv_heads, page, head), 4096, &bars[slot]);
        bulk_g2s(dst + kVCodeOff, L.v_code + page_head_offset(64, L.kv_heads, page, head), 4096, &bars[slot]);
        bulk_g2s(dst + kKScaleOff, L.k_scale + page_head_offset(5, L.kv_heads, page, head), 640, &bars[slot]);
        bulk_g2s(dst + kVScaleOff, L.v_scale + page_head_offset(4, L.kv_heads, page, head), 512, &bars[slot]);
    };
    // Page table entries are read 32 at a time, one per lane, a full batch ahead of their use: lane l of `ids`
    // knows the physical page of logical page ids_base + l, `ids_next` the 32 after those.
    int w0 = 0, w1 = 0, ids_base = 0;
    int32_t ids = -1, ids_next = -1;
    auto load_ids = [&](int base) -> int32_t { return base + lane < w1 ? L.page_of(tbl, base + lane) : -1; };
    auto page_id = [&](int lp) -> int32_t {  // whole warp; lp in [ids_base, ids_base + 64)
        const int k = lp - ids_base;
        const int32_t a = __shfl_sync(0xffffffffu, ids, k & 31), b = __shfl_sync(0xffffffffu, ids_next, k & 31);
        return k < 32 ? a : b;
    };
    uint32_t ok_mask = 0;  // bit s: slot s holds a page in flight / ready
    int32_t second_page = -1;
    if (split < P.nsplit) {  // sealed pages of this CTA, then of this warp
        const int pb = min(key_begin / kPage, sealed_pages), pe = min((key_end + kPage - 1) / kPage, sealed_pages);
        const int n = max(pe - pb, 0);
        const int c0 = pb + static_cast<int>(static_cast<int64_t>(n) * split / P.nsplit);
        const int c1 = pb + static_cast<int>(static_cast<int64_t>(n) * (split + 1) / P.nsplit);
        // A warp that starts in the middle of a tile pays the per-tile set-up (scale transpose, q digits) for two
        // tiles where one would do: around one or two tiles per warp, warps take whole tiles (measured: 6 % faster at
        // 32,768 tokens; with longer ranges the extra set-up no longer shows and page granularity balances better).
        const int u0 = c0 >> 1, u1 = (c1 + 1) >> 1;  // tiles the CTA touches
        if (u1 - u0 >= kWarps - 1 && u1 - u0 <= 2 * kWarps) {
            w0 = max(c0, 2 * (u0 + (u1 - u0) * warp / kWarps));
            w1 = min(c1, 2 * (u0 + (u1 - u0) * (warp + 1) / kWarps));
            if (w1 < w0) w1 = w0;
        } else {
            w0 = c0 + (c1 - c0) * warp / kWarps;
            w1 = c0 + (c1 - c0) * (warp + 1) / kWarps;
        }
        ids_base = w0;
        ids = load_ids(w0);
        ids_next = load_ids(w0 + 32);
        const int32_t p0 = __shfl_sync(0xffffffffu, ids, 0), p1 = __shfl_sync(0xffffffffu, ids, 1);  // -1 beyond w1 or bad
        ok_mask = (p0 >= 0 ? 1u : 0u) | (p1 >= 0 ? 2u : 0u);
        second_page = p1;
        if (lane == 0 && p0 >= 0) issue(p0, 0);
    }

    // ---- q' = H q * scale * log2(e) for the rows of this block, stored in fragment order
#pragma unroll
    for (int i = 0; i < NB; ++i) {
        const int r = warp + kWarps * i;
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
    if (lane == 0 && second_page >= 0) issue(second_page, 1);
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
        for (int mb = 0; mb < 8; ++mb) acc.o[nb][mb][0] = acc.o[nb][mb][1] = acc.o[nb][mb][2] = acc.o[nb][mb][3] = 0.0f;
        acc.m[nb][0] = acc.m[nb][1] = -INFINITY;
        acc.l[nb][0] = acc.l[nb][1] = acc.z[nb][0] = acc.z[nb][1] = 0.0f;
    }
    QFrag<NB> qf;   // fp16 fragments for the open tile (stage rows)
    QInt<NB> qi;    // 8-bit digits for the quantised pages
    bool timed_out = false;

    if (split < P.nsplit) {
        uint8_t* scratch = sm.scratch[warp];
        uint32_t phase[2] = {0, 0};
        int cur_tile = -1;
        for (int lp = w0; lp < w1; ++lp) {
            const int slot = (lp - w0) & 1;
            if (lp - ids_base >= 32) {
                ids = ids_next;
                ids_base += 32;
                ids_next = load_ids(ids_base + 32);
            }
            const bool valid = (ok_mask >> slot) & 1u;
            if (valid) {
                if (!mbar_wait_bounded(&bars[slot], phase[slot])) { timed_out = true; break; }
                phase[slot] ^= 1u;
                const uint8_t* pg = sm.slots[warp][slot];
                if ((lp >> 1) != cur_tile) {  // per-dim scale / zero point are per tile (stored in both pages)
                    cur_tile = lp >> 1;
                    __syncwarp();
                    transpose_k_scale(pg + kKScaleOff, scratch, lane);
                    __syncwarp();
                    build_qint<NB>(sm, scratch, lane, qi);
                } else if constexpr (kOther) {
                    __syncwarp();
                    transpose_k_scale(pg + kKScaleOff, scratch, lane);
                    __syncwarp();
                }
                const int first = lp * kPage;
                const bool need_mask = first + kPage - 1 > min_lim || first < key_begin || first + kPage > key_end;
                float s[NB][4][4];
                qk_page<NB, kOther>(pg, scratch, qi, s, lane, need_mask, first, row_lim, key_begin, key_end);
                softmax_block<NB, 4>(s, acc);
                pv_page<NB>(pg, s, acc, lane);
            }
            // refill this slot with the page after next; the generic-proxy reads above must be ordered first
            __syncwarp();
            const int32_t np = lp + 2 < w1 ? page_id(lp + 2) : -1;
            const uint32_t nv = np >= 0 ? 1u : 0u;
            if (lane == 0 && nv) {
                fence_proxy_async();
                issue(np, slot);
            }
            ok_mask = (ok_mask & ~(1u << slot)) | (nv << slot);
        }
        if (timed_out) {
            if (lane == 0) L.flag(KVB_ERR_WAIT_TIMEOUT);
            // copies already issued must land before the CTA's shared memory is released: bounded second wait
            for (int s2 = 0; s2 < kSlots; ++s2)
                if ((ok_mask >> s2) & 1u) mbar_wait_bounded(&bars[s2], phase[s2]);
        }
    } else {
        // ---- open tile: warp w takes keys 16w .. 16w+15 of the tile, un-quantised, from the stage
        const int tile = kv_total / kTile, base = tile * kTile;
        const int first = base + 16 * warp;
        if (first < key_end && first + 16 > key_begin && first < kv_total) {
            build_qfrag<false, NB>(sm, nullptr, lane, qf);
            process_stage_group<NB>(L.stage_row(0, tile & 1, head, 16 * warp), L.stage_row(1, tile & 1, head, 16 * warp), qf,
                                    acc, lane, first, kv_total, row_lim, key_begin, key_end);
        }
    }

    // ---- merge the 8 warps of the CTA (log-sum-exp) and store one partial per row
    __syncthreads();  // every slot has been consumed: the ring memory becomes the merge buffer
    constexpr int kORow = D + 4, kWarpFloats = 3 * kRows + kRows * kORow;
    float* mbuf = reinterpret_cast<float*>(sm.slots) + warp * kWarpFloats;
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
        float* ob = mbuf + 3 * kRows + (8 * nb + 2 * t) * kORow + 16 * g;
#pragma unroll
        for (int e = 0; e < 4; ++e) {  // component e: row 2t + (e & 1), dims 16g + 8 (e >> 1) ..
            float* dst = ob + (e & 1) * kORow + (e >> 1) * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(acc.o[nb][0][e], acc.o[nb][1][e], acc.o[nb][2][e], acc.o[nb][3][e]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(acc.o[nb][4][e], acc.o[nb][5][e], acc.o[nb][6][e], acc.o[nb][7][e]);
        }
    }
    __syncthreads();
    const float* all = reinterpret_cast<const float*>(sm.slots);
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

template <int NB, bool kOther>
__global__ void __launch_bounds__(kThreads, 1) attn_kernel(const AttnParams P) {
    grid_dependency_wait();  // q, the positions and the cache come from the kernels before this one
    const int head = blockIdx.y, zb = blockIdx.z, split = blockIdx.x;
    attn_cta<NB, kOther>(P, split, head, zb, ((static_cast<int64_t>(head) * gridDim.z + zb) * (P.nsplit + 1) + split) * kRows);
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

template <int NB>
__global__ void __launch_bounds__(kThreads, 1) attn_batch_kernel(const BatchParams B) {
    grid_dependency_wait();
    const int part = blockIdx.x, head = blockIdx.y;
    const int b = batch_entry_of(B.plan, part);
    AttnParams P;
    P.L = B.layers[b];
    if ((P.L.head_dim != D || P.L.iters != 0) && threadIdx.x == 0) P.L.flag(KVB_ERR_GEOMETRY);  // results undefined, no fault
    P.q = B.q + static_cast<int64_t>(b) * P.L.q_heads * D;
    P.pos = B.pos + b;
    P.total_pos = B.pos + b;
    P.T = 1;
    P.scale_log2 = B.scale_log2;
    P.nsplit = B.plan.prefix[b + 1] - B.plan.prefix[b] - 1;
    P.key_begin = 0;
    P.key_end = INT_MAX;
    P.ws_m = B.ws_m;
    P.ws_l = B.ws_l;
    P.ws_o = B.ws_o;
    attn_cta<NB, false>(P, part - B.plan.prefix[b], head, 0, (static_cast<int64_t>(head) * gridDim.x + part) * kRows);
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
__device__ __forceinline__ void ring_store2(unsigned long long* p, float a, float b, uint32_t call) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(a)), "r"(call), "r"(__float_as_uint(b)),
                 "r"(call)
                 : "memory");
}
__device__ __forceinline__ uint4 ring_load2(const unsigned long long* p) {
    uint4 w;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ bool ring_arrived(const uint4& w, uint32_t call) { return w.y == call && w.w == call; }

__global__ void __launch_bounds__(kReduceWarps * 32) reduce_kernel(const float* __restrict__ ws_m, const float* __restrict__ ws_l,
                                                                  const float* __restrict__ ws_o, int parts, int T, int q_heads,
                                                                  int kv_heads, int zblocks, int dtype, uint16_t* __restrict__ out,
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
        const int R = tq * G + gq, zb = R / kRows, r = R % kRows;
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
        // (m, l) of every rank
        float rm[kRingMaxWorld], rl[kRingMaxWorld];
        uint32_t pending = everyone;
        while (pending != 0u && spins < push.max_spins) {
            uint4 w[kRingMaxWorld];
#pragma unroll
            for (int p = 0; p < kRingMaxWorld; ++p)
                if (pending >> p & 1u) w[p] = ring_load2(in + p * block + ml_off);
#pragma unroll
            for (int p = 0; p < kRingMaxWorld; ++p)
                if ((pending >> p & 1u) && ring_arrived(w[p], call)) {
                    rm[p] = __uint_as_float(w[p].x);
                    rl[p] = __uint_as_float(w[p].z);
                    pending &= ~(1u << p);
                }
            if (pending != 0u) { ++spins; __nanosleep(32); }
        }
        bool ok = pending == 0u;
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
            pending = everyone >> g & ((1u << kRingGroup) - 1u);
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

int zblocks_of(int q_heads, int kv_heads, int rows) { return (rows * (q_heads / kv_heads) + kRows - 1) / kRows; }

// Splits over the sealed pages: one CTA per SM in total, the open-tile CTAs included, at least one
// page per warp where the context is long enough.
int split_count(int kv_len_max, int kv_heads, int zblocks) {
    const int pages = 2 * (kv_len_max / kTile);
    const int per = kv_heads * zblocks;
    int n = (sm_count() - per) / per;
    n = n < 1 ? 1 : n;
    const int by_pages = (pages + 1) / 2;  // at least two pages per CTA
    if (n > by_pages) n = by_pages;
    if (n > kReduceWarps * kMaxPartsPerWarp - 1) n = kReduceWarps * kMaxPartsPerWarp - 1;  // reduce_kernel holds 64 parts
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
    if ((layer->head_dim != 128 || layer->sinkhorn_iters != 0) && push != nullptr)
        return fail(KVB_ERANGE, "%s: the sharded decode covers head_dim 128 caches written with sinkhorn_iters = 0", who);
    if (layer->head_dim != 128 || layer->sinkhorn_iters != 0)  // shapes outside the tuned kernels: general kernel, same semantics
        return launch_general_attention(layer, q, pos_dev, total_pos_dev, T, scale, kv_len_max, key_begin, key_end, workspace, out,
                                        part_m, part_l, part_o, stream);
    const int Z = zblocks_of(layer->q_heads, layer->kv_heads, T);
    const int nsplit = split_count(kv_len_max, layer->kv_heads, Z);
    const int parts = nsplit + 1;
    AttnParams P;
    P.L = make_view(*layer);
    P.q = static_cast<const uint16_t*>(q);
    P.pos = pos_dev;
    P.total_pos = total_pos_dev;
    P.T = T;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.nsplit = nsplit;
    P.key_begin = key_begin;
    P.key_end = key_end;
    const size_t rows = static_cast<size_t>(layer->kv_heads) * Z * parts * kRows;
    P.ws_m = static_cast<float*>(workspace);
    P.ws_l = P.ws_m + rows;
    P.ws_o = P.ws_l + rows;
    const bool upper = T * (layer->q_heads / layer->kv_heads) > 8;
    const int smem = static_cast<int>(sizeof(AttnSmem));
    static unsigned long long opted = 0;
    if (first_call_on_device(opted)) {
        KVB_CUDA_OK(cudaFuncSetAttribute(attn_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        KVB_CUDA_OK(cudaFuncSetAttribute(attn_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    const dim3 grid(parts, layer->kv_heads, Z);
    KVB_CUDA_OK(launch_early(upper ? attn_kernel<2, false> : attn_kernel<1, false>, grid, dim3(kThreads), smem, stream, P));
    const int total_rows = T * layer->q_heads;
    KVB_CUDA_OK(launch_early(reduce_kernel, dim3(total_rows), dim3(kReduceWarps * 32), 0, stream, P.ws_m, P.ws_l, P.ws_o, parts, T,
                             layer->q_heads, layer->kv_heads, Z, layer->dtype, static_cast<uint16_t*>(out), part_m, part_l, part_o,
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
    return kvb::split_count(kv_len_max, kv_heads, kvb::zblocks_of(q_heads, kv_heads, rows)) + 1;
}

extern "C" size_t kvb_workspace_bytes(int kv_len_max, int kv_heads, int q_heads, int head_dim, int rows, int batch) {
    if (kv_heads < 1 || q_heads < kv_heads || rows < 1 || batch < 1) return 0;
    const int Z = kvb::zblocks_of(q_heads, kv_heads, rows);
    const size_t parts = kvb::split_count(kv_len_max, kv_heads, Z) + 1;
    size_t bytes = static_cast<size_t>(kv_heads) * Z * parts * kvb::kRows * (head_dim + 2) * sizeof(float);
    const size_t general = kvb::general_workspace_bytes(kv_len_max, q_heads, head_dim, rows);
    if (general > bytes) bytes = general;
    if (rows * (q_heads / kv_heads) >= kDenseRows) {  // verify steps this wide run on the chunk-attention kernel
        const size_t dense = kvb_prefill_workspace_bytes(kv_len_max, kv_heads, q_heads, head_dim, rows);
        if (dense > bytes) bytes = dense;
    }
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

extern "C" int kvb_attn_decode_sharded(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale, int kv_len_max,
                                       void* workspace, const kvb_peer_ring* ring, void* out, void* stream) {
    using namespace kvb;
    if (ring == nullptr || ring->peer_bufs == nullptr || ring->local_buf == nullptr || ring->state == nullptr || out == nullptr)
        return fail(KVB_EINVAL, "kvb_attn_decode_sharded: null ring / buffers / out");
    if (ring->world < 1 || ring->world > kRingMaxWorld || ring->rank < 0 || ring->rank >= ring->world)
        return fail(KVB_EINVAL, "kvb_attn_decode_sharded: rank %d of world %d (1..%d ranks)", ring->rank, ring->world, kRingMaxWorld);
    PushTarget push{};
    for (int p = 0; p < ring->world; ++p) {
        if (ring->peer_bufs[p] == nullptr || (reinterpret_cast<uintptr_t>(ring->peer_bufs[p]) & 15u) != 0)
            return fail(KVB_EINVAL, "kvb_attn_decode_sharded: ring buffer of rank %d is null or not 16-byte aligned", p);
        push.peers[p] = static_cast<unsigned long long*>(ring->peer_bufs[p]);
    }
    if ((reinterpret_cast<uintptr_t>(ring->local_buf) & 15u) != 0)
        return fail(KVB_EINVAL, "kvb_attn_decode_sharded: local ring buffer is not 16-byte aligned");
    push.state = ring->state;
    push.local_buf = static_cast<const unsigned long long*>(ring->local_buf);
    push.max_spins = ring->max_spins ? ring->max_spins : (1u << 20);
    push.error_word = layer != nullptr ? layer->error_word : nullptr;
    push.rank = ring->rank;
    push.world = ring->world;
    return launch_attention(layer, q, pos_dev, pos_dev, 1, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), "kvb_attn_decode_sharded", &push);
}

// ---------------------------------------------------------------------------------------------------------
// Batched decode of independent sequences.
namespace kvb {
namespace {

static_assert(sizeof(LayerView) == sizeof(kvb_layer) && offsetof(LayerView, error_word) == offsetof(kvb_layer, error_word) &&
                  offsetof(LayerView, table_stride) == offsetof(kvb_layer, table_stride) &&
                  offsetof(LayerView, iters) == offsetof(kvb_layer, sinkhorn_iters),
              "the device reads kvb_layer structs as LayerView");

// Parts (splits over sealed pages + the open tile) of every sequence from the host's bounds of their lengths:
// about eight CTAs per SM in total, at least 16 pages per split, at most 63 splits per sequence.
int plan_batch(const int32_t* kv_len_max, int batch, int kv_heads, BatchPlan& plan) {
    int64_t total_pages = 0;
    for (int b = 0; b < batch; ++b) total_pages += 2 * (kv_len_max[b] / kTile);
    const int64_t want = std::max<int64_t>(batch, static_cast<int64_t>(8) * sm_count() / kv_heads);
    const int64_t chunk = std::max<int64_t>(16, (total_pages + want - 1) / want);
    plan.n = batch;
    plan.prefix[0] = 0;
    for (int b = 0; b < batch; ++b) {
        const int64_t pages = 2 * (kv_len_max[b] / kTile);
        int nsplit = static_cast<int>((pages + chunk - 1) / chunk);
        nsplit = std::min(std::max(nsplit, 1), kReduceWarps * kMaxPartsPerWarp - 1);
        plan.prefix[b + 1] = plan.prefix[b] + nsplit + 1;
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
    B.ws_m = static_cast<float*>(workspace);
    B.ws_l = B.ws_m + rows;
    B.ws_o = B.ws_l + rows;
    const int smem = static_cast<int>(sizeof(AttnSmem));
    static unsigned long long opted = 0;
    if (first_call_on_device(opted)) {
        KVB_CUDA_OK(cudaFuncSetAttribute(attn_batch_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        KVB_CUDA_OK(cudaFuncSetAttribute(attn_batch_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool upper = q_heads / kv_heads > 8;
    KVB_CUDA_OK(launch_early(upper ? attn_batch_kernel<2> : attn_batch_kernel<1>, dim3(total, kv_heads, 1), dim3(kThreads), smem, st, B));
    KVB_CUDA_OK(launch_early(reduce_kernel, dim3(batch * q_heads), dim3(kReduceWarps * 32), 0, st, B.ws_m, B.ws_l, B.ws_o, 0, batch, q_heads,
                             kv_heads, 1, dtype, static_cast<uint16_t*>(out), static_cast<float*>(nullptr), static_cast<float*>(nullptr),
                             static_cast<float*>(nullptr), PushTarget{}, B.plan));
    return KVB_OK;
}

namespace kvb {
int launch_chunk_attention(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int tokens, float scale,
                           int kv_len_max, void* workspace, void* out, cudaStream_t s);  // kvb_prefill.cu
}

extern "C" int kvb_attn_verify(const kvb_layer* layer, const void* q, const void* k, const void* v,
                               const int32_t* positions_dev, int width, float scale, int kv_len_max, void* workspace,
                               void* out, void* stream) {
    if (width < 1 || width > 8) return kvb::fail(KVB_ERANGE, "kvb_attn_verify: width %d (1..8; the reference rejects more, too)", width);
    if (int st = kvb::check_layer(layer, "kvb_attn_verify")) return st;
    if (int st = kvb_append(layer, k, v, positions_dev, width, stream)) return st;
    if (width * (layer->q_heads / layer->kv_heads) >= kDenseRows && layer->head_dim == 128 && layer->sinkhorn_iters == 0) {
        if (q == nullptr || workspace == nullptr || out == nullptr) return kvb::fail(KVB_EINVAL, "kvb_attn_verify: null q / workspace / out");
        return kvb::launch_chunk_attention(layer, q, positions_dev, width, scale, kv_len_max, workspace, out, static_cast<cudaStream_t>(stream));
    }
    return kvb::launch_attention(layer, q, positions_dev, positions_dev + (width - 1), width, scale, kv_len_max, 0, INT_MAX, workspace, out, nullptr, nullptr,
                                 nullptr, static_cast<cudaStream_t>(stream), "kvb_attn_verify");
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
