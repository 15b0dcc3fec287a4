// kvb_append.cu -- quantise-append into the paged pool, and the tile decode used for verification.
//
// One launch covers any token count: the grid is (tile slot of the append, kv head, K|V).  A CTA
// keeps the whole 128 x head_dim fp16 tile in shared memory, rotates the new rows into it with one
// warp per row (Walsh-Hadamard in registers + shuffles), and -- when the append completes the tile --
// quantises it in place: per-row min/max -> fp16 scale / zero-point -> 4-bit codes, written to the two
// pages of the tile with 128-bit stores.  There is no intermediate record and no bit-serial packing.
//
// Arithmetic that decides bytes (reference kvarn128_codec.cuh:188-217 == bee_oracle.cpp:328-341) is
// spelled with round-to-nearest intrinsics so that no multiply-add contraction can change a code:
//   scale = fmaxf((hi - lo) / 15, 1e-10f);  q = clamp(roundf((x - lo) / scale), 0, 15)
//   scale_axis = fp16(best_row * scale);  zp_axis = fp16(best_row * lo);  other_axis = fp16(best_col)
#include "kvb_common.cuh"

namespace kvb {
namespace {

constexpr int kThreads = 256;
constexpr int kRowPad = 8;  // halves of padding per staged row: keeps 128-bit row reads conflict-free

// Tile geometry of one append, derived on the device from the first and last position
// (reference kvarn128_launch.cu:53-77; positions are contiguous, single sequence).
struct AppendTile {
    int t0, tlast, tile, base, begin, end;
    bool in_range, sealed;
};

__device__ __forceinline__ AppendTile append_tile(int pos0, int last, int index) {
    AppendTile r;
    r.t0 = pos0 / kTile;
    r.tlast = last / kTile;
    r.tile = r.t0 + index;
    r.in_range = r.tile <= r.tlast;
    r.base = r.tile * kTile;
    r.begin = pos0 > r.base ? pos0 - r.base : 0;
    r.end = last + 1 < r.base + kTile ? last + 1 - r.base : kTile;
    r.sealed = r.base + kTile <= last + 1;
    return r;
}

template <int D> struct AppendSmem {
    static constexpr int S = D / kSlice;
    static constexpr int kStride = D + kRowPad;
    alignas(16) __half rows[kTile * kStride];  // rotated rows of the tile, fp16 (what the stage holds)
    alignas(16) uint8_t codes[kTile * (D / 2)];  // token-major code rows, both pages back to back
    float red_lo[4 * D];                    // partial minima / maxima of the row scan
    float red_hi[4 * D];
    float best_col[kSlice], best_row[kSlice];  // Sinkhorn factors of the slice being quantised
    float std_col[kSlice], std_row[kSlice], log_col[kSlice], log_row[kSlice], cur_col[kSlice], cur_row[kSlice];
    float rcp_col[kSlice], rcp_row[kSlice];  // 1 / cur_col, 1 / cur_row
    float scal[8];
    __half ax_scale[S * kSlice];            // scale_axis / zp_axis / other_axis of every slice
    __half ax_zp[S * kSlice];
    __half ax_other[S * kSlice];
    alignas(16) __half scale_page[2 * kPage * 5 * S];  // the two scale pages, assembled before the store
};

// Element (r, c) of the slice matrix: K has row = dim, col = token; V has row = token, col = dim
// (reference kvarn128_codec.cuh:366-379).
template <int D, bool kValue>
__device__ __forceinline__ float mat(const AppendSmem<D>& sm, int slice, int r, int c) {
    const int tok = kValue ? r : c, dim = kValue ? c : r;
    return __half2float(sm.rows[tok * AppendSmem<D>::kStride + slice * kSlice + dim]);
}

// Sinkhorn variance balancing, `iters` rounds, in the reference's order of updates
// (kvarn128_codec.cuh:104-186 == bee_oracle.cpp:210-255): columns, rows, then "keep the best so far".
// iters > 0 is the tolerance-checked regime (the reference's own CUDA kernel does not reproduce its host oracle
// byte for byte there either), so the standard deviations are computed the fast way: every thread of the CTA
// takes part, x / (s_col * s_row) becomes x * (1/s_col) * (1/s_row) with the reciprocals taken once per update
// and the factor of the reduced-over axis pulled out of the sums, and partial sums meet in shared memory.
// In memory terms a standard deviation runs either over the dims of a token (contiguous) or over the tokens of a
// dim (strided); which of the two is the "row" depends on K / V (see mat()).
template <int D, bool kValue>
__device__ void sinkhorn(AppendSmem<D>& sm, int slice, int iters) {
    constexpr int kStride = AppendSmem<D>::kStride;
    const int i = threadIdx.x;
    auto finish = [](float sum, float sq) {  // sample standard deviation of 128 values from their sum and sum of squares
        const float mean = sum * (1.0f / 128.0f);
        return sqrtf(fmaxf((sq - 128.0f * mean * mean) * (1.0f / 127.0f), 0.0f));
    };
    // out[tok] = std over the 128 dims of x[tok][dim] * rd[dim] * rt[tok]; thread = (token, half of the dims)
    auto std_over_dims = [&](float* out, const float* rt, const float* rd) {
        const int t = i & 127, hf = i >> 7;
        const __half* row = &sm.rows[t * kStride + slice * kSlice + hf * 64];
        float s0 = 0.0f, s1 = 0.0f, q0 = 0.0f, q1 = 0.0f;
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
            const uint4 pk = *reinterpret_cast<const uint4*>(row + j);
            const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float a = __low2float(h2[e]) * rd[hf * 64 + j + 2 * e], b = __high2float(h2[e]) * rd[hf * 64 + j + 2 * e + 1];
                s0 += a; q0 = fmaf(a, a, q0);
                s1 += b; q1 = fmaf(b, b, q1);
            }
        }
        sm.red_lo[hf * kTile + t] = s0 + s1;
        sm.red_hi[hf * kTile + t] = q0 + q1;
        __syncthreads();
        if (i < kSlice) {
            const float f = rt[i];
            out[i] = finish((sm.red_lo[i] + sm.red_lo[kTile + i]) * f, (sm.red_hi[i] + sm.red_hi[kTile + i]) * f * f);
        }
        __syncthreads();
    };
    // out[dim] = std over the 128 tokens; thread = (dim pair, quarter of the tokens)
    auto std_over_tokens = [&](float* out, const float* rt, const float* rd) {
        const int b = i & 63, qtr = i >> 6;
        float s0 = 0.0f, s1 = 0.0f, q0 = 0.0f, q1 = 0.0f;
#pragma unroll 8
        for (int c = qtr * 32; c < qtr * 32 + 32; ++c) {
            const __half2 h = *reinterpret_cast<const __half2*>(&sm.rows[c * kStride + slice * kSlice + 2 * b]);
            const float f = rt[c];
            const float x0 = __low2float(h) * f, x1 = __high2float(h) * f;
            s0 += x0; q0 = fmaf(x0, x0, q0);
            s1 += x1; q1 = fmaf(x1, x1, q1);
        }
        sm.red_lo[qtr * kSlice + 2 * b] = s0; sm.red_lo[qtr * kSlice + 2 * b + 1] = s1;
        sm.red_hi[qtr * kSlice + 2 * b] = q0; sm.red_hi[qtr * kSlice + 2 * b + 1] = q1;
        __syncthreads();
        if (i < kSlice) {
            const float f = rd[i];
            const float sum = (sm.red_lo[i] + sm.red_lo[kSlice + i]) + (sm.red_lo[2 * kSlice + i] + sm.red_lo[3 * kSlice + i]);
            const float sq = (sm.red_hi[i] + sm.red_hi[kSlice + i]) + (sm.red_hi[2 * kSlice + i] + sm.red_hi[3 * kSlice + i]);
            out[i] = finish(sum * f, sq * f * f);
        }
        __syncthreads();
    };
    // K: row = dim, col = token.  V: row = token, col = dim.
    auto col_std = [&]() {
        if constexpr (kValue) std_over_tokens(sm.std_col, sm.rcp_row, sm.rcp_col);
        else std_over_dims(sm.std_col, sm.rcp_col, sm.rcp_row);
    };
    auto row_std = [&]() {
        if constexpr (kValue) std_over_dims(sm.std_row, sm.rcp_row, sm.rcp_col);
        else std_over_tokens(sm.std_row, sm.rcp_col, sm.rcp_row);
    };
    auto keep_best = [&]() {  // imbalance of the current factors; "<=" lets a later tie win
        if (i < 32) {
            float cmin = 3.402823466e+38f, cmax = 0.0f, rmin = 3.402823466e+38f, rmax = 0.0f;
#pragma unroll
            for (int j = i; j < kSlice; j += 32) {
                cmin = fminf(cmin, sm.std_col[j]); cmax = fmaxf(cmax, sm.std_col[j]);
                rmin = fminf(rmin, sm.std_row[j]); rmax = fmaxf(rmax, sm.std_row[j]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                cmin = fminf(cmin, __shfl_xor_sync(0xffffffffu, cmin, o)); cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
                rmin = fminf(rmin, __shfl_xor_sync(0xffffffffu, rmin, o)); rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
            }
            if (i == 0) {
                const float imb = __fadd_rn(__fdiv_rn(cmax, fmaxf(cmin, 1e-8f)), __fdiv_rn(rmax, fmaxf(rmin, 1e-8f)));
                sm.scal[1] = imb <= sm.scal[0] ? 1.0f : 0.0f;
                if (imb <= sm.scal[0]) sm.scal[0] = imb;
            }
        }
        __syncthreads();
        if (i < kSlice && sm.scal[1] != 0.0f) { sm.best_col[i] = sm.cur_col[i]; sm.best_row[i] = sm.cur_row[i]; }
        __syncthreads();
    };
    if (i < kSlice) {
        sm.log_col[i] = sm.log_row[i] = 0.0f;
        sm.cur_col[i] = sm.cur_row[i] = sm.best_col[i] = sm.best_row[i] = 1.0f;
        sm.rcp_col[i] = sm.rcp_row[i] = 1.0f;
    }
    if (i == 0) sm.scal[0] = 3.402823466e+38f;
    __syncthreads();
    if (iters <= 0) return;
    col_std();
    row_std();
    keep_best();
    for (int it = 0; it < iters; ++it) {
        if (i < kSlice) {
            const float c = fminf(fmaxf(sm.std_col[i], 1e-3f), 1e3f);
            sm.log_col[i] = fminf(fmaxf(__fadd_rn(sm.log_col[i], logf(c)), -0.3f), 10.0f);
            sm.cur_col[i] = expf(sm.log_col[i]);
            sm.rcp_col[i] = __fdiv_rn(1.0f, sm.cur_col[i]);
        }
        __syncthreads();
        row_std();
        if (i < kSlice) {
            const float r = fminf(fmaxf(sm.std_row[i], 1e-3f), 1e3f);
            sm.log_row[i] = fminf(fmaxf(__fadd_rn(sm.log_row[i], logf(r)), -0.3f), 10.0f);
            sm.cur_row[i] = expf(sm.log_row[i]);
            sm.rcp_row[i] = __fdiv_rn(1.0f, sm.cur_row[i]);
        }
        __syncthreads();
        row_std();
        col_std();
        keep_best();
    }
}

__device__ __forceinline__ float quant_scale(float lo, float hi) {
    return fmaxf(__fdiv_rn(__fsub_rn(hi, lo), 15.0f), 1e-10f);
}
__device__ __forceinline__ uint32_t quant_code(float x, float lo, float scale) {
    return static_cast<uint32_t>(fminf(fmaxf(roundf(__fdiv_rn(__fsub_rn(x, lo), scale)), 0.0f), 15.0f));
}

// Quantise slice `slice` of the staged tile.  kSink = false is the iters == 0 regime (all factors 1,
// x == v exactly); kSink = true divides by the Sinkhorn factors first.
template <int D, bool kValue, bool kSink>
__device__ void quantize_slice(AppendSmem<D>& sm, int slice) {
    constexpr int kStride = AppendSmem<D>::kStride;
    const int tid = threadIdx.x;
    if constexpr (!kValue) {
        // K: row = dim.  Thread = (dim pair b, token quarter).
        const int b = tid & 63, qtr = tid >> 6, r0 = 2 * b;
        float lo0 = 3.402823466e+38f, hi0 = -3.402823466e+38f, lo1 = lo0, hi1 = hi0;
        float br0 = 1.0f, br1 = 1.0f;
        if constexpr (kSink) { br0 = sm.best_row[r0]; br1 = sm.best_row[r0 + 1]; }
        for (int c = qtr * 32; c < qtr * 32 + 32; ++c) {
            const __half2 h = *reinterpret_cast<const __half2*>(&sm.rows[c * kStride + slice * kSlice + r0]);
            float x0 = __low2float(h), x1 = __high2float(h);
            if constexpr (kSink) {
                x0 = __fdiv_rn(x0, __fmul_rn(sm.best_col[c], br0));
                x1 = __fdiv_rn(x1, __fmul_rn(sm.best_col[c], br1));
            }
            lo0 = fminf(lo0, x0); hi0 = fmaxf(hi0, x0);
            lo1 = fminf(lo1, x1); hi1 = fmaxf(hi1, x1);
        }
        sm.red_lo[qtr * D + r0] = lo0; sm.red_hi[qtr * D + r0] = hi0;
        sm.red_lo[qtr * D + r0 + 1] = lo1; sm.red_hi[qtr * D + r0 + 1] = hi1;
        __syncthreads();
        lo0 = fminf(fminf(sm.red_lo[r0], sm.red_lo[D + r0]), fminf(sm.red_lo[2 * D + r0], sm.red_lo[3 * D + r0]));
        hi0 = fmaxf(fmaxf(sm.red_hi[r0], sm.red_hi[D + r0]), fmaxf(sm.red_hi[2 * D + r0], sm.red_hi[3 * D + r0]));
        lo1 = fminf(fminf(sm.red_lo[r0 + 1], sm.red_lo[D + r0 + 1]), fminf(sm.red_lo[2 * D + r0 + 1], sm.red_lo[3 * D + r0 + 1]));
        hi1 = fmaxf(fmaxf(sm.red_hi[r0 + 1], sm.red_hi[D + r0 + 1]), fmaxf(sm.red_hi[2 * D + r0 + 1], sm.red_hi[3 * D + r0 + 1]));
        const float s0 = quant_scale(lo0, hi0), s1 = quant_scale(lo1, hi1);
        for (int c = qtr * 32; c < qtr * 32 + 32; ++c) {
            const __half2 h = *reinterpret_cast<const __half2*>(&sm.rows[c * kStride + slice * kSlice + r0]);
            float x0 = __low2float(h), x1 = __high2float(h);
            if constexpr (kSink) {
                x0 = __fdiv_rn(x0, __fmul_rn(sm.best_col[c], br0));
                x1 = __fdiv_rn(x1, __fmul_rn(sm.best_col[c], br1));
            }
            sm.codes[c * (D / 2) + slice * 64 + b] =
                static_cast<uint8_t>(quant_code(x0, lo0, s0) | (quant_code(x1, lo1, s1) << 4));
        }
        if (qtr == 0) {
            sm.ax_scale[slice * kSlice + r0] = __float2half_rn(__fmul_rn(br0, s0));
            sm.ax_scale[slice * kSlice + r0 + 1] = __float2half_rn(__fmul_rn(br1, s1));
            sm.ax_zp[slice * kSlice + r0] = __float2half_rn(__fmul_rn(br0, lo0));
            sm.ax_zp[slice * kSlice + r0 + 1] = __float2half_rn(__fmul_rn(br1, lo1));
        }
        if (tid < kSlice) sm.ax_other[slice * kSlice + tid] = __float2half_rn(kSink ? sm.best_col[tid] : 1.0f);
    } else {
        // V: row = token.  Thread = (token, half of the slice's dims).
        const int t = tid & 127, hf = tid >> 7;
        const __half* row = &sm.rows[t * kStride + slice * kSlice + hf * 64];
        float br = 1.0f;
        if constexpr (kSink) br = sm.best_row[t];
        float lo = 3.402823466e+38f, hi = -3.402823466e+38f;
        for (int j = 0; j < 64; j += 8) {
            const uint4 pk = *reinterpret_cast<const uint4*>(row + j);
            const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x0 = __low2float(h2[e]), x1 = __high2float(h2[e]);
                if constexpr (kSink) {
                    x0 = __fdiv_rn(x0, __fmul_rn(sm.best_col[hf * 64 + j + 2 * e], br));
                    x1 = __fdiv_rn(x1, __fmul_rn(sm.best_col[hf * 64 + j + 2 * e + 1], br));
                }
                lo = fminf(lo, fminf(x0, x1));
                hi = fmaxf(hi, fmaxf(x0, x1));
            }
        }
        sm.red_lo[hf * kTile + t] = lo; sm.red_hi[hf * kTile + t] = hi;
        __syncthreads();
        lo = fminf(sm.red_lo[t], sm.red_lo[kTile + t]);
        hi = fmaxf(sm.red_hi[t], sm.red_hi[kTile + t]);
        const float sc = quant_scale(lo, hi);
        uint32_t words[8];
        for (int j = 0; j < 64; j += 8) {
            const uint4 pk = *reinterpret_cast<const uint4*>(row + j);
            const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
            uint32_t w = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x0 = __low2float(h2[e]), x1 = __high2float(h2[e]);
                if constexpr (kSink) {
                    x0 = __fdiv_rn(x0, __fmul_rn(sm.best_col[hf * 64 + j + 2 * e], br));
                    x1 = __fdiv_rn(x1, __fmul_rn(sm.best_col[hf * 64 + j + 2 * e + 1], br));
                }
                w |= (quant_code(x0, lo, sc) | (quant_code(x1, lo, sc) << 4)) << (8 * e);
            }
            words[j / 8] = w;
        }
        uint4* dst = reinterpret_cast<uint4*>(&sm.codes[t * (D / 2) + slice * 64 + hf * 32]);
        dst[0] = make_uint4(words[0], words[1], words[2], words[3]);
        dst[1] = make_uint4(words[4], words[5], words[6], words[7]);
        if (hf == 0) {
            sm.ax_scale[slice * kSlice + t] = __float2half_rn(__fmul_rn(br, sc));
            sm.ax_zp[slice * kSlice + t] = __float2half_rn(__fmul_rn(br, lo));
        }
        if (tid < kSlice) sm.ax_other[slice * kSlice + tid] = __float2half_rn(kSink ? sm.best_col[tid] : 1.0f);
    }
    __syncthreads();
}

// phase 0: rotate + stage + seal.  phase 1: stage rows of tiles whose stage slot could still be read by
// the first tile's CTA during phase 0 (only launched when the append can span three tiles or more).
//
// Which tiles keep their rows in the stage: only the last two tiles of an append (one per slot) can be
// looked at again -- the open tile by attention and later appends, the one before it by a roll-back that
// re-opens it.  Earlier tiles of a long append would be overwritten within the same call anyway.
template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads) append_kernel(LayerView L, const uint16_t* __restrict__ k,
                                                          const uint16_t* __restrict__ v,
                                                          const int32_t* __restrict__ positions, int tokens,
                                                          int phase) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    AppendSmem<D>& sm = *reinterpret_cast<AppendSmem<D>*>(smem_raw);
    using G = Geo<D>;
    constexpr int kStride = AppendSmem<D>::kStride;
    const int pos0 = positions[0], last = positions[tokens - 1];
    if (pos0 < 0 || last - pos0 != tokens - 1) {  // positions must be contiguous and non-negative
        if (threadIdx.x == 0) L.flag(KVB_ERR_POSITIONS);
        return;
    }
    const AppendTile t = append_tile(pos0, last, blockIdx.x);
    if (!t.in_range) return;
    const int head = blockIdx.y, which = blockIdx.z, slot = t.tile & 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool keeps_stage = t.tile >= t.tlast - 1;
    const bool early = t.tile <= t.t0 + 1;  // no other CTA of phase 0 touches this tile's stage slot
    if (phase == 1 && (!keeps_stage || early)) return;
    const bool write_stage = keeps_stage && (phase == 1 || early);
    const bool seal = t.sealed && phase == 0;
    if (!seal && !write_stage) return;

    // rows appended by earlier calls (first tile only) come from the stage
    if (seal && t.begin > 0) {
        const __half* src = L.stage_row(which, slot, head, 0);
        for (int i = threadIdx.x; i < t.begin * (D / 8); i += kThreads) {
            const int r = i / (D / 8), c = i % (D / 8);
            *reinterpret_cast<uint4*>(&sm.rows[r * kStride + c * 8]) =
                *reinterpret_cast<const uint4*>(src + static_cast<int64_t>(r) * D + c * 8);
        }
    }
    // new rows: one warp per row, lane l holds dims l + 32 r.  A warp has up to 16 rows of the tile: it reads them
    // eight at a time before rotating any, so that it waits for global memory twice, not sixteen times.
    const uint16_t* src = which ? v : k;
    constexpr int kBatch = 8, kWarpsPerCta = kThreads / 32;
    for (int t0 = t.begin + warp; t0 < t.end; t0 += kBatch * kWarpsPerCta) {
        uint16_t raw[kBatch][D / 32];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int tt = t0 + u * kWarpsPerCta;
            if (tt < t.end) {
                const uint16_t* row = src + (static_cast<int64_t>(t.base + tt - pos0) * L.kv_heads + head) * D;
#pragma unroll
                for (int r = 0; r < D / 32; ++r) raw[u][r] = row[lane + 32 * r];
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int tt = t0 + u * kWarpsPerCta;
            if (tt >= t.end) break;
            float val[D / 32];
#pragma unroll
            for (int r = 0; r < D / 32; ++r) val[r] = in_to_f32<kBf16>(raw[u][r]);
            hadamard_warp<D>(val, lane);
            __half* st = L.stage_row(which, slot, head, tt);
#pragma unroll
            for (int r = 0; r < D / 32; ++r) {
                const __half h = __float2half_rn(val[r]);
                sm.rows[tt * kStride + lane + 32 * r] = h;
                if (write_stage) st[lane + 32 * r] = h;
            }
        }
    }
    if (!seal) return;
    __syncthreads();

    const int32_t* tbl = L.table();
    const int32_t page0 = L.page_of(tbl, 2 * t.tile), page1 = L.page_of(tbl, 2 * t.tile + 1);
    if (page0 < 0 || page1 < 0) return;  // error word already set; skip the tile instead of faulting

    for (int s = 0; s < G::S; ++s) {
        if (L.iters > 0) {
            if (which) { sinkhorn<D, true>(sm, s, L.iters); quantize_slice<D, true, true>(sm, s); }
            else { sinkhorn<D, false>(sm, s, L.iters); quantize_slice<D, false, true>(sm, s); }
        } else {
            if (which) quantize_slice<D, true, false>(sm, s);
            else quantize_slice<D, false, false>(sm, s);
        }
    }

    // code rows -> the two pages (each page-head is one contiguous run of the plane)
    uint8_t* code = which ? L.v_code : L.k_code;
    for (int i = threadIdx.x; i < 2 * G::kCodePageBytes / 16; i += kThreads) {
        const int pg = i / (G::kCodePageBytes / 16), o = i % (G::kCodePageBytes / 16);
        uint8_t* dst = code + page_head_offset(G::kCodeLeading, L.kv_heads, pg ? page1 : page0, head);
        reinterpret_cast<uint4*>(dst)[o] = reinterpret_cast<const uint4*>(sm.codes + pg * G::kCodePageBytes)[o];
    }
    // scale pages: dim-axis entries go to both pages, token-axis entries to the page of the token
    const int SL = which ? G::kVScaleLeading : G::kKScaleLeading;
    constexpr int c = G::kAxisCols, S = G::S;
    for (int i = threadIdx.x; i < 2 * kPage * SL; i += kThreads) {
        const int pg = i / (kPage * SL), r = (i / SL) % kPage, j = i % SL, tok = pg * kPage + r;
        __half h;
        if (!which) {
            if (j < c) h = sm.ax_scale[c * r + j];
            else if (j < 2 * c) h = sm.ax_zp[c * r + j - c];
            else h = sm.ax_other[(j - 2 * c) * kSlice + tok];
        } else {
            if (j < c) h = sm.ax_other[c * r + j];
            else if (j < c + S) h = sm.ax_scale[(j - c) * kSlice + tok];
            else h = sm.ax_zp[(j - c - S) * kSlice + tok];
        }
        sm.scale_page[i] = h;
    }
    __syncthreads();
    __half* scale = which ? L.v_scale : L.k_scale;
    const int page_halves = kPage * SL;
    for (int i = threadIdx.x; i < 2 * page_halves / 8; i += kThreads) {
        const int pg = i / (page_halves / 8), o = i % (page_halves / 8);
        __half* dst = scale + page_head_offset(SL, L.kv_heads, pg ? page1 : page0, head);
        reinterpret_cast<uint4*>(dst)[o] = reinterpret_cast<const uint4*>(sm.scale_page + pg * page_halves)[o];
    }
}

// One tile of one head -> rotated-domain fp16 [128][D]: val = (q * scale_axis + zp_axis) * other_axis,
// each step rounded (reference kvarn128_codec.cuh:314-350).
template <int D>
__global__ void __launch_bounds__(kThreads) decode_tile_kernel(LayerView L, int tile, int head, __half* out_k,
                                                               __half* out_v) {
    using G = Geo<D>;
    constexpr int c = G::kAxisCols, S = G::S;
    const int32_t* tbl = L.table();
    for (int i = threadIdx.x; i < kTile * D; i += kThreads) {
        const int tok = i / D, d = i % D, s = d / kSlice;
        const int32_t page = L.page_of(tbl, 2 * tile + tok / kPage);
        if (page < 0) continue;
        const int off = tok % kPage;
        const int64_t cb = page_head_offset(G::kCodeLeading, L.kv_heads, page, head) + off * G::kCodeLeading + d / 2;
        const int sh = (d & 1) * 4;
        const float qk = static_cast<float>((L.k_code[cb] >> sh) & 15), qv = static_cast<float>((L.v_code[cb] >> sh) & 15);
        const __half* ks = L.k_scale + page_head_offset(G::kKScaleLeading, L.kv_heads, page, head);
        const __half* vs = L.v_scale + page_head_offset(G::kVScaleLeading, L.kv_heads, page, head);
        const float ksa = __half2float(ks[G::kKScaleLeading * (d / c) + d % c]);
        const float kzp = __half2float(ks[G::kKScaleLeading * (d / c) + c + d % c]);
        const float koa = __half2float(ks[G::kKScaleLeading * off + 2 * c + s]);
        const float voa = __half2float(vs[G::kVScaleLeading * (d / c) + d % c]);
        const float vsa = __half2float(vs[G::kVScaleLeading * off + c + s]);
        const float vzp = __half2float(vs[G::kVScaleLeading * off + c + S + s]);
        out_k[i] = __float2half_rn(__fmul_rn(__fadd_rn(__fmul_rn(qk, ksa), kzp), koa));
        out_v[i] = __float2half_rn(__fmul_rn(__fadd_rn(__fmul_rn(qv, vsa), vzp), voa));
    }
}

template <int D, bool kBf16>
int launch_append(const LayerView& V, const void* k, const void* v, const int32_t* positions, int tokens,
                  cudaStream_t stream) {
    static unsigned long long opted = 0;  // per template instance; setting the attribute again is harmless
    const int smem = static_cast<int>(sizeof(AppendSmem<D>));
    if (first_call_on_device(opted)) {
        KVB_CUDA_OK(cudaFuncSetAttribute(append_kernel<D, kBf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    const dim3 grid(tokens / kTile + 2, V.kv_heads, 2);
    append_kernel<D, kBf16><<<grid, kThreads, smem, stream>>>(V, static_cast<const uint16_t*>(k),
                                                             static_cast<const uint16_t*>(v), positions, tokens, 0);
    KVB_CUDA_OK(cudaGetLastError());
    if (tokens > kTile) {  // only then can an append touch three tiles
        append_kernel<D, kBf16><<<grid, kThreads, smem, stream>>>(V, static_cast<const uint16_t*>(k),
                                                                 static_cast<const uint16_t*>(v), positions, tokens, 1);
        KVB_CUDA_OK(cudaGetLastError());
    }
    return KVB_OK;
}

}  // namespace
}  // namespace kvb

extern "C" int kvb_append(const kvb_layer* layer, const void* k, const void* v, const int32_t* positions_dev,
                          int tokens, void* stream) {
    using namespace kvb;
    if (tokens == 0) return KVB_OK;  // the reference returns silently for an empty append
    if (int st = check_layer(layer, "kvb_append")) return st;
    if (tokens < 0) return fail(KVB_EINVAL, "kvb_append: tokens = %d", tokens);
    if (k == nullptr || v == nullptr || positions_dev == nullptr)
        return fail(KVB_EINVAL, "kvb_append: null k / v / positions");
    if (layer->stage == nullptr) return fail(KVB_EINVAL, "kvb_append: layer has no stage buffer");
    const LayerView V = make_view(*layer);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool bf = layer->dtype == KVB_DTYPE_BF16;
    if (layer->head_dim == 128) return bf ? launch_append<128, true>(V, k, v, positions_dev, tokens, s)
                                          : launch_append<128, false>(V, k, v, positions_dev, tokens, s);
    return bf ? launch_append<256, true>(V, k, v, positions_dev, tokens, s)
              : launch_append<256, false>(V, k, v, positions_dev, tokens, s);
}

extern "C" int kvb_decode_tile(const kvb_layer* layer, int tile, int head, void* out_k, void* out_v, void* stream) {
    using namespace kvb;
    if (int st = check_layer(layer, "kvb_decode_tile")) return st;
    if (out_k == nullptr || out_v == nullptr) return fail(KVB_EINVAL, "kvb_decode_tile: null output");
    if (tile < 0 || head < 0 || head >= layer->kv_heads || 2 * tile + 1 >= layer->table_len)
        return fail(KVB_EINVAL, "kvb_decode_tile: tile %d / head %d out of range", tile, head);
    const LayerView V = make_view(*layer);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (layer->head_dim == 128)
        decode_tile_kernel<128><<<1, kThreads, 0, s>>>(V, tile, head, static_cast<__half*>(out_k), static_cast<__half*>(out_v));
    else
        decode_tile_kernel<256><<<1, kThreads, 0, s>>>(V, tile, head, static_cast<__half*>(out_k), static_cast<__half*>(out_v));
    KVB_CUDA_OK(cudaGetLastError());
    return KVB_OK;
}
