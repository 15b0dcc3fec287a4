// kvb_attn_general.cu -- attention over the quantised cache for the shapes the tuned kernels do not cover:
// head_dim 256 (two 128-dim slices, the reference engine's own geometry) and, for prefill chunks and verify steps
// of 32 merged rows or more, caches written with Sinkhorn iterations > 0 (per-key and per-dim `other` factors
// different from 1; decode and narrower verify steps of such caches run on the int8 kernel).  Same semantics and
// the same entry points; a plain CUDA-core kernel: one CTA per (key range, KV head, query token), one warp per key, every
// element de-quantised as (q * scale_axis + zp_axis) * other_axis in fp32 (reference kvarn128_codec.cuh:331-347),
// fp32 dot products with warp-shuffle reductions, running softmax per warp, log-sum-exp merges at the end.
// Lane l owns the contiguous dims R l .. R l + R - 1 (R = head_dim / 32): its codes of a key are one 16- or 32-bit
// word, its per-dim factors stay in registers for a page, its query values for the whole call.
#include <climits>

#include "kvb_common.cuh"

namespace kvb {
namespace {

constexpr int kGWarps = 8, kGThreads = kGWarps * 32, kMaxG = 8;

struct GeneralParams {
    LayerView L;
    const uint16_t* q;         // [T][q_heads][D]
    const int32_t* pos;        // [T]
    const int32_t* total_pos;
    int T, nsplit, key_begin, key_end;
    float scale;
    float* ws_m;               // [T][H][nsplit][G]
    float* ws_l;
    float* ws_o;               // [T][H][nsplit][G][D]
};

template <int DD> struct GeneralSmem {
    float q[kMaxG][DD];        // rotated, scaled query rows of this KV head
    float wm[kGWarps][kMaxG], wl[kGWarps][kMaxG];
    float wo[kGWarps][kMaxG][DD];
};

template <int DD>
__global__ void __launch_bounds__(kGThreads) general_attn_kernel(const GeneralParams P) {
    using Geo_ = Geo<DD>;
    constexpr int R = DD / 32, S = Geo_::S, c = Geo_::kAxisCols;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    GeneralSmem<DD>& sm = *reinterpret_cast<GeneralSmem<DD>*>(smem_raw);
    const LayerView& L = P.L;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x, head = blockIdx.y, tq = blockIdx.z;
    const int G = L.q_heads / L.kv_heads;
    const int kv_total = *P.total_pos + 1;
    const int my_pos = P.pos[tq];
    const int key_end = min(min(P.key_end, kv_total), my_pos + 1), key_begin = max(P.key_begin, 0);

    for (int g = warp; g < G; g += kGWarps) {  // q' = H q * scale
        const uint16_t* qrow = P.q + (static_cast<int64_t>(tq) * L.q_heads + head * G + g) * DD;
        float v[R];
#pragma unroll
        for (int j = 0; j < R; ++j)
            v[j] = L.dtype == KVB_DTYPE_BF16 ? in_to_f32<true>(qrow[lane + 32 * j]) : in_to_f32<false>(qrow[lane + 32 * j]);
        hadamard_warp<DD>(v, lane);
#pragma unroll
        for (int j = 0; j < R; ++j) sm.q[g][lane + 32 * j] = v[j] * P.scale;
    }
    float m[kMaxG], l[kMaxG], o[kMaxG][R];
#pragma unroll
    for (int g = 0; g < kMaxG; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < R; ++j) o[g][j] = 0.0f;
    }
    __syncthreads();
    float qr[kMaxG][R];  // this lane's dims of the query rows
#pragma unroll
    for (int g = 0; g < kMaxG; ++g)
#pragma unroll
        for (int j = 0; j < R; ++j) qr[g][j] = g < G ? sm.q[g][R * lane + j] : 0.0f;
    auto attend = [&](const float (&kv)[R], const float (&vv)[R]) {  // one key against the G query rows
#pragma unroll
        for (int g = 0; g < kMaxG; ++g) {
            if (g >= G) break;
            float dot = 0.0f;
#pragma unroll
            for (int j = 0; j < R; ++j) dot = fmaf(qr[g][j], kv[j], dot);
#pragma unroll
            for (int sft = 16; sft > 0; sft >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, sft);
            const float mn = fmaxf(m[g], dot), a = __expf(m[g] - mn), p = __expf(dot - mn);
            m[g] = mn;
            l[g] = l[g] * a + p;
#pragma unroll
            for (int j = 0; j < R; ++j) o[g][j] = fmaf(o[g][j], a, p * vv[j]);
        }
    };

    const int sealed_end = (kv_total / kTile) * kTile;  // keys below this are in pages
    const int32_t* tbl = L.table();
    // pages of this split (the last split also takes the open tile)
    const int pb = min(key_begin, sealed_end) / kPage, pe = (min(key_end, sealed_end) + kPage - 1) / kPage;
    const int n = max(pe - pb, 0);
    const int p0 = pb + static_cast<int>(static_cast<int64_t>(n) * split / P.nsplit);
    const int p1 = pb + static_cast<int>(static_cast<int64_t>(n) * (split + 1) / P.nsplit);
    __syncthreads();
    for (int lp = p0; lp < p1; ++lp) {
        const int32_t page = L.page_of(tbl, lp);
        if (page < 0) continue;
        const __half* ks = L.k_scale + page_head_offset(Geo_::kKScaleLeading, L.kv_heads, page, head);
        const __half* vs = L.v_scale + page_head_offset(Geo_::kVScaleLeading, L.kv_heads, page, head);
        float ksc[R], kzp[R], vot[R];  // per-dim factors of the tile for this lane's dims (the same in both pages)
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const int d = R * lane + j;
            ksc[j] = __half2float(ks[Geo_::kKScaleLeading * (d / c) + d % c]);
            kzp[j] = __half2float(ks[Geo_::kKScaleLeading * (d / c) + c + d % c]);
            vot[j] = __half2float(vs[Geo_::kVScaleLeading * (d / c) + d % c]);
        }
        const int s = (R * lane) / kSlice;  // the slice this lane's dims lie in
        const uint8_t* kc = L.k_code + page_head_offset(Geo_::kCodeLeading, L.kv_heads, page, head);
        const uint8_t* vc = L.v_code + page_head_offset(Geo_::kCodeLeading, L.kv_heads, page, head);
        // the warp's eight keys of the page: every load is issued before the first key is used
        constexpr int kKeys = kPage / kGWarps;
        uint32_t wk[kKeys], wv[kKeys];  // R codes of 4 bits, dim R lane + j at bits 4 j
        __half ko[kKeys], vsa[kKeys], vzp[kKeys];
#pragma unroll
        for (int u = 0; u < kKeys; ++u) {
            const int off = warp + kGWarps * u;
            if constexpr (R == 8) {
                wk[u] = *reinterpret_cast<const uint32_t*>(kc + off * Geo_::kCodeLeading + 4 * lane);
                wv[u] = *reinterpret_cast<const uint32_t*>(vc + off * Geo_::kCodeLeading + 4 * lane);
            } else {
                wk[u] = *reinterpret_cast<const uint16_t*>(kc + off * Geo_::kCodeLeading + 2 * lane);
                wv[u] = *reinterpret_cast<const uint16_t*>(vc + off * Geo_::kCodeLeading + 2 * lane);
            }
            ko[u] = ks[Geo_::kKScaleLeading * off + 2 * c + s];
            vsa[u] = vs[Geo_::kVScaleLeading * off + c + s];
            vzp[u] = vs[Geo_::kVScaleLeading * off + c + S + s];
        }
#pragma unroll
        for (int u = 0; u < kKeys; ++u) {
            const int p = lp * kPage + warp + kGWarps * u;
            if (p < key_begin || p >= key_end) continue;  // warp-uniform
            const float kof = __half2float(ko[u]), vsf = __half2float(vsa[u]), vzf = __half2float(vzp[u]);
            float kv[R], vv[R];
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const float qk = static_cast<float>((wk[u] >> (4 * j)) & 15u), qv = static_cast<float>((wv[u] >> (4 * j)) & 15u);
                kv[j] = __fmul_rn(__fadd_rn(__fmul_rn(qk, ksc[j]), kzp[j]), kof);
                vv[j] = __fmul_rn(__fadd_rn(__fmul_rn(qv, vsf), vzf), vot[j]);
            }
            attend(kv, vv);
        }
    }
    if (split == P.nsplit - 1) {  // open tile: un-quantised rows of the stage
        const int tile = kv_total / kTile;
        for (int tt = warp; sealed_end + tt < kv_total; tt += kGWarps) {
            const int p = sealed_end + tt;
            if (p < key_begin || p >= key_end) continue;
            const __half* kr = L.stage_row(0, tile & 1, head, tt);
            const __half* vr = L.stage_row(1, tile & 1, head, tt);
            float kv[R], vv[R];
#pragma unroll
            for (int j = 0; j < R; ++j) { kv[j] = __half2float(kr[R * lane + j]); vv[j] = __half2float(vr[R * lane + j]); }
            attend(kv, vv);
        }
    }
    // merge the warps
    __syncthreads();
#pragma unroll
    for (int g = 0; g < kMaxG; ++g) {
        if (g >= G) break;
        if (lane == 0) { sm.wm[warp][g] = m[g]; sm.wl[warp][g] = l[g]; }
#pragma unroll
        for (int j = 0; j < R; ++j) sm.wo[warp][g][R * lane + j] = o[g][j];
    }
    __syncthreads();
    const int64_t base = ((static_cast<int64_t>(tq) * L.kv_heads + head) * P.nsplit + split) * G;
    for (int e = threadIdx.x; e < G * DD; e += kGThreads) {
        const int g = e / DD, d = e % DD;
        float mm = -INFINITY;
        for (int w = 0; w < kGWarps; ++w) mm = fmaxf(mm, sm.wm[w][g]);
        float ll = 0.0f, oo = 0.0f;
        if (mm != -INFINITY)
            for (int w = 0; w < kGWarps; ++w) {
                const float wt = __expf(sm.wm[w][g] - mm);
                ll += wt * sm.wl[w][g];
                oo += wt * sm.wo[w][g][d];
            }
        P.ws_o[(base + g) * DD + d] = oo;
        if (d == 0) { P.ws_m[base + g] = mm; P.ws_l[base + g] = ll; }
    }
}

// Merge the key ranges of one (token, q head), then either export the partial or normalise, rotate back and store.
template <int DD>
__global__ void __launch_bounds__(128) general_reduce_kernel(const float* __restrict__ ws_m, const float* __restrict__ ws_l,
                                                             const float* __restrict__ ws_o, int nsplit, int T, int q_heads,
                                                             int kv_heads, int dtype, uint16_t* __restrict__ out,
                                                             float* __restrict__ part_m, float* __restrict__ part_l,
                                                             float* __restrict__ part_o) {
    constexpr int R = DD / 32;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= T * q_heads) return;
    const int G = q_heads / kv_heads, tq = row / q_heads, qh = row % q_heads, head = qh / G, g = qh % G;
    const int64_t base = ((static_cast<int64_t>(tq) * kv_heads + head) * nsplit) * G + g;
    float m = -INFINITY;
    for (int z = 0; z < nsplit; ++z) m = fmaxf(m, ws_m[base + static_cast<int64_t>(z) * G]);
    float l = 0.0f, o[R];
#pragma unroll
    for (int j = 0; j < R; ++j) o[j] = 0.0f;
    if (m != -INFINITY)
        for (int z = 0; z < nsplit; ++z) {
            const int64_t i = base + static_cast<int64_t>(z) * G;
            const float w = __expf(ws_m[i] - m);
            l += w * ws_l[i];
#pragma unroll
            for (int j = 0; j < R; ++j) o[j] += w * ws_o[i * DD + lane + 32 * j];
        }
    if (part_m != nullptr) {
        if (lane == 0) { part_m[row] = m; part_l[row] = l; }
#pragma unroll
        for (int j = 0; j < R; ++j) part_o[static_cast<int64_t>(row) * DD + lane + 32 * j] = o[j];
        return;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int j = 0; j < R; ++j) o[j] *= inv;
    hadamard_warp<DD>(o, lane);
#pragma unroll
    for (int j = 0; j < R; ++j)
        out[static_cast<int64_t>(row) * DD + lane + 32 * j] = dtype == KVB_DTYPE_BF16 ? f32_to_out<true>(o[j]) : f32_to_out<false>(o[j]);
}

int general_splits(int kv_len_max, int T) {
    if (T > 8) return 1;  // a chunk already brings one CTA per token and head
    const int pages = kv_len_max / kPage;
    int n = pages / 8;
    return n < 1 ? 1 : (n > 36 ? 36 : n);  // with four KV heads: one CTA per SM of a 148-SM part
}

template <int DD>
int launch_general_t(const kvb_layer* layer, const GeneralParams& P, void* out, float* pm, float* pl, float* po, cudaStream_t s) {
    const int smem = static_cast<int>(sizeof(GeneralSmem<DD>));
    static unsigned long long opted = 0;
    if (first_call_on_device(opted)) {
        KVB_CUDA_OK(cudaFuncSetAttribute(general_attn_kernel<DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    general_attn_kernel<DD><<<dim3(P.nsplit, layer->kv_heads, P.T), kGThreads, smem, s>>>(P);
    KVB_CUDA_OK(cudaGetLastError());
    const int rows = P.T * layer->q_heads;
    general_reduce_kernel<DD><<<(rows + 3) / 4, 128, 0, s>>>(P.ws_m, P.ws_l, P.ws_o, P.nsplit, P.T, layer->q_heads, layer->kv_heads,
                                                            layer->dtype, static_cast<uint16_t*>(out), pm, pl, po);
    KVB_CUDA_OK(cudaGetLastError());
    return KVB_OK;
}

}  // namespace

// Bytes of workspace the general path needs for `rows` query tokens.
size_t general_workspace_bytes(int kv_len_max, int q_heads, int head_dim, int rows) {
    return static_cast<size_t>(rows) * q_heads * general_splits(kv_len_max, rows) * (head_dim + 2) * sizeof(float);
}

// Attention of T already-appended query tokens on the general kernel (any supported head_dim / Sinkhorn setting).
int launch_general_attention(const kvb_layer* layer, const void* q, const int32_t* pos_dev, const int32_t* total_pos_dev, int T,
                             float scale, int kv_len_max, int key_begin, int key_end, void* workspace, void* out, float* part_m,
                             float* part_l, float* part_o, cudaStream_t stream) {
    GeneralParams P;
    P.L = make_view(*layer);
    P.q = static_cast<const uint16_t*>(q);
    P.pos = pos_dev;
    P.total_pos = total_pos_dev;
    P.T = T;
    P.nsplit = general_splits(kv_len_max, T);
    P.key_begin = key_begin;
    P.key_end = key_end;
    P.scale = scale;
    const size_t rows = static_cast<size_t>(T) * layer->q_heads * P.nsplit;
    P.ws_m = static_cast<float*>(workspace);
    P.ws_l = P.ws_m + rows;
    P.ws_o = P.ws_l + rows;
    if (layer->head_dim == 128) return launch_general_t<128>(layer, P, out, part_m, part_l, part_o, stream);
    return launch_general_t<256>(layer, P, out, part_m, part_l, part_o, stream);
}

}  // namespace kvb
