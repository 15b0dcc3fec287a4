// kvb_prefill.cu -- prefill-chunk attention over the quantised cache on the 5th-generation tensor cores.
//
// The chunk's (token, q head) rows of one KV head are GQA-packed into tiles of 128 rows; a CTA owns one such
// tile, one KV head and one range of 128-key tiles, and walks its keys flash-attention style:
//   S = Q K^T   tcgen05.mma, A = Q tile and B = de-quantised K tile in shared memory (K-major, 128-byte swizzle),
//               accumulator S[128 x 128] fp32 in tensor memory;
//   softmax     thread r owns row r (= TMEM lane r): loads S with tcgen05.ld, running max / sum in registers,
//               writes P (fp16) over the K tile (S is complete by then), rescales the O accumulator in TMEM only
//               when a row maximum moved;
//   O += P V    tcgen05.mma, A = P tile (K-major over keys), B = de-quantised V tile (MN-major: one 128-byte row
//               of 64 dims per key), accumulator O[128 x 128] fp32 in tensor memory.
// K and V tiles are de-quantised by the CUDA cores straight from the planes (thread = key): nibbles -> fp16 with
// the exact unpack of the decode kernel, then one fused multiply-add with the tile's per-dim (K) or the key's
// (V) fp16 scale and zero point.  Dims inside every group of eight are kept in the order the unpack yields
// (0,4,1,5,2,6,3,7); Q is written in the same order, so the contraction is unaffected, and the merge kernel
// puts the output dims back.  Keys of the open tile come un-quantised from the stage.
// Three 32 KB tiles (Q, K/P, V) and 256 TMEM columns per CTA let two CTAs share an SM, so one CTA's CUDA-core
// phases (de-quantisation, softmax) overlap the other's MMAs.
// Every wait on an mbarrier is bounded; a wait that gives up sets KVB_ERR_WAIT_TIMEOUT and the CTA leaves
// through the normal exit (TMEM is freed).
#include <climits>

#include "kvb_common.cuh"
#include "kvb_tcgen05.cuh"

namespace kvb {
namespace {

constexpr int D = 128;
constexpr int kM = 128;        // query rows per CTA
constexpr int kN = 128;        // keys per step = one quantisation tile
constexpr int kThreads = 128;  // thread r <-> query row r <-> TMEM lane r
constexpr int kTileBytes = kM * D * 2;
constexpr uint32_t kTmemCols = 256;  // S at columns [0,128), O at [128,256)

struct PrefillParams {
    LayerView L;
    const uint16_t* q;         // [T][q_heads][D]
    const int32_t* pos;        // [T]
    const int32_t* total_pos;  // newest position in the cache
    int T, mtiles, ksplit;
    float scale_log2;
    float* ws_m;               // [H][mtiles][ksplit][128]
    float* ws_l;
    float* ws_o;               // [H][mtiles][ksplit][128][D], dims in tile order
};

struct __align__(1024) PrefillSmem {
    uint8_t q[kTileBytes];
    uint8_t k[kTileBytes];  // the K tile, then -- once S = Q K^T has completed -- the P tile of the same step
    uint8_t v[kTileBytes];
    __half ks[D], kz[D];  // per-dim scale / zero point of the K tile, in tile dim order
    __half vo[D];         // per-dim other_V of the tile (balanced caches), in tile dim order
    uint64_t bar_s, bar_o;
    uint32_t tmem_base;
    int row_pos[kM];
    int flags[4];
};

// Byte offset of element (row, col) in a [128 rows][128 cols] fp16 tile stored as two 64-column blocks of
// 128-byte rows, 8-row groups 1024 bytes apart, 16-byte chunks XOR-swizzled with the row (128-byte swizzle).
__device__ __forceinline__ uint32_t tile_off(int row, int col) {
    return (col >> 6) * 16384 + (row >> 3) * 1024 + (row & 7) * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4) + (col & 7) * 2;
}
// Position of dim d inside its group of eight: order 0,4,1,5,2,6,3,7.
__device__ __forceinline__ int dim_slot(int d) { return (d & ~7) | ((d & 3) << 1) | ((d >> 2) & 1); }

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// De-quantise one key row (64 code bytes) into the tile: out = code * scale + zp, pairs (d, d+4).
// kPerDim: scale / zp pairs come from the per-dim tables (K); otherwise s2 / z2 hold the key's pair (V).
// `other` (caches written with variance balancing): the result is multiplied by the key's other_K (K: o2, both halves)
// or by the per-dim other_V table (V), reference kvarn128_codec.cuh:331-347; fp16 like the rest of this kernel.
// ks / kz / vo: the per-dim tables of the tile in shared memory (tile dim order).
template <bool kPerDim, bool other>
__device__ __forceinline__ void dequant_row(const uint4 (&codes)[4], uint8_t* tile, int row, const __half* ks, const __half* kz,
                                            const __half* vo, uint32_t s2, uint32_t z2, uint32_t o2) {
#pragma unroll
    for (int v4 = 0; v4 < 4; ++v4) {
        const uint4 pk = codes[v4];
        const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int chunk = v4 * 4 + i;  // dims 8 chunk .. 8 chunk + 7
            uint32_t u[4];
            unpack8(w[i], u);
            uint4 out;
            if constexpr (kPerDim) {
                const uint4 sc = *reinterpret_cast<const uint4*>(&ks[8 * chunk]);
                const uint4 zp = *reinterpret_cast<const uint4*>(&kz[8 * chunk]);
                out = make_uint4(hfma2_u32(u[0], sc.x, zp.x), hfma2_u32(u[1], sc.y, zp.y), hfma2_u32(u[2], sc.z, zp.z),
                                 hfma2_u32(u[3], sc.w, zp.w));
                if constexpr (other) out = make_uint4(hmul2_u32(out.x, o2), hmul2_u32(out.y, o2), hmul2_u32(out.z, o2), hmul2_u32(out.w, o2));
            } else {
                out = make_uint4(hfma2_u32(u[0], s2, z2), hfma2_u32(u[1], s2, z2), hfma2_u32(u[2], s2, z2), hfma2_u32(u[3], s2, z2));
                if constexpr (other) {
                    const uint4 ot = *reinterpret_cast<const uint4*>(&vo[8 * chunk]);
                    out = make_uint4(hmul2_u32(out.x, ot.x), hmul2_u32(out.y, ot.y), hmul2_u32(out.z, ot.z), hmul2_u32(out.w, ot.w));
                }
            }
            *reinterpret_cast<uint4*>(tile + tile_off(row, 8 * chunk)) = out;
        }
    }
}

// Copy one un-quantised fp16 row of the stage into the tile (dims re-ordered inside every group of eight).
__device__ __forceinline__ void stage_row_to_tile(const __half* __restrict__ src, uint8_t* tile, int row, bool live) {
#pragma unroll
    for (int chunk = 0; chunk < 16; ++chunk) {
        uint4 r = live ? reinterpret_cast<const uint4*>(src)[chunk] : make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(tile + tile_off(row, 8 * chunk)) =
            make_uint4(prmt(r.x, r.z, 0x5410), prmt(r.x, r.z, 0x7632), prmt(r.y, r.w, 0x5410), prmt(r.y, r.w, 0x7632));
    }
}

// The Q tile of a CTA: rows (token, q head of this KV head) `first_row` .. + 127 rotated, scaled, rounded to fp16 and
// stored in tile dim order; rows beyond the chunk are zeros.  One warp per row, lane l holds dims l + 32 j; the rows of
// a warp are taken eight at a time with every global load issued before the first rotation (a row per iteration cost
// one memory latency each: 32 us per CTA with four warps).
__device__ __forceinline__ void build_q_tile(const PrefillParams& P, const LayerView& L, int first_row, int head, int G, uint8_t* q_tile,
                                             int* row_pos, int warp, int lane) {
    constexpr int kWarps = kThreads / 32, kBatch = 8;
    for (int j0 = 0; j0 < kM / kWarps; j0 += kBatch) {
        uint16_t raw[kBatch][4];
        int rp[kBatch];
#pragma unroll
        for (int jj = 0; jj < kBatch; ++jj) {
            const int r = warp + kWarps * (j0 + jj), R = first_row + r, tq = R / G, gq = R % G;
            rp[jj] = -1;
            raw[jj][0] = raw[jj][1] = raw[jj][2] = raw[jj][3] = 0;
            if (tq < P.T) {
                const uint16_t* qrow = P.q + (static_cast<int64_t>(tq) * L.q_heads + head * G + gq) * D;
#pragma unroll
                for (int j = 0; j < 4; ++j) raw[jj][j] = qrow[lane + 32 * j];
                rp[jj] = P.pos[tq];
            }
        }
#pragma unroll
        for (int jj = 0; jj < kBatch; ++jj) {
            const int r = warp + kWarps * (j0 + jj);
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = L.dtype == KVB_DTYPE_BF16 ? in_to_f32<true>(raw[jj][j]) : in_to_f32<false>(raw[jj][j]);
            if (rp[jj] >= 0) hadamard_warp<D>(v, lane);  // warp-uniform: a row is real or not for the whole warp
            if (lane == 0) row_pos[r] = rp[jj];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<__half*>(q_tile + tile_off(r, dim_slot(lane + 32 * j))) = __float2half_rn(v[j] * P.scale_log2);
        }
    }
}

// kOther: the cache carries balancing factors different from 1 (Sinkhorn iterations > 0).
template <bool kOther>
__global__ void __launch_bounds__(kThreads, 2) prefill_kernel(const PrefillParams P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // the swizzled tiles need a 1024-byte aligned base; the launch reserves 1024 spare bytes for this
    PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const LayerView& L = P.L;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mt = blockIdx.x, head = blockIdx.y, zs = blockIdx.z;
    const int G = L.q_heads / L.kv_heads;
    const int kv_total = *P.total_pos + 1;

    if (warp == 0) tc::tmem_alloc(&sm.tmem_base, kTmemCols);
    if (tid == 0) {
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_fence_init();
        sm.flags[0] = 0;
    }
    build_q_tile(P, L, mt * kM, head, G, sm.q, sm.row_pos, warp, lane);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_s = sm.tmem_base, tmem_o = sm.tmem_base + kN;
    const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;

    int max_pos = -1, min_pos = INT_MAX;
    for (int r = 0; r < kM; ++r) {
        const int p = sm.row_pos[r];
        if (p >= 0) { max_pos = max(max_pos, p); min_pos = min(min_pos, p); }
    }
    const int my_pos = sm.row_pos[tid];
    // key tiles this CTA walks: those a row of the tile can see, cut into ksplit ranges
    const int ntiles = max_pos < 0 ? 0 : min((kv_total + kN - 1) / kN, max_pos / kN + 1);
    const int t0 = static_cast<int>(static_cast<int64_t>(ntiles) * zs / P.ksplit);
    const int t1 = static_cast<int>(static_cast<int64_t>(ntiles) * (zs + 1) / P.ksplit);
    const int32_t* tbl = L.table();
    constexpr bool other = kOther;
    const uint32_t idesc_qk = tc::idesc_f16(kM, kN, false, false), idesc_pv = tc::idesc_f16(kM, D, false, true);
    const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v);

    float m_run = -INFINITY, l_run = 0.0f;
    bool have_o = false, failed = false;
    uint32_t it = 0;
    const bool warp_has_rows = __any_sync(0xffffffffu, my_pos >= 0);  // warps without a valid row skip the softmax

    // Everything a tile needs from global memory before its K side can be de-quantised; fetched one tile ahead
    // so that the page-table lookup and the load latency hide behind the previous tile's softmax.
    struct KFetch {
        uint4 codes[4], vcodes[4];
        uint32_t vsz;
        __half ks, kz;
        __half ko, vo;  // balanced caches: other_K of this thread's key, other_V of this thread's dim
        int32_t page;  // page of this thread's key (-1: tile unusable)
        bool sealed, ok;
    };
    // The physical pages of a tile are looked up one step before its codes are requested (ids_a / ids_b: pages of the
    // tile the next fetch_k asks for): page id -> code address is a dependent trip to L2 that would otherwise stall
    // every step for about 0.3 us.
    int32_t ids_a = -1, ids_b = -1;
    auto lookup = [&](int t) {
        ids_a = ids_b = -1;
        if (t < t1 && t * kN + kN <= kv_total) {
            ids_a = L.page_of(tbl, 2 * t);
            ids_b = L.page_of(tbl, 2 * t + 1);
        }
    };
    auto fetch_k = [&](int t, KFetch& f) {  // uses the pages `lookup(t)` found, then looks up those of tile t + 1
        f.sealed = t * kN + kN <= kv_total;
        f.ok = t < t1;
        f.page = -1;
        const int32_t pg0 = ids_a, pg1 = ids_b;
        lookup(t + 1);
        if (!f.ok || !f.sealed) return;
        if (pg0 < 0 || pg1 < 0) { f.ok = false; return; }  // reported in the error word; every thread skips the tile alike
        f.page = tid < 64 ? pg0 : pg1;
        const uint4* kc = reinterpret_cast<const uint4*>(L.k_code + page_head_offset(64, L.kv_heads, f.page, head) + (tid & 63) * 64);
#pragma unroll
        for (int i = 0; i < 4; ++i) f.codes[i] = kc[i];
        const uint4* vc = reinterpret_cast<const uint4*>(L.v_code + page_head_offset(64, L.kv_heads, f.page, head) + (tid & 63) * 64);
#pragma unroll
        for (int i = 0; i < 4; ++i) f.vcodes[i] = vc[i];
        f.vsz = *reinterpret_cast<const uint32_t*>(L.v_scale + page_head_offset(4, L.kv_heads, f.page, head) + (tid & 63) * 4 + 2);
        // per-dim scale / zero point of the tile (stored in both pages): page row d/2 = [s s z z other]
        const __half* ksp = L.k_scale + page_head_offset(5, L.kv_heads, pg0, head);
        f.ks = ksp[(tid >> 1) * 5 + (tid & 1)];
        f.kz = ksp[(tid >> 1) * 5 + 2 + (tid & 1)];
        if constexpr (other) {  // K scale row of a token ends with its other_K; V scale row d / 2 starts with other_V(d), other_V(d + 1)
            f.ko = L.k_scale[page_head_offset(5, L.kv_heads, f.page, head) + (tid & 63) * 5 + 4];
            f.vo = L.v_scale[page_head_offset(4, L.kv_heads, pg0, head) + (tid >> 1) * 4 + (tid & 1)];
        }
    };
    KFetch cur, nxt;
    lookup(t0);
    fetch_k(t0, nxt);
    bool tables_ready = false;  // the scale tables of this tile were written during the previous step (saves a barrier)
    for (int t = t0; t < t1; ++t) {
        cur = nxt;
        const int base = t * kN;
        const bool sealed = cur.sealed;
        if (!cur.ok) { fetch_k(t + 1, nxt); tables_ready = false; continue; }
        if (!tables_ready) {
            if (sealed) {
                sm.ks[dim_slot(tid)] = cur.ks;
                sm.kz[dim_slot(tid)] = cur.kz;
                if constexpr (other) sm.vo[dim_slot(tid)] = cur.vo;
            }
            __syncthreads();  // scale tables visible
        }
        // ---- K tile -> shared memory (the previous P V does not touch the K buffer: P lives in tensor memory)
        if (sealed) {
            dequant_row<true, other>(cur.codes, sm.k, tid, sm.ks, sm.kz, sm.vo, 0, 0, other ? __half_as_ushort(cur.ko) * 0x10001u : 0u);
        } else {
            stage_row_to_tile(L.stage_row(0, t & 1, head, tid), sm.k, tid, base + tid < kv_total);
        }
        // ---- the previous P V reads P from the columns S = Q K^T is about to overwrite, and the V buffer: drain it
        if (have_o && !mbar_wait_bounded(&sm.bar_o, (it - 1) & 1)) { failed = true; }
        fence_proxy_async();
        __syncthreads();
        if (warp == 0) {  // the whole warp computes the (warp-uniform) operands, one elected lane issues
            tc::fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t o = (kk >> 2) * 16384 + (kk & 3) * 32;
                tc::mma_f16_ss(tmem_s, tc::smem_desc(q_addr + o, 16, 1024), tc::smem_desc(k_addr + o, 16, 1024), idesc_qk, kk > 0);
            }
            tc::commit(&sm.bar_s);
        }
        // ---- V tile -> shared memory (overlaps the QK MMA), then start fetching the next tile
        if (sealed) {
            dequant_row<false, other>(cur.vcodes, sm.v, tid, sm.ks, sm.kz, sm.vo, prmt(cur.vsz, cur.vsz, 0x1010), prmt(cur.vsz, cur.vsz, 0x3232), 0u);
        } else {
            stage_row_to_tile(L.stage_row(1, t & 1, head, tid), sm.v, tid, base + tid < kv_total);
        }
        fetch_k(t + 1, nxt);  // (issuing this at the top of the step was measured slower)
        // ---- softmax of row `tid`
        if (!mbar_wait_bounded(&sm.bar_s, it & 1)) { failed = true; }  // a warp that gave up reads stale S; the CTA agrees below
        tc::fence_after_sync();
        if (warp_has_rows) {
        float s[kN];
        {  // the four loads are in flight together: one round trip to tensor memory, not four
            uint32_t r0[32], r1[32], r2[32], r3[32];
            tc::tmem_ld32(tmem_s + lane_base, r0);
            tc::tmem_ld32(tmem_s + lane_base + 32, r1);
            tc::tmem_ld32(tmem_s + lane_base + 64, r2);
            tc::tmem_ld32(tmem_s + lane_base + 96, r3);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                s[j] = __uint_as_float(r0[j]);
                s[32 + j] = __uint_as_float(r1[j]);
                s[64 + j] = __uint_as_float(r2[j]);
                s[96 + j] = __uint_as_float(r3[j]);
            }
        }
        if (base + kN - 1 > min_pos || !sealed) {
#pragma unroll
            for (int j = 0; j < kN; ++j)
                if (base + j > my_pos || base + j >= kv_total) s[j] = -INFINITY;
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains: two warps per scheduler hide little latency
#pragma unroll
        for (int j = 0; j < kN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // The reference point of the row's exponentials follows the running maximum lazily: it moves only when the
        // maximum has grown by more than 2^kLazy, so P stays below 2^kLazy (exact enough in fp16, whose precision is
        // relative) and the O accumulator is rescaled a few times per walk instead of at every new maximum.
        constexpr float kLazy = 8.0f;
        const bool grown = mx > m_run + kLazy || (m_run == -INFINITY && mx > -INFINITY);
        const float m_new = grown ? mx : m_run;
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;
        const float alpha = grown ? fast_exp2(m_run - m_use) : 1.0f;
        const bool moved = have_o && grown;
        m_run = m_new;
        float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        // P stays in tensor memory: fp16 pairs over the first 64 columns of S (already in registers), the A operand
        // of the P V product -- no shared-memory round trip for P
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t pk[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float p0 = fast_exp2(s[64 * c + 2 * j] - m_use), p1 = fast_exp2(s[64 * c + 2 * j + 1] - m_use);
                sum4[j & 3] += p0 + p1;
                pk[j] = pack_half2(p0, p1);
            }
            tc::tmem_st32(tmem_s + lane_base + 32 * c, pk);
        }
        tc::tmem_st_wait();
        l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        if (__any_sync(0xffffffffu, moved)) {  // rescale this warp's 32 rows of O (alpha = 1 for rows that did not move)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tc::tmem_ld32(tmem_o + lane_base + 32 * c, r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                tc::tmem_st32(tmem_o + lane_base + 32 * c, r);
            }
            tc::tmem_st_wait();
        }
        }  // warp_has_rows (rows of the other warps are never read: their P and O may hold anything)
        // the scale tables of the next tile: this tile's K rows were de-quantised two barriers ago
        tables_ready = nxt.ok;
        if (nxt.ok && nxt.sealed) {
            sm.ks[dim_slot(tid)] = nxt.ks;
            sm.kz[dim_slot(tid)] = nxt.kz;
        }
        // ---- O += P V (every warp has its V rows in shared memory and its P rows in tensor memory; any failed wait ends the walk)
        fence_proxy_async();
        tc::fence_before_sync();
        if (__syncthreads_or(failed)) { failed = true; break; }
        if constexpr (other) {
            if (nxt.ok && nxt.sealed) sm.vo[dim_slot(tid)] = nxt.vo;  // every thread is past this tile's V rows
        }
        if (warp == 0) {  // the whole warp computes the (warp-uniform) operands, one elected lane issues
            tc::fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                tc::mma_f16_ts(tmem_o, tmem_s + 8 * kk, tc::smem_desc(v_addr + kk * 2048, 16384, 1024), idesc_pv, have_o || kk > 0);  // 16 keys = 8 columns of P
            }
            tc::commit(&sm.bar_o);
        }
        have_o = true;
        ++it;
    }
    if (have_o && !failed && !mbar_wait_bounded(&sm.bar_o, (it - 1) & 1)) failed = true;
    if (failed && tid == 0) L.flag(KVB_ERR_WAIT_TIMEOUT);
    tc::fence_after_sync();

    // ---- partial of this (row tile, key range): m (log2 units), l, o in tile dim order
    const int64_t idx = ((static_cast<int64_t>(head) * P.mtiles + mt) * P.ksplit + zs) * kM + tid;
    if (my_pos >= 0) {
        P.ws_m[idx] = failed ? -INFINITY : m_run;
        P.ws_l[idx] = failed ? 0.0f : l_run;
    }
    float* orow = P.ws_o + idx * D;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (!warp_has_rows) break;
        uint32_t r[32];
        if (have_o) {
            tc::tmem_ld32(tmem_o + lane_base + 32 * c, r);
            tc::tmem_ld_wait();
        }
        if (my_pos < 0) continue;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(orow + 32 * c + j) =
                have_o && !failed ? make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]))
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(sm.tmem_base, kTmemCols);
}

// ---------------------------------------------------------------------------------------------------------
// verify_kernel: the same attention for a verify step (at most 64 GQA-merged rows: 8 tokens x 8 query heads per KV
// head), with the two halves of the CTA given different work.  Only TMEM lanes 0-63 hold rows, so only warps 0 and 1
// have a softmax to do; in prefill_kernel warps 2 and 3 idle through it and every warp de-quantises a quarter of
// each tile in between.  Here
//   warps 2, 3   de-quantise: K(t+1) into the K buffer as soon as S(t) = Q K(t)^T has completed -- while warps 0, 1
//                are busy with the softmax of step t -- and V(t+1) as soon as P V(t) has completed; thread = one key
//                row of each page of the tile; codes fetched a tile ahead;
//   warps 0, 1   softmax of their rows; warp 0 also issues the MMAs (one elected lane): Q K^T when the K tile is
//                ready, P V when both warps have stored P and the V tile is ready.
// The chain of a step shrinks from de-quantise + issue + softmax + issue to issue + softmax + issue.  Hand-offs are
// mbarriers (bounded waits that also watch a CTA-wide abort flag); the two warps of a half meet at a named barrier
// once per step, and a warp whose wait gave up still goes to that barrier before it leaves, so nobody is left waiting.
struct __align__(1024) VerifySmem {
    uint8_t q[kTileBytes];
    uint8_t k[kTileBytes];
    uint8_t v[kTileBytes];
    __half ks[2][D], kz[2][D], vo[2][D];  // per-dim tables of the tile, by step parity
    uint64_t bar_s, bar_o, k_ready, v_ready;
    uint32_t tmem_base;
    int row_pos[kM];
    int abort_flag, bad_tile;
};

__device__ __forceinline__ bool verify_wait(uint64_t* bar, uint32_t parity, VerifySmem& sm) {
    bool ok = false;
    for (uint32_t i = 0; i < kSpinLimit && !ok; ++i) {
        ok = mbar_try_wait(bar, parity);
        if (!ok && *reinterpret_cast<volatile int*>(&sm.abort_flag) != 0) break;
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) *reinterpret_cast<volatile int*>(&sm.abort_flag) = 1;
    return ok;
}

template <bool kOther>
__global__ void __launch_bounds__(kThreads, 2) verify_kernel(const PrefillParams P) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    VerifySmem& sm = *reinterpret_cast<VerifySmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const LayerView& L = P.L;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.y, zs = blockIdx.z;
    const int G = L.q_heads / L.kv_heads;
    const int kv_total = *P.total_pos + 1;

    if (warp == 0) tc::tmem_alloc(&sm.tmem_base, kTmemCols);
    if (tid == 0) {
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_init(&sm.k_ready, 2);  // lane 0 of each de-quantising warp
        mbar_init(&sm.v_ready, 2);
        mbar_fence_init();
        sm.abort_flag = 0;
        sm.bad_tile = 0;
    }
    build_q_tile(P, L, 0, head, G, sm.q, sm.row_pos, warp, lane);  // rows beyond the step's are zeros; the MMA reads all 128
    fence_proxy_async();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_s = sm.tmem_base, tmem_o = sm.tmem_base + kN;
    int max_pos = -1, min_pos = INT_MAX;
    for (int r = 0; r < 64; ++r) {
        const int p = sm.row_pos[r];
        if (p >= 0) { max_pos = max(max_pos, p); min_pos = min(min_pos, p); }
    }
    const int ntiles = max_pos < 0 ? 0 : min((kv_total + kN - 1) / kN, max_pos / kN + 1);
    const int t0 = static_cast<int>(static_cast<int64_t>(ntiles) * zs / P.ksplit);
    const int t1 = static_cast<int>(static_cast<int64_t>(ntiles) * (zs + 1) / P.ksplit);
    const int n = t1 - t0;
    bool failed = false;
    volatile int* abort_flag = &sm.abort_flag;

    if (warp >= 2) {
        // =========================== de-quantise ===========================
        const int dt = tid - 64;  // key rows dt of both pages of the tile (tile rows dt and dt + 64); dims dt and dt + 64
        const int32_t* tbl = L.table();
        struct Fetch {
            uint4 codes[2][4], vcodes[2][4];
            uint32_t vsz[2];
            __half ks[2], kz[2], ko[2], vo[2];
            bool bad;
        };
        int32_t ids_a = -1, ids_b = -1;  // pages of the tile the next fetch asks for, looked up a step earlier
        auto sealed_tile = [&](int t) { return t * kN + kN <= kv_total; };
        auto lookup = [&](int t) {
            ids_a = ids_b = -1;
            if (t < t1 && sealed_tile(t)) {
                ids_a = L.page_of(tbl, 2 * t);
                ids_b = L.page_of(tbl, 2 * t + 1);
            }
        };
        auto fetch = [&](int t, Fetch& f) {
            int32_t pg[2] = {ids_a, ids_b};
            lookup(t + 1);
            f.bad = false;
            if (t >= t1 || !sealed_tile(t)) return;
            if (pg[0] < 0 || pg[1] < 0) { f.bad = true; pg[0] = pg[1] = 0; }  // reported in the error word; the tile is masked
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4* kc = reinterpret_cast<const uint4*>(L.k_code + page_head_offset(64, L.kv_heads, pg[h], head) + dt * 64);
                const uint4* vc = reinterpret_cast<const uint4*>(L.v_code + page_head_offset(64, L.kv_heads, pg[h], head) + dt * 64);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    f.codes[h][i] = kc[i];
                    f.vcodes[h][i] = vc[i];
                }
                f.vsz[h] = *reinterpret_cast<const uint32_t*>(L.v_scale + page_head_offset(4, L.kv_heads, pg[h], head) + dt * 4 + 2);
                // per-dim entries of the tile (stored in both pages): this thread's dims are dt and dt + 64
                const int d = dt + 64 * h;
                const __half* ksp = L.k_scale + page_head_offset(5, L.kv_heads, pg[0], head);
                f.ks[h] = ksp[(d >> 1) * 5 + (d & 1)];
                f.kz[h] = ksp[(d >> 1) * 5 + 2 + (d & 1)];
                if constexpr (kOther) {
                    f.ko[h] = L.k_scale[page_head_offset(5, L.kv_heads, pg[h], head) + dt * 5 + 4];
                    f.vo[h] = L.v_scale[page_head_offset(4, L.kv_heads, pg[0], head) + (d >> 1) * 4 + (d & 1)];
                }
            }
        };
        Fetch cur, nxt;
        if (n > 0) {
            lookup(t0);
            fetch(t0, nxt);
        }
        for (int i = 0; i < n; ++i) {
            const int t = t0 + i, base = t * kN, par = i & 1;
            const bool sealed = sealed_tile(t);
            cur = nxt;
            // ---- K: the buffer (and the tables of this parity) are free once S(i-1) has completed
            if (!failed && i > 0 && !verify_wait(&sm.bar_s, (i - 1) & 1, sm)) failed = true;
            if (!failed && sealed) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    sm.ks[par][dim_slot(dt + 64 * h)] = cur.ks[h];
                    sm.kz[par][dim_slot(dt + 64 * h)] = cur.kz[h];
                    if constexpr (kOther) sm.vo[par][dim_slot(dt + 64 * h)] = cur.vo[h];
                }
                if (dt == 0 && cur.bad) sm.bad_tile = 1;  // sticky: the error word is set, the result is void anyway
            }
            named_barrier_sync(2, 64);  // tables visible to both warps; a warp that gave up meets its partner here
            if (*abort_flag) break;
            if (sealed) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    dequant_row<true, kOther>(cur.codes[h], sm.k, dt + 64 * h, sm.ks[par], sm.kz[par], sm.vo[par], 0, 0,
                                              kOther ? __half_as_ushort(cur.ko[h]) * 0x10001u : 0u);
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    stage_row_to_tile(L.stage_row(0, t & 1, head, dt + 64 * h), sm.k, dt + 64 * h, base + dt + 64 * h < kv_total);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.k_ready);
            fetch(t + 1, nxt);
            // ---- V: the buffer is free once P V(i-1) has completed
            if (i > 0 && !verify_wait(&sm.bar_o, (i - 1) & 1, sm)) { failed = true; continue; }
            if (sealed) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    dequant_row<false, kOther>(cur.vcodes[h], sm.v, dt + 64 * h, sm.ks[par], sm.kz[par], sm.vo[par],
                                               prmt(cur.vsz[h], cur.vsz[h], 0x1010), prmt(cur.vsz[h], cur.vsz[h], 0x3232), 0u);
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    stage_row_to_tile(L.stage_row(1, t & 1, head, dt + 64 * h), sm.v, dt + 64 * h, base + dt + 64 * h < kv_total);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.v_ready);
        }
    } else {
        // =========================== softmax (warps 0, 1) and MMA issue (warp 0) ===========================
        const uint32_t lane_base = static_cast<uint32_t>(32 * warp) << 16;
        const int my_pos = sm.row_pos[tid];
        const bool warp_has_rows = __any_sync(0xffffffffu, my_pos >= 0);
        const uint32_t idesc_qk = tc::idesc_f16(kM, kN, false, false), idesc_pv = tc::idesc_f16(kM, D, false, true);
        const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v);
        float m_run = -INFINITY, l_run = 0.0f;
        for (int i = 0; i < n; ++i) {
            const int base = (t0 + i) * kN;
            const bool sealed = base + kN <= kv_total;
            if (warp == 0 && !failed) {  // S(i) = Q K(i)^T: the K tile is ready; P V(i-1), which reads P from the columns of S, has completed
                if (!verify_wait(&sm.k_ready, i & 1, sm) || (i > 0 && !verify_wait(&sm.bar_o, (i - 1) & 1, sm))) {
                    failed = true;
                } else {
                    tc::fence_after_sync();
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        const uint32_t o = (kk >> 2) * 16384 + (kk & 3) * 32;
                        tc::mma_f16_ss(tmem_s, tc::smem_desc(q_addr + o, 16, 1024), tc::smem_desc(k_addr + o, 16, 1024), idesc_qk, kk > 0);
                    }
                    tc::commit(&sm.bar_s);
                }
            }
            if (!failed && !verify_wait(&sm.bar_s, i & 1, sm)) failed = true;
            tc::fence_after_sync();
            if (!failed && warp_has_rows) {
                const bool all_masked = *reinterpret_cast<volatile int*>(&sm.bad_tile) != 0;
                float s[kN];
                {
                    uint32_t r0[32], r1[32], r2[32], r3[32];
                    tc::tmem_ld32(tmem_s + lane_base, r0);
                    tc::tmem_ld32(tmem_s + lane_base + 32, r1);
                    tc::tmem_ld32(tmem_s + lane_base + 64, r2);
                    tc::tmem_ld32(tmem_s + lane_base + 96, r3);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        s[j] = __uint_as_float(r0[j]);
                        s[32 + j] = __uint_as_float(r1[j]);
                        s[64 + j] = __uint_as_float(r2[j]);
                        s[96 + j] = __uint_as_float(r3[j]);
                    }
                }
                if (base + kN - 1 > min_pos || !sealed || all_masked) {
#pragma unroll
                    for (int j = 0; j < kN; ++j)
                        if (base + j > my_pos || base + j >= kv_total || all_masked) s[j] = -INFINITY;
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < kN; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], s[j]);
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                constexpr float kLazy = 8.0f;  // lazy reference point, as in prefill_kernel
                const bool grown = mx > m_run + kLazy || (m_run == -INFINITY && mx > -INFINITY);
                const float m_new = grown ? mx : m_run;
                const float m_use = m_new == -INFINITY ? 0.0f : m_new;
                const float alpha = grown ? fast_exp2(m_run - m_use) : 1.0f;
                const bool moved = i > 0 && grown;
                m_run = m_new;
                float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t pk[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float p0 = fast_exp2(s[64 * c + 2 * j] - m_use), p1 = fast_exp2(s[64 * c + 2 * j + 1] - m_use);
                        sum4[j & 3] += p0 + p1;
                        pk[j] = pack_half2(p0, p1);
                    }
                    tc::tmem_st32(tmem_s + lane_base + 32 * c, pk);
                }
                tc::tmem_st_wait();
                l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
                if (__any_sync(0xffffffffu, moved)) {  // P V(i-1) completed before S(i) was issued: O may be rescaled
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t r[32];
                        tc::tmem_ld32(tmem_o + lane_base + 32 * c, r);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * alpha);
                        tc::tmem_st32(tmem_o + lane_base + 32 * c, r);
                    }
                    tc::tmem_st_wait();
                }
            }
            tc::fence_before_sync();
            named_barrier_sync(1, 64);  // P of both warps is in tensor memory; a warp that gave up meets its partner here
            if (*abort_flag) { failed = true; break; }
            if (warp == 0) {  // O += P V(i)
                if (!verify_wait(&sm.v_ready, i & 1, sm)) {
                    failed = true;
                } else {
                    tc::fence_after_sync();
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        tc::mma_f16_ts(tmem_o, tmem_s + 8 * kk, tc::smem_desc(v_addr + kk * 2048, 16384, 1024), idesc_pv, i > 0 || kk > 0);
                    tc::commit(&sm.bar_o);
                }
            }
        }
        // ---- partial of this key range: m (log2 units), l, o in tile dim order
        if (n > 0 && !failed && !verify_wait(&sm.bar_o, (n - 1) & 1, sm)) failed = true;
        if (*abort_flag) failed = true;
        tc::fence_after_sync();
        const bool have = n > 0 && !failed;
        const int64_t idx = (static_cast<int64_t>(head) * P.ksplit + zs) * kM + tid;
        if (my_pos >= 0) {
            P.ws_m[idx] = have ? m_run : -INFINITY;
            P.ws_l[idx] = have ? l_run : 0.0f;
        }
        float* orow = P.ws_o + idx * D;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (!warp_has_rows) break;
            uint32_t r[32];
            if (have) {
                tc::tmem_ld32(tmem_o + lane_base + 32 * c, r);
                tc::tmem_ld_wait();
            }
            if (my_pos < 0) continue;
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(orow + 32 * c + j) =
                    have ? make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if ((failed || *abort_flag) && lane == 0) L.flag(KVB_ERR_WAIT_TIMEOUT);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(sm.tmem_base, kTmemCols);
}

// Merge the key ranges of one query row, normalise, undo the tile dim order, rotate back, store -- or, for a cache
// that holds only a range of the sequence, export the merged partial instead (m in natural-log units, l, o in the
// rotated domain and natural dim order, not normalised).
// One CTA of 8 warps per row: warp w takes ranges w, w+8, ..; lane l owns dims l + 32 j.  The loop is pure load
// latency, so it is unrolled to keep several ranges in flight; the warp sums meet in shared memory.
template <int kPer>  // ranges per warp: ksplit <= 8 kPer
__global__ void __launch_bounds__(256) prefill_merge_kernel(const float* __restrict__ ws_m, const float* __restrict__ ws_l,
                                                            const float* __restrict__ ws_o, int T, int q_heads, int kv_heads,
                                                            int mtiles, int ksplit, int dtype, uint16_t* __restrict__ out,
                                                            float* __restrict__ part_m, float* __restrict__ part_l,
                                                            float* __restrict__ part_o) {
    __shared__ float so[8][D];
    __shared__ float sl[8], smx[8];
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = q_heads / kv_heads, tq = row / q_heads, qh = row % q_heads, head = qh / G, R = tq * G + qh % G;
    const int64_t base = ((static_cast<int64_t>(head) * mtiles + R / kM) * ksplit) * kM + R % kM;
    // Warp w merges ranges w, w + 8, .. (kPer of them; at most 16: ksplit <= 128) relative to their own maximum, every
    // load issued before the first use: one trip to memory for the whole row; the eight warp results meet in shared
    // memory.  kPer is a template parameter so that a chunk (a few ranges, tens of thousands of rows) keeps the
    // registers low and the occupancy high.
    float pm[kPer], pl[kPer], po[kPer][4];
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
        const int z = warp + 8 * k;
        const bool on = z < ksplit;
        const int64_t i = base + static_cast<int64_t>(on ? z : 0) * kM;
        pm[k] = on ? ws_m[i] : -INFINITY;
        pl[k] = on ? ws_l[i] : 0.0f;
#pragma unroll
        for (int j = 0; j < 4; ++j) po[k][j] = on ? ws_o[i * D + dim_slot(lane + 32 * j)] : 0.0f;
    }
    float mw = -INFINITY;
#pragma unroll
    for (int k = 0; k < kPer; ++k) mw = fmaxf(mw, pm[k]);
    float l = 0.0f, o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (mw != -INFINITY) {
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const float w = fast_exp2(pm[k] - mw);  // 0 for a range that is not there
            l += w * pl[k];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] += w * po[k][j];
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) so[warp][lane + 32 * j] = o[j];
    if (lane == 0) { sl[warp] = l; smx[warp] = mw; }
    __syncthreads();
    if (warp != 0) return;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) m = fmaxf(m, smx[w]);
    l = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const float wt = smx[w] == -INFINITY ? 0.0f : fast_exp2(smx[w] - m);
        l += wt * sl[w];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] += wt * so[w][lane + 32 * j];
    }
    if (part_m != nullptr) {
        if (lane == 0) { part_m[row] = m * 0.6931471805599453f; part_l[row] = l; }
#pragma unroll
        for (int j = 0; j < 4; ++j) part_o[static_cast<int64_t>(row) * D + lane + 32 * j] = o[j];
        return;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] *= inv;
    hadamard_warp<D>(o, lane);
#pragma unroll
    for (int j = 0; j < 4; ++j)
        out[static_cast<int64_t>(row) * D + lane + 32 * j] = dtype == KVB_DTYPE_BF16 ? f32_to_out<true>(o[j]) : f32_to_out<false>(o[j]);
}

int prefill_sm_count() { return device_sm_count(); }

void prefill_shape(int kv_len_max, int kv_heads, int q_heads, int tokens, int* mtiles, int* ksplit) {
    const int rows = tokens * (q_heads / kv_heads);
    *mtiles = (rows + kM - 1) / kM;
    const int ctas = *mtiles * kv_heads, ntiles = (kv_len_max + kN - 1) / kN;
    // two CTAs share an SM: about six waves of CTAs for a chunk, rounded down so that the last wave is full (measured on
    // 1,024 x 262,144: 9 key ranges 4.94 ms, 7: 5.19, 10: 5.03, 12: 4.98, 14: 5.25); one wave for a few rows (verify),
    // where every extra key range costs a partial per row
    int ks = ctas >= 64 ? (6 * 2 * prefill_sm_count()) / ctas : (2 * prefill_sm_count() + ctas - 1) / ctas;
    if (ks > ntiles / 2) ks = ntiles / 2;
    if (ks > 128) ks = 128;
    *ksplit = ks < 1 ? 1 : ks;
}

}  // namespace
}  // namespace kvb

namespace kvb {
// kvb_attn_general.cu: head_dim 256 and caches written with Sinkhorn iterations > 0
size_t general_workspace_bytes(int kv_len_max, int q_heads, int head_dim, int rows);
int launch_general_attention(const kvb_layer* layer, const void* q, const int32_t* pos_dev, const int32_t* total_pos_dev, int T,
                             float scale, int kv_len_max, int key_begin, int key_end, void* workspace, void* out, float* part_m,
                             float* part_l, float* part_o, cudaStream_t stream);
}  // namespace kvb

extern "C" size_t kvb_prefill_workspace_bytes(int kv_len_max, int kv_heads, int q_heads, int head_dim, int tokens) {
    if (kv_heads < 1 || q_heads < kv_heads || tokens < 1) return 0;
    int mtiles, ksplit;
    kvb::prefill_shape(kv_len_max, kv_heads, q_heads, tokens, &mtiles, &ksplit);
    const size_t tuned = static_cast<size_t>(kv_heads) * mtiles * ksplit * kvb::kM * (head_dim + 2) * sizeof(float);
    const size_t general = kvb::general_workspace_bytes(kv_len_max, q_heads, head_dim, tokens);  // head_dim 256, Sinkhorn caches
    return tuned > general ? tuned : general;
}

namespace kvb {
// Chunk attention of `tokens` rows that are already appended (shared by the prefill and the verify entry points).
int launch_chunk_attention(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int tokens, float scale,
                           int kv_len_max, void* workspace, void* out, cudaStream_t s, float* part_m, float* part_l,
                           float* part_o, const int32_t* total_pos_dev) {
    PrefillParams P;
    P.L = make_view(*layer);
    P.q = static_cast<const uint16_t*>(q);
    P.pos = positions_dev;
    P.total_pos = total_pos_dev != nullptr ? total_pos_dev : positions_dev + (tokens - 1);
    P.T = tokens;
    prefill_shape(kv_len_max, layer->kv_heads, layer->q_heads, tokens, &P.mtiles, &P.ksplit);
    P.scale_log2 = scale * 1.4426950408889634f;
    const size_t rows = static_cast<size_t>(layer->kv_heads) * P.mtiles * P.ksplit * kM;
    P.ws_m = static_cast<float*>(workspace);
    P.ws_l = P.ws_m + rows;
    P.ws_o = P.ws_l + rows;
    const int smem = static_cast<int>(sizeof(PrefillSmem)) + 1024;  // room to align the tiles to 1024 bytes
    static unsigned long long opted = 0;
    if (first_call_on_device(opted)) {
        KVB_CUDA_OK(cudaFuncSetAttribute(prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        KVB_CUDA_OK(cudaFuncSetAttribute(prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    }
    const bool few_rows = tokens * (layer->q_heads / layer->kv_heads) <= 64;  // a verify step: the role-split kernel
    if (few_rows) {
        const int vsmem = static_cast<int>(sizeof(VerifySmem)) + 1024;
        static unsigned long long vopted = 0;
        if (first_call_on_device(vopted)) {
            KVB_CUDA_OK(cudaFuncSetAttribute(verify_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, vsmem));
            KVB_CUDA_OK(cudaFuncSetAttribute(verify_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, vsmem));
        }
        if (layer->sinkhorn_iters > 0) {
            verify_kernel<true><<<dim3(1, layer->kv_heads, P.ksplit), kThreads, vsmem, s>>>(P);
        } else {
            verify_kernel<false><<<dim3(1, layer->kv_heads, P.ksplit), kThreads, vsmem, s>>>(P);
        }
    } else if (layer->sinkhorn_iters > 0) {
        prefill_kernel<true><<<dim3(P.mtiles, layer->kv_heads, P.ksplit), kThreads, smem, s>>>(P);
    } else {
        prefill_kernel<false><<<dim3(P.mtiles, layer->kv_heads, P.ksplit), kThreads, smem, s>>>(P);
    }
    KVB_CUDA_OK(cudaGetLastError());
    const int total_rows = tokens * layer->q_heads;
    auto merge = P.ksplit <= 16 ? prefill_merge_kernel<2> : P.ksplit <= 32 ? prefill_merge_kernel<4> : P.ksplit <= 64 ? prefill_merge_kernel<8>
                                                                                                                      : prefill_merge_kernel<16>;
    merge<<<total_rows, 256, 0, s>>>(P.ws_m, P.ws_l, P.ws_o, tokens, layer->q_heads, layer->kv_heads, P.mtiles, P.ksplit, layer->dtype,
                                     static_cast<uint16_t*>(out), part_m, part_l, part_o);
    KVB_CUDA_OK(cudaGetLastError());
    return KVB_OK;
}
}  // namespace kvb

extern "C" int kvb_attn_prefill(const kvb_layer* layer, const void* q, const void* k, const void* v,
                                const int32_t* positions_dev, int tokens, float scale, int kv_len_max, void* workspace,
                                void* out, void* stream) {
    using namespace kvb;
    if (int st = check_layer(layer, "kvb_attn_prefill")) return st;
    if (tokens < 1) return fail(KVB_EINVAL, "kvb_attn_prefill: tokens = %d", tokens);
    if (q == nullptr || workspace == nullptr || out == nullptr) return fail(KVB_EINVAL, "kvb_attn_prefill: null q / workspace / out");
    if (layer->stage == nullptr) return fail(KVB_EINVAL, "kvb_attn_prefill: layer has no stage buffer");
    if (tokens > 65535) return fail(KVB_ERANGE, "kvb_attn_prefill: %d tokens in one chunk (at most 65535)", tokens);
    if (int st = kvb_append(layer, k, v, positions_dev, tokens, stream)) return st;
    if (layer->head_dim != 128)  // two slices per key: general kernel, same semantics
        return launch_general_attention(layer, q, positions_dev, positions_dev + (tokens - 1), tokens, scale, kv_len_max, 0, INT_MAX,
                                        workspace, out, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream));
    return launch_chunk_attention(layer, q, positions_dev, tokens, scale, kv_len_max, workspace, out, static_cast<cudaStream_t>(stream),
                                  nullptr, nullptr, nullptr, nullptr);
}
