// Runs the engine-shaped launchers on the GPU and checks them against the C ABI called directly on a second,
// identical cache: append of a prompt chunk + prompt attention, a verify step, a single-token append + cached
// decode, a 12-column step attended in two column blocks.  Outputs must match bit for bit (same kernels, same
// inputs); the error words must stay zero.  Both caches are written with 0 Sinkhorn iterations.
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

#include "ninfer_engine_shim.hpp"

#define OK(x)                                                                      \
    do {                                                                           \
        cudaError_t e_ = (x);                                                      \
        if (e_ != cudaSuccess) { std::printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); return 2; } \
    } while (0)

static unsigned short f2h(float f) {  // fp32 -> fp16, round to nearest even, normal range only (test inputs are small)
    unsigned int x;
    std::memcpy(&x, &f, 4);
    const unsigned int sign = (x >> 16) & 0x8000u;
    int exp = static_cast<int>((x >> 23) & 0xff) - 127 + 15;
    unsigned int man = x & 0x7fffffu;
    if (exp <= 0) return static_cast<unsigned short>(sign);
    unsigned int h = sign | (static_cast<unsigned int>(exp) << 10) | (man >> 13);
    const unsigned int rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return static_cast<unsigned short>(h);
}

int main() {
    using namespace ninfer;
    using namespace ninfer::ops;
    const int D = 128, H = 4, QH = 24, pages = 16, prompt = 300, width = 5;
    kvarn128_set_sinkhorn_iters(0);
    unsigned int seed = 12345u;
    auto rnd = [&]() { seed = seed * 1664525u + 1013904223u; return (static_cast<float>(seed >> 8) / 8388608.0f - 1.0f); };
    auto rows = [&](int n, int heads) { std::vector<unsigned short> h(static_cast<size_t>(n) * heads * D); for (auto& x : h) x = f2h(rnd()); return h; };
    auto dev = [&](const void* src, size_t bytes) { void* p = nullptr; cudaMalloc(&p, bytes); if (src) cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice); else cudaMemset(p, 0, bytes); return p; };

    // two identical caches: A driven through the engine-shaped launchers, B through the C ABI
    const size_t code_b = kvb_plane_bytes(0, D, H, pages), ks_b = kvb_plane_bytes(1, D, H, pages), vs_b = kvb_plane_bytes(3, D, H, pages);
    void *kc[2], *vc[2], *ks[2], *vs[2];
    for (int i = 0; i < 2; ++i) { kc[i] = dev(nullptr, code_b); vc[i] = dev(nullptr, code_b); ks[i] = dev(nullptr, ks_b); vs[i] = dev(nullptr, vs_b); }
    std::vector<int> table(pages);
    for (int i = 0; i < pages; ++i) table[i] = (i * 5 + 3) % pages;  // a permutation: 5 and 16 are coprime
    void* table_dev = dev(table.data(), pages * sizeof(int));
    const int zero = 0;
    void* table_rows_dev = dev(&zero, sizeof(int));
    void* stage_b = dev(nullptr, kvb_stage_bytes(D, H));
    void* err_b = dev(nullptr, 4);
    const size_t ws_bytes = kvb_prefill_workspace_bytes(pages * 64, H, QH, D, prompt) + kvb_workspace_bytes(pages * 64, H, QH, D, 8, 1);
    void* ws_b = dev(nullptr, ws_bytes);

    PagedKVLayerView one;
    PagedKVBatchLayerView many;
    auto plane = [&](void* p, int leading) { Tensor t; t.data = p; t.dtype = DType::U8; t.ne[0] = leading; t.ne[1] = 64; t.ne[2] = H; t.ne[3] = pages; return t; };
    one.k_pages = many.k_pages = plane(kc[0], D / 2);
    one.v_pages = many.v_pages = plane(vc[0], D / 2);
    one.k_scale_pages = many.k_scale_pages = plane(ks[0], 5);
    one.v_scale_pages = many.v_scale_pages = plane(vs[0], 4);
    one.block_table.data = table_dev; one.block_table.dtype = DType::I32; one.block_table.ne[0] = pages;
    many.block_tables.data = table_dev; many.block_tables.dtype = DType::I32; many.block_tables.ne[0] = pages; many.block_tables.ne[1] = 1;
    one.num_kv_heads = many.num_kv_heads = H;
    Tensor table_rows; table_rows.data = table_rows_dev; table_rows.dtype = DType::I32;
    Tensor none, pa, pm, pl;
    CausalAttentionExecutionEnvelope env; env.max_visible_keys = pages * 64;

    KvarnTile128BlockTable bt(static_cast<const std::int32_t*>(table_dev), pages);
    Kvarn128Geometry geo; geo.head_dim = D; geo.q_heads = QH; geo.error_word = static_cast<std::uint32_t*>(err_b);
    Kvarn128LayerView vb;
    vb.layer = detail::make_layer(bt, static_cast<unsigned char*>(kc[1]), ks[1], static_cast<unsigned char*>(vc[1]), vs[1], stage_b, H, pages, geo);
    vb.kv_len_max = pages * 64;

    auto tensor_rows = [&](void* p, int heads, int n) { Tensor t; t.data = p; t.ne[0] = D; t.ne[1] = heads; t.ne[2] = n; return t; };
    auto positions = [&](int first, int n) { std::vector<int> h(n); for (int i = 0; i < n; ++i) h[i] = first + i; return dev(h.data(), n * sizeof(int)); };
    int failures = 0;
    auto same = [&](const char* what, void* a, void* b, size_t bytes) {
        std::vector<unsigned char> ha(bytes), hb(bytes);
        cudaMemcpy(ha.data(), a, bytes, cudaMemcpyDeviceToHost);
        cudaMemcpy(hb.data(), b, bytes, cudaMemcpyDeviceToHost);
        bool nonzero = false;
        for (unsigned char c : ha) nonzero |= c != 0;
        if (std::memcmp(ha.data(), hb.data(), bytes) != 0 || !nonzero) { std::printf("FAIL: %s differs or is empty\n", what); ++failures; }
    };

    // 1. prompt chunk: quantise-append + causal attention
    {
        auto hk = rows(prompt, H), hv = rows(prompt, H), hq = rows(prompt, QH);
        void *k = dev(hk.data(), hk.size() * 2), *v = dev(hv.data(), hv.size() * 2), *q = dev(hq.data(), hq.size() * 2);
        void *oa = dev(nullptr, hq.size() * 2), *ob = dev(nullptr, hq.size() * 2), *pos = positions(0, prompt);
        Tensor tk = tensor_rows(k, H, prompt), tv = tensor_rows(v, H, prompt), tq = tensor_rows(q, QH, prompt), to = tensor_rows(oa, QH, prompt);
        Tensor tp; tp.data = pos; tp.dtype = DType::I32; tp.ne[0] = prompt;
        causal_attention_prompt_launch(tq, tk, tv, tp, none, table_rows, 0.088f, many, to, true, nullptr);
        causal_attention_prompt_launch(q, k, v, static_cast<const std::int32_t*>(pos), 0.088f, vb, prompt, ws_b, ob, nullptr);
        OK(cudaDeviceSynchronize());
        same("prompt output", oa, ob, hq.size() * 2);
        same("K codes after the prompt", kc[0], kc[1], code_b);
        same("V scales after the prompt", vs[0], vs[1], vs_b);
    }
    // 2. verify step of `width` rows
    {
        auto hk = rows(width, H), hv = rows(width, H), hq = rows(width, QH);
        void *k = dev(hk.data(), hk.size() * 2), *v = dev(hv.data(), hv.size() * 2), *q = dev(hq.data(), hq.size() * 2);
        void *oa = dev(nullptr, hq.size() * 2), *ob = dev(nullptr, hq.size() * 2), *pos = positions(prompt, width);
        Tensor tk = tensor_rows(k, H, width), tv = tensor_rows(v, H, width), tq = tensor_rows(q, QH, width), to = tensor_rows(oa, QH, width);
        Tensor tp; tp.data = pos; tp.dtype = DType::I32; tp.ne[0] = width;
        causal_attention_small_t_launch(tq, tk, tv, tp, none, table_rows, 0.088f, many, env, 0, width, pa, pm, pl, to, nullptr);
        causal_attention_small_t_launch(q, k, v, static_cast<const std::int32_t*>(pos), 0.088f, vb, width, ws_b, ob, nullptr);
        OK(cudaDeviceSynchronize());
        same("verify output", oa, ob, hq.size() * 2);
    }
    // 3. one more token, then cached decode
    {
        auto hk = rows(1, H), hv = rows(1, H), hq = rows(1, QH);
        void *k = dev(hk.data(), hk.size() * 2), *v = dev(hv.data(), hv.size() * 2), *q = dev(hq.data(), hq.size() * 2);
        void *oa = dev(nullptr, hq.size() * 2), *ob = dev(nullptr, hq.size() * 2), *pos = positions(prompt + width, 1);
        Tensor tk = tensor_rows(k, H, 1), tv = tensor_rows(v, H, 1), tq = tensor_rows(q, QH, 1), to = tensor_rows(oa, QH, 1);
        Tensor tp; tp.data = pos; tp.dtype = DType::I32; tp.ne[0] = 1;
        kv_cache_append_launch(tk, tv, tp, one, nullptr);
        causal_attention_cached_small_t_launch(tq, tp, 0.088f, one, env, pa, pm, pl, to, nullptr);
        kv_cache_append_kvarn128_launch(k, v, static_cast<const std::int32_t*>(pos), bt, static_cast<unsigned char*>(kc[1]), ks[1],
                                        static_cast<unsigned char*>(vc[1]), vs[1], stage_b, 1, H, pages, nullptr, geo);
        causal_attention_cached_small_t_launch(q, static_cast<const std::int32_t*>(pos), 0.088f, vb, ws_b, ob, nullptr);
        OK(cudaDeviceSynchronize());
        same("decode output", oa, ob, hq.size() * 2);
    }
    // 4. a step of 12 columns: appended whole by the first block (columns 0..7), attended in two column blocks; a masked
    //    variant (valid_columns given) appends and attends the same
    {
        const int wide = 12, first = prompt + width + 1;
        auto hk = rows(wide, H), hv = rows(wide, H), hq = rows(wide, QH);
        void *k = dev(hk.data(), hk.size() * 2), *v = dev(hv.data(), hv.size() * 2), *q = dev(hq.data(), hq.size() * 2);
        void *oa = dev(nullptr, hq.size() * 2), *ob = dev(nullptr, hq.size() * 2), *pos = positions(first, wide);
        const int valid = wide;
        void* valid_dev = dev(&valid, sizeof(int));
        Tensor tk = tensor_rows(k, H, wide), tv = tensor_rows(v, H, wide), tq = tensor_rows(q, QH, wide), to = tensor_rows(oa, QH, wide);
        Tensor tp; tp.data = pos; tp.dtype = DType::I32; tp.ne[0] = wide;
        Tensor tvalid; tvalid.data = valid_dev; tvalid.dtype = DType::I32; tvalid.ne[0] = 1;
        causal_attention_small_t_launch(tq, tk, tv, tp, tvalid, table_rows, 0.088f, many, env, 0, 8, pa, pm, pl, to, nullptr);
        causal_attention_small_t_launch(tq, tk, tv, tp, tvalid, table_rows, 0.088f, many, env, 8, 4, pa, pm, pl, to, nullptr);
        const std::int32_t* p = static_cast<const std::int32_t*>(pos);
        const size_t row_bytes = static_cast<size_t>(QH) * D * 2;
        if (kvb_append(&vb.layer, k, v, p, wide, nullptr) != KVB_OK) { std::printf("FAIL: append of the wide step\n"); ++failures; }
        for (int c0 = 0; c0 < wide; c0 += 4)  // other block boundaries on the C-ABI side: the rows do not depend on them
            if (kvb_attn_rows(&vb.layer, static_cast<char*>(q) + c0 * row_bytes, p + c0, 4, p + (wide - 1), 0.088f, vb.kv_len_max, ws_b,
                              static_cast<char*>(ob) + c0 * row_bytes, nullptr) != KVB_OK) { std::printf("FAIL: kvb_attn_rows\n"); ++failures; }
        OK(cudaDeviceSynchronize());
        same("K codes after the wide step", kc[0], kc[1], code_b);
        // blocks of 8 + 4 columns against blocks of 4: different kernels may serve blocks of different widths, so the
        // comparison is within the tolerance of the wider one (2^-8 of the largest magnitude)
        std::vector<unsigned short> ha(hq.size()), hb(hq.size());
        cudaMemcpy(ha.data(), oa, hq.size() * 2, cudaMemcpyDeviceToHost);
        cudaMemcpy(hb.data(), ob, hq.size() * 2, cudaMemcpyDeviceToHost);
        auto h2f = [](unsigned short h) { const int e = (h >> 10) & 31, m = h & 1023; float v = e ? (1.0f + m / 1024.0f) * std::ldexp(1.0f, e - 15) : m / 1024.0f * std::ldexp(1.0f, -14); return (h & 0x8000) ? -v : v; };
        float worst = 0.0f, ref = 0.0f;
        for (size_t i = 0; i < ha.size(); ++i) { worst = std::max(worst, std::fabs(h2f(ha[i]) - h2f(hb[i]))); ref = std::max(ref, std::fabs(h2f(hb[i]))); }
        if (!(worst <= ref / 256.0f) || ref == 0.0f) { std::printf("FAIL: column blocks differ: %g of %g\n", worst, ref); ++failures; }
    }
    unsigned int ea = 1, eb = 1;
    cudaMemcpy(&ea, detail::layer_states()[kc[0]].error_word, 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(&eb, err_b, 4, cudaMemcpyDeviceToHost);
    if (ea != 0 || eb != 0) { std::printf("FAIL: error words %u %u\n", ea, eb); ++failures; }
    kvarn128_release_all();
    std::printf(failures ? "engine shim on the GPU: %d failure(s)\n" : "engine shim on the GPU: ok\n", failures);
    return failures;
}
