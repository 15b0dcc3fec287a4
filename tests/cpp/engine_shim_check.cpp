// Compiles the engine-shaped adapter (ninfer::ops launchers over Tensor / PagedKV*LayerView values) and checks the
// host-side behaviour that needs no GPU: the five launcher signatures exist; multi-sequence positions, column blocks
// that leave the step and foreign storage kinds are refused with std::invalid_argument before anything is allocated
// or launched; empty appends return silently; the encoder's iteration count defaults to the reference's 16.
#include <cstdio>
#include <stdexcept>

#include "ninfer_engine_shim.hpp"

template <typename F> static int expect_refusal(const char* what, F&& f) {
    try {
        f();
    } catch (const std::invalid_argument&) {
        return 0;
    } catch (const std::exception& e) {
        std::printf("FAIL: %s threw %s\n", what, e.what());
        return 1;
    }
    std::printf("FAIL: %s was accepted\n", what);
    return 1;
}

int main() {
    using namespace ninfer;
    using namespace ninfer::ops;
    int failures = 0;
    void* fake = reinterpret_cast<void*>(0x1000);  // never dereferenced
    Tensor k, v, q, out, pos, none, rows, pa, pm, pl;
    k.data = v.data = q.data = out.data = pos.data = rows.data = fake;
    k.ne[0] = v.ne[0] = q.ne[0] = 128; k.ne[1] = v.ne[1] = 4; q.ne[1] = 24;
    pos.dtype = rows.dtype = DType::I32;
    PagedKVLayerView one;
    PagedKVBatchLayerView many;
    one.k_pages.data = many.k_pages.data = fake;
    one.k_pages.ne[3] = many.k_pages.ne[3] = 8;
    CausalAttentionExecutionEnvelope env;
    env.max_visible_keys = 512;

    // empty appends are silent no-ops (reference: `if (tokens <= 0) return;`)
    k.ne[2] = v.ne[2] = 0;
    kv_cache_append_launch(k, v, pos, one, nullptr);
    kv_cache_append_batch_launch(k, v, pos, none, rows, many, nullptr);
    k.ne[2] = v.ne[2] = q.ne[2] = 4;

    // multi-sequence positions are refused loudly
    Tensor pos2 = pos;
    pos2.ne[1] = 2;
    failures += expect_refusal("append with multi-sequence positions", [&] { kv_cache_append_launch(k, v, pos2, one, nullptr); });
    failures += expect_refusal("prompt with multi-sequence positions",
                               [&] { causal_attention_prompt_launch(q, k, v, pos2, none, rows, 0.1f, many, out, true, nullptr); });
    // column blocks must lie inside the step and hold 1..8 columns
    failures += expect_refusal("verify columns [2, 6) of a 4-column step", [&] {
        causal_attention_small_t_launch(q, k, v, pos, none, rows, 0.1f, many, env, 2, 4, pa, pm, pl, out, nullptr);
    });
    failures += expect_refusal("verify block of 0 columns", [&] {
        causal_attention_small_t_launch(q, k, v, pos, none, rows, 0.1f, many, env, 0, 0, pa, pm, pl, out, nullptr);
    });
    // the encoder runs the reference's iteration count unless told otherwise
    if (kvarn128_sinkhorn_iters() != 16) { std::printf("FAIL: default Sinkhorn iterations %d, the reference's are 16\n", kvarn128_sinkhorn_iters()); ++failures; }
    failures += expect_refusal("65 Sinkhorn iterations", [&] { kvarn128_set_sinkhorn_iters(65); });
    kvarn128_set_sinkhorn_iters(0);
    if (kvarn128_sinkhorn_iters() != 0) { std::printf("FAIL: the iteration count did not change\n"); ++failures; }
    // decode takes one token
    failures += expect_refusal("cached decode with 4 tokens",
                               [&] { causal_attention_cached_small_t_launch(q, pos, 0.1f, one, env, pa, pm, pl, out, nullptr); });
    // other storage kinds are not this shim's business
    one.storage = KvCacheStorage::BFloat16;
    failures += expect_refusal("bf16 storage", [&] { kv_cache_append_launch(k, v, pos, one, nullptr); });
    std::printf(failures ? "engine shim: %d failure(s)\n" : "engine shim: ok\n", failures);
    return failures;
}
