// Compiles the C++ host mirror of the reference interface (ninfer::ops::*) against the C ABI and checks the
// host-side behaviour that needs no GPU: names and signatures exist, bad arguments throw std::invalid_argument
// the way the reference's launcher does, an empty append is a silent no-op.
#include <cstdio>
#include <cstring>
#include <stdexcept>

#include "ninfer_kvarn128.hpp"

int main() {
    using namespace ninfer::ops;
    int failures = 0;
    unsigned char* fake = reinterpret_cast<unsigned char*>(0x1000);  // never dereferenced: checks fail before any launch
    KvarnTile128BlockTable table(reinterpret_cast<const std::int32_t*>(fake), 8);
    Kvarn128Geometry geo;
    // empty append returns silently (reference: `if (tokens <= 0) return;`)
    kv_cache_append_kvarn128_launch(fake, fake, reinterpret_cast<const std::int32_t*>(fake), table, fake, fake, fake, fake, fake, 0, 4, 8,
                                    nullptr, geo);
    // unsupported head count -> std::invalid_argument (reference: "KVarN128 unsupported KV head count")
    try {
        kv_cache_append_kvarn128_launch(fake, fake, reinterpret_cast<const std::int32_t*>(fake), table, fake, fake, fake, fake, fake, 1, 0,
                                        8, nullptr, geo);
        std::printf("FAIL: kv_heads = 0 accepted\n");
        ++failures;
    } catch (const std::invalid_argument& e) {
        if (std::strstr(e.what(), "kv_heads") == nullptr) { std::printf("FAIL: message %s\n", e.what()); ++failures; }
    }
    // null plane -> std::invalid_argument (reference: "KVarN128 missing arguments")
    try {
        kv_cache_append_kvarn128_launch(fake, fake, reinterpret_cast<const std::int32_t*>(fake), table, nullptr, fake, fake, fake, fake, 1, 4,
                                        8, nullptr, geo);
        std::printf("FAIL: null plane accepted\n");
        ++failures;
    } catch (const std::invalid_argument&) {
    }
    // tile out of the table -> std::invalid_argument
    try {
        kvarn128_decode_tile(fake, fake, fake, fake, table, 100, 0, 4, 8, fake, fake, nullptr, geo);
        std::printf("FAIL: tile 100 of an 8-entry table accepted\n");
        ++failures;
    } catch (const std::invalid_argument&) {
    }
    Kvarn128LayerView view;
    view.layer = detail::make_layer(table, fake, fake, fake, fake, fake, 4, 8, geo);
    view.kv_len_max = 32768;
    if (causal_attention_split_capacity_kvarn128(view, 1) < 2) { std::printf("FAIL: split capacity\n"); ++failures; }
    if (causal_attention_workspace_bytes_kvarn128(view, 1) == 0) { std::printf("FAIL: workspace bytes\n"); ++failures; }
    // batched decode: more than 64 sequences per call are refused before anything is launched
    {
        std::int32_t bounds[2] = {100, 100};
        if (causal_attention_batch_workspace_bytes_kvarn128(bounds, 2, 4, geo) == 0) { std::printf("FAIL: batch workspace bytes\n"); ++failures; }
        try {
            causal_attention_cached_small_t_batch_launch(reinterpret_cast<const kvb_layer*>(fake), 65, 4, fake, reinterpret_cast<const std::int32_t*>(fake),
                                                         0.1f, bounds, fake, fake, nullptr, geo);
            std::printf("FAIL: 65 sequences accepted\n");
            ++failures;
        } catch (const std::invalid_argument&) {
        }
    }
    if (kvarn128_stage_slots() != 2) { std::printf("FAIL: stage slots\n"); ++failures; }
    std::printf(failures ? "host mirror: %d failure(s)\n" : "host mirror: ok\n", failures);
    return failures;
}
