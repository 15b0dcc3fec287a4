// ninfer_kvarn128.hpp -- C++ host mirror of the reference's kvarn128 operator interface over the C ABI.
//
// Same names, argument meaning and error behaviour as the reference's
// kvarn-port/engine/src/ops/kv_cache/append/kvarn128_launch.h (lines 21-58): functions live in
// namespace ninfer::ops, take raw device pointers and a cudaStream_t, print to stderr and throw
// std::invalid_argument on a bad argument (kvarn128_launch.cu:1024-1061) and std::runtime_error when a
// CUDA call fails (the reference's CUDA_CHECK).  Differences, all forced by the drop-in being a library
// without hidden global state:
//   * the per-layer fp16 stage is caller-owned and passed in (the reference allocates it lazily in a
//     process-global table keyed by the K code plane, kvarn128_launch.cu:275-322);
//   * there is no bf16 "consumer window": attention reads the quantised planes directly
//     (causal_attention_*_kvarn128 below), so kvarn128_window* have no counterpart;
//   * head_dim and the input dtype are arguments (the reference is fixed to 256 / bf16).
// Header-only; link with libkvarn_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <stdexcept>
#include <string>

#include "../../include/kvarn_b200.h"

namespace ninfer::ops {

// Block-table descriptor, passed by value: either a resolved table or tables + table_rows[0] * stride.
// Resolution happens on the device only (kvarn128_launch.h:21-36).
struct KvarnTile128BlockTable {
    const std::int32_t* direct = nullptr;
    const std::int32_t* tables = nullptr;
    const std::int32_t* table_rows = nullptr;
    std::int32_t table_stride = 0;
    std::int32_t table_len = 0;  // entries readable in the resolved table (device-side bounds check)

    KvarnTile128BlockTable() = default;
    KvarnTile128BlockTable(const std::int32_t* table, std::int32_t len) : direct(table), table_len(len) {}
};

// Geometry the reference fixes at compile time (kvarn_layout.h:34-42).
struct Kvarn128Geometry {
    int head_dim = 128;
    int q_heads = 24;
    int dtype = KVB_DTYPE_F16;
    int sinkhorn_iters = 0;
    std::uint32_t* error_word = nullptr;
};

namespace detail {
inline void raise(int status, const char* who) {
    if (status == KVB_OK) return;
    const std::string msg = std::string(who) + ": " + kvb_last_error_string();
    if (status == KVB_EINVAL || status == KVB_ERANGE) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}
inline kvb_layer make_layer(KvarnTile128BlockTable table, unsigned char* k_code, void* k_scale, unsigned char* v_code,
                            void* v_scale, void* stage, int kv_heads, int pages, const Kvarn128Geometry& geo) {
    kvb_layer L{};
    L.k_code = k_code; L.k_scale = k_scale; L.v_code = v_code; L.v_scale = v_scale; L.stage = stage;
    L.table_direct = table.direct; L.tables = table.tables; L.table_rows = table.table_rows;
    L.table_stride = table.table_stride; L.table_len = table.table_len;
    L.pages = pages; L.kv_heads = kv_heads; L.q_heads = geo.q_heads; L.head_dim = geo.head_dim;
    L.dtype = geo.dtype; L.sinkhorn_iters = geo.sinkhorn_iters; L.error_word = geo.error_word;
    return L;
}
}  // namespace detail

// kvarn128_launch.h:40-44.  `stage` is the layer's persistent fp16 stage (kvb_stage_bytes() bytes, zeroed once).
inline void kv_cache_append_kvarn128_launch(const void* k, const void* v, const std::int32_t* positions,
                                            KvarnTile128BlockTable table, unsigned char* k_code, void* k_scale,
                                            unsigned char* v_code, void* v_scale, void* stage, int tokens, int kv_heads,
                                            int pages, cudaStream_t stream, const Kvarn128Geometry& geo = {}) {
    if (tokens <= 0) return;  // kvarn128_launch.cu:1023
    const kvb_layer L = detail::make_layer(table, k_code, k_scale, v_code, v_scale, stage, kv_heads, pages, geo);
    detail::raise(kvb_append(&L, k, v, positions, tokens, stream), "kv_cache_append");
}

// kvarn128_launch.h:56-58: one tile -> rotated-domain fp16 [128][head_dim].
inline void kvarn128_decode_tile(const void* k_code, const void* k_scale, const void* v_code, const void* v_scale,
                                 KvarnTile128BlockTable table, int tile, int head, int kv_heads, int pages, void* out_k,
                                 void* out_v, cudaStream_t stream, const Kvarn128Geometry& geo = {}) {
    const kvb_layer L = detail::make_layer(table, static_cast<unsigned char*>(const_cast<void*>(k_code)),
                                           const_cast<void*>(k_scale), static_cast<unsigned char*>(const_cast<void*>(v_code)),
                                           const_cast<void*>(v_scale), nullptr, kv_heads, pages, geo);
    detail::raise(kvb_decode_tile(&L, tile, head, out_k, out_v, stream), "kvarn128_decode_tile");
}

inline int kvarn128_stage_slots() { return 2; }  // kvarn128_launch.h:51

// A layer view for the attention launchers (stands in for the engine's PagedKVLayerView with storage
// KvarnTile128, patches/0003 lines 3612-3631).
struct Kvarn128LayerView {
    kvb_layer layer{};
    int kv_len_max = 0;  // host upper bound of the sequence length (sizes the split grid, graph-stable)
};

// causal_attention_split_capacity (patches/0003:3326-3380)
inline int causal_attention_split_capacity_kvarn128(const Kvarn128LayerView& view, int tokens, int batch = 1) {
    return kvb_split_capacity(view.kv_len_max, view.layer.kv_heads, view.layer.q_heads, tokens, batch);
}
inline std::size_t causal_attention_workspace_bytes_kvarn128(const Kvarn128LayerView& view, int tokens, int batch = 1) {
    return kvb_workspace_bytes(view.kv_len_max, view.layer.kv_heads, view.layer.q_heads, view.layer.head_dim, tokens, batch);
}

// causal_attention_cached_small_t_launch (patches/0003:3612-3616): q [D, QH, 1, 1], pos [1] on the device.
// `partials` replaces the three tensors partial_acc / partial_m / partial_l.
inline void causal_attention_cached_small_t_launch(const void* q, const std::int32_t* pos, float scale,
                                                   const Kvarn128LayerView& view, void* partials, void* out,
                                                   cudaStream_t stream) {
    detail::raise(kvb_attn_decode(&view.layer, q, pos, scale, view.kv_len_max, partials, out, stream),
                  "causal_attention_cached_small_t");
}

// causal_attention_small_t_launch (patches/0003:3508-3515): appends the `width` new rows, then causal attention.
inline void causal_attention_small_t_launch(const void* q, const void* k, const void* v, const std::int32_t* pos, float scale,
                                            const Kvarn128LayerView& view, int width, void* partials, void* out,
                                            cudaStream_t stream) {
    detail::raise(kvb_attn_verify(&view.layer, q, k, v, pos, width, scale, view.kv_len_max, partials, out, stream),
                  "causal_attention_small_t");
}

// causal_attention_prompt_launch (patches/0003:2362-2366): quantise-append the chunk, then causal chunk attention.
inline void causal_attention_prompt_launch(const void* q, const void* k, const void* v, const std::int32_t* positions,
                                           float scale, const Kvarn128LayerView& view, int tokens, void* workspace, void* out,
                                           cudaStream_t stream) {
    detail::raise(kvb_attn_prefill(&view.layer, q, k, v, positions, tokens, scale, view.kv_len_max, workspace, out, stream),
                  "causal_attention_prompt");
}

// ---- calls without a counterpart in the reference (one GPU, one sequence per call there)

// Decode for up to 64 independent sequences in one call.  `layers_dev`: device array of kvb_layer descriptors (upload
// once); `kv_len_max`: host array of upper bounds of the lengths; q, out: [batch][q_heads][head_dim]; pos: [batch].
inline std::size_t causal_attention_batch_workspace_bytes_kvarn128(const std::int32_t* kv_len_max, int batch, int kv_heads,
                                                                  const Kvarn128Geometry& geo = {}) {
    return kvb_batch_workspace_bytes(kv_len_max, batch, kv_heads, geo.q_heads, geo.head_dim);
}
inline void causal_attention_cached_small_t_batch_launch(const kvb_layer* layers_dev, int batch, int kv_heads, const void* q,
                                                         const std::int32_t* pos, float scale, const std::int32_t* kv_len_max,
                                                         void* workspace, void* out, cudaStream_t stream,
                                                         const Kvarn128Geometry& geo = {}) {
    detail::raise(kvb_attn_decode_batch(layers_dev, batch, kv_heads, geo.q_heads, geo.head_dim, geo.dtype, q, pos, scale, kv_len_max,
                                        workspace, out, stream),
                  "causal_attention_cached_small_t_batch");
}

// Decode of one sequence whose tile ranges live on several GPUs: this rank's range in `view`, partials exchanged by
// the kernels through the peer-mapped ring buffers of `ring` (see kvb_peer_ring in the C header).
inline void causal_attention_cached_small_t_sharded_launch(const void* q, const std::int32_t* local_pos, float scale,
                                                           const Kvarn128LayerView& view, const kvb_peer_ring& ring, void* workspace,
                                                           void* out, cudaStream_t stream) {
    detail::raise(kvb_attn_decode_sharded(&view.layer, q, local_pos, scale, view.kv_len_max, workspace, &ring, out, stream),
                  "causal_attention_cached_small_t_sharded");
}

// A verify step of `width` (1..8) rows over such a sequence: the rank that owns the open tile appends the rows
// first (k, v non-null there, null elsewhere), every rank attends its own range, the partials are exchanged by the
// kernels (the ring buffers must hold width * q_heads rows: kvb_peer_ring::rows).
inline void causal_attention_small_t_sharded_launch(const void* q, const void* k, const void* v, const std::int32_t* local_pos,
                                                    int width, float scale, const Kvarn128LayerView& view, const kvb_peer_ring& ring,
                                                    void* workspace, void* out, cudaStream_t stream) {
    if (k != nullptr && v != nullptr)
        detail::raise(kvb_append(&view.layer, k, v, local_pos, width, stream), "causal_attention_small_t_sharded (append)");
    detail::raise(kvb_attn_rows_sharded(&view.layer, q, local_pos, width, scale, view.kv_len_max, workspace, &ring, out, stream),
                  "causal_attention_small_t_sharded");
}

// One decode step as one call: append the token at *pos, then attend (ring: null, or the ring of a sharded sequence on
// the rank that owns the open tile).
inline void kv_cache_append_then_decode_launch(const void* q, const void* k, const void* v, const std::int32_t* pos, float scale,
                                               const Kvarn128LayerView& view, const kvb_peer_ring* ring, void* workspace, void* out,
                                               cudaStream_t stream) {
    detail::raise(kvb_append_decode(&view.layer, q, k, v, pos, scale, view.kv_len_max, workspace, ring, out, stream),
                  "kv_cache_append_then_decode");
}

}  // namespace ninfer::ops
