// ninfer_engine_shim.hpp -- the reference engine's own launcher signatures over the C ABI.
//
// The reference routes a KvarnTile128 cache through five engine-level launchers that take the engine's `Tensor`
// and `PagedKV*LayerView` values (kvarn-port/patches/0003-*.patch: kv_cache_append_launch :1379,
// kv_cache_append_batch_launch :1397, causal_attention_prompt_launch :2362, causal_attention_small_t_launch :3508,
// causal_attention_cached_small_t_launch :3612).  The engine's headers are not part of the reference tree, so the
// value types below carry only the members those launchers read (data pointer, dtype, ne[4] with ne[0] fastest;
// storage kind, the four planes, block table(s), KV head count; the visible-key envelope).  An engine build would
// drop these stand-ins, include its own headers and keep the function bodies.
//
// What differs from the reference's bodies, by design of the replacement:
//   * no bf16 consumer window: the attention launchers read the quantised planes directly, so
//     kvarn128_mirror_layer / _batch and the window pool have no counterpart;
//   * the per-layer fp16 stage is still owned by the op and keyed by the K code plane (kvarn128_launch.cu:275-322),
//     but lives in a table the caller can pre-populate (kvarn128_reserve_stage) so that nothing allocates during
//     CUDA-graph capture; like the reference, a first use inside a capture is an error, not a silent allocation;
//   * partial_acc / partial_m / partial_l are accepted for signature compatibility; the split-K partials live in
//     one workspace allocation per layer, sized by kvb_workspace_bytes and kept beside the stage;
//   * multi-sequence positions are refused loudly, as in the reference (patches/0003:1183-1190): tile sealing is
//     defined for one sequence with contiguous positions.
// Header-only; link with libkvarn_b200.so and the CUDA runtime.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

#include "ninfer_kvarn128.hpp"

namespace ninfer {

enum class DType : std::int32_t { F16 = 0, BF16 = 1, F32 = 2, I32 = 3, U8 = 4 };

// data + dtype + four extents, ne[0] fastest (q: {D, QH, T, B}; k, v: {D, H, T, B}; planes: {leading, 64, H, pages};
// block_tables: {stride, rows}), patches/0003:1060,1586-1587,3304-3321.
struct Tensor {
    void* data = nullptr;
    DType dtype = DType::F16;
    std::int32_t ne[4] = {1, 1, 1, 1};
};

enum class KvCacheStorage : std::int32_t { BFloat16 = 0, KvarnTile128 = 1 };

struct PagedKVLayerView {
    KvCacheStorage storage = KvCacheStorage::KvarnTile128;
    Tensor k_pages, v_pages, k_scale_pages, v_scale_pages;  // u8 codes {D/2, 64, H, pages}; fp16 axes {5S | 4S, 64, H, pages}
    Tensor block_table;                                     // int32 {entries}: resolved table of the sequence
    std::int32_t num_kv_heads = 4;
};

struct PagedKVBatchLayerView {
    KvCacheStorage storage = KvCacheStorage::KvarnTile128;
    Tensor k_pages, v_pages, k_scale_pages, v_scale_pages;
    Tensor block_tables;  // int32 {stride, rows}: row table_rows[b] belongs to batch entry b
    std::int32_t num_kv_heads = 4;
};

// Host-known bounds of the number of visible keys; sizes the split grid so that it is stable under graph replay.
struct CausalAttentionExecutionEnvelope {
    std::int32_t min_visible_keys = 0, max_visible_keys = 0;
    std::int32_t min_count = 1, max_count = 1;
};

namespace ops {

// ---- op-owned per-layer state (stage + split-K workspace), keyed by the K code plane like the reference's stage
struct Kvarn128LayerState {
    void* stage = nullptr;
    void* workspace = nullptr;
    std::size_t workspace_bytes = 0;
    std::uint32_t* error_word = nullptr;
};

namespace detail {
inline std::unordered_map<const void*, Kvarn128LayerState>& layer_states() {
    static std::unordered_map<const void*, Kvarn128LayerState> table;
    return table;
}
inline std::mutex& layer_states_lock() {
    static std::mutex m;
    return m;
}
inline void cuda_ok(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
[[noreturn]] inline void refuse(const char* msg) {
    std::fprintf(stderr, "ninfer: %s\n", msg);
    std::fflush(stderr);
    throw std::invalid_argument(msg);
}
inline bool capturing(cudaStream_t stream) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    return cudaStreamIsCapturing(stream, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone;
}
}  // namespace detail

// Allocates (once) and zeroes the stage of the layer whose K code plane is `k_code`, and a split-K workspace for
// contexts up to `max_visible_keys` with up to `max_rows` query tokens.  Call it before any graph capture; the
// launchers below call it themselves on first use outside a capture.
inline Kvarn128LayerState& kvarn128_reserve_stage(const void* k_code, int head_dim, int kv_heads, int q_heads, int max_visible_keys,
                                                  int max_rows, cudaStream_t stream) {
    std::lock_guard<std::mutex> guard(detail::layer_states_lock());
    Kvarn128LayerState& s = detail::layer_states()[k_code];
    const std::size_t need = kvb_workspace_bytes(max_visible_keys, kv_heads, q_heads, head_dim, max_rows < 8 ? max_rows : 8, 1);
    const std::size_t need_chunk = kvb_prefill_workspace_bytes(max_visible_keys, kv_heads, q_heads, head_dim, max_rows);
    const std::size_t want = need > need_chunk ? need : need_chunk;
    if (s.stage != nullptr && s.workspace_bytes >= want) return s;
    if (detail::capturing(stream))
        detail::refuse("KVarN128: the stage / workspace of a layer must be reserved before CUDA-graph capture begins");
    if (s.stage == nullptr) {
        const std::size_t bytes = kvb_stage_bytes(head_dim, kv_heads);
        detail::cuda_ok(cudaMalloc(&s.stage, bytes), "KVarN128 stage");
        detail::cuda_ok(cudaMemsetAsync(s.stage, 0, bytes, stream), "KVarN128 stage");
        void* ew = nullptr;
        detail::cuda_ok(cudaMalloc(&ew, sizeof(std::uint32_t)), "KVarN128 error word");
        detail::cuda_ok(cudaMemsetAsync(ew, 0, sizeof(std::uint32_t), stream), "KVarN128 error word");
        s.error_word = static_cast<std::uint32_t*>(ew);
    }
    if (s.workspace_bytes < want) {
        if (s.workspace != nullptr) detail::cuda_ok(cudaFree(s.workspace), "KVarN128 workspace");
        detail::cuda_ok(cudaMalloc(&s.workspace, want), "KVarN128 workspace");
        s.workspace_bytes = want;
    }
    return s;
}

// Frees everything kvarn128_reserve_stage allocated (the reference never frees its pools; tests and tools do).
inline void kvarn128_release_all() {
    std::lock_guard<std::mutex> guard(detail::layer_states_lock());
    for (auto& kv : detail::layer_states()) {
        if (kv.second.stage) cudaFree(kv.second.stage);
        if (kv.second.workspace) cudaFree(kv.second.workspace);
        if (kv.second.error_word) cudaFree(kv.second.error_word);
    }
    detail::layer_states().clear();
}

// Sinkhorn iterations of the encoder for every layer routed through this shim.  The reference fixes them at compile time,
// kKvarnIters = 16 (kvarn-port/engine/src/ops/kv_cache/kvarn_layout.h:40-42); that is the default here.  0 selects the
// regime in which codes are bit-exact against the CPU oracle and the tuned attention kernels apply.  Set it before the
// first append of a cache: a cache must be read with the iteration count it was written with.
inline int& kvarn128_sinkhorn_iters() {
    static int iters = 16;
    return iters;
}
inline void kvarn128_set_sinkhorn_iters(int iters) {
    if (iters < 0 || iters > 64) throw std::invalid_argument("KVarN128: sinkhorn iterations must be 0..64");
    kvarn128_sinkhorn_iters() = iters;
}

namespace detail {
inline Kvarn128Geometry geometry_of(const Tensor& rows, int q_heads, const Kvarn128LayerState& st) {
    Kvarn128Geometry g;
    g.head_dim = rows.ne[0];
    g.q_heads = q_heads;
    g.dtype = rows.dtype == DType::BF16 ? KVB_DTYPE_BF16 : KVB_DTYPE_F16;
    g.sinkhorn_iters = kvarn128_sinkhorn_iters();
    g.error_word = st.error_word;
    return g;
}
inline void single_sequence(const Tensor& positions, const char* who) {
    if (positions.ne[1] > 1 || positions.ne[3] > 1) {
        std::fprintf(stderr, "ninfer: %s: KVarN128 takes single-sequence positions (got ne = [%d, %d, %d, %d])\n", who, positions.ne[0],
                     positions.ne[1], positions.ne[2], positions.ne[3]);
        std::fflush(stderr);
        throw std::invalid_argument("KVarN128 requires single-sequence positions");
    }
}
inline KvarnTile128BlockTable direct_table(const Tensor& block_table) {
    return KvarnTile128BlockTable(static_cast<const std::int32_t*>(block_table.data), block_table.ne[0]);
}
inline KvarnTile128BlockTable batch_table(const Tensor& block_tables, const Tensor& table_rows) {
    KvarnTile128BlockTable t;
    t.tables = static_cast<const std::int32_t*>(block_tables.data);
    t.table_rows = static_cast<const std::int32_t*>(table_rows.data);
    t.table_stride = block_tables.ne[0];
    t.table_len = block_tables.ne[0];
    return t;
}
template <typename View>
inline Kvarn128LayerView layer_view(const View& cache, KvarnTile128BlockTable table, const Tensor& rows, int q_heads,
                                    const CausalAttentionExecutionEnvelope* envelope, int max_rows, cudaStream_t stream) {
    if (cache.storage != KvCacheStorage::KvarnTile128) refuse("this shim routes KvarnTile128 storage only");
    const int pages = cache.k_pages.ne[3], kv_heads = cache.num_kv_heads;
    const int bound = envelope != nullptr && envelope->max_visible_keys > 0 ? envelope->max_visible_keys : pages * 64;
    Kvarn128LayerState& st = kvarn128_reserve_stage(cache.k_pages.data, rows.ne[0], kv_heads, q_heads > 0 ? q_heads : kv_heads, bound,
                                                    max_rows, stream);
    Kvarn128LayerView view;
    view.layer = make_layer(table, static_cast<unsigned char*>(cache.k_pages.data), cache.k_scale_pages.data,
                            static_cast<unsigned char*>(cache.v_pages.data), cache.v_scale_pages.data, st.stage, kv_heads, pages,
                            geometry_of(rows, q_heads > 0 ? q_heads : kv_heads, st));
    view.kv_len_max = bound;
    return view;
}
}  // namespace detail

// patches/0003:1379-1395.  k, v: {D, H, tokens, 1}; positions: int32 {tokens}.
inline void kv_cache_append_launch(const Tensor& k, const Tensor& v, const Tensor& positions, PagedKVLayerView cache,
                                   cudaStream_t stream) {
    detail::single_sequence(positions, "kv_cache_append");
    const int tokens = k.ne[2];
    if (tokens <= 0) return;
    const Kvarn128LayerView view = detail::layer_view(cache, detail::direct_table(cache.block_table), k, 0, nullptr, 8, stream);
    detail::raise(kvb_append(&view.layer, k.data, v.data, static_cast<const std::int32_t*>(positions.data), tokens, stream),
                       "kv_cache_append");
}

// patches/0003:1397-1428.  The block table of the sequence is row table_rows[0] of cache.block_tables.  valid_columns
// selects the masked metadata variant in the reference, but its KvarnTile128 branch takes only tables / table_rows /
// table_stride from the metadata (patches/0003:1159-1189) and appends all `tokens` rows: the same here.
inline void kv_cache_append_batch_launch(const Tensor& k, const Tensor& v, const Tensor& positions, const Tensor& /*valid_columns*/,
                                         const Tensor& table_rows, PagedKVBatchLayerView cache, cudaStream_t stream) {
    detail::single_sequence(positions, "kv_cache_append_batch");
    const int tokens = k.ne[2];
    if (tokens <= 0) return;
    const Kvarn128LayerView view = detail::layer_view(cache, detail::batch_table(cache.block_tables, table_rows), k, 0, nullptr, 8, stream);
    detail::raise(kvb_append(&view.layer, k.data, v.data, static_cast<const std::int32_t*>(positions.data), tokens, stream),
                       "kv_cache_append_batch");
}

// patches/0003:3612-3616: decode over a cache that already holds the newest token.  q: {D, QH, 1, 1}.
inline void causal_attention_cached_small_t_launch(const Tensor& q, const Tensor& pos, float scale, const PagedKVLayerView& cache,
                                                   CausalAttentionExecutionEnvelope envelope, Tensor& /*partial_acc*/,
                                                   Tensor& /*partial_m*/, Tensor& /*partial_l*/, Tensor& out, cudaStream_t stream) {
    if (q.ne[2] != 1 || q.ne[3] != 1) detail::refuse("causal_attention_cached_small_t: one query token, one sequence");
    const Kvarn128LayerView view = detail::layer_view(cache, detail::direct_table(cache.block_table), q, q.ne[1], &envelope, 8, stream);
    const Kvarn128LayerState& st = detail::layer_states()[cache.k_pages.data];
    causal_attention_cached_small_t_launch(q.data, static_cast<const std::int32_t*>(pos.data), scale, view, st.workspace, out.data, stream);
}

// patches/0003:3508-3515: verify.  q: {D, QH, full_width, 1}; k, v: {D, H, full_width, 1}; pos: int32 {full_width}.
// As in the reference's KvarnTile128 branch (patches/0003:3517-3545): the whole step (all full_width rows) is appended
// when column_begin == 0; every call then attends the columns [column_begin, column_begin + width) of q, so a step
// wider than 8 columns is one call with column_begin == 0 followed by calls that only attend.  valid_columns (the
// count of real columns of a padded step) does not change what is appended there, nor here; the padded columns'
// outputs are computed like the others and are the caller's to ignore.
inline void causal_attention_small_t_launch(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& pos,
                                            const Tensor& /*valid_columns*/, const Tensor& table_rows, float scale,
                                            PagedKVBatchLayerView cache, CausalAttentionExecutionEnvelope envelope,
                                            std::int32_t column_begin, std::int32_t width, Tensor& /*partial_acc*/, Tensor& /*partial_m*/,
                                            Tensor& /*partial_l*/, Tensor& out, cudaStream_t stream, const void* /*gate*/ = nullptr) {
    detail::single_sequence(pos, "causal_attention_small_t");
    if (q.ne[3] != 1) detail::refuse("causal_attention_small_t: one sequence per call");
    const int full_width = q.ne[2];
    if (width < 1 || width > 8 || column_begin < 0 || column_begin + width > full_width)
        detail::refuse("causal_attention_small_t: columns [column_begin, column_begin + width) must lie in the step, width 1..8");
    const Kvarn128LayerView view = detail::layer_view(cache, detail::batch_table(cache.block_tables, table_rows), q, q.ne[1], &envelope, 8, stream);
    const Kvarn128LayerState& st = detail::layer_states()[cache.k_pages.data];
    const std::int32_t* positions = static_cast<const std::int32_t*>(pos.data);
    if (column_begin == 0)
        detail::raise(kvb_append(&view.layer, k.data, v.data, positions, full_width, stream), "causal_attention_small_t (append)");
    const std::size_t row_bytes = static_cast<std::size_t>(q.ne[0]) * q.ne[1] * 2;  // fp16 / bf16 rows of all q heads
    detail::raise(kvb_attn_rows(&view.layer, static_cast<const char*>(q.data) + column_begin * row_bytes, positions + column_begin, width,
                                positions + (full_width - 1), scale, view.kv_len_max, st.workspace,
                                static_cast<char*>(out.data) + column_begin * row_bytes, stream),
                  "causal_attention_small_t");
}

// patches/0003:2362-2366: prefill chunk.  q: {D, QH, tokens, 1}; k, v: {D, H, tokens, 1}.  `fast` selects between two
// kernels of equal results in the reference and is ignored here; valid_columns as in kv_cache_append_batch_launch.
inline void causal_attention_prompt_launch(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& positions,
                                           const Tensor& valid_columns, const Tensor& table_rows, float scale,
                                           PagedKVBatchLayerView cache, Tensor& out, bool /*fast*/, cudaStream_t stream) {
    detail::single_sequence(positions, "causal_attention_prompt");
    (void)valid_columns;  // as for the append: the reference's KvarnTile128 branch does not read it
    if (q.ne[3] != 1) detail::refuse("causal_attention_prompt: one sequence per call");
    const int tokens = q.ne[2];
    if (tokens <= 0) return;
    const Kvarn128LayerView view =
        detail::layer_view(cache, detail::batch_table(cache.block_tables, table_rows), q, q.ne[1], nullptr, tokens, stream);
    const Kvarn128LayerState& st = detail::layer_states()[cache.k_pages.data];
    causal_attention_prompt_launch(q.data, k.data, v.data, static_cast<const std::int32_t*>(positions.data), scale, view, tokens,
                                   st.workspace, out.data, stream);
}

}  // namespace ops
}  // namespace ninfer
