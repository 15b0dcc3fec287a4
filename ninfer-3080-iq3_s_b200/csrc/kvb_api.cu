// kvb_api.cu -- argument checks, error text and size queries of the C ABI.
#include <cstdarg>
#include <cstring>

#include "kvb_common.cuh"

namespace kvb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(kvb_status st, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    // loud failure, like the reference's fprintf + fflush before it throws (kvarn128_launch.cu:1024-1061)
    std::fprintf(stderr, "kvarn_b200: %s\n", g_error);
    std::fflush(stderr);
    return static_cast<int>(st);
}

LayerView make_view(const kvb_layer& L) {
    LayerView V;
    V.k_code = L.k_code;
    V.k_scale = static_cast<__half*>(L.k_scale);
    V.v_code = L.v_code;
    V.v_scale = static_cast<__half*>(L.v_scale);
    V.stage = static_cast<__half*>(L.stage);
    V.table_direct = L.table_direct;
    V.tables = L.tables;
    V.table_rows = L.table_rows;
    V.table_stride = L.table_stride;
    V.table_len = L.table_len;
    V.pages = L.pages;
    V.kv_heads = L.kv_heads;
    V.q_heads = L.q_heads;
    V.head_dim = L.head_dim;
    V.dtype = L.dtype;
    V.iters = L.sinkhorn_iters;
    V.error_word = L.error_word;
    return V;
}

int check_layer(const kvb_layer* L, const char* who) {
    if (L == nullptr) return fail(KVB_EINVAL, "%s: null layer", who);
    if (L->k_code == nullptr || L->k_scale == nullptr || L->v_code == nullptr || L->v_scale == nullptr)
        return fail(KVB_EINVAL, "%s: a plane pointer is null", who);
    if (L->table_direct == nullptr && (L->tables == nullptr || L->table_rows == nullptr))
        return fail(KVB_EINVAL, "%s: no block table (table_direct, or tables + table_rows)", who);
    if (L->head_dim != 128 && L->head_dim != 256)
        return fail(KVB_EINVAL, "%s: head_dim %d unsupported (128 or 256)", who, L->head_dim);
    if (L->kv_heads < 1 || L->kv_heads > 8) return fail(KVB_EINVAL, "%s: kv_heads %d unsupported (1..8)", who, L->kv_heads);
    if (L->q_heads < L->kv_heads || L->q_heads % L->kv_heads != 0 || L->q_heads / L->kv_heads > 8)
        return fail(KVB_EINVAL, "%s: q_heads %d must be kv_heads * (1..8)", who, L->q_heads);
    if (L->dtype != KVB_DTYPE_F16 && L->dtype != KVB_DTYPE_BF16) return fail(KVB_EINVAL, "%s: dtype %d", who, L->dtype);
    if (L->pages < 1 || L->table_len < 1) return fail(KVB_EINVAL, "%s: pages %d / table_len %d", who, L->pages, L->table_len);
    if (L->sinkhorn_iters < 0 || L->sinkhorn_iters > 64) return fail(KVB_EINVAL, "%s: sinkhorn_iters %d", who, L->sinkhorn_iters);
    return KVB_OK;
}

}  // namespace kvb

extern "C" const char* kvb_last_error_string(void) { return kvb::g_error; }
extern "C" int kvb_version(void) { return 1; }

extern "C" size_t kvb_stage_bytes(int head_dim, int kv_heads) {
    return static_cast<size_t>(2) * 2 * kv_heads * kvb::kTile * head_dim * sizeof(__half);
}

extern "C" size_t kvb_plane_bytes(int which, int head_dim, int kv_heads, int pages) {
    const int S = head_dim / kvb::kSlice;
    const size_t per_token = which == 0 || which == 2 ? head_dim / 2 : (which == 1 ? 5 * S * 2 : 4 * S * 2);
    return per_token * kvb::kPage * kv_heads * pages;
}
