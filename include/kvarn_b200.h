/*
 * kvarn_b200.h -- C ABI of the B200 (sm_100a) KVarN quantized paged KV-cache library.
 *
 * Drop-in boundary for the reference's kvarn-port operator API.  Every entry point names the
 * reference interface it replaces (paths relative to the reference repository root;
 * LAUNCH.h = kvarn-port/engine/src/ops/kv_cache/append/kvarn128_launch.h,
 * LAUNCH.cu = the .cu beside it, P3 = kvarn-port/patches/0003-*.patch).
 *
 * Conventions
 *   - plain pointers and sizes; every buffer is caller-owned DEVICE memory unless stated.
 *   - `stream` is a cudaStream_t passed as void*.
 *   - calls are asynchronous on `stream`; none synchronises, none allocates.
 *   - no exceptions cross the ABI: functions return a kvb_status; kvb_last_error_string()
 *     gives the text of the calling thread's last failure.
 *   - positions and block tables are read on the device only (the reference's hard rule,
 *     LAUNCH.cu:5-11): the host never dereferences them.
 *
 * Memory layout (identical to the reference's P1 planes, kvarn_layout.h:61-131, generalised to
 * S = head_dim/128 in {1,2} slices):
 *   k_code, v_code : u8  {head_dim/2, 64, kv_heads, pages}   byte b of a token row = dims 2b | 2b+1<<4
 *   k_scale        : f16 {5S, 64, kv_heads, pages}           cols [0,2S) scale_axis[dim 2S*row+col],
 *                                                            [2S,4S) zp_axis, 4S+s other_axis[token row]
 *   v_scale        : f16 {4S, 64, kv_heads, pages}           cols [0,2S) other_axis[dim], 2S+s scale_axis[token],
 *                                                            3S+s zp_axis[token]
 *   element offset = L*64*(head + kv_heads*page) + L*page_off + slot   (kvarn_layout.h:90-97)
 *   stage          : f16 [K|V][slot = tile%2][kv_heads][128][head_dim] rotated, un-quantised rows of the
 *                    open tile; persistent state of the layer (LAUNCH.cu:262-273), kvb_stage_bytes().
 *   tile t (128 tokens) = logical pages 2t, 2t+1 -> physical pages table[2t], table[2t+1].
 */
#ifndef KVARN_B200_H
#define KVARN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum kvb_status {
    KVB_OK = 0,
    KVB_EINVAL = 1,   /* bad argument (the reference throws std::invalid_argument, LAUNCH.cu:1024-1061) */
    KVB_ECUDA = 2,    /* a CUDA call failed (the reference's CUDA_CHECK, LAUNCH.cu:1075-1091) */
    KVB_ERANGE = 3,   /* a size exceeds what the call supports */
    KVB_ETIMEOUT = 4  /* a bounded device-side wait gave up (read from the error word) */
} kvb_status;

enum { KVB_DTYPE_F16 = 0, KVB_DTYPE_BF16 = 1 };

/* One layer's cache, passed by pointer to every call (host struct of device pointers).
 * Replaces the argument list of kv_cache_append_kvarn128_launch (LAUNCH.h:40-44) and the
 * KvarnTile128BlockTable descriptor (LAUNCH.h:21-36). */
typedef struct kvb_layer {
    uint8_t* k_code;
    void* k_scale;
    uint8_t* v_code;
    void* v_scale;
    void* stage;                 /* kvb_stage_bytes(head_dim, kv_heads) bytes, zero-initialised by the caller */
    const int32_t* table_direct; /* resolved table, or NULL to use tables + table_rows[0]*table_stride */
    const int32_t* tables;
    const int32_t* table_rows;
    int32_t table_stride;
    int32_t table_len;           /* entries readable in the resolved table (bounds check on device) */
    int32_t pages;               /* physical pages in the planes */
    int32_t kv_heads;            /* 1..8 */
    int32_t q_heads;             /* multiple of kv_heads; q_heads/kv_heads <= 8 */
    int32_t head_dim;            /* 128 or 256 */
    int32_t dtype;               /* KVB_DTYPE_* of k, v, q and out */
    int32_t sinkhorn_iters;      /* 0 = bit-exact regime; the reference engine's default is 16 */
    uint32_t* error_word;        /* optional device word: kernels OR in a code instead of faulting */
} kvb_layer;

/* bits OR-ed into *error_word */
enum { KVB_ERR_PAGE_RANGE = 1u, KVB_ERR_TABLE_RANGE = 2u, KVB_ERR_WAIT_TIMEOUT = 4u, KVB_ERR_POSITIONS = 8u, KVB_ERR_GEOMETRY = 16u };

const char* kvb_last_error_string(void);
int kvb_version(void);

/* Sizes. */
size_t kvb_stage_bytes(int head_dim, int kv_heads);
size_t kvb_plane_bytes(int which /*0 k_code,1 k_scale,2 v_code,3 v_scale*/, int head_dim, int kv_heads, int pages);

/* Append `tokens` contiguous positions positions_dev[0..tokens) of one sequence: rotate the rows into the
 * stage, and quantise every tile the append completes into its two pages.
 * k, v: [tokens][kv_heads][head_dim], dim fastest (LAUNCH.cu:111-113).
 * Replaces kv_cache_append_kvarn128_launch (LAUNCH.h:40-44, LAUNCH.cu:1018-1097). */
int kvb_append(const kvb_layer* layer, const void* k, const void* v, const int32_t* positions_dev, int tokens,
               void* stream);

/* De-quantise tile `tile` of head `head` to rotated-domain fp16 [128][head_dim] (out_k, out_v).
 * Replaces kvarn128_decode_tile (LAUNCH.h:56-58, LAUNCH.cu:1099-1115). */
int kvb_decode_tile(const kvb_layer* layer, int tile, int head, void* out_k, void* out_v, void* stream);

/* The compact tile record at every code width of the reference (bits = 2, 3, 4, 5, 6 or 8): each 128 x 128 fp32 matrix
 * (a K tile with the dims as rows, a V tile with the tokens as rows, as the caller lays it out) becomes
 *     payload (LSB-first bit string, row-major, 16 * bits bytes per row) || scale_axis[128] || zp_axis[128] || other_axis[128]
 * (axes fp16), kvb_record_bytes(bits) = 2048 * bits + 768 bytes: 140 B per token and KV head for K4V4, 108 B for K4V2.
 * No variance balancing (other_axis = 1): codes and axes equal the host oracle's bit for bit
 * (kvarn-evidence/oracle/bee_oracle.cpp:152-172 bit string, :309-357 quantiser, :359-374 inverse; the engine's kernels are
 * templated on the same widths, kvarn128_launch.cu:126,158,248).  tiles: [n_tiles][128][128] fp32; records:
 * n_tiles * kvb_record_bytes(bits) bytes; all device memory.  The attention entry points read 4-bit P1 planes only. */
size_t kvb_record_bytes(int bits);
int kvb_records_encode(const float* tiles, int n_tiles, int bits, void* records, void* stream);
int kvb_records_decode(const void* records, int n_tiles, int bits, float* tiles, void* stream);

/* Split count and workspace size for the attention calls.
 * Replace causal_attention_split_capacity (P3:3326-3380) and the partial_acc/partial_m/partial_l tensors
 * the reference's callers allocate (P3:3612-3616). rows = query tokens per call (1 decode, 1..8 verify). */
int kvb_split_capacity(int kv_len_max, int kv_heads, int q_heads, int rows, int batch);
size_t kvb_workspace_bytes(int kv_len_max, int kv_heads, int q_heads, int head_dim, int rows, int batch);

/* Decode attention of one query token over the cache (the token at *pos_dev is already appended):
 * out = softmax(scale * q K^T) V over keys 0..pos, keys of sealed tiles read from the quantised pages
 * (de-quantisation fused into the QK and PV loops), keys of the open tile from the stage.
 * q, out: [q_heads][head_dim].  kv_len_max: host upper bound of pos+1 (sizes the grid, graph-stable).
 * workspace: kvb_workspace_bytes(kv_len_max, ..., rows=1, batch=1) bytes.
 * Replaces causal_attention_cached_small_t_launch (P3:3612-3696). */
int kvb_attn_decode(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale, int kv_len_max,
                    void* workspace, void* out, void* stream);

/* Decode attention without a caller-supplied workspace.  No counterpart in the reference.
 * For hosts that cannot get device memory while they run -- an engine whose KV pool took the whole GPU at
 * start-up, a serving thread that must stay away from the allocator -- the split-K partials live in a fixed
 * 2 MiB array inside the library (kvb_static_scratch_bytes()); every GPU that loads the library holds it until
 * the process exits.  Same arguments and result as kvb_attn_decode minus the workspace.  The call allocates
 * nothing.  The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current); make that first call before any stream capture begins.  Shapes whose partials do not fit
 * (kvb_workspace_bytes(...) > kvb_static_scratch_bytes()) are refused with KVB_ERANGE.  All calls on a device
 * share the one array, which keeps what the previous call left in it -- nothing in it needs clearing, each call
 * writes every entry before reading it -- so two calls that overlap on the GPU (different streams) race. */
size_t kvb_static_scratch_bytes(void);
int kvb_attn_decode_static(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale, int kv_len_max,
                           void* out, void* stream);

/* Decode for `batch` (1..64) independent sequences in one pair of launches; larger batches: several calls.
 * No counterpart in the reference, whose kvarn128 path is single-sequence (patches/0003:1181-1190).
 * `layers_dev` is a DEVICE array of `batch` kvb_layer structs (upload it once: the descriptors only hold
 * pointers and sizes), all with the geometry given here (kv_heads, q_heads, head_dim = 128, dtype) and
 * sinkhorn_iters = 0; an entry that disagrees sets KVB_ERR_GEOMETRY in its error word.  The caches may share
 * planes (one pool, one block table per sequence) or not.  q, out: [batch][q_heads][head_dim]; pos_dev: [batch]
 * positions of the newest token of each sequence (device).  kv_len_max: HOST array of upper bounds of the lengths:
 * it shapes the grid -- every sequence gets splits in proportion to its bound -- and must be the same at capture
 * and replay.  Workspace: kvb_batch_workspace_bytes(same bounds). */
size_t kvb_batch_workspace_bytes(const int32_t* kv_len_max, int batch, int kv_heads, int q_heads, int head_dim);
int kvb_attn_decode_batch(const kvb_layer* layers_dev, int batch, int kv_heads, int q_heads, int head_dim, int dtype,
                          const void* q, const int32_t* pos_dev, float scale, const int32_t* kv_len_max, void* workspace,
                          void* out, void* stream);

/* Same, but stops before the final normalisation: writes the log-sum-exp partial of keys
 * [key_begin, key_end) -- part_m[q_heads] (max logit, natural log units), part_l[q_heads] (sum of
 * exp(logit - m)), part_o[q_heads][head_dim] (sum of exp(logit - m) * V, rotated domain), fp32.
 * One GPU's contribution to a sequence-range sharded decode. No counterpart in the reference (single GPU). */
int kvb_attn_decode_partial(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale,
                            int kv_len_max, int key_begin, int key_end, void* workspace, float* part_m,
                            float* part_l, float* part_o, void* stream);

/* Merge `parts` partial sets laid out [parts][q_heads](m), [parts][q_heads](l), [parts][q_heads][head_dim](o):
 * log-sum-exp merge, normalise, inverse rotation, write out [q_heads][head_dim] in `dtype`.
 * Replaces causal_attention_small_t_reduce_output_kernel (P3:3467-3482) for the cross-GPU step. */
int kvb_merge_partials(const float* parts_m, const float* parts_l, const float* parts_o, int parts, int q_heads,
                       int head_dim, int dtype, void* out, void* stream);

/* Same merge for partials that travel as one block per part: block p = m[q_heads] | l[q_heads] | o[q_heads][head_dim]
 * (q_heads * (head_dim + 2) floats), the layout one all-gather of kvb_attn_decode_partial outputs produces when
 * part_m, part_l, part_o point into one send buffer.  No counterpart in the reference (single GPU). */
int kvb_merge_partials_packed(const float* packed, int parts, int q_heads, int head_dim, int dtype, void* out, void* stream);

/* Sequence-range sharded decode without a collective library on the data path.  No counterpart in the reference
 * (single GPU).  Every rank holds its tile range of the sequence as a local cache and owns a ring buffer of
 * kvb_peer_ring_bytes() bytes that all ranks can write (peer memory over NVLink, e.g. a symmetric-memory
 * allocation); `peer_bufs` is a host array with the ring buffer address (16-byte aligned) of every rank in rank
 * order, this rank's own included; it is read during the call only.  One call = attention over the local range, then one kernel in which the CTA of each query
 * row stores its (m, l, o) partial of the row straight into every peer's ring buffer -- each fp32 value in one
 * 8-byte word together with the call number, so a word that shows the expected call number also shows its value
 * and no fence or flag is needed -- waits, bounded by `max_spins` polling rounds (0 = default), for the peers'
 * partials of the same row, merges them in rank order (all ranks write the same bits), rotates back and writes
 * `out`: two launches, like the single-GPU decode.
 * A wait that runs out sets KVB_ERR_WAIT_TIMEOUT in *layer->error_word and writes zeros; nothing traps or hangs.
 * `state` is three zero-initialised device words owned by this rank.  Ring buffer and state must be zeroed once
 * before the first call; all ranks must make the same sequence of calls on a ring; calls on one ring must not
 * overlap on the GPU.  head_dim 128, at most 16 ranks. */
typedef struct kvb_peer_ring {
    void* const* peer_bufs;
    void* local_buf;
    uint32_t* state;
    int32_t rank, world;
    uint32_t max_spins;
    uint32_t rows;  /* query rows (tokens x q heads) the ring buffers hold: they were sized with
                       kvb_peer_ring_bytes(world, rows, head_dim); 0 = the layer's q_heads (one token per call) */
} kvb_peer_ring;
size_t kvb_peer_ring_bytes(int world, int q_heads, int head_dim);
int kvb_attn_decode_sharded(const kvb_layer* layer, const void* q, const int32_t* pos_dev, float scale, int kv_len_max,
                            void* workspace, const kvb_peer_ring* ring, void* out, void* stream);

/* The same exchange for a verify step of 1..8 query tokens over a range-sharded sequence: causal attention of the
 * `rows` tokens (q: [rows][q_heads][head_dim], the same on every rank) over THIS rank's cache, partials pushed to
 * the peers and merged inside the reduce kernel, the finished rows in `out` on every rank.  positions_dev[rows] are
 * positions in this cache's own coordinates: on the rank that owns the open tile -- which has appended the rows
 * with kvb_append before this call -- the rows' own positions, on the other ranks their last position, repeated.
 * The ring buffers must hold rows * q_heads query rows (kvb_peer_ring.rows).  No counterpart in the reference
 * (single GPU); the single-GPU operator is causal_attention_small_t_launch (P3:3508-3545). */
int kvb_attn_rows_sharded(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int rows, float scale,
                          int kv_len_max, void* workspace, const kvb_peer_ring* ring, void* out, void* stream);

/* One decode step: append the token at *pos_dev (k, v: [kv_heads][head_dim]), then decode attention of q over the
 * cache including it -- kvb_append followed by kvb_attn_decode (ring == NULL) or kvb_attn_decode_sharded (ring given:
 * the rank that owns the open tile of a range-sharded sequence), same results bit for bit, one host call instead of
 * two (an attention kernel that started before the append had finished was measured slower).  The reference's decode
 * step makes the same pair of calls (kv_cache_append_launch, then causal_attention_cached_small_t_launch, P3:1379, 3612). */
int kvb_append_decode(const kvb_layer* layer, const void* q, const void* k, const void* v, const int32_t* pos_dev, float scale,
                      int kv_len_max, void* workspace, const kvb_peer_ring* ring, void* out, void* stream);

/* MTP verify: append `width` (1..8) new rows, then causal attention of those rows (row i sees keys
 * 0..positions[i]).  q, out: [width][q_heads][head_dim]; k, v: [width][kv_heads][head_dim].
 * Replaces causal_attention_small_t_launch (P3:3508-3610). */
int kvb_attn_verify(const kvb_layer* layer, const void* q, const void* k, const void* v, const int32_t* positions_dev,
                    int width, float scale, int kv_len_max, void* workspace, void* out, void* stream);

/* The attention half of a verify step alone: causal attention of `rows` (1..8) query tokens whose K/V rows are already
 * in the cache.  *total_pos_dev is the position of the newest token the cache holds (it decides which tile is the open
 * one), positions_dev[i] the position of query row i (it sees keys 0..positions[i]).  For the reference's column-block
 * form of causal_attention_small_t_launch (P3:3508-3545: the whole step is appended when column_begin == 0, the
 * blocks column_begin > 0 attend only).  Workspace as for kvb_attn_verify. */
int kvb_attn_rows(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int rows, const int32_t* total_pos_dev,
                  float scale, int kv_len_max, void* workspace, void* out, void* stream);

/* Prefill chunk: quantise-append `tokens` rows, then causal attention of the chunk over prefix + chunk.
 * q, out: [tokens][q_heads][head_dim].  Replaces causal_attention_prompt_launch (P3:2362-2416). */
int kvb_attn_prefill(const kvb_layer* layer, const void* q, const void* k, const void* v,
                     const int32_t* positions_dev, int tokens, float scale, int kv_len_max, void* workspace,
                     void* out, void* stream);
size_t kvb_prefill_workspace_bytes(int kv_len_max, int kv_heads, int q_heads, int head_dim, int tokens);

/* Verify steps and prefill chunks over a sequence whose tile ranges live on several GPUs: causal attention of `tokens`
 * query rows over THIS cache alone, stopped before the normalisation -- part_m[tokens * q_heads] (max logit, natural
 * log), part_l (sum of exp(logit - m)), part_o[tokens * q_heads][head_dim] (rotated domain), fp32, row = token * q_heads
 * + q head.  Nothing is appended: the rank that owns the open tile calls kvb_append for the new rows first.
 * positions_dev are in this cache's own coordinates (row i sees keys 0..positions[i]; the last entry also tells the
 * length of the cache): the owner of the new rows passes their local positions, a rank that holds an earlier range
 * passes its last position for every row.  The partials of all ranks merge with kvb_merge_partials(_packed), passing
 * tokens * q_heads as the row count.  Workspace: kvb_workspace_bytes(..., rows = tokens, 1) for tokens <= 8,
 * kvb_prefill_workspace_bytes(..., tokens) for longer chunks.  No counterpart in the reference (single GPU); the
 * single-GPU operators it extends are causal_attention_small_t_launch and causal_attention_prompt_launch
 * (P3:3508-3610, 2362-2416), the merge it feeds repeats their split reduction (P3:3149-3170, 3467-3482). */
int kvb_attn_chunk_partial(const kvb_layer* layer, const void* q, const int32_t* positions_dev, int tokens, float scale,
                           int kv_len_max, void* workspace, float* part_m, float* part_l, float* part_o, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KVARN_B200_H */
