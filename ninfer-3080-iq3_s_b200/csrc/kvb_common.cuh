// kvb_common.cuh -- geometry, rotation and small device helpers shared by every kernel of the library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../../include/kvarn_b200.h"

namespace kvb {

constexpr int kTile = 128;   // tokens per quantisation tile          (reference kvarn_layout.h:34)
constexpr int kPage = 64;    // tokens per page                       (kvarn_layout.h:35)
constexpr int kSlice = 128;  // dims per quantisation record          (kvarn_layout.h:38)

// Host-side error text of the calling thread.
void set_error(const char* fmt, ...);
int fail(kvb_status st, const char* fmt, ...);
#define KVB_CUDA_OK(expr)                                                                      \
    do {                                                                                       \
        cudaError_t e_ = (expr);                                                               \
        if (e_ != cudaSuccess) return ::kvb::fail(KVB_ECUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

// Plane geometry for S = D/128 slices (kvarn_layout.h:61-131 generalised).
template <int D> struct Geo {
    static constexpr int S = D / kSlice;
    static constexpr int kCodeLeading = D / 2;      // bytes per token row
    static constexpr int kKScaleLeading = 5 * S;    // halves per token row
    static constexpr int kVScaleLeading = 4 * S;
    static constexpr int kAxisCols = 2 * S;         // dim-axis entries per page row
    static constexpr int kCodePageBytes = kCodeLeading * kPage;
    static constexpr int kKScalePageBytes = kKScaleLeading * kPage * 2;
    static constexpr int kVScalePageBytes = kVScaleLeading * kPage * 2;
};

// Offset (in elements) of the first element of (page, head) in a plane of leading extent L.
__host__ __device__ __forceinline__ int64_t page_head_offset(int L, int heads, int page, int head) {
    return static_cast<int64_t>(L) * kPage * (static_cast<int64_t>(head) + static_cast<int64_t>(heads) * page);
}

// Device view of a layer (kvb_layer copied by value into kernel parameters).
struct LayerView {
    uint8_t* k_code;
    __half* k_scale;
    uint8_t* v_code;
    __half* v_scale;
    __half* stage;
    const int32_t* table_direct;
    const int32_t* tables;
    const int32_t* table_rows;
    int32_t table_stride, table_len, pages, kv_heads, q_heads, head_dim, dtype, iters;
    uint32_t* error_word;

    __device__ __forceinline__ const int32_t* table() const {
        return table_direct != nullptr ? table_direct
                                       : tables + static_cast<int64_t>(table_rows[0]) * table_stride;
    }
    __device__ __forceinline__ void flag(uint32_t bit) const {
        if (error_word != nullptr) atomicOr(error_word, bit);
    }
    // Physical page of a logical page, range-checked: a bad entry sets the error word and yields -1.
    __device__ __forceinline__ int32_t page_of(const int32_t* tbl, int logical) const {
        if (logical < 0 || logical >= table_len) { flag(KVB_ERR_TABLE_RANGE); return -1; }
        const int32_t p = tbl[logical];
        if (p < 0 || p >= pages) { flag(KVB_ERR_PAGE_RANGE); return -1; }
        return p;
    }
    __device__ __forceinline__ __half* stage_row(int which, int slot, int head, int tok) const {
        const int64_t plane = static_cast<int64_t>(2) * kv_heads * kTile * head_dim;
        return stage + which * plane + ((static_cast<int64_t>(slot) * kv_heads + head) * kTile + tok) * head_dim;
    }
};

// Launch with programmatic stream serialization: the kernel may become resident while its predecessor in the
// stream still runs and must call grid_dependency_wait() (kvb_ptx.cuh) before its first global memory access.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_early(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// True the first time it is called on the current device for this `seen` mask: for set-up CUDA keeps per device
// (the opt-in to large dynamic shared memory).  Not synchronised -- two threads making the first call at once
// both do the set-up, which is harmless.
inline bool first_call_on_device(unsigned long long& seen) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return true;
    const unsigned long long bit = 1ull << (dev & 63);
    if (seen & bit) return false;
    seen |= bit;
    return true;
}
// SM count of the current device (cached per device; 148 if the query fails).
inline int device_sm_count() {
    static int cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    int& n = cache[dev & 63];
    if (n <= 0 && (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)) n = 148;
    return n;
}

LayerView make_view(const kvb_layer& L);
int check_layer(const kvb_layer* L, const char* who);

// 16-bit input element -> fp32.
template <bool kBf16> __device__ __forceinline__ float in_to_f32(const uint16_t v) {
    if constexpr (kBf16) return __uint_as_float(static_cast<uint32_t>(v) << 16);
    else return __half2float(__ushort_as_half(v));
}
template <bool kBf16> __device__ __forceinline__ uint16_t f32_to_out(float v) {
    if constexpr (kBf16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}

// Normalised Sylvester-Hadamard of one head row held by one warp: lane l carries dims l + 32 r in
// v[r], r < D/32.  Five shuffle stages (strides 1..16), then register butterflies for strides
// 32, 64 (,128), then one scale: exactly 2^-4 for D = 256, the 128-point constant for D = 128.
// Same butterfly order and roundings as the reference rotation
// (kvarn-evidence/wht-gate/ninfer_hadamard_d256_verbatim.h:16-71).  Self-inverse.
template <int D> __device__ __forceinline__ void hadamard_warp(float (&v)[D / 32], int lane) {
    constexpr int R = D / 32;
#pragma unroll
    for (int stride = 1; stride <= 16; stride <<= 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float peer = __shfl_xor_sync(0xffffffffu, v[r], stride);
            v[r] = (lane & stride) == 0 ? __fadd_rn(v[r], peer) : __fsub_rn(peer, v[r]);
        }
    }
#pragma unroll
    for (int span = 1; span < R; span <<= 1) {
#pragma unroll
        for (int base = 0; base < R; base += 2 * span) {
#pragma unroll
            for (int o = 0; o < span; ++o) {
                const float lo = v[base + o], hi = v[base + o + span];
                v[base + o] = __fadd_rn(lo, hi);
                v[base + o + span] = __fsub_rn(lo, hi);
            }
        }
    }
    constexpr float norm = D == 256 ? 0.0625f : 0.08838834764831845f;
#pragma unroll
    for (int r = 0; r < R; ++r) v[r] = __fmul_rn(v[r], norm);
}

}  // namespace kvb
