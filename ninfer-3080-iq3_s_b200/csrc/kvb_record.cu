// kvb_record.cu -- the compact tile record at every code width: a 128 x 128 fp32 matrix quantised row by row to
// `bits`-bit codes (2, 3, 4, 5, 6 or 8), stored as
//     payload (LSB-first bit string, row-major, 16 * bits bytes per row) || scale_axis[128] || zp_axis[128] || other_axis[128]
// with the three axes in fp16 (reference kvarn-evidence/oracle/bee_oracle.cpp:152-172 for the bit string, :309-374 for
// the quantiser and its inverse; the engine's kernel is templated on the same widths, kvarn128_launch.cu:126,158,248).
// This is the 70 * bits / 4 + 6 bytes-per-row record the reference's compact geometry stores once per tile (K4V4: 140 B per
// token and KV head); the attention kernels of this library read the 4-bit P1 planes, which hold the same codes and
// axes.  Regime: no variance balancing (all balancing factors 1), where codes and axes are bit-exact against the host
// oracle: x - lo, the division by the scale and roundf are done with round-to-nearest intrinsics, nothing is contracted.
// One CTA per tile, thread = row: min / max, scale, codes packed by the thread that owns the row (a row is a whole
// number of bytes at every width).  A codec for export / import and for the byte-level gates, not a hot path.
#include "kvb_common.cuh"

namespace kvb {
namespace {

constexpr int kRecDim = 128;

__host__ __device__ constexpr size_t record_payload(int bits) { return static_cast<size_t>(kRecDim) * kRecDim * bits / 8; }
__host__ __device__ constexpr size_t record_bytes(int bits) { return record_payload(bits) + 3 * kRecDim * sizeof(__half); }

__global__ void __launch_bounds__(kRecDim) record_encode_kernel(const float* __restrict__ tiles, int bits, uint8_t* __restrict__ records) {
    const int r = threadIdx.x;
    const float* row = tiles + (static_cast<size_t>(blockIdx.x) * kRecDim + r) * kRecDim;  // the row is read twice; the second pass hits L1
    uint8_t* rec = records + static_cast<size_t>(blockIdx.x) * record_bytes(bits);
    __half* axes = reinterpret_cast<__half*>(rec + record_payload(bits));
    const int qmax = (1 << bits) - 1;
    float lo = row[0], hi = row[0];
    for (int c4 = 0; c4 < kRecDim / 4; ++c4) {
        const float4 x = reinterpret_cast<const float4*>(row)[c4];
        lo = fminf(fminf(lo, fminf(x.x, x.y)), fminf(x.z, x.w));
        hi = fmaxf(fmaxf(hi, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
    }
    const float scale = fmaxf(__fdiv_rn(__fsub_rn(hi, lo), static_cast<float>(qmax)), 1e-10f);
    uint8_t* out = rec + static_cast<size_t>(r) * (kRecDim * bits / 8);
    unsigned long long buf = 0;  // bit string of the row, flushed a byte at a time
    int have = 0;
    for (int c4 = 0; c4 < kRecDim / 4; ++c4) {
        const float4 x4 = reinterpret_cast<const float4*>(row)[c4];
        const float x[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float q = fminf(fmaxf(roundf(__fdiv_rn(__fsub_rn(x[e], lo), scale)), 0.0f), static_cast<float>(qmax));
            buf |= static_cast<unsigned long long>(static_cast<unsigned>(q)) << have;
            have += bits;
            while (have >= 8) {
                *out++ = static_cast<uint8_t>(buf & 0xFFu);
                buf >>= 8;
                have -= 8;
            }
        }
    }
    axes[r] = __float2half_rn(scale);
    axes[kRecDim + r] = __float2half_rn(lo);
    axes[2 * kRecDim + r] = __float2half_rn(1.0f);
}

// x[r][c] = (q * scale_axis[r] + zp_axis[r]) * other_axis[c], every step rounded to fp32 (bee_oracle.cpp:359-374).
__global__ void __launch_bounds__(kRecDim) record_decode_kernel(const uint8_t* __restrict__ records, int bits, float* __restrict__ tiles) {
    __shared__ float other[kRecDim];
    const int r = threadIdx.x;
    const uint8_t* rec = records + static_cast<size_t>(blockIdx.x) * record_bytes(bits);
    const __half* axes = reinterpret_cast<const __half*>(rec + record_payload(bits));
    other[r] = __half2float(axes[2 * kRecDim + r]);
    const float sa = __half2float(axes[r]), zp = __half2float(axes[kRecDim + r]);
    __syncthreads();
    const uint8_t* in = rec + static_cast<size_t>(r) * (kRecDim * bits / 8);
    unsigned long long buf = 0;
    int have = 0;
    const unsigned mask = (1u << bits) - 1u;
    float* dst = tiles + (static_cast<size_t>(blockIdx.x) * kRecDim + r) * kRecDim;
    for (int c4 = 0; c4 < kRecDim / 4; ++c4) {
        float x[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            while (have < bits) {
                buf |= static_cast<unsigned long long>(*in++) << have;
                have += 8;
            }
            const unsigned q = static_cast<unsigned>(buf) & mask;
            buf >>= bits;
            have -= bits;
            x[e] = __fmul_rn(__fadd_rn(__fmul_rn(static_cast<float>(q), sa), zp), other[4 * c4 + e]);
        }
        reinterpret_cast<float4*>(dst)[c4] = make_float4(x[0], x[1], x[2], x[3]);
    }
}

bool width_ok(int bits) { return bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8; }

}  // namespace
}  // namespace kvb

extern "C" size_t kvb_record_bytes(int bits) { return kvb::width_ok(bits) ? kvb::record_bytes(bits) : 0; }

extern "C" int kvb_records_encode(const float* tiles, int n_tiles, int bits, void* records, void* stream) {
    using namespace kvb;
    if (!width_ok(bits)) return fail(KVB_EINVAL, "kvb_records_encode: %d-bit codes (2, 3, 4, 5, 6 or 8)", bits);
    if (n_tiles < 0 || (n_tiles > 0 && (tiles == nullptr || records == nullptr))) return fail(KVB_EINVAL, "kvb_records_encode: null tiles / records");
    if (n_tiles == 0) return KVB_OK;
    record_encode_kernel<<<n_tiles, kRecDim, 0, static_cast<cudaStream_t>(stream)>>>(tiles, bits, static_cast<uint8_t*>(records));
    KVB_CUDA_OK(cudaGetLastError());
    return KVB_OK;
}

extern "C" int kvb_records_decode(const void* records, int n_tiles, int bits, float* tiles, void* stream) {
    using namespace kvb;
    if (!width_ok(bits)) return fail(KVB_EINVAL, "kvb_records_decode: %d-bit codes (2, 3, 4, 5, 6 or 8)", bits);
    if (n_tiles < 0 || (n_tiles > 0 && (tiles == nullptr || records == nullptr))) return fail(KVB_EINVAL, "kvb_records_decode: null tiles / records");
    if (n_tiles == 0) return KVB_OK;
    record_decode_kernel<<<n_tiles, kRecDim, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(records), bits, tiles);
    KVB_CUDA_OK(cudaGetLastError());
    return KVB_OK;
}
