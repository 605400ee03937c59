// Warp-level row quantisation used by the dispatch kernels.
//   fp8 1x128 : inv = 448 / max(amax_blk, 1e-4);  q = e4m3_rn_sat(x * inv);  scale = max(amax_blk, 1e-4) / 448
//   fp8 1x128 with power-of-two scales: scale = 2^ceil(log2(max(amax_blk, 1e-4) / 448)), inv = 1 / scale
//   int8 token: inv = 127 / (amax_row + 1e-12);   q = rint(x * inv);         scale = 1 / inv
// The int8 form follows the per-token dynamic quantisation of the reference's dispatch kernels
// (moe_dispatch_normal.h:289-315); the fp8 form is the DeepSeek-style block scaling.
#pragma once
#include "ptx.cuh"

namespace cam {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    // cvt packs (hi, lo) -> the first source lands in the upper byte.
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}

// Power-of-two ("UE8M0") block scale: the smallest 2^k >= amax / 448, and its exact reciprocal.
// The tensor core's block-scaled MMA takes only the exponent byte of a scale, so scales meant for
// it must be exact powers of two.  amax is clamped to 1e-4 first, like the fp32-scale form.
__device__ __forceinline__ void ue8m0_scale(float amax, float& scale, float& inv) {
    const uint32_t b = __float_as_uint(__fdiv_rn(fmaxf(amax, 1e-4f), 448.f));
    const uint32_t e = (b >> 23) + ((b & 0x7FFFFFu) ? 1u : 0u);
    scale = __uint_as_float(e << 23);
    inv = __uint_as_float((254u - e) << 23);
}

// One warp quantises one bf16 row of `h` elements (h % 256 == 0 handled fast, h % 128 == 0 in
// general) to e4m3 with 1x128 scales (arbitrary fp32 scales, or powers of two when UE8M0).
// Output goes to the warp's staging area in shared memory: `q` (h bytes, 16-byte aligned) and
// `s` (h/128 floats).
// Quantises the 8 bf16 values a lane holds (`v`) as part of a 128-element block spread over 16
// consecutive lanes; all 32 lanes must call it together.  Returns the packed e4m3 bytes and the
// block's scale.
template <bool UE8M0>
__device__ __forceinline__ uint2 quant8_in_block16(const uint4& v, float& scale) {
    float f[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                  bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    float inv;
    if (UE8M0) {
        ue8m0_scale(amax, scale, inv);
    } else {
        const float a = fmaxf(amax, 1e-4f);
        inv = 448.f / a;
        scale = a / 448.f;
    }
    uint2 o2;
    o2.x = pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
    o2.y = pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
    return o2;
}

template <bool UE8M0 = false>
__device__ __forceinline__ void warp_quant_fp8_1x128(const __nv_bfloat16* __restrict__ row, int h,
                                                     uint8_t* q, float* s) {
    const uint32_t lane = lane_id();
    // Each lane owns 8 consecutive elements per step of 256; 16 lanes cover one 128-element block.
    // The loads of four steps are issued together (the steps are independent), which divides the
    // number of exposed memory latencies per row by four.
    for (int base = 0; base < h; base += 1024) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = base + u * 256 + static_cast<int>(lane) * 8;
            v[u] = (c < h) ? ld_nc_v4(row + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = base + u * 256 + static_cast<int>(lane) * 8;
            float sc;
            const uint2 o2 = quant8_in_block16<UE8M0>(v[u], sc);
            if (c < h) {
                *reinterpret_cast<uint2*>(q + c) = o2;
                if ((lane & 15u) == 0u) s[c >> 7] = sc;
            }
        }
    }
}

// The whole CTA quantises one bf16 row (every thread must call it; no barrier inside): thread i
// owns elements [8 i, 8 i + 8) of every pass of 8 * blockDim.x elements, so a 7168-element row
// costs a 512-thread CTA two loads per thread, issued together.
template <bool UE8M0>
__device__ __forceinline__ void block_quant_fp8_1x128(const __nv_bfloat16* __restrict__ row, int h,
                                                      uint8_t* q, float* s) {
    const int stride = static_cast<int>(blockDim.x) * 8;
    const int c0 = static_cast<int>(threadIdx.x) * 8;
    for (int base = 0; base < h; base += 2 * stride) {
        const int ca = base + c0, cb = base + stride + c0;
        const uint4 va = (ca < h) ? ld_nc_v4(row + ca) : make_uint4(0, 0, 0, 0);
        const uint4 vb = (cb < h) ? ld_nc_v4(row + cb) : make_uint4(0, 0, 0, 0);
        float sa, sb;
        const uint2 oa = quant8_in_block16<UE8M0>(va, sa);
        const uint2 ob = quant8_in_block16<UE8M0>(vb, sb);
        if (ca < h) {
            *reinterpret_cast<uint2*>(q + ca) = oa;
            if ((threadIdx.x & 15u) == 0u) s[ca >> 7] = sa;
        }
        if (cb < h) {
            *reinterpret_cast<uint2*>(q + cb) = ob;
            if ((threadIdx.x & 15u) == 0u) s[cb >> 7] = sb;
        }
    }
}

// One warp quantises one bf16 row to int8 with a single dynamic scale.  `q` holds h bytes,
// s[0] receives the dequantisation scale.
// `smooth` (optional, h floats) multiplies the row element-wise first (moe_dispatch_shmem.h:693-733).
__device__ __forceinline__ void warp_quant_int8_token(const __nv_bfloat16* __restrict__ row, int h,
                                                      uint8_t* q, float* s,
                                                      const float* __restrict__ smooth = nullptr) {
    const uint32_t lane = lane_id();
    float amax = 0.f;
    for (int col = static_cast<int>(lane) * 8; col < h; col += 256) {
        uint4 v = ld_nc_v4(row + col);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float m0 = smooth ? smooth[col + 2 * i] : 1.f, m1 = smooth ? smooth[col + 2 * i + 1] : 1.f;
            amax = fmaxf(amax, fabsf(bf16_lo(w[i]) * m0));
            amax = fmaxf(amax, fabsf(bf16_hi(w[i]) * m1));
        }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float inv = 127.f / (amax + 1e-12f);
    for (int col = static_cast<int>(lane) * 8; col < h; col += 256) {
        uint4 v = ld_nc_v4(row + col);  // second read hits L1/L2
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t out[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float m0 = smooth ? smooth[col + 2 * i] : 1.f, m1 = smooth ? smooth[col + 2 * i + 1] : 1.f;
            int a = __float2int_rn(bf16_lo(w[i]) * m0 * inv);
            int b = __float2int_rn(bf16_hi(w[i]) * m1 * inv);
            a = max(-127, min(127, a));
            b = max(-127, min(127, b));
            const uint32_t two = (static_cast<uint32_t>(a) & 0xFFu) | ((static_cast<uint32_t>(b) & 0xFFu) << 8);
            out[i >> 1] |= two << ((i & 1) * 16);
        }
        *reinterpret_cast<uint2*>(q + col) = make_uint2(out[0], out[1]);
    }
    if (lane == 0) s[0] = 1.f / inv;
}

}  // namespace cam
