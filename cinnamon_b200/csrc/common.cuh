// Shared helpers for the cinnamon_b200 CUDA library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>

// ---- status codes returned by every extern "C" entry point -----------------
#define CINN_OK 0
#define CINN_ERR_INVALID 1      // bad argument (null pointer, shape, alignment, dtype)
#define CINN_ERR_CUDA 2         // a CUDA runtime/driver call failed
#define CINN_ERR_UNSUPPORTED 3  // valid request that this build cannot serve
#define CINN_ERR_DEVICE 4       // a kernel reported a device-side problem (bounded wait ran out)

// dtype tags of the C-ABI
#define CINN_BF16 0
#define CINN_F32 1
#define CINN_F16 2
#define CINN_F32_BF16 3   // GEMM output only: fp32 storage of the value rounded to bf16

// division flavour of the quantisers
#define CINN_DIV_FULL 0   // PTX div.full.f32: what Triton emits for the reference kernels on a GPU
#define CINN_DIV_RN 1     // IEEE round-to-nearest: what a CPU restatement computes

namespace cinn {

void set_error(const char* fmt, ...);

#define CINN_CHECK_ARG(cond, ...)                      \
    do {                                               \
        if (!(cond)) {                                 \
            cinn::set_error(__VA_ARGS__);              \
            return CINN_ERR_INVALID;                   \
        }                                              \
    } while (0)

#define CINN_CHECK_CUDA(expr)                                                          \
    do {                                                                               \
        cudaError_t _e = (expr);                                                       \
        if (_e != cudaSuccess) {                                                       \
            cinn::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),    \
                            __FILE__, __LINE__);                                       \
            return CINN_ERR_CUDA;                                                      \
        }                                                                              \
    } while (0)

#define CINN_CHECK_LAUNCH()  CINN_CHECK_CUDA(cudaGetLastError())

int sm_count();   // SMs of the current device (cached per device)

// ---- arithmetic shared by every quantiser ---------------------------------
constexpr float kFp8Max = 448.0f;
constexpr float kAmaxFloor = 1e-4f;   // 0x38D1B717

template <int DIV>
__device__ __forceinline__ float div_f32(float a, float b) {
    if constexpr (DIV == CINN_DIV_FULL) {
        float r;
        asm("div.full.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
        return r;
    } else {
        return __fdiv_rn(a, b);
    }
}

// amax (>= 0, NaN already dropped) -> scale.
// round_scale: 2^ceil(log2(amax/448)) with log2 evaluated by CUDA's fp32 log2f,
// rounded up by cvt.rpi and exponentiated by ex2.approx (exact for integers).
template <int DIV, bool ROUND>
__device__ __forceinline__ float scale_from_amax(float amax) {
    amax = fmaxf(amax, kAmaxFloor);
    float s = div_f32<DIV>(amax, kFp8Max);
    if constexpr (ROUND) {
        float lg = log2f(s);
        float e, r;
        asm("cvt.rpi.ftz.f32.f32 %0, %1;" : "=f"(e) : "f"(lg));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e));
        s = r;
    }
    return s;
}

// Many elements are divided by one scale.  In the div.full.f32 flavour the quotient x / s is formed as
// x * rcp.approx(s) with the reciprocal taken once per scale: for every divisor in [2^-126, 2^126] (all scales these
// kernels produce: the amax has a floor of 1e-4 and is finite) that product has the very bits of
// div.full.f32(x, s), which cinn_selfcheck_division confirms on the GPU at hand for every 16-bit x and every
// scale a 16-bit amax can give.  The IEEE flavour divides element by element.
template <int DIV>
__device__ __forceinline__ float divisor_of(float s) {
    if constexpr (DIV == CINN_DIV_FULL) {
        float r;
        asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(s));
        return r;
    } else {
        return s;
    }
}

// x / s (d = divisor_of(s)), clamped from below.
template <int DIV>
__device__ __forceinline__ float scaled_clamped(float x, float d) {
    float y;
    if constexpr (DIV == CINN_DIV_FULL) y = __fmul_rn(x, d);
    else y = __fdiv_rn(x, d);
    // The reference clamps with max(y, -448) then min(., 448), both dropping a NaN operand.
    // Only the max is kept: it turns NaN into -448 as the reference does; the upper (and lower)
    // clamp is what the saturating e4m3 conversion that always follows does anyway.
    return fmaxf(y, -kFp8Max);
}

// two fp32 -> two e4m3 bytes (lo in bits 0-7, hi in bits 8-15), RNE, finite saturation
__device__ __forceinline__ uint16_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
    return (uint32_t)cvt_e4m3x2(a, b) | ((uint32_t)cvt_e4m3x2(c, d) << 16);
}

// e4m3 byte -> fp32 (exact): via the hardware e4m3x2 -> f16x2 conversion
__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t v) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(v));
    __half2 h = *reinterpret_cast<__half2*>(&h2);
    return __half22float2(h);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

}  // namespace cinn
