// Shared host-side plumbing of the cellerator_b200 library: status + thread-local error text,
// a process-wide kernel-launch counter, and small device helpers used by several kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/cellerator_b200.h"

namespace cb200 {

// Thread-local message of the last failing call (the convention of the reference's public
// C ABI, src/abi/abi.cu:40-74).
char *last_error_buffer();
cb200_status fail(cb200_status status, const char *fmt, ...);
void clear_error();

// Every kernel launch of this library goes through count_launch() so that callers can
// report how many of its kernels ran inside a timed region.
extern std::atomic<std::uint64_t> g_kernel_launches;
inline void count_launch(std::uint64_t n = 1) { g_kernel_launches.fetch_add(n, std::memory_order_relaxed); }

#define CB200_CUDA_OK(expr)                                                                       \
    do {                                                                                          \
        const cudaError_t cb200_err_ = (expr);                                                    \
        if (cb200_err_ != cudaSuccess)                                                            \
            return ::cb200::fail(CB200_STATUS_CUDA_ERROR, "%s: %s", #expr, cudaGetErrorString(cb200_err_)); \
    } while (0)

// Sets the device for the scope and restores the previous one (launchers may be called with
// another device current).
struct device_scope {
    int previous = -1;
    cudaError_t status = cudaSuccess;
    explicit device_scope(int device) {
        status = cudaGetDevice(&previous);
        if (status == cudaSuccess && previous != device) status = cudaSetDevice(device);
    }
    ~device_scope() {
        int now = -1;
        if (cudaGetDevice(&now) == cudaSuccess && previous >= 0 && now != previous) cudaSetDevice(previous);
    }
};

#if defined(__CUDACC__)
// bf16 pair (low half = element 0) -> two floats, exact.
__device__ __forceinline__ void bf16x2_to_f32(std::uint32_t packed, float &lo, float &hi) {
    lo = __uint_as_float(packed << 16);
    hi = __uint_as_float(packed & 0xffff0000u);
}

// Eight consecutive elements of a dense row as floats (16-byte aligned address).
__device__ __forceinline__ void load8(const float *p, float (&w)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p));
    const float4 b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
    w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16 *p, float (&w)[8]) {
    const uint4 a = __ldg(reinterpret_cast<const uint4 *>(p));
    bf16x2_to_f32(a.x, w[0], w[1]);
    bf16x2_to_f32(a.y, w[2], w[3]);
    bf16x2_to_f32(a.z, w[4], w[5]);
    bf16x2_to_f32(a.w, w[6], w[7]);
}
// Composed epilogue of the forward projections: act(value + bias), the rule of the reference's
// referee (src/compute/math/referee.cc:81-97).  `value` already holds alpha * product + beta * out.
__device__ __forceinline__ bool epilogue_has_bias(int kind) {
    return kind == CB200_EPILOGUE_BIAS || kind >= CB200_EPILOGUE_BIAS_RELU;
}
// Not inlined: the output stages are unrolled dozens of times, and a copy of erff / tanhf in each
// of them costs the kernels that ask for no epilogue their instruction cache (the Blocked-ELL
// tensor kernel ran 19 % slower with it inlined).
static __device__ __noinline__ float apply_epilogue(float value, float bias, int kind) {
    if (epilogue_has_bias(kind)) value += bias;
    if (kind == CB200_EPILOGUE_RELU || kind == CB200_EPILOGUE_BIAS_RELU) return fmaxf(value, 0.0f);
    if (kind == CB200_EPILOGUE_GELU_ERF || kind == CB200_EPILOGUE_BIAS_GELU_ERF)
        return 0.5f * value * (1.0f + erff(value * 0.70710678118654752f));
    if (kind == CB200_EPILOGUE_GELU_TANH || kind == CB200_EPILOGUE_BIAS_GELU_TANH)
        return 0.5f * value * (1.0f + tanhf(0.79788456080286536f * (value + 0.044715f * value * value * value)));
    return value;
}
// The epilogue of one output element at column `col`; `bias` may be null for kinds without bias.
__device__ __forceinline__ float finish_output(float value, const float *bias, int col, int kind) {
    if (kind == CB200_EPILOGUE_NONE) return value;
    return apply_epilogue(value, epilogue_has_bias(kind) ? __ldg(bias + col) : 0.0f, kind);
}

// One thread's 32 consecutive output columns of a row, starting at column col0 (16-byte aligned):
//     out = act(alpha * v + beta * out + bias).
// The phases are kept apart -- every load, then the arithmetic, then the optional epilogue calls,
// then every store -- so that the eight loads of a beta != 0 launch are in flight together; with a
// call between each load and store they would follow one another.
__device__ __forceinline__ void store_row32(float *out, float (&v)[32], float alpha, float beta, const float *bias, int col0,
                                            int kind) {
#pragma unroll
    for (int c = 0; c < 32; ++c) v[c] *= alpha;
    if (beta != 0.0f) {
        float4 o[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) o[c] = *reinterpret_cast<const float4 *>(out + 4 * c);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            v[4 * c + 0] = fmaf(beta, o[c].x, v[4 * c + 0]); v[4 * c + 1] = fmaf(beta, o[c].y, v[4 * c + 1]);
            v[4 * c + 2] = fmaf(beta, o[c].z, v[4 * c + 2]); v[4 * c + 3] = fmaf(beta, o[c].w, v[4 * c + 3]);
        }
    }
    if (kind != CB200_EPILOGUE_NONE) {
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] = finish_output(v[c], bias, col0 + c, kind);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c)
        *reinterpret_cast<float4 *>(out + 4 * c) = make_float4(v[4 * c + 0], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}

__device__ __forceinline__ float load1(const float *p) { return __ldg(p); }
__device__ __forceinline__ float load1(const __nv_bfloat16 *p) {
    return __uint_as_float(static_cast<std::uint32_t>(__ldg(reinterpret_cast<const unsigned short *>(p))) << 16);
}
#endif

} // namespace cb200
