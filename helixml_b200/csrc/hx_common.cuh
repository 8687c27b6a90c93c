// Shared helpers of the helix_b200 CUDA library: error reporting, dtype access, fast math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/helix_b200.h"

namespace hx {

// Records a printf-style message for the calling thread and returns `st`.
hx_status fail(hx_status st, const char *fmt, ...);

inline hx_status cuda_fail(cudaError_t e, const char *what) {
    return fail(HX_ERR_BACKEND, "%s: %s", what, cudaGetErrorString(e));
}

#define HX_CUDA(call)                                              \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) return hx::cuda_fail(e__, #call);  \
    } while (0)

#define HX_REQUIRE(cond, st, ...)                       \
    do {                                                \
        if (!(cond)) return hx::fail(st, __VA_ARGS__);  \
    } while (0)

// Checks the launch that was just made.
inline hx_status check_launch(const char *kernel) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(HX_ERR_BACKEND, "launch of %s failed: %s", kernel, cudaGetErrorString(e));
    return HX_OK;
}

inline size_t dtype_size(int dt) { return dt == HX_F32 ? 4 : dt == HX_BF16 ? 2 : 1; }

// Number of SMs of the current device, cached per device.
int sm_count();

// resid[i] += x[i] (x fp32 or bf16): the residual update where no GEMM epilogue can do it.
hx_status residual_add(float *resid, const void *x, int x_dtype, int64_t n, cudaStream_t st);

// The kernel HX_SCAN_AUTO picks for a d_state == 16 problem on the current device (selective_scan.cu); the Mamba
// block plans its launches and its workspace with the same rule.
namespace scan {
enum class ScanKind { Tiled, Direct, LookBack };
ScanKind auto_kind(const hx_scan_args *a);
int auto_channels_per_lane(const hx_scan_args *a);  // 1 or 2: what the one-lane-per-channel kernel would run with
}  // namespace scan

// Translation units with bounded device-side waits keep a status word each; these read (and
// optionally clear) them.  hx_device_status() ORs them together.
hx_status read_status_scan(int *v, bool clear);
hx_status read_status_gemm(int *v, bool clear);
hx_status read_status_convx(int *v, bool clear);

// ---------------------------------------------------------------- device-side helpers
template <typename T> __device__ __forceinline__ float ld_f32(const T *p);
template <> __device__ __forceinline__ float ld_f32<float>(const float *p) { return *p; }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat162float(*p); }

template <typename T> __device__ __forceinline__ void st_f32(T *p, float v);
template <> __device__ __forceinline__ void st_f32<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f32<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// x / (1 + exp(-x)) with one ex2 and one rcp on the special-function unit.
__device__ __forceinline__ float silu_fast(float x) {
    return x * rcp_approx(1.0f + ex2_approx(-kLog2e * x));
}
// The same through tanh: x sigmoid(x) = h + h tanh(h), h = x / 2.  One special-function result instead of two;
// tanh.approx is good to about 2^-11 relative, which is below the rounding of a bf16 result.
__device__ __forceinline__ float silu_tanh(float x) {
    const float h = 0.5f * x;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return fmaf(h, t, h);
}
// Accurate forms used by the parity-baseline kernels.
__device__ __forceinline__ float silu_acc(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplus_acc(float v) { return v > 20.0f ? v : logf(1.0f + expf(v)); }

}  // namespace hx
