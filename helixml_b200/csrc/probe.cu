// Pipe-throughput probes: how many fp32 fused multiply-adds and how many special-function results
// (ex2.approx) this GPU retires per second.  The selective scan is bound by these two pipes, not by
// HBM, once its traffic is down to one pass; the benchmark measures both on the device it runs on and
// reports the scan against max(bytes / bandwidth, special-function results / rate, fp32 operations / rate).
//
// Each probe is a register-only loop of independent dependency chains (8 per thread, 2048 threads
// per SM), long enough that launch and drain are below 1 % of the run.
#include "hx_common.cuh"
#include "hx_tma.cuh"

namespace hx {
namespace probe {

constexpr int kChains = 8, kThreads = 256, kBlocksPerSm = 8, kIters = 4096;

__global__ void __launch_bounds__(kThreads) fma_kernel(float *out, int iters, float a, float b) {
    float v[kChains];
#pragma unroll
    for (int i = 0; i < kChains; ++i) v[i] = threadIdx.x * 0.001f + i;
    for (int it = 0; it < iters; ++it)
#pragma unroll
        for (int i = 0; i < kChains; ++i) v[i] = fmaf(v[i], a, b);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kChains; ++i) s += v[i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

__global__ void __launch_bounds__(kThreads) fma2_kernel(float *out, int iters, float a, float b) {
    float2 v[kChains];
#pragma unroll
    for (int i = 0; i < kChains; ++i) v[i] = make_float2(threadIdx.x * 0.001f + i, (float)i);
    const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
    for (int it = 0; it < iters; ++it)
#pragma unroll
        for (int i = 0; i < kChains; ++i) v[i] = fma2(v[i], a2, b2);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kChains; ++i) s += v[i].x + v[i].y;
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

__global__ void __launch_bounds__(kThreads) ex2_kernel(float *out, int iters) {
    float v[kChains];
#pragma unroll
    for (int i = 0; i < kChains; ++i) v[i] = -(float)threadIdx.x * 0.001f - i;
    for (int it = 0; it < iters; ++it)
#pragma unroll
        for (int i = 0; i < kChains; ++i) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(v[i]));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kChains; ++i) s += v[i];
    out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace probe
}  // namespace hx

extern "C" hx_status hx_probe_pipe(int32_t kind, void *scratch, size_t scratch_bytes, double *per_second, void *stream) {
    using namespace hx::probe;
    HX_REQUIRE(per_second, HX_ERR_INVALID_INPUT, "hx_probe_pipe: NULL result pointer");
    HX_REQUIRE(kind >= HX_PROBE_FMA && kind <= HX_PROBE_EX2, HX_ERR_INVALID_INPUT, "hx_probe_pipe: unknown kind %d", kind);
    const int blocks = hx::sm_count() * kBlocksPerSm;
    const size_t need = (size_t)blocks * kThreads * sizeof(float);
    HX_REQUIRE(scratch && scratch_bytes >= need, HX_ERR_INVALID_INPUT, "hx_probe_pipe needs %zu bytes of device scratch (got %zu)",
               need, scratch_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *out = static_cast<float *>(scratch);
    auto launch = [&]() {
        if (kind == HX_PROBE_FMA) fma_kernel<<<blocks, kThreads, 0, st>>>(out, kIters, 1.0001f, 0.5f);
        else if (kind == HX_PROBE_FMA2) fma2_kernel<<<blocks, kThreads, 0, st>>>(out, kIters, 1.0001f, 0.5f);
        else ex2_kernel<<<blocks, kThreads, 0, st>>>(out, kIters);
    };
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    HX_CUDA(cudaEventCreate(&e0));
    HX_CUDA(cudaEventCreate(&e1));
    float best = 1e30f;
    hx_status rc = HX_OK;
    launch();  // warm-up
    for (int r = 0; r < 5 && rc == HX_OK; ++r) {
        cudaEventRecord(e0, st);
        launch();
        cudaEventRecord(e1, st);
        if (cudaEventSynchronize(e1) != cudaSuccess) { rc = hx::fail(HX_ERR_BACKEND, "hx_probe_pipe: the probe kernel failed"); break; }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (ms < best) best = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != HX_OK) return rc;
    if (hx::check_launch("probe kernel") != HX_OK) return HX_ERR_BACKEND;
    const double per_thread = (double)kIters * kChains * (kind == HX_PROBE_FMA2 ? 2.0 : 1.0);
    *per_second = per_thread * blocks * kThreads / (best * 1e-3);
    return HX_OK;
}
