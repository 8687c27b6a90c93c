// Library-level entry points: version, error strings, device memory and copies.
#include <cstring>
#include <mutex>

#include "hx_common.cuh"

namespace hx {

static thread_local char g_err[512] = "";

hx_status fail(hx_status st, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return st;
}

int sm_count() {
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace hx

extern "C" {

const char *hx_version(void) { return "helix_b200 0.1 (sm_100a)"; }

const char *hx_last_error(void) { return hx::g_err; }

const char *hx_status_name(hx_status s) {
    switch (s) {
        case HX_OK: return "Ok";
        case HX_ERR_SHAPE_MISMATCH: return "ShapeMismatch";
        case HX_ERR_INVALID_DIMENSION: return "InvalidDimension";
        case HX_ERR_DEVICE_MISMATCH: return "DeviceMismatch";
        case HX_ERR_DTYPE_MISMATCH: return "DTypeMismatch";
        case HX_ERR_UNSUPPORTED_OPERATION: return "UnsupportedOperation";
        case HX_ERR_ALLOCATION_FAILED: return "AllocationFailed";
        case HX_ERR_BACKEND: return "BackendError";
        case HX_ERR_SERIALIZATION: return "SerializationError";
        case HX_ERR_INVALID_CHECKPOINT: return "InvalidCheckpoint";
        case HX_ERR_INVALID_INPUT: return "InvalidInput";
    }
    return "Unknown";
}

hx_status hx_device_count(int *count) {
    HX_REQUIRE(count != nullptr, HX_ERR_INVALID_INPUT, "hx_device_count: count is NULL");
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) {
        *count = 0;
        return hx::cuda_fail(e, "cudaGetDeviceCount");
    }
    return HX_OK;
}

hx_status hx_set_device(int device) {
    HX_CUDA(cudaSetDevice(device));
    return HX_OK;
}

hx_status hx_alloc(void **dptr, size_t bytes) {
    HX_REQUIRE(dptr != nullptr, HX_ERR_INVALID_INPUT, "hx_alloc: dptr is NULL");
    *dptr = nullptr;
    if (bytes == 0) return HX_OK;
    cudaError_t e = cudaMalloc(dptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return hx::fail(HX_ERR_ALLOCATION_FAILED, "cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
    }
    return HX_OK;
}

hx_status hx_free(void *dptr) {
    if (dptr) HX_CUDA(cudaFree(dptr));
    return HX_OK;
}

hx_status hx_host_alloc(void **hptr, size_t bytes) {
    HX_REQUIRE(hptr != nullptr, HX_ERR_INVALID_INPUT, "hx_host_alloc: hptr is NULL");
    *hptr = nullptr;
    if (bytes == 0) return HX_OK;
    cudaError_t e = cudaMallocHost(hptr, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return hx::fail(HX_ERR_ALLOCATION_FAILED, "cudaMallocHost(%zu bytes): %s", bytes, cudaGetErrorString(e));
    }
    return HX_OK;
}

hx_status hx_host_free(void *hptr) {
    if (hptr) HX_CUDA(cudaFreeHost(hptr));
    return HX_OK;
}

hx_status hx_memcpy_h2d(void *dst, const void *src_host, size_t bytes, void *stream) {
    if (bytes == 0) return HX_OK;
    HX_REQUIRE(dst && src_host, HX_ERR_INVALID_INPUT, "hx_memcpy_h2d: NULL pointer");
    HX_CUDA(cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return HX_OK;
}

hx_status hx_memcpy_d2h(void *dst_host, const void *src, size_t bytes, void *stream) {
    if (bytes == 0) return HX_OK;
    HX_REQUIRE(dst_host && src, HX_ERR_INVALID_INPUT, "hx_memcpy_d2h: NULL pointer");
    HX_CUDA(cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return HX_OK;
}

hx_status hx_memset(void *dptr, int value, size_t bytes, void *stream) {
    if (bytes == 0) return HX_OK;
    HX_REQUIRE(dptr != nullptr, HX_ERR_INVALID_INPUT, "hx_memset: NULL pointer");
    HX_CUDA(cudaMemsetAsync(dptr, value, bytes, (cudaStream_t)stream));
    return HX_OK;
}

hx_status hx_device_status(int32_t *status, int32_t clear) {
    HX_REQUIRE(status != nullptr, HX_ERR_INVALID_INPUT, "hx_device_status: status is NULL");
    HX_CUDA(cudaDeviceSynchronize());
    int a = 0, b = 0, c = 0;
    hx_status s = hx::read_status_scan(&a, clear != 0);
    if (s != HX_OK) return s;
    if ((s = hx::read_status_gemm(&b, clear != 0)) != HX_OK) return s;
    if ((s = hx::read_status_convx(&c, clear != 0)) != HX_OK) return s;
    *status = a | b | c;
    return HX_OK;
}

hx_status hx_device_check(void) {
    int32_t st = 0;
    hx_status s = hx_device_status(&st, 1);
    if (s != HX_OK) return s;
    if (st == 0) return HX_OK;
    return hx::fail(HX_ERR_BACKEND,
                    "a bounded device-side wait ran out (status 0x%x:%s%s%s%s%s%s%s); outputs since the last check are not valid", st,
                    (st & 1) ? " tile load" : "", (st & 2) ? " stage release" : "", (st & 4) ? " output tile" : "",
                    (st & 8) ? " output release" : "", (st & 16) ? " segment carry" : "", (st & 32) ? " GEMM pipeline" : "", (st & 64) ? " conv + x_proj pipeline" : "");
}

hx_status hx_stream_synchronize(void *stream) {
    HX_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return HX_OK;
}

}  // extern "C"
