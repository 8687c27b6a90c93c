// Tensor primitives on device-resident tensors: what `impl TensorOps / TensorBroadcast / TensorRandom /
// TensorMixedPrecision / TensorActivation for DeviceTensor` binds, so that the reference's generic blocks
// (`MambaBlock<T>`, `S4Block<T>` with T: Tensor + TensorOps + TensorRandom + TensorBroadcast + TensorMixedPrecision,
// crates/nn/src/lib.rs:846, crates/nn/src/ssm.rs:37) type-check and run with the device tensor as T.
//
// Semantics follow the CPU tensor of the reference, crates/backend-cpu/src/lib.rs:
//   element-wise binary ops need identical shapes (:570-632, :852-899, :951-975), unary ops map every element
//   (:759-850, :900-949, :1100-1198), matmul is (2,2), (1,2) or (2,1) with the sum over k ascending in one fp32
//   accumulator, product and sum rounded separately (:634-757), transpose materialises the permuted tensor
//   (:115-137), slice is 2-D only (:139-183), cat is 1-D only (:184-252), stack of 1-/2-/3-D tensors lays the
//   operands one after the other whatever `dim` says and only the shape label gets the new axis at `dim`
//   (:254-335), broadcast_to repeats along leading axes (:1352-1518).
// These are utility kernels (one thread per element); the hot path does not go through them.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>

#include "helix_host.hpp"
#include "hx_common.cuh"

namespace helix {
namespace tops {

namespace {

TensorError terr(hx_status code, const std::string &msg) { return TensorError{code, msg}; }

#define TOPS_TRY(expr)                     \
    do {                                   \
        auto r__ = (expr);                 \
        if (!r__.ok()) return r__.error(); \
    } while (0)

Result<Unit> on_device(const DeviceTensor &t) {
    if (!t.device().is_cuda()) return terr(HX_ERR_DEVICE_MISMATCH, "expected a CUDA tensor");
    if (hx_set_device(t.device().id) != HX_OK) return terr(HX_ERR_BACKEND, hx_last_error());
    return Unit{};
}

Result<Unit> launched(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return terr(HX_ERR_BACKEND, std::string(what) + ": " + cudaGetErrorString(e));
    return Unit{};
}

bool is_float(DType d) { return d == DType::F32 || d == DType::BF16; }

std::string shape_str(const Shape &s) {
    std::string r = "[";
    for (size_t i = 0; i < s.ndim(); ++i) r += (i ? ", " : "") + std::to_string(s.dim(i));
    return r + "]";
}

template <typename T> __device__ __forceinline__ float ldf(const T *p, int64_t i) { return hx::ld_f32<T>(p + i); }
template <typename T> __device__ __forceinline__ void stf(T *p, int64_t i, float v) { hx::st_f32<T>(p + i, v); }

// ---------------------------------------------------------------- element-wise
__device__ __forceinline__ float apply_binary(int op, float a, float b) {
    switch (op) {
        case HX_OP_ADD: return __fadd_rn(a, b);
        case HX_OP_SUB: return __fsub_rn(a, b);
        case HX_OP_MUL: return __fmul_rn(a, b);
        case HX_OP_DIV: return __fdiv_rn(a, b);
        case HX_OP_MAX: return fmaxf(a, b);
        case HX_OP_MIN: return fminf(a, b);
        default: return a > b ? 1.f : 0.f;  // HX_OP_GT
    }
}

__device__ __forceinline__ float apply_unary(int op, float x, float p0, float p1) {
    switch (op) {
        case HX_OP_SQRT: return sqrtf(x);
        case HX_OP_EXP: return expf(x);
        case HX_OP_LOG: return logf(x);
        case HX_OP_SIN: return sinf(x);
        case HX_OP_COS: return cosf(x);
        case HX_OP_TAN: return tanf(x);
        case HX_OP_ABS: return fabsf(x);
        case HX_OP_SIGN: return isnan(x) ? x : copysignf(1.f, x);  // f32::signum: +-1 also for +-0
        case HX_OP_NEG: return -x;
        case HX_OP_RELU: return fmaxf(x, 0.f);
        case HX_OP_GELU: {
            const float c = sqrtf(2.0f / 3.14159265358979323846f);
            const float x3 = __fmul_rn(__fmul_rn(x, x), x);
            return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x3)));
        }
        case HX_OP_SILU: return x / (1.0f + expf(-x));
        case HX_OP_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case HX_OP_TANH: return tanhf(x);
        case HX_OP_POW: return powf(x, p0);
        case HX_OP_CLAMP: return fminf(fmaxf(x, p0), p1);
        case HX_OP_ADD_SCALAR: return __fadd_rn(x, p0);
        case HX_OP_MUL_SCALAR: return __fmul_rn(x, p0);
        case HX_OP_GT_SCALAR: return x > p0 ? 1.f : 0.f;
        default: return x >= 0.f ? x : __fmul_rn(p0, x);  // HX_OP_LEAKY_RELU
    }
}

template <typename T> __global__ void binary_kernel(int op, const T *a, const T *b, T *o, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        stf(o, i, apply_binary(op, ldf(a, i), ldf(b, i)));
}
template <typename T> __global__ void unary_kernel(int op, const T *a, T *o, int64_t n, float p0, float p1) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        stf(o, i, apply_unary(op, ldf(a, i), p0, p1));
}
template <typename TI, typename TO> __global__ void cast_kernel(const TI *a, TO *o, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        hx::st_f32<TO>(o + i, hx::ld_f32<TI>(a + i));
}
template <typename T> __global__ void fill_kernel(T *o, int64_t n, float v) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        stf(o, i, v);
}

int grid_for(int64_t n) {
    const int64_t b = (n + 255) / 256;
    return (int)(b < 1 ? 1 : (b > 65535 ? 65535 : b));
}

// ---------------------------------------------------------------- strided gather (transpose, slice, broadcast)
struct Gather {
    int ndim;
    int64_t out_dims[8];
    int64_t in_strides[8];  // element stride of the source per OUTPUT axis (0 = broadcast)
    int64_t in_offset;
};
template <typename T> __global__ void gather_kernel(const T *a, T *o, int64_t n, Gather g) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = i, src = g.in_offset;
        for (int k = g.ndim - 1; k >= 0; --k) {
            const int64_t c = rem % g.out_dims[k];
            rem /= g.out_dims[k];
            src += c * g.in_strides[k];
        }
        o[i] = a[src];
    }
}

Result<DeviceTensor> gather(const DeviceTensor &a, const Shape &out_shape, const Gather &g) {
    auto out = DeviceTensor::empty(out_shape, a.dtype(), a.device());
    if (!out.ok()) return out.error();
    const int64_t n = out_shape.numel();
    if (n == 0) return out;
    if (a.dtype() == DType::F32)
        gather_kernel<float><<<grid_for(n), 256>>>(static_cast<const float *>(a.data()), static_cast<float *>(out.value().data()), n, g);
    else if (a.dtype() == DType::BF16)
        gather_kernel<uint16_t><<<grid_for(n), 256>>>(static_cast<const uint16_t *>(a.data()),
                                                      static_cast<uint16_t *>(out.value().data()), n, g);
    else
        gather_kernel<uint8_t><<<grid_for(n), 256>>>(static_cast<const uint8_t *>(a.data()), static_cast<uint8_t *>(out.value().data()), n, g);
    TOPS_TRY(launched("gather_kernel"));
    return out;
}

std::vector<int64_t> row_major_strides(const Shape &s) {
    std::vector<int64_t> st(s.ndim(), 1);
    for (int i = (int)s.ndim() - 2; i >= 0; --i) st[i] = st[i + 1] * s.dim(i + 1);
    return st;
}

// ---------------------------------------------------------------- matmul in the reference's arithmetic
// C[i][j] = sum_k A[i][k] * B[k][j], k ascending, one fp32 accumulator, product and sum rounded separately
// (the reference's Rust loop does not fuse them): crates/backend-cpu/src/lib.rs:657-668.
template <typename T>
__global__ void __launch_bounds__(256) matmul_ref_kernel(const T *A, const T *B, T *C, int M, int N, int K) {
    __shared__ float sa[16][17], sb[16][17];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int i = blockIdx.y * 16 + ty, j = blockIdx.x * 16 + tx;
    float sum = 0.f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        sa[ty][tx] = (i < M && k0 + tx < K) ? ldf(A, (int64_t)i * K + k0 + tx) : 0.f;
        sb[ty][tx] = (k0 + ty < K && j < N) ? ldf(B, (int64_t)(k0 + ty) * N + j) : 0.f;
        __syncthreads();
        const int kk = min(16, K - k0);
        for (int k = 0; k < kk; ++k) sum = __fadd_rn(sum, __fmul_rn(sa[ty][k], sb[k][tx]));
        __syncthreads();
    }
    if (i < M && j < N) stf(C, (int64_t)i * N + j, sum);
}

}  // namespace

// ================================================================================================ API
Result<DeviceTensor> binary(int op, const DeviceTensor &a, const DeviceTensor &b) {
    if (op < HX_OP_ADD || op > HX_OP_GT) return terr(HX_ERR_INVALID_INPUT, "unknown binary op " + std::to_string(op));
    if (!(a.shape() == b.shape()))
        return terr(HX_ERR_SHAPE_MISMATCH, "binary op on shapes " + shape_str(a.shape()) + " and " + shape_str(b.shape()));
    if (a.dtype() != b.dtype() || !is_float(a.dtype())) return terr(HX_ERR_DTYPE_MISMATCH, "binary op needs two F32 or two BF16 tensors");
    if (!(a.device() == b.device())) return terr(HX_ERR_DEVICE_MISMATCH, "binary op on tensors of different devices");
    TOPS_TRY(on_device(a));
    auto out = DeviceTensor::empty(a.shape(), a.dtype(), a.device());
    if (!out.ok()) return out.error();
    const int64_t n = a.numel();
    if (n == 0) return out;
    if (a.dtype() == DType::F32)
        binary_kernel<float><<<grid_for(n), 256>>>(op, static_cast<const float *>(a.data()), static_cast<const float *>(b.data()),
                                                   static_cast<float *>(out.value().data()), n);
    else
        binary_kernel<__nv_bfloat16><<<grid_for(n), 256>>>(op, static_cast<const __nv_bfloat16 *>(a.data()),
                                                           static_cast<const __nv_bfloat16 *>(b.data()),
                                                           static_cast<__nv_bfloat16 *>(out.value().data()), n);
    TOPS_TRY(launched("binary_kernel"));
    return out;
}

Result<DeviceTensor> unary(int op, const DeviceTensor &a, float p0, float p1) {
    if (op < HX_OP_SQRT || op > HX_OP_LEAKY_RELU) return terr(HX_ERR_INVALID_INPUT, "unknown unary op " + std::to_string(op));
    if (!is_float(a.dtype())) return terr(HX_ERR_DTYPE_MISMATCH, "unary op needs an F32 or BF16 tensor");
    TOPS_TRY(on_device(a));
    auto out = DeviceTensor::empty(a.shape(), a.dtype(), a.device());
    if (!out.ok()) return out.error();
    const int64_t n = a.numel();
    if (n == 0) return out;
    if (a.dtype() == DType::F32)
        unary_kernel<float><<<grid_for(n), 256>>>(op, static_cast<const float *>(a.data()), static_cast<float *>(out.value().data()), n, p0, p1);
    else
        unary_kernel<__nv_bfloat16><<<grid_for(n), 256>>>(op, static_cast<const __nv_bfloat16 *>(a.data()),
                                                          static_cast<__nv_bfloat16 *>(out.value().data()), n, p0, p1);
    TOPS_TRY(launched("unary_kernel"));
    return out;
}

Result<DeviceTensor> matmul(const DeviceTensor &a, const DeviceTensor &b) {
    if (a.ndim() == 0 || b.ndim() == 0) return terr(HX_ERR_UNSUPPORTED_OPERATION, "matrix multiplication requires at least 1D tensors");
    if (a.dtype() != b.dtype() || !is_float(a.dtype())) return terr(HX_ERR_DTYPE_MISMATCH, "matmul needs two F32 or two BF16 tensors");
    if (!(a.device() == b.device())) return terr(HX_ERR_DEVICE_MISMATCH, "matmul on tensors of different devices");
    int64_t M, K, Kb, N;
    Shape out_shape;
    if (a.ndim() == 2 && b.ndim() == 2) {
        M = a.shape().dim(0); K = a.shape().dim(1); Kb = b.shape().dim(0); N = b.shape().dim(1);
        out_shape = Shape({M, N});
    } else if (a.ndim() == 1 && b.ndim() == 2) {
        M = 1; K = a.shape().dim(0); Kb = b.shape().dim(0); N = b.shape().dim(1);
        out_shape = Shape({N});
    } else if (a.ndim() == 2 && b.ndim() == 1) {
        M = a.shape().dim(0); K = a.shape().dim(1); Kb = b.shape().dim(0); N = 1;
        out_shape = Shape({M});
    } else {
        return terr(HX_ERR_UNSUPPORTED_OPERATION, "batch matrix multiplication for >2D tensors not implemented yet");
    }
    if (K != Kb) return terr(HX_ERR_SHAPE_MISMATCH, "matmul inner dimensions " + std::to_string(K) + " and " + std::to_string(Kb));
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return terr(HX_ERR_INVALID_DIMENSION, "matmul dimension exceeds 2^31");
    TOPS_TRY(on_device(a));
    auto out = DeviceTensor::empty(out_shape, a.dtype(), a.device());
    if (!out.ok()) return out.error();
    if (M * N == 0) return out;
    if (hx_matmul_ref(a.data(), b.data(), out.value().data(), (int)M, (int)N, (int)K, (int)a.dtype(), nullptr) != HX_OK)
        return terr(HX_ERR_BACKEND, hx_last_error());
    return out;
}

Result<DeviceTensor> transpose(const DeviceTensor &a, int64_t d0, int64_t d1) {
    const int nd = (int)a.ndim();
    if (d0 < 0 || d1 < 0 || d0 >= nd || d1 >= nd)
        return terr(HX_ERR_INVALID_DIMENSION, "transpose(" + std::to_string(d0) + ", " + std::to_string(d1) + ") of " + shape_str(a.shape()));
    if (nd > 8) return terr(HX_ERR_UNSUPPORTED_OPERATION, "more than 8 dimensions");
    TOPS_TRY(on_device(a));
    std::vector<int64_t> dims = a.shape().as_slice();
    std::vector<int64_t> st = row_major_strides(a.shape());
    std::swap(dims[d0], dims[d1]);
    std::swap(st[d0], st[d1]);
    Gather g{};
    g.ndim = nd;
    g.in_offset = 0;
    for (int i = 0; i < nd; ++i) { g.out_dims[i] = dims[i]; g.in_strides[i] = st[i]; }
    return gather(a, Shape(dims), g);
}

Result<DeviceTensor> slice(const DeviceTensor &a, const std::vector<int64_t> &start, const std::vector<int64_t> &end) {
    const size_t nd = a.ndim();
    if (start.size() != nd || end.size() != nd)
        return terr(HX_ERR_SHAPE_MISMATCH, "slice: " + std::to_string(std::max(start.size(), end.size())) + " indices for " + shape_str(a.shape()));
    for (size_t i = 0; i < nd; ++i)
        if (start[i] < 0 || start[i] >= a.shape().dim(i) || end[i] > a.shape().dim(i) || start[i] >= end[i])
            return terr(HX_ERR_INVALID_DIMENSION, "slice bounds outside dimension " + std::to_string(i) + " of " + shape_str(a.shape()));
    if (nd != 2) return terr(HX_ERR_UNSUPPORTED_OPERATION, "Slicing for " + std::to_string(nd) + "D tensors not implemented yet");
    TOPS_TRY(on_device(a));
    Gather g{};
    g.ndim = 2;
    g.out_dims[0] = end[0] - start[0];
    g.out_dims[1] = end[1] - start[1];
    g.in_strides[0] = a.shape().dim(1);
    g.in_strides[1] = 1;
    g.in_offset = start[0] * a.shape().dim(1) + start[1];
    return gather(a, Shape({g.out_dims[0], g.out_dims[1]}), g);
}

// cat (1-D operands) and stack (1- to 3-D operands): the operands' buffers one after the other.
static Result<DeviceTensor> concat_buffers(const std::vector<const DeviceTensor *> &ts, const Shape &out_shape) {
    const DeviceTensor &f = *ts[0];
    TOPS_TRY(on_device(f));
    auto out = DeviceTensor::empty(out_shape, f.dtype(), f.device());
    if (!out.ok()) return out.error();
    size_t off = 0;
    const size_t es = dtype_size(f.dtype());
    for (const DeviceTensor *t : ts) {
        const size_t bytes = (size_t)t->numel() * es;
        if (bytes && cudaMemcpyAsync(static_cast<char *>(out.value().data()) + off, t->data(), bytes, cudaMemcpyDeviceToDevice, nullptr) != cudaSuccess)
            return terr(HX_ERR_BACKEND, "device copy failed");
        off += bytes;
    }
    return out;
}

Result<DeviceTensor> cat(const std::vector<const DeviceTensor *> &ts, int64_t dim) {
    if (ts.empty()) return terr(HX_ERR_UNSUPPORTED_OPERATION, "concatenation of empty tensor list");
    for (auto *t : ts)
        if (!t) return terr(HX_ERR_INVALID_INPUT, "cat: NULL tensor");
    if (ts.size() == 1) return ts[0]->clone();
    const Shape &fs = ts[0]->shape();
    if (dim < 0 || dim >= (int64_t)fs.ndim()) return terr(HX_ERR_INVALID_DIMENSION, "cat along dimension " + std::to_string(dim) + " of " + shape_str(fs));
    int64_t total = 0;
    for (auto *t : ts) {
        if (t->ndim() != fs.ndim()) return terr(HX_ERR_SHAPE_MISMATCH, "cat: operands of different rank");
        for (size_t i = 0; i < fs.ndim(); ++i)
            if ((int64_t)i != dim && t->shape().dim(i) != fs.dim(i)) return terr(HX_ERR_SHAPE_MISMATCH, "cat: operands differ outside the joined dimension");
        if (t->dtype() != ts[0]->dtype()) return terr(HX_ERR_DTYPE_MISMATCH, "cat: operands of different dtype");
        if (!(t->device() == ts[0]->device())) return terr(HX_ERR_DEVICE_MISMATCH, "cat: operands on different devices");
        total += t->shape().dim(dim);
    }
    if (fs.ndim() != 1) return terr(HX_ERR_UNSUPPORTED_OPERATION, "Concatenation for " + std::to_string(fs.ndim()) + "D tensors not implemented yet");
    return concat_buffers(ts, Shape({total}));
}

Result<DeviceTensor> stack(const std::vector<const DeviceTensor *> &ts, int64_t dim) {
    if (ts.empty()) return terr(HX_ERR_UNSUPPORTED_OPERATION, "stacking of empty tensor list");
    for (auto *t : ts)
        if (!t) return terr(HX_ERR_INVALID_INPUT, "stack: NULL tensor");
    if (ts.size() == 1) return ts[0]->clone();
    const Shape &fs = ts[0]->shape();
    for (auto *t : ts) {
        if (!(t->shape() == fs)) return terr(HX_ERR_SHAPE_MISMATCH, "stack: " + shape_str(t->shape()) + " against " + shape_str(fs));
        if (t->dtype() != ts[0]->dtype()) return terr(HX_ERR_DTYPE_MISMATCH, "stack: operands of different dtype");
        if (!(t->device() == ts[0]->device())) return terr(HX_ERR_DEVICE_MISMATCH, "stack: operands on different devices");
    }
    if (dim < 0 || dim > (int64_t)fs.ndim()) return terr(HX_ERR_INVALID_DIMENSION, "stack at dimension " + std::to_string(dim) + " of " + shape_str(fs));
    if (fs.ndim() < 1 || fs.ndim() > 3) return terr(HX_ERR_UNSUPPORTED_OPERATION, "stack of " + std::to_string(fs.ndim()) + "D tensors");
    // the buffer is [count, operand shape...] whatever `dim`; the label carries the new axis at `dim`
    std::vector<int64_t> label = fs.as_slice();
    label.insert(label.begin() + dim, (int64_t)ts.size());
    return concat_buffers(ts, Shape(label));
}

Result<DeviceTensor> broadcast_to(const DeviceTensor &a, const Shape &shape) {
    const Shape &s = a.shape();
    if (s.ndim() > shape.ndim()) return terr(HX_ERR_SHAPE_MISMATCH, "broadcast of " + shape_str(s) + " to fewer dimensions " + shape_str(shape));
    if (s == shape) return a.clone();
    if (shape.ndim() > 8) return terr(HX_ERR_UNSUPPORTED_OPERATION, "more than 8 dimensions");
    const size_t pad = shape.ndim() - s.ndim();
    for (size_t i = 0; i < shape.ndim(); ++i) {
        const int64_t sd = i < pad ? 1 : s.dim(i - pad);
        if (sd != 1 && sd != shape.dim(i)) return terr(HX_ERR_SHAPE_MISMATCH, "cannot broadcast " + shape_str(s) + " to " + shape_str(shape));
    }
    // rank extensions the reference has a case for: (1,2), (2,3), (1,3); equal ranks broadcast axis by axis
    if (pad != 0) {
        const bool ok12 = s.ndim() == 1 && shape.ndim() == 2 && (s.dim(0) == shape.dim(1) || s.dim(0) == shape.dim(0));
        const bool ok23 = s.ndim() == 2 && shape.ndim() == 3 &&
                          ((s.dim(0) == shape.dim(1) && s.dim(1) == shape.dim(2)) || (s.dim(0) == 1 && s.dim(1) == shape.dim(2)));
        const bool ok13 = s.ndim() == 1 && shape.ndim() == 3 && s.dim(0) == shape.dim(2);
        if (!(ok12 || ok23 || ok13)) {
            if ((s.ndim() == 1 && shape.ndim() <= 3) || (s.ndim() == 2 && shape.ndim() == 3))
                return terr(HX_ERR_SHAPE_MISMATCH, "cannot broadcast " + shape_str(s) + " to " + shape_str(shape));
            return terr(HX_ERR_UNSUPPORTED_OPERATION, "broadcast from " + std::to_string(s.ndim()) + " to " + std::to_string(shape.ndim()) + " dimensions");
        }
    }
    TOPS_TRY(on_device(a));
    const std::vector<int64_t> st = row_major_strides(s);
    Gather g{};
    g.ndim = (int)shape.ndim();
    g.in_offset = 0;
    for (size_t i = 0; i < shape.ndim(); ++i) {
        g.out_dims[i] = shape.dim(i);
        g.in_strides[i] = (i < pad || s.dim(i - pad) == 1) ? 0 : st[i - pad];
    }
    return gather(a, shape, g);
}

Result<DeviceTensor> cast(const DeviceTensor &a, DType dtype) {
    if (!is_float(a.dtype()) || !is_float(dtype)) return terr(HX_ERR_UNSUPPORTED_OPERATION, "cast between F32 and BF16 only");
    if (a.dtype() == dtype) return a.clone();
    TOPS_TRY(on_device(a));
    auto out = DeviceTensor::empty(a.shape(), dtype, a.device());
    if (!out.ok()) return out.error();
    const int64_t n = a.numel();
    if (n == 0) return out;
    if (dtype == DType::BF16)
        cast_kernel<float, __nv_bfloat16><<<grid_for(n), 256>>>(static_cast<const float *>(a.data()), static_cast<__nv_bfloat16 *>(out.value().data()), n);
    else
        cast_kernel<__nv_bfloat16, float><<<grid_for(n), 256>>>(static_cast<const __nv_bfloat16 *>(a.data()), static_cast<float *>(out.value().data()), n);
    TOPS_TRY(launched("cast_kernel"));
    return out;
}

Result<float> to_scalar(const DeviceTensor &a) {
    if (a.numel() != 1) return terr(HX_ERR_INVALID_INPUT, "Cannot convert tensor with " + std::to_string(a.numel()) + " elements to scalar");
    float v = 0.f;
    auto r = a.to_host_f32(&v, 1);
    if (!r.ok()) return r.error();
    return v;
}

Result<DeviceTensor> full(float value, const Shape &shape, DType dtype, const Device &device) {
    if (!is_float(dtype)) return terr(HX_ERR_DTYPE_MISMATCH, "full: dtype must be F32 or BF16");
    auto out = DeviceTensor::empty(shape, dtype, device);
    if (!out.ok()) return out.error();
    const int64_t n = shape.numel();
    if (n == 0) return out;
    if (dtype == DType::F32) fill_kernel<float><<<grid_for(n), 256>>>(static_cast<float *>(out.value().data()), n, value);
    else fill_kernel<__nv_bfloat16><<<grid_for(n), 256>>>(static_cast<__nv_bfloat16 *>(out.value().data()), n, value);
    TOPS_TRY(launched("fill_kernel"));
    return out;
}

Result<DeviceTensor> eye(int64_t n, DType dtype, const Device &device) {
    if (n < 0) return terr(HX_ERR_INVALID_DIMENSION, "eye: negative size");
    std::vector<float> h((size_t)n * n, 0.f);
    for (int64_t i = 0; i < n; ++i) h[(size_t)i * n + i] = 1.f;
    return DeviceTensor::from_host_f32(h.data(), Shape({n, n}), dtype, device);
}

Result<DeviceTensor> arange(float start, float end, float step, DType dtype, const Device &device) {
    if (!(step > 0.f) || !std::isfinite(start) || !std::isfinite(end)) return terr(HX_ERR_INVALID_INPUT, "arange needs a positive step and finite bounds");
    std::vector<float> h;
    // the reference's loop: current += step in fp32, while current < end
    for (float cur = start; cur < end; cur += step) {
        if (h.size() > (size_t)1 << 28) return terr(HX_ERR_INVALID_INPUT, "arange of more than 2^28 elements");
        h.push_back(cur);
    }
    return DeviceTensor::from_host_f32(h.data(), Shape({(int64_t)h.size()}), dtype, device);
}

}  // namespace tops
}  // namespace helix

// ================================================================================================ C handles
namespace {
hx_status fail_from(const helix::TensorError &e) { return hx::fail(e.code, "%s", e.message.c_str()); }
template <typename R> hx_status give(R &&r, hx_tensor **out) {
    if (!r.ok()) return fail_from(r.error());
    *out = new hx_tensor{std::move(r.value())};
    return HX_OK;
}
bool shape_from(const int64_t *dims, int32_t ndim, helix::Shape *s) {
    if (ndim < 0 || ndim > 8 || (ndim > 0 && !dims)) return false;
    *s = helix::Shape(std::vector<int64_t>(dims, dims + ndim));
    return true;
}
}  // namespace

extern "C" {

hx_status hx_matmul_ref(const void *A, const void *B, void *C, int32_t M, int32_t N, int32_t K, int32_t dtype, void *stream) {
    HX_REQUIRE(M >= 0 && N >= 0 && K >= 0, HX_ERR_INVALID_DIMENSION, "hx_matmul_ref: negative dimension");
    HX_REQUIRE(dtype == HX_F32 || dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "hx_matmul_ref: dtype must be F32 or BF16");
    if (M == 0 || N == 0) return HX_OK;
    HX_REQUIRE(C && (K == 0 || (A && B)), HX_ERR_INVALID_INPUT, "hx_matmul_ref: NULL operand");
    dim3 grid((unsigned)((N + 15) / 16), (unsigned)((M + 15) / 16));
    HX_REQUIRE(grid.y <= 65535, HX_ERR_INVALID_DIMENSION, "hx_matmul_ref: more than 2^20 rows; use hx_gemm_bf16 / hx_gemm_simt");
    cudaStream_t st = (cudaStream_t)stream;
    using namespace helix::tops;
    if (dtype == HX_F32)
        matmul_ref_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float *>(A), static_cast<const float *>(B),
                                                       static_cast<float *>(C), M, N, K);
    else
        matmul_ref_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16 *>(A), static_cast<const __nv_bfloat16 *>(B),
                                                               static_cast<__nv_bfloat16 *>(C), M, N, K);
    return hx::check_launch("matmul_ref_kernel");
}

hx_status hx_tensor_binary(int32_t op, const hx_tensor *a, const hx_tensor *b, hx_tensor **out) {
    HX_REQUIRE(a && b && out, HX_ERR_INVALID_INPUT, "hx_tensor_binary: NULL argument");
    return give(helix::tops::binary(op, a->t, b->t), out);
}

hx_status hx_tensor_unary(int32_t op, const hx_tensor *a, float p0, float p1, hx_tensor **out) {
    HX_REQUIRE(a && out, HX_ERR_INVALID_INPUT, "hx_tensor_unary: NULL argument");
    return give(helix::tops::unary(op, a->t, p0, p1), out);
}

hx_status hx_tensor_matmul(const hx_tensor *a, const hx_tensor *b, hx_tensor **out) {
    HX_REQUIRE(a && b && out, HX_ERR_INVALID_INPUT, "hx_tensor_matmul: NULL argument");
    return give(helix::tops::matmul(a->t, b->t), out);
}

hx_status hx_tensor_transpose(const hx_tensor *a, int64_t dim0, int64_t dim1, hx_tensor **out) {
    HX_REQUIRE(a && out, HX_ERR_INVALID_INPUT, "hx_tensor_transpose: NULL argument");
    return give(helix::tops::transpose(a->t, dim0, dim1), out);
}

hx_status hx_tensor_slice(const hx_tensor *a, const int64_t *start, const int64_t *end, int32_t n, hx_tensor **out) {
    HX_REQUIRE(a && out && n >= 0 && n <= 8 && (n == 0 || (start && end)), HX_ERR_INVALID_INPUT, "hx_tensor_slice: bad arguments");
    return give(helix::tops::slice(a->t, std::vector<int64_t>(start, start + n), std::vector<int64_t>(end, end + n)), out);
}

hx_status hx_tensor_cat(const hx_tensor *const *tensors, int32_t count, int64_t dim, hx_tensor **out) {
    HX_REQUIRE(out && count >= 0 && (count == 0 || tensors), HX_ERR_INVALID_INPUT, "hx_tensor_cat: bad arguments");
    std::vector<const helix::DeviceTensor *> ts;
    for (int32_t i = 0; i < count; ++i) ts.push_back(tensors[i] ? &tensors[i]->t : nullptr);
    return give(helix::tops::cat(ts, dim), out);
}

hx_status hx_tensor_stack(const hx_tensor *const *tensors, int32_t count, int64_t dim, hx_tensor **out) {
    HX_REQUIRE(out && count >= 0 && (count == 0 || tensors), HX_ERR_INVALID_INPUT, "hx_tensor_stack: bad arguments");
    std::vector<const helix::DeviceTensor *> ts;
    for (int32_t i = 0; i < count; ++i) ts.push_back(tensors[i] ? &tensors[i]->t : nullptr);
    return give(helix::tops::stack(ts, dim), out);
}

hx_status hx_tensor_broadcast_to(const hx_tensor *a, const int64_t *dims, int32_t ndim, hx_tensor **out) {
    helix::Shape s;
    HX_REQUIRE(a && out && shape_from(dims, ndim, &s), HX_ERR_INVALID_INPUT, "hx_tensor_broadcast_to: bad arguments");
    return give(helix::tops::broadcast_to(a->t, s), out);
}

hx_status hx_tensor_reshape(const hx_tensor *a, const int64_t *dims, int32_t ndim, hx_tensor **out) {
    helix::Shape s;
    HX_REQUIRE(a && out && shape_from(dims, ndim, &s), HX_ERR_INVALID_INPUT, "hx_tensor_reshape: bad arguments");
    // the reference's reshape returns an owned copy (crates/backend-cpu/src/lib.rs:94-113)
    auto c = a->t.clone();
    if (!c.ok()) return fail_from(c.error());
    return give(c.value().reshape(s), out);
}

hx_status hx_tensor_clone(const hx_tensor *a, hx_tensor **out) {
    HX_REQUIRE(a && out, HX_ERR_INVALID_INPUT, "hx_tensor_clone: NULL argument");
    return give(a->t.clone(), out);
}

hx_status hx_tensor_cast(const hx_tensor *a, int32_t dtype, hx_tensor **out) {
    HX_REQUIRE(a && out, HX_ERR_INVALID_INPUT, "hx_tensor_cast: NULL argument");
    HX_REQUIRE(dtype == HX_F32 || dtype == HX_BF16, HX_ERR_UNSUPPORTED_OPERATION,
               "hx_tensor_cast: the device tensor stores F32 or BF16 (asked for dtype %d)", dtype);
    return give(helix::tops::cast(a->t, (helix::DType)dtype), out);
}

hx_status hx_tensor_to_scalar(const hx_tensor *a, float *value) {
    HX_REQUIRE(a && value, HX_ERR_INVALID_INPUT, "hx_tensor_to_scalar: NULL argument");
    auto r = helix::tops::to_scalar(a->t);
    if (!r.ok()) return fail_from(r.error());
    *value = r.value();
    return HX_OK;
}

hx_status hx_tensor_full(float value, const int64_t *dims, int32_t ndim, int32_t dtype, int32_t device_id, hx_tensor **out) {
    helix::Shape s;
    HX_REQUIRE(out && shape_from(dims, ndim, &s), HX_ERR_INVALID_INPUT, "hx_tensor_full: bad arguments");
    HX_REQUIRE(dtype == HX_F32 || dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "hx_tensor_full: dtype must be F32 or BF16");
    return give(helix::tops::full(value, s, (helix::DType)dtype, helix::Device::cuda(device_id)), out);
}

hx_status hx_tensor_eye(int64_t n, int32_t dtype, int32_t device_id, hx_tensor **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_tensor_eye: out is NULL");
    HX_REQUIRE(dtype == HX_F32 || dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "hx_tensor_eye: dtype must be F32 or BF16");
    return give(helix::tops::eye(n, (helix::DType)dtype, helix::Device::cuda(device_id)), out);
}

hx_status hx_tensor_arange(float start, float end, float step, int32_t dtype, int32_t device_id, hx_tensor **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_tensor_arange: out is NULL");
    HX_REQUIRE(dtype == HX_F32 || dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "hx_tensor_arange: dtype must be F32 or BF16");
    return give(helix::tops::arange(start, end, step, (helix::DType)dtype, helix::Device::cuda(device_id)), out);
}

hx_status hx_tensor_random(int32_t kind, const int64_t *dims, int32_t ndim, float p0, float p1, int32_t device_id, hx_tensor **out) {
    helix::Shape s;
    HX_REQUIRE(out && shape_from(dims, ndim, &s), HX_ERR_INVALID_INPUT, "hx_tensor_random: bad arguments");
    const helix::Device dev = helix::Device::cuda(device_id);
    switch (kind) {
        case HX_RANDOM_NORMAL: return give(helix::init_normal(s, (double)p1, helix::DType::F32, dev, (double)p0), out);
        case HX_RANDOM_UNIFORM:
            HX_REQUIRE(p0 < p1, HX_ERR_INVALID_INPUT, "hx_tensor_random: empty range [%g, %g)", p0, p1);
            return give(helix::init_uniform(s, (double)p0, (double)p1, helix::DType::F32, dev), out);
        case HX_RANDOM_BERNOULLI: return give(helix::init_bernoulli(s, (double)p0, helix::DType::F32, dev), out);
        default: return hx::fail(HX_ERR_INVALID_INPUT, "hx_tensor_random: unknown kind %d", kind);
    }
}

}  // extern "C"
