// Implementation of the C++ host layer (helix_host.hpp) and of its C handles (hx_tensor_* / hx_module_*).
#include "helix_host.hpp"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cmath>
#include <cstring>
#include <mutex>

#include "hx_common.cuh"

namespace helix {

// ------------------------------------------------------------------------------------------ helpers
static TensorError err(hx_status code, const std::string &msg) { return TensorError{code, msg}; }
static TensorError last_abi_error(hx_status code) { return TensorError{code, hx_last_error()}; }

#define HELIX_TRY_ABI(call)                             \
    do {                                                \
        hx_status st__ = (call);                        \
        if (st__ != HX_OK) return last_abi_error(st__); \
    } while (0)

#define HELIX_TRY(expr)                              \
    do {                                             \
        auto r__ = (expr);                           \
        if (!r__.ok()) return r__.error();           \
    } while (0)

static Result<Unit> use_device(const Device &d) {
    if (!d.is_cuda()) return err(HX_ERR_DEVICE_MISMATCH, "expected a CUDA device, got " + d.to_string());
    HELIX_TRY_ABI(hx_set_device(d.id));
    return Unit{};
}

static std::string shape_str(const Shape &s) {
    std::string r = "[";
    for (size_t i = 0; i < s.ndim(); ++i) r += (i ? ", " : "") + std::to_string(s.dim(i));
    return r + "]";
}

// ---- seeded initialisers: SplitMix64 counter streams, Box-Muller normals
static std::atomic<uint64_t> g_seed{0x243F6A8885A308D3ull};
static std::atomic<uint64_t> g_stream{0};
void manual_seed(uint64_t seed) {
    g_seed = seed;
    g_stream = 0;
}
static inline uint64_t mix64(uint64_t x) {
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
struct Rng {
    uint64_t key, ctr = 0;
    Rng() : key(mix64(g_seed.load() * 0x9E3779B97F4A7C15ull + g_stream.fetch_add(1))) {}
    double uniform01() { return (double)(mix64(key + (++ctr) * 0x9E3779B97F4A7C15ull) >> 40) * (1.0 / 16777216.0); }
    double normal() {
        const double u1 = 1.0 - uniform01(), u2 = uniform01();
        return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
    }
};

static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

// ------------------------------------------------------------------------------------------ DeviceTensor
Result<DeviceTensor> DeviceTensor::empty(const Shape &shape, DType dtype, const Device &device) {
    for (auto d : shape.as_slice())
        if (d < 0) return err(HX_ERR_INVALID_DIMENSION, "negative dimension in shape " + shape_str(shape));
    HELIX_TRY(use_device(device));
    DeviceTensor t;
    t.shape_ = shape;
    t.dtype_ = dtype;
    t.device_ = device;
    const size_t bytes = (size_t)shape.numel() * dtype_size(dtype);
    if (bytes > 0) {
        void *p = nullptr;
        HELIX_TRY_ABI(hx_alloc(&p, bytes));
        const int dev = device.id;
        t.storage_ = std::shared_ptr<void>(p, [dev](void *q) {
            int cur = 0;
            cudaGetDevice(&cur);
            if (cur != dev) cudaSetDevice(dev);
            cudaFree(q);
            if (cur != dev) cudaSetDevice(cur);
        });
        t.ptr_ = p;
    }
    return t;
}

Result<DeviceTensor> DeviceTensor::zeros(const Shape &shape, DType dtype, const Device &device) {
    auto r = empty(shape, dtype, device);
    if (!r.ok()) return r;
    if (r.value().numel() > 0)
        HELIX_TRY_ABI(hx_memset(r.value().data(), 0, (size_t)r.value().numel() * dtype_size(dtype), nullptr));
    return r;
}

Result<Unit> DeviceTensor::copy_from_host_f32(const float *data, int64_t n) {
    if (n != numel())
        return err(HX_ERR_SHAPE_MISMATCH, "copy_from_host: got " + std::to_string(n) + " values for shape " + shape_str(shape_));
    if (n == 0) return Unit{};
    if (!data) return err(HX_ERR_INVALID_INPUT, "copy_from_host: data is NULL");
    HELIX_TRY(use_device(device_));
    if (dtype_ == DType::F32) {
        HELIX_TRY_ABI(hx_memcpy_h2d(ptr_, data, (size_t)n * 4, nullptr));
    } else if (dtype_ == DType::BF16) {
        std::vector<uint16_t> tmp((size_t)n);
        for (int64_t i = 0; i < n; ++i) tmp[(size_t)i] = f32_to_bf16_bits(data[i]);
        HELIX_TRY_ABI(hx_memcpy_h2d(ptr_, tmp.data(), (size_t)n * 2, nullptr));
        HELIX_TRY_ABI(hx_stream_synchronize(nullptr));  // tmp dies at scope end
    } else {
        return err(HX_ERR_DTYPE_MISMATCH, "copy_from_host_f32 into a U8 tensor");
    }
    HELIX_TRY_ABI(hx_stream_synchronize(nullptr));
    return Unit{};
}

Result<DeviceTensor> DeviceTensor::from_host_f32(const float *data, const Shape &shape, DType dtype, const Device &device) {
    auto r = empty(shape, dtype, device);
    if (!r.ok()) return r;
    HELIX_TRY(r.value().copy_from_host_f32(data, shape.numel()));
    return r;
}

Result<DeviceTensor> DeviceTensor::from_host_u8(const uint8_t *data, const Shape &shape, const Device &device) {
    auto r = empty(shape, DType::U8, device);
    if (!r.ok()) return r;
    if (shape.numel() > 0) {
        if (!data) return err(HX_ERR_INVALID_INPUT, "from_host_u8: data is NULL");
        HELIX_TRY_ABI(hx_memcpy_h2d(r.value().data(), data, (size_t)shape.numel(), nullptr));
        HELIX_TRY_ABI(hx_stream_synchronize(nullptr));
    }
    return r;
}

Result<Unit> DeviceTensor::to_host_f32(float *out, int64_t n) const {
    if (n != numel()) return err(HX_ERR_SHAPE_MISMATCH, "to_host: buffer of " + std::to_string(n) + " for shape " + shape_str(shape_));
    if (n == 0) return Unit{};
    if (!out) return err(HX_ERR_INVALID_INPUT, "to_host: out is NULL");
    HELIX_TRY(use_device(device_));
    if (dtype_ == DType::F32) {
        HELIX_TRY_ABI(hx_memcpy_d2h(out, ptr_, (size_t)n * 4, nullptr));
        HELIX_TRY_ABI(hx_stream_synchronize(nullptr));
    } else if (dtype_ == DType::BF16) {
        std::vector<uint16_t> tmp((size_t)n);
        HELIX_TRY_ABI(hx_memcpy_d2h(tmp.data(), ptr_, (size_t)n * 2, nullptr));
        HELIX_TRY_ABI(hx_stream_synchronize(nullptr));
        for (int64_t i = 0; i < n; ++i) out[i] = bf16_bits_to_f32(tmp[(size_t)i]);
    } else {
        std::vector<uint8_t> tmp((size_t)n);
        HELIX_TRY_ABI(hx_memcpy_d2h(tmp.data(), ptr_, (size_t)n, nullptr));
        HELIX_TRY_ABI(hx_stream_synchronize(nullptr));
        for (int64_t i = 0; i < n; ++i) out[i] = (float)tmp[(size_t)i];
    }
    return Unit{};
}

Result<DeviceTensor> DeviceTensor::clone() const {
    auto r = empty(shape_, dtype_, device_);
    if (!r.ok()) return r;
    const size_t bytes = (size_t)numel() * dtype_size(dtype_);
    if (bytes > 0) {
        if (cudaMemcpyAsync(r.value().data(), ptr_, bytes, cudaMemcpyDeviceToDevice, nullptr) != cudaSuccess)
            return err(HX_ERR_BACKEND, "device-to-device copy failed");
    }
    return r;
}

Result<DeviceTensor> DeviceTensor::reshape(const Shape &shape) const {
    if (shape.numel() != numel())
        return err(HX_ERR_SHAPE_MISMATCH, "reshape " + shape_str(shape_) + " -> " + shape_str(shape));
    DeviceTensor t = *this;
    t.shape_ = shape;
    return t;
}

// Normal(mean, std) / uniform / Bernoulli / constant initialisers (TensorRandom, crates/tensor-core/src/tensor.rs:212-233),
// drawn on the host from the seeded counter streams above
Result<DeviceTensor> init_normal(const Shape &shape, double stddev, DType dtype, const Device &device, double mean) {
    if (shape.numel() < 0) return err(HX_ERR_INVALID_DIMENSION, "negative dimension in shape " + shape_str(shape));
    std::vector<float> h((size_t)shape.numel());
    Rng rng;
    for (auto &v : h) v = (float)(mean + stddev * rng.normal());
    return DeviceTensor::from_host_f32(h.data(), shape, dtype, device);
}
Result<DeviceTensor> init_uniform(const Shape &shape, double lo, double hi, DType dtype, const Device &device) {
    if (shape.numel() < 0) return err(HX_ERR_INVALID_DIMENSION, "negative dimension in shape " + shape_str(shape));
    std::vector<float> h((size_t)shape.numel());
    Rng rng;
    for (auto &v : h) v = (float)(lo + (hi - lo) * rng.uniform01());
    return DeviceTensor::from_host_f32(h.data(), shape, dtype, device);
}
Result<DeviceTensor> init_bernoulli(const Shape &shape, double p, DType dtype, const Device &device) {
    if (shape.numel() < 0) return err(HX_ERR_INVALID_DIMENSION, "negative dimension in shape " + shape_str(shape));
    std::vector<float> h((size_t)shape.numel());
    Rng rng;
    for (auto &v : h) v = rng.uniform01() < p ? 1.f : 0.f;
    return DeviceTensor::from_host_f32(h.data(), shape, dtype, device);
}
static Result<DeviceTensor> init_const(const Shape &shape, float value, DType dtype, const Device &device) {
    std::vector<float> h((size_t)shape.numel(), value);
    return DeviceTensor::from_host_f32(h.data(), shape, dtype, device);
}

#define HELIX_ASSIGN(dst, expr)                   \
    do {                                          \
        auto r__ = (expr);                        \
        if (!r__.ok()) return r__.error();        \
        dst = std::move(r__.value());             \
    } while (0)

// Splits an input of shape [.., d] into (rows, d); the reference modules take [L, d] and [B, L, d].
static Result<Unit> rows_of(const DeviceTensor &x, int64_t last, const char *who, int64_t *rows) {
    if (x.ndim() < 2 || x.ndim() > 3)
        return err(HX_ERR_SHAPE_MISMATCH, std::string(who) + ": expected a 2-D or 3-D input, got " + shape_str(x.shape()));
    if (x.shape().dim(x.ndim() - 1) != last)
        return err(HX_ERR_SHAPE_MISMATCH, std::string(who) + ": last dimension is " +
                                              std::to_string(x.shape().dim(x.ndim() - 1)) + ", expected " + std::to_string(last));
    *rows = x.numel() / last;
    return Unit{};
}

// ------------------------------------------------------------------------------------------ Linear
Result<std::unique_ptr<Linear>> Linear::create(int64_t in_f, int64_t out_f, bool bias, DType dtype, const Device &device) {
    if (in_f <= 0 || out_f <= 0) return err(HX_ERR_INVALID_DIMENSION, "Linear: features must be positive");
    auto m = std::unique_ptr<Linear>(new Linear());
    m->device_ = device;
    m->has_bias = bias;
    HELIX_ASSIGN(m->weight, init_normal(Shape({out_f, in_f}), std::sqrt(2.0 / (double)in_f), dtype, device));
    if (bias) HELIX_ASSIGN(m->bias, DeviceTensor::zeros(Shape({out_f}), DType::F32, device));
    return std::move(m);
}

Result<DeviceTensor> Linear::forward(const DeviceTensor &x) const {
    const int64_t in_f = weight.shape().dim(1), out_f = weight.shape().dim(0);
    int64_t rows = 0;
    HELIX_TRY(rows_of(x, in_f, "Linear", &rows));
    if (!(x.device() == device_)) return err(HX_ERR_DEVICE_MISMATCH, "Linear: input on " + x.device().to_string());
    if (x.dtype() != weight.dtype()) return err(HX_ERR_DTYPE_MISMATCH, "Linear: input and weight dtypes differ");
    std::vector<int64_t> od = x.shape().as_slice();
    od.back() = out_f;
    DeviceTensor y;
    HELIX_ASSIGN(y, DeviceTensor::empty(Shape(od), x.dtype(), device_));
    const float *b = has_bias ? static_cast<const float *>(bias.data()) : nullptr;
    if (x.dtype() == DType::BF16 && in_f % 8 == 0)
        HELIX_TRY_ABI(hx_gemm_bf16(x.data(), in_f, weight.data(), in_f, b, y.data(), out_f, HX_BF16, (int)rows, (int)out_f,
                                   (int)in_f, 0, nullptr));
    else
        HELIX_TRY_ABI(hx_gemm_simt(x.data(), in_f, weight.data(), in_f, b, y.data(), out_f, (int)x.dtype(), (int)x.dtype(),
                                   (int)rows, (int)out_f, (int)in_f, 0, nullptr));
    return y;
}
std::vector<const DeviceTensor *> Linear::parameters() const {
    if (has_bias) return {&weight, &bias};
    return {&weight};
}
std::vector<DeviceTensor *> Linear::parameters_mut() {
    if (has_bias) return {&weight, &bias};
    return {&weight};
}

// ------------------------------------------------------------------------------------------ RMSNorm
Result<std::unique_ptr<RMSNorm>> RMSNorm::create(int64_t d_model, float eps, const Device &device) {
    if (d_model <= 0) return err(HX_ERR_INVALID_DIMENSION, "RMSNorm: d_model must be positive");
    auto m = std::unique_ptr<RMSNorm>(new RMSNorm());
    m->device_ = device;
    m->eps = eps;
    HELIX_ASSIGN(m->weight, init_const(Shape({d_model}), 1.0f, DType::F32, device));
    return std::move(m);
}
Result<DeviceTensor> RMSNorm::forward(const DeviceTensor &x) const {
    const int64_t d = weight.shape().dim(0);
    int64_t rows = 0;
    HELIX_TRY(rows_of(x, d, "RMSNorm", &rows));
    if (x.dtype() == DType::U8) return err(HX_ERR_DTYPE_MISMATCH, "RMSNorm: U8 input");
    DeviceTensor y;
    HELIX_ASSIGN(y, DeviceTensor::empty(x.shape(), x.dtype(), device_));
    HELIX_TRY_ABI(hx_rmsnorm_fwd(x.data(), (int)x.dtype(), nullptr, static_cast<const float *>(weight.data()), y.data(),
                                 (int)x.dtype(), rows, (int)d, eps, nullptr));
    return y;
}

// ------------------------------------------------------------------------------------------ S4Block
Result<std::unique_ptr<S4Block>> S4Block::create(int64_t d_model, int64_t d_state, const Device &device) {
    if (d_model <= 0 || d_state <= 0 || d_state > 256)
        return err(HX_ERR_INVALID_DIMENSION, "S4Block: need d_model > 0 and 0 < d_state <= 256");
    auto m = std::unique_ptr<S4Block>(new S4Block());
    m->device_ = device;
    m->d_model = d_model;
    m->d_state = d_state;
    const DType f = DType::F32;
    // crates/nn/src/ssm.rs:39-100: A_real zeros, A_imag ~ N(0,1), B ~ N(0,0.1) [N,M], C ~ N(0,0.1) [M,N],
    // D zeros, delta ~ U(0.001, 0.1), Lambda ~ N(0,1)
    HELIX_ASSIGN(m->A_real, DeviceTensor::zeros(Shape({d_state}), f, device));
    HELIX_ASSIGN(m->A_imag, init_normal(Shape({d_state}), 1.0, f, device));
    HELIX_ASSIGN(m->B, init_normal(Shape({d_state, d_model}), 0.1, f, device));
    HELIX_ASSIGN(m->C, init_normal(Shape({d_model, d_state}), 0.1, f, device));
    HELIX_ASSIGN(m->D, DeviceTensor::zeros(Shape({d_model}), f, device));
    HELIX_ASSIGN(m->delta, init_uniform(Shape({d_model}), 0.001, 0.1, f, device));
    HELIX_ASSIGN(m->Lambda, init_normal(Shape({d_state}), 1.0, f, device));
    // per-channel diagonal form: A[d,n] = -(n+1)/2, B and C ~ N(0, 1/N)
    {
        std::vector<float> a((size_t)(d_model * d_state));
        for (int64_t d = 0; d < d_model; ++d)
            for (int64_t n = 0; n < d_state; ++n) a[(size_t)(d * d_state + n)] = -0.5f * (float)(n + 1);
        HELIX_ASSIGN(m->A_diag, DeviceTensor::from_host_f32(a.data(), Shape({d_model, d_state}), f, device));
    }
    HELIX_ASSIGN(m->B_diag, init_normal(Shape({d_model, d_state}), std::sqrt(1.0 / (double)d_state), f, device));
    HELIX_ASSIGN(m->C_diag, init_normal(Shape({d_model, d_state}), std::sqrt(1.0 / (double)d_state), f, device));
    return std::move(m);
}

Result<DeviceTensor> S4Block::forward_ssm(const DeviceTensor &u) const {
    // crates/nn/src/ssm.rs:138-147: dim 0 must equal d_model
    if (u.ndim() != 2) return err(HX_ERR_SHAPE_MISMATCH, "S4Block::forward_ssm: expected [d_model, seq_len], got " + shape_str(u.shape()));
    if (u.shape().dim(0) != d_model)
        return TensorError{HX_ERR_SHAPE_MISMATCH, "S4Block::forward_ssm: expected [" + std::to_string(d_model) + "], got [" +
                                                      std::to_string(u.shape().dim(0)) + "]"};
    if (u.dtype() != DType::F32) return err(HX_ERR_DTYPE_MISMATCH, "S4Block::forward_ssm takes f32");
    const int64_t L = u.shape().dim(1);
    // the reference labels the result [d_model, L] although its buffer is time-major; here the shape says what
    // the buffer holds: [L, d_model]
    DeviceTensor y, ws;
    HELIX_ASSIGN(y, DeviceTensor::empty(Shape({L, d_model}), DType::F32, device_));
    const size_t wb = hx_s4_ref_workspace_bytes((int)L, (int)d_state);
    HELIX_ASSIGN(ws, DeviceTensor::empty(Shape({(int64_t)wb}), DType::U8, device_));
    auto f = [](const DeviceTensor &t) { return static_cast<const float *>(t.data()); };
    HELIX_TRY_ABI(hx_s4_ref_forward_ssm(f(u), f(A_real), f(A_imag), f(B), f(C), f(D), 0.1f, static_cast<float *>(y.data()),
                                        (int)d_model, (int)L, (int)d_state, ws.data(), wb, nullptr));
    HELIX_TRY_ABI(hx_stream_synchronize(nullptr));  // ws is released on return
    return y;
}

Result<DeviceTensor> S4Block::forward(const DeviceTensor &u) const {
    int64_t rows = 0;
    HELIX_TRY(rows_of(u, d_model, "S4Block", &rows));
    if (u.dtype() == DType::U8) return err(HX_ERR_DTYPE_MISMATCH, "S4Block: U8 input");
    const int64_t L = u.shape().dim(u.ndim() - 2), Bsz = rows / L;
    DeviceTensor y;
    HELIX_ASSIGN(y, DeviceTensor::empty(u.shape(), u.dtype(), device_));
    auto f = [](const DeviceTensor &t) { return static_cast<const float *>(t.data()); };
    HELIX_TRY_ABI(hx_s4_diag_fwd(u.data(), f(A_diag), f(B_diag), f(C_diag), f(delta), f(D), y.data(), (int)Bsz, (int)L,
                                 (int)d_model, (int)d_state, (int)u.dtype(), nullptr));
    return y;
}
std::vector<const DeviceTensor *> S4Block::parameters() const {
    return {&A_real, &A_imag, &B, &C, &D, &delta, &Lambda, &A_diag, &B_diag, &C_diag};
}
std::vector<DeviceTensor *> S4Block::parameters_mut() {
    return {&A_real, &A_imag, &B, &C, &D, &delta, &Lambda, &A_diag, &B_diag, &C_diag};
}

// ------------------------------------------------------------------------------------------ MambaBlock
Result<std::unique_ptr<MambaBlock>> MambaBlock::create(int64_t d_model, int64_t d_state, int64_t d_conv, int64_t expand,
                                                       DType dtype, const Device &device) {
    if (d_model <= 0 || d_state <= 0 || d_state > 256 || expand <= 0)
        return err(HX_ERR_INVALID_DIMENSION, "MambaBlock: need d_model > 0, 0 < d_state <= 256, expand > 0");
    if (d_conv < 1 || d_conv > 4) return err(HX_ERR_INVALID_DIMENSION, "MambaBlock: d_conv must be in [1, 4]");
    if (dtype == DType::U8) return err(HX_ERR_DTYPE_MISMATCH, "MambaBlock: dtype must be F32 or BF16");
    auto m = std::unique_ptr<MambaBlock>(new MambaBlock());
    m->device_ = device;
    m->d_model = d_model; m->d_state = d_state; m->d_conv = d_conv; m->expand = expand;
    m->d_inner = d_model * expand;
    m->dt_rank = (d_model + 15) / 16;
    m->dtype = dtype;
    const int64_t E = m->d_inner, R = m->dt_rank, N = d_state;
    const DType f = DType::F32;
    HELIX_ASSIGN(m->W_in, init_normal(Shape({2 * E, d_model}), std::sqrt(2.0 / (double)d_model), dtype, device));
    HELIX_ASSIGN(m->conv_w, init_uniform(Shape({E, d_conv}), -0.5, 0.5, f, device));
    HELIX_ASSIGN(m->conv_b, DeviceTensor::zeros(Shape({E}), f, device));
    HELIX_ASSIGN(m->W_x, init_normal(Shape({R + 2 * N, E}), std::sqrt(2.0 / (double)E), dtype, device));
    HELIX_ASSIGN(m->W_dt, init_normal(Shape({E, R}), std::sqrt(2.0 / (double)R), dtype, device));
    {
        // dt bias = softplus^-1(dt0), dt0 log-uniform in [1e-3, 1e-1]
        std::vector<float> b((size_t)E);
        Rng rng;
        for (auto &v : b) {
            const double dt0 = std::exp(std::log(1e-3) + rng.uniform01() * (std::log(1e-1) - std::log(1e-3)));
            v = (float)(dt0 + std::log(-std::expm1(-dt0)));
        }
        HELIX_ASSIGN(m->b_dt, DeviceTensor::from_host_f32(b.data(), Shape({E}), f, device));
    }
    {
        // A = -exp(A_log), A_log[d, n] = log(n + 1)
        std::vector<float> a((size_t)(E * N));
        for (int64_t d = 0; d < E; ++d)
            for (int64_t n = 0; n < N; ++n) a[(size_t)(d * N + n)] = -std::exp(std::log((float)(n + 1)));
        HELIX_ASSIGN(m->A, DeviceTensor::from_host_f32(a.data(), Shape({E, N}), f, device));
    }
    HELIX_ASSIGN(m->D, init_const(Shape({E}), 1.0f, f, device));
    HELIX_ASSIGN(m->W_out, init_normal(Shape({d_model, E}), std::sqrt(2.0 / (double)E), dtype, device));
    HELIX_TRY(m->parameters_updated());
    return std::move(m);
}

Result<Unit> MambaBlock::parameters_updated() {
    int32_t g = 0;
    HELIX_TRY(use_device(device_));
    HELIX_TRY_ABI(hx_scan_check_geometric(static_cast<const float *>(A.data()), (int)d_inner, (int)d_state, &g));
    a_geometric = g != 0;
    return Unit{};
}

static hx_mamba_block_args block_args(const MambaBlock &m, int64_t batch, int64_t seq_len) {
    hx_mamba_block_args a;
    std::memset(&a, 0, sizeof(a));
    a.batch = (int)batch; a.seq_len = (int)seq_len;
    a.d_model = (int)m.d_model; a.d_inner = (int)m.d_inner; a.d_state = (int)m.d_state; a.d_conv = (int)m.d_conv;
    a.dt_rank = (int)m.dt_rank;
    a.io_dtype = (int)m.dtype;
    a.W_in = m.W_in.data(); a.W_x = m.W_x.data(); a.W_dt = m.W_dt.data(); a.W_out = m.W_out.data();
    a.conv_w = static_cast<const float *>(m.conv_w.data());
    a.conv_b = static_cast<const float *>(m.conv_b.data());
    a.b_dt = static_cast<const float *>(m.b_dt.data());
    a.A = static_cast<const float *>(m.A.data());
    a.Dskip = static_cast<const float *>(m.D.data());
    a.scan_variant = HX_SCAN_AUTO;
    a.a_geometric = m.a_geometric ? 1 : 0;
    return a;
}

size_t MambaBlock::workspace_bytes(int64_t batch, int64_t seq_len) const {
    hx_mamba_block_args a = block_args(*this, batch, seq_len);
    size_t n = 0;
    hx_mamba_block_workspace_bytes(&a, &n);
    return n;
}

Result<Unit> MambaBlock::forward_into(const void *x, void *out, int64_t batch, int64_t seq_len, void *workspace,
                                      size_t ws_bytes, void *stream, void **stage_events, float *h_last,
                                      void *conv_state, float *residual) const {
    hx_mamba_block_args a = block_args(*this, batch, seq_len);
    a.x = x; a.out = out; a.workspace = workspace; a.workspace_bytes = ws_bytes;
    a.stage_events = stage_events;
    a.h_last = h_last; a.conv_state = conv_state; a.residual = residual;
    HELIX_TRY_ABI(hx_mamba_block_fwd(&a, stream));
    return Unit{};
}

static hx_mamba_step_args step_args(const MambaBlock &m, int64_t batch) {
    hx_mamba_step_args a;
    std::memset(&a, 0, sizeof(a));
    a.batch = (int)batch;
    a.d_model = (int)m.d_model; a.d_inner = (int)m.d_inner; a.d_state = (int)m.d_state; a.d_conv = (int)m.d_conv;
    a.dt_rank = (int)m.dt_rank;
    a.io_dtype = (int)m.dtype;
    a.W_in = m.W_in.data(); a.W_x = m.W_x.data(); a.W_dt = m.W_dt.data(); a.W_out = m.W_out.data();
    a.conv_w = static_cast<const float *>(m.conv_w.data());
    a.conv_b = static_cast<const float *>(m.conv_b.data());
    a.b_dt = static_cast<const float *>(m.b_dt.data());
    a.A = static_cast<const float *>(m.A.data());
    a.Dskip = static_cast<const float *>(m.D.data());
    return a;
}

size_t MambaBlock::step_workspace_bytes(int64_t batch) const {
    hx_mamba_step_args a = step_args(*this, batch);
    size_t n = 0;
    hx_mamba_step_workspace_bytes(&a, &n);
    return n;
}

Result<Unit> MambaBlock::step_into(const void *x, void *out, int64_t batch, float *h, void *conv_state, void *workspace,
                                   size_t ws_bytes, void *stream, float *residual, const float *norm_w, float norm_eps) const {
    hx_mamba_step_args a = step_args(*this, batch);
    a.x = x; a.out = out; a.h = h; a.conv_state = conv_state;
    a.workspace = workspace; a.workspace_bytes = ws_bytes;
    a.residual = residual; a.norm_w = norm_w; a.norm_eps = norm_eps;
    HELIX_TRY_ABI(hx_mamba_block_step(&a, stream));
    return Unit{};
}

Result<DeviceTensor> MambaBlock::forward(const DeviceTensor &x) const {
    int64_t rows = 0;
    HELIX_TRY(rows_of(x, d_model, "MambaBlock", &rows));
    if (!(x.device() == device_)) return err(HX_ERR_DEVICE_MISMATCH, "MambaBlock: input on " + x.device().to_string());
    if (x.dtype() != dtype) return err(HX_ERR_DTYPE_MISMATCH, "MambaBlock: input dtype differs from the block's");
    const int64_t L = x.shape().dim(x.ndim() - 2), Bsz = rows / L;
    HELIX_TRY(use_device(device_));
    DeviceTensor y, ws;
    HELIX_ASSIGN(y, DeviceTensor::empty(x.shape(), dtype, device_));
    if (rows == 0) return y;
    const size_t wb = workspace_bytes(Bsz, L);
    HELIX_ASSIGN(ws, DeviceTensor::empty(Shape({(int64_t)wb}), DType::U8, device_));
    HELIX_TRY(forward_into(x.data(), y.data(), Bsz, L, ws.data(), wb, nullptr));
    HELIX_TRY_ABI(hx_stream_synchronize(nullptr));  // the workspace is released on return
    return y;
}
std::vector<const DeviceTensor *> MambaBlock::parameters() const {
    return {&W_in, &conv_w, &conv_b, &W_x, &W_dt, &b_dt, &A, &D, &W_out};
}
std::vector<DeviceTensor *> MambaBlock::parameters_mut() {
    return {&W_in, &conv_w, &conv_b, &W_x, &W_dt, &b_dt, &A, &D, &W_out};
}

// ------------------------------------------------------------------------------------------ Sequential
Result<DeviceTensor> Sequential::forward(const DeviceTensor &input) const {
    auto cur = input.clone();  // `let mut output = input.clone()` (crates/nn/src/lib.rs:605)
    if (!cur.ok()) return cur.error();
    DeviceTensor t = std::move(cur.value());
    for (const auto &m : modules_) {
        auto r = m->forward(t);
        if (!r.ok()) return r.error();
        t = std::move(r.value());
    }
    return t;
}
std::vector<const DeviceTensor *> Sequential::parameters() const {
    std::vector<const DeviceTensor *> p;
    for (const auto &m : modules_)
        for (auto *t : static_cast<const Module *>(m.get())->parameters()) p.push_back(t);
    return p;
}
std::vector<DeviceTensor *> Sequential::parameters_mut() {
    std::vector<DeviceTensor *> p;
    for (auto &m : modules_)
        for (auto *t : m->parameters_mut()) p.push_back(t);
    return p;
}
Result<Unit> Sequential::parameters_updated() {
    for (auto &m : modules_) HELIX_TRY(m->parameters_updated());
    return Unit{};
}

// ------------------------------------------------------------------------------------------ ByteLM
struct ByteLM::Buffers {
    int64_t batch = 0, seq_len = 0;
    DeviceTensor tokens, resid, normed, block_out, logits, workspace;
};

// Decode state of one batch: per layer the scan state and the conv window, the step's own buffers, and the
// captured graph of one step over those buffers.
struct ByteLM::Decode {
    int64_t batch = 0;
    std::vector<DeviceTensor> h, conv;  // per layer: [B, E, N] fp32, [B, 3, E] model dtype
    DeviceTensor tokens, resid, normed, block_out, logits, workspace;
    cudaStream_t capture_stream = nullptr;
    cudaGraphExec_t exec = nullptr;
    int64_t steps = 0;
    ~Decode() {
        if (exec) cudaGraphExecDestroy(exec);
        if (capture_stream) cudaStreamDestroy(capture_stream);
    }
};

// Event-based stage timing: per forward, events[0] before the embedding, then per layer one event before the
// norm and the block's seven, then events before the final norm, before the head and after it.
struct ByteLM::Profile {
    std::vector<cudaEvent_t> ev;       // events of the forwards not read yet, in recording order
    std::vector<int> cls;              // stage class that STARTS at each event (-1: end marker)
    std::vector<cudaEvent_t> pool;
    size_t used = 0;
    int forwards = 0;
    cudaEvent_t next() {
        if (used == pool.size()) {
            cudaEvent_t e;
            cudaEventCreate(&e);
            pool.push_back(e);
        }
        return pool[used++];
    }
    ~Profile() {
        for (auto e : pool) cudaEventDestroy(e);
    }
};

// Captured forwards, keyed by what a graph bakes in: the caller's two pointers, the shape and whether the decode
// state is kept.  `seen` counts plain runs of a key: the first call runs as plain launches (it also sets the
// kernels' attributes), the second is captured.
struct ByteLM::FwdGraphs {
    struct Entry {
        const void *tok = nullptr;
        void *logits = nullptr;
        int64_t batch = 0, seq_len = 0;
        bool keep = false;
        int seen = 0;
        cudaGraphExec_t exec = nullptr;
        uint64_t used = 0;
    };
    std::vector<Entry> entries;
    cudaStream_t capture_stream = nullptr;
    uint64_t tick = 0;
    void clear() {
        for (auto &e : entries)
            if (e.exec) cudaGraphExecDestroy(e.exec);
        entries.clear();
    }
    ~FwdGraphs() {
        clear();
        if (capture_stream) cudaStreamDestroy(capture_stream);
    }
};

void ByteLM::set_forward_graph(bool enable) {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    forward_graph_ = enable;
    if (!enable && fwd_) fwd_->clear();
}

ByteLM::~ByteLM() {
    delete fwd_;
    delete buf_;
    delete prof_;
    delete dec_;
}

Result<Unit> ByteLM::set_profile(bool enable) {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    delete prof_;
    prof_ = enable ? new Profile() : nullptr;
    return Unit{};
}

Result<Unit> ByteLM::read_profile(float *ms9, int *forwards) {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    if (!ms9 || !forwards) return err(HX_ERR_INVALID_INPUT, "read_profile: NULL argument");
    for (int i = 0; i < 9; ++i) ms9[i] = 0.f;
    *forwards = 0;
    if (!prof_) return Unit{};
    HELIX_TRY(use_device(device_));
    if (cudaDeviceSynchronize() != cudaSuccess) return err(HX_ERR_BACKEND, "cudaDeviceSynchronize failed");
    for (size_t i = 0; i + 1 < prof_->ev.size(); ++i) {
        if (prof_->cls[i] < 0) continue;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, prof_->ev[i], prof_->ev[i + 1]);
        ms9[prof_->cls[i]] += ms;
    }
    *forwards = prof_->forwards;
    prof_->ev.clear();
    prof_->cls.clear();
    prof_->used = 0;
    prof_->forwards = 0;
    return Unit{};
}

Result<std::unique_ptr<ByteLM>> ByteLM::create(int64_t n_layer, int64_t d_model, int64_t d_state, int64_t d_conv,
                                               int64_t expand, DType dtype, const Device &device) {
    if (n_layer <= 0) return err(HX_ERR_INVALID_DIMENSION, "ByteLM: n_layer must be positive");
    auto m = std::unique_ptr<ByteLM>(new ByteLM());
    m->device_ = device;
    m->d_model = d_model;
    m->dtype = dtype;
    HELIX_ASSIGN(m->embedding, init_normal(Shape({256, d_model}), 0.02, dtype, device));
    for (int64_t l = 0; l < n_layer; ++l) {
        auto n = RMSNorm::create(d_model, m->eps, device);
        if (!n.ok()) return n.error();
        m->norms.push_back(std::move(n.value()));
        auto b = MambaBlock::create(d_model, d_state, d_conv, expand, dtype, device);
        if (!b.ok()) return b.error();
        // serving-style init: N(0, 0.02) for the projections
        for (DeviceTensor *w : {&b.value()->W_in, &b.value()->W_x, &b.value()->W_dt, &b.value()->W_out})
            HELIX_ASSIGN(*w, init_normal(w->shape(), 0.02, dtype, device));
        m->blocks.push_back(std::move(b.value()));
    }
    HELIX_ASSIGN(m->norm_f, init_const(Shape({d_model}), 1.0f, DType::F32, device));
    return std::move(m);
}

Result<Unit> ByteLM::parameters_updated() {
    {
        std::lock_guard<std::recursive_mutex> lock(mu_);
        if (fwd_) fwd_->clear();  // a captured forward bakes in the kernel choice the parameters imply
    }
    for (auto &b : blocks) HELIX_TRY(b->parameters_updated());
    return Unit{};
}

Result<Unit> ByteLM::ensure_buffers(int64_t batch, int64_t seq_len) {
    if (buf_ && buf_->batch == batch && buf_->seq_len == seq_len) return Unit{};
    delete buf_;
    buf_ = new Buffers();
    const int64_t T = batch * seq_len;
    HELIX_ASSIGN(buf_->tokens, DeviceTensor::empty(Shape({T}), DType::U8, device_));
    HELIX_ASSIGN(buf_->resid, DeviceTensor::empty(Shape({T, d_model}), DType::F32, device_));
    HELIX_ASSIGN(buf_->normed, DeviceTensor::empty(Shape({T, d_model}), dtype, device_));
    HELIX_ASSIGN(buf_->block_out, DeviceTensor::empty(Shape({T, d_model}), dtype, device_));
    HELIX_ASSIGN(buf_->logits, DeviceTensor::empty(Shape({T, 256}), dtype, device_));
    const size_t wb = blocks[0]->workspace_bytes(batch, seq_len);
    HELIX_ASSIGN(buf_->workspace, DeviceTensor::empty(Shape({(int64_t)wb}), DType::U8, device_));
    buf_->batch = batch;
    buf_->seq_len = seq_len;
    return Unit{};
}

int64_t ByteLM::launches_per_forward() const {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    // embedding + per layer (norm + the block's 5 or 6 kernels) + final norm + logits GEMM
    int32_t per_block = 6;
    if (buf_ && buf_->batch > 0 && !blocks.empty()) {
        hx_mamba_block_args a = block_args(*blocks[0], buf_->batch, buf_->seq_len);
        hx_mamba_block_kernel_launches(&a, &per_block);
    }
    return 1 + (int64_t)blocks.size() * (1 + per_block) + 2;
}

Result<Unit> ByteLM::forward_device(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream) {
    return run_layers(tokens_dev, logits_dev, batch, seq_len, stream, false);
}

Result<Unit> ByteLM::prefill_device(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream) {
    return run_layers(tokens_dev, logits_dev, batch, seq_len, stream, true);
}

Result<Unit> ByteLM::ensure_decode(int64_t batch) {
    if (dec_ && dec_->batch == batch) return Unit{};
    delete dec_;
    dec_ = new Decode();
    const MambaBlock &b0 = *blocks[0];
    for (size_t l = 0; l < blocks.size(); ++l) {
        DeviceTensor h, c;
        HELIX_ASSIGN(h, DeviceTensor::zeros(Shape({batch, b0.d_inner, b0.d_state}), DType::F32, device_));
        HELIX_ASSIGN(c, DeviceTensor::zeros(Shape({batch, 3, b0.d_inner}), dtype, device_));
        dec_->h.push_back(std::move(h));
        dec_->conv.push_back(std::move(c));
    }
    HELIX_ASSIGN(dec_->tokens, DeviceTensor::empty(Shape({batch}), DType::U8, device_));
    HELIX_ASSIGN(dec_->resid, DeviceTensor::empty(Shape({batch, d_model}), DType::F32, device_));
    HELIX_ASSIGN(dec_->normed, DeviceTensor::empty(Shape({batch, d_model}), dtype, device_));
    HELIX_ASSIGN(dec_->block_out, DeviceTensor::empty(Shape({batch, d_model}), dtype, device_));
    HELIX_ASSIGN(dec_->logits, DeviceTensor::empty(Shape({batch, 256}), dtype, device_));
    HELIX_ASSIGN(dec_->workspace, DeviceTensor::empty(Shape({(int64_t)b0.step_workspace_bytes(batch)}), DType::U8, device_));
    dec_->batch = batch;
    return Unit{};
}

// One step over the module's own buffers (dec_->tokens in, dec_->logits out): what the graph captures.
Result<Unit> ByteLM::enqueue_step(void *stream) {
    const int64_t B = dec_->batch;
    float *resid = static_cast<float *>(dec_->resid.data());
    HELIX_TRY_ABI(hx_embedding_fwd(static_cast<const uint8_t *>(dec_->tokens.data()), embedding.data(), (int)dtype, resid, HX_F32,
                                   B, (int)d_model, stream));
    for (size_t l = 0; l < blocks.size(); ++l) {
        // residual form: the norm runs inside the step (inside its in_proj kernel on the bf16 path) and the block
        // output is added into the stream by out_proj
        HELIX_TRY(blocks[l]->step_into(nullptr, dec_->block_out.data(), B, static_cast<float *>(dec_->h[l].data()),
                                       dec_->conv[l].data(), dec_->workspace.data(), (size_t)dec_->workspace.numel(), stream,
                                       resid, static_cast<const float *>(norms[l]->weight.data()), eps));
    }
    HELIX_TRY_ABI(hx_rmsnorm_fwd(nullptr, (int)dtype, resid, static_cast<const float *>(norm_f.data()),
                                 dec_->normed.data(), (int)dtype, B, (int)d_model, eps, stream));
    if (dtype == DType::BF16 && d_model % 8 == 0)
        HELIX_TRY_ABI(hx_gemm_bf16(dec_->normed.data(), d_model, embedding.data(), d_model, nullptr, dec_->logits.data(), 256,
                                   HX_BF16, (int)B, 256, (int)d_model, 0, stream));
    else
        HELIX_TRY_ABI(hx_gemm_simt(dec_->normed.data(), d_model, embedding.data(), d_model, nullptr, dec_->logits.data(), 256,
                                   (int)dtype, (int)dtype, (int)B, 256, (int)d_model, 0, stream));
    return Unit{};
}

int64_t ByteLM::launches_per_decode_step() const {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    // embedding + per layer (fused: in_proj with norm and conv step, x_proj, state step, out_proj with the add;
    // otherwise: norm, in_proj, conv step, x_proj, state step, out_proj, residual add) + final norm + head
    const int64_t batch = dec_ ? dec_->batch : 1;
    const int64_t per_layer = (!blocks.empty() && blocks[0]->step_is_fused(batch)) ? 4 : 7;
    return 1 + (int64_t)blocks.size() * per_layer + 2;
}

Result<Unit> ByteLM::decode_step_device(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, void *stream) {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    if (!tokens_dev || !logits_dev) return err(HX_ERR_INVALID_INPUT, "ByteLM::decode_step_device: NULL buffer");
    if (!dec_ || dec_->batch != batch)
        return err(HX_ERR_INVALID_INPUT, "ByteLM::decode_step_device: no prefill state for batch " + std::to_string(batch));
    HELIX_TRY(use_device(device_));
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemcpyAsync(dec_->tokens.data(), tokens_dev, (size_t)batch, cudaMemcpyDeviceToDevice, st) != cudaSuccess)
        return err(HX_ERR_BACKEND, "ByteLM::decode_step_device: token copy failed");
    // The first step runs as plain launches (it also sets the kernels' attributes); the second one is captured
    // on a private stream (capture is not allowed on the legacy default stream) and every later step replays it.
    if (decode_graph_ && dec_->steps >= 1 && !dec_->exec) {
        if (!dec_->capture_stream && cudaStreamCreateWithFlags(&dec_->capture_stream, cudaStreamNonBlocking) != cudaSuccess)
            return err(HX_ERR_BACKEND, "ByteLM::decode_step_device: cannot create the capture stream");
        if (cudaStreamBeginCapture(dec_->capture_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
            return err(HX_ERR_BACKEND, "ByteLM::decode_step_device: cudaStreamBeginCapture failed");
        auto r = enqueue_step(dec_->capture_stream);
        cudaGraph_t graph = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(dec_->capture_stream, &graph);
        if (!r.ok()) {
            if (graph) cudaGraphDestroy(graph);
            return r.error();
        }
        if (ce != cudaSuccess || !graph) return err(HX_ERR_BACKEND, "ByteLM::decode_step_device: stream capture failed");
        const cudaError_t ie = cudaGraphInstantiate(&dec_->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ie != cudaSuccess) {
            dec_->exec = nullptr;
            return err(HX_ERR_BACKEND, "ByteLM::decode_step_device: cudaGraphInstantiate failed");
        }
    }
    if (decode_graph_ && dec_->exec) {
        if (cudaGraphLaunch(dec_->exec, st) != cudaSuccess) return err(HX_ERR_BACKEND, "ByteLM::decode_step_device: graph launch failed");
    } else {
        HELIX_TRY(enqueue_step(stream));
    }
    dec_->steps += 1;
    if (cudaMemcpyAsync(logits_dev, dec_->logits.data(), (size_t)batch * 256 * dtype_size(dtype), cudaMemcpyDeviceToDevice, st) !=
        cudaSuccess)
        return err(HX_ERR_BACKEND, "ByteLM::decode_step_device: logits copy failed");
    return Unit{};
}

Result<Unit> ByteLM::run_layers(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream,
                                bool keep_state) {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    if (batch <= 0 || seq_len <= 0) return err(HX_ERR_INVALID_DIMENSION, "ByteLM: batch and seq_len must be positive");
    HELIX_TRY(use_device(device_));
    const bool had_buffers = buf_ && buf_->batch == batch && buf_->seq_len == seq_len;
    HELIX_TRY(ensure_buffers(batch, seq_len));
    if (!had_buffers && fwd_) fwd_->clear();  // the graphs point into the old activation buffers
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing((cudaStream_t)stream, &cap);
    if (!forward_graph_ || prof_ || cap != cudaStreamCaptureStatusNone)
        return run_layers_plain(tokens_dev, logits_dev, batch, seq_len, stream, keep_state);
    if (keep_state) {
        const bool had_decode = dec_ && dec_->batch == batch;
        HELIX_TRY(ensure_decode(batch));  // allocate outside any capture
        if (!had_decode && fwd_) fwd_->clear();  // graphs that keep the state point into the old state buffers
        dec_->steps = 0;
    }
    if (!fwd_) fwd_ = new FwdGraphs();
    FwdGraphs::Entry *e = nullptr;
    for (auto &c : fwd_->entries)
        if (c.tok == tokens_dev && c.logits == logits_dev && c.batch == batch && c.seq_len == seq_len && c.keep == keep_state) e = &c;
    if (!e) {
        if (fwd_->entries.size() >= 4) {  // drop the least recently used
            size_t lru = 0;
            for (size_t i = 1; i < fwd_->entries.size(); ++i)
                if (fwd_->entries[i].used < fwd_->entries[lru].used) lru = i;
            if (fwd_->entries[lru].exec) cudaGraphExecDestroy(fwd_->entries[lru].exec);
            fwd_->entries.erase(fwd_->entries.begin() + lru);
        }
        FwdGraphs::Entry n;
        n.tok = tokens_dev; n.logits = logits_dev; n.batch = batch; n.seq_len = seq_len; n.keep = keep_state;
        fwd_->entries.push_back(n);
        e = &fwd_->entries.back();
    }
    e->used = ++fwd_->tick;
    if (!e->exec && e->seen >= 1) {
        if (!fwd_->capture_stream && cudaStreamCreateWithFlags(&fwd_->capture_stream, cudaStreamNonBlocking) != cudaSuccess)
            return err(HX_ERR_BACKEND, "ByteLM: cannot create the capture stream");
        if (cudaStreamBeginCapture(fwd_->capture_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
            return err(HX_ERR_BACKEND, "ByteLM: cudaStreamBeginCapture failed");
        auto r = run_layers_plain(tokens_dev, logits_dev, batch, seq_len, fwd_->capture_stream, keep_state);
        cudaGraph_t graph = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(fwd_->capture_stream, &graph);
        if (!r.ok()) {
            if (graph) cudaGraphDestroy(graph);
            return r.error();
        }
        if (ce != cudaSuccess || !graph) {
            cudaGetLastError();
            return err(HX_ERR_BACKEND, "ByteLM: stream capture of the forward failed");
        }
        const cudaError_t ie = cudaGraphInstantiate(&e->exec, graph, 0);
        cudaGraphDestroy(graph);
        if (ie != cudaSuccess) {
            e->exec = nullptr;
            cudaGetLastError();
            return err(HX_ERR_BACKEND, "ByteLM: cudaGraphInstantiate of the forward failed");
        }
    }
    if (e->exec) {
        if (cudaGraphLaunch(e->exec, (cudaStream_t)stream) != cudaSuccess) return err(HX_ERR_BACKEND, "ByteLM: graph launch failed");
        return Unit{};
    }
    e->seen += 1;
    return run_layers_plain(tokens_dev, logits_dev, batch, seq_len, stream, keep_state);
}

Result<Unit> ByteLM::run_layers_plain(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream,
                                      bool keep_state) {
    HELIX_TRY(ensure_buffers(batch, seq_len));
    if (keep_state) {
        HELIX_TRY(ensure_decode(batch));
        dec_->steps = 0;
    }
    const int64_t T = batch * seq_len;
    float *resid = static_cast<float *>(buf_->resid.data());
    auto mark = [&](int cls) {
        if (!prof_) return;
        cudaEvent_t e = prof_->next();
        cudaEventRecord(e, (cudaStream_t)stream);
        prof_->ev.push_back(e);
        prof_->cls.push_back(cls);
    };
    mark(0);
    // h = emb[tokens] (fp32 residual stream)
    HELIX_TRY_ABI(hx_embedding_fwd(tokens_dev, embedding.data(), (int)dtype, resid, HX_F32, T, (int)d_model, stream));
    for (size_t l = 0; l < blocks.size(); ++l) {
        // normed = rmsnorm(residual); the block adds its output into the residual stream itself (out_proj epilogue)
        mark(1);
        HELIX_TRY_ABI(hx_rmsnorm_fwd(nullptr, (int)dtype, resid, static_cast<const float *>(norms[l]->weight.data()),
                                     buf_->normed.data(), (int)dtype, T, (int)d_model, eps, stream));
        void *sev[7];
        void **sevp = nullptr;
        if (prof_) {
            for (int k = 0; k < 7; ++k) {
                cudaEvent_t e = prof_->next();
                sev[k] = e;
                prof_->ev.push_back(e);
                prof_->cls.push_back(k < 6 ? 2 + k : -1);  // in_proj, conv, x_proj, dt_proj, scan, out_proj, end
            }
            sevp = sev;
        }
        HELIX_TRY(blocks[l]->forward_into(buf_->normed.data(), buf_->block_out.data(), batch, seq_len, buf_->workspace.data(),
                                          (size_t)buf_->workspace.numel(), stream, sevp,
                                          keep_state ? static_cast<float *>(dec_->h[l].data()) : nullptr,
                                          keep_state ? dec_->conv[l].data() : nullptr, resid));
    }
    mark(1);
    HELIX_TRY_ABI(hx_rmsnorm_fwd(nullptr, (int)dtype, resid, static_cast<const float *>(norm_f.data()),
                                 buf_->normed.data(), (int)dtype, T, (int)d_model, eps, stream));
    mark(8);
    // tied head: logits = normed . emb^T
    if (dtype == DType::BF16 && d_model % 8 == 0)
        HELIX_TRY_ABI(hx_gemm_bf16(buf_->normed.data(), d_model, embedding.data(), d_model, nullptr, logits_dev, 256, HX_BF16,
                                   (int)T, 256, (int)d_model, 0, stream));
    else
        HELIX_TRY_ABI(hx_gemm_simt(buf_->normed.data(), d_model, embedding.data(), d_model, nullptr, logits_dev, 256, (int)dtype,
                                   (int)dtype, (int)T, 256, (int)d_model, 0, stream));
    mark(-1);
    if (prof_) prof_->forwards += 1;
    return Unit{};
}

Result<Unit> ByteLM::forward_host(const uint8_t *tokens_host, void *logits_host, int64_t batch, int64_t seq_len, void *stream) {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    if (!tokens_host || !logits_host) return err(HX_ERR_INVALID_INPUT, "ByteLM::forward_host: NULL buffer");
    HELIX_TRY(use_device(device_));
    HELIX_TRY(ensure_buffers(batch, seq_len));
    const int64_t T = batch * seq_len;
    HELIX_TRY_ABI(hx_memcpy_h2d(buf_->tokens.data(), tokens_host, (size_t)T, stream));
    HELIX_TRY(forward_device(static_cast<const uint8_t *>(buf_->tokens.data()), buf_->logits.data(), batch, seq_len, stream));
    HELIX_TRY_ABI(hx_memcpy_d2h(logits_host, buf_->logits.data(), (size_t)T * 256 * dtype_size(dtype), stream));
    return Unit{};
}

Result<DeviceTensor> ByteLM::forward(const DeviceTensor &tokens) const {
    std::lock_guard<std::recursive_mutex> lock(mu_);
    if (tokens.dtype() != DType::U8) return err(HX_ERR_DTYPE_MISMATCH, "ByteLM: tokens must be U8");
    if (tokens.ndim() != 2) return err(HX_ERR_SHAPE_MISMATCH, "ByteLM: expected tokens [batch, seq_len], got " + shape_str(tokens.shape()));
    const int64_t B = tokens.shape().dim(0), L = tokens.shape().dim(1);
    DeviceTensor logits;
    HELIX_ASSIGN(logits, DeviceTensor::empty(Shape({B, L, 256}), dtype, device_));
    if (B * L == 0) return logits;
    // forward() is const in the interface; the activation buffers are a cache
    HELIX_TRY(const_cast<ByteLM *>(this)->forward_device(static_cast<const uint8_t *>(tokens.data()), logits.data(), B, L, nullptr));
    HELIX_TRY_ABI(hx_device_check());  // synchronises; a device-side wait that ran out is a BackendError
    return logits;
}

std::vector<const DeviceTensor *> ByteLM::parameters() const {
    std::vector<const DeviceTensor *> p{&embedding};
    for (size_t l = 0; l < blocks.size(); ++l) {
        p.push_back(&norms[l]->weight);
        for (auto *t : blocks[l]->parameters()) p.push_back(t);
    }
    p.push_back(&norm_f);
    return p;
}
std::vector<DeviceTensor *> ByteLM::parameters_mut() {
    std::vector<DeviceTensor *> p{&embedding};
    for (size_t l = 0; l < blocks.size(); ++l) {
        p.push_back(&norms[l]->weight);
        for (auto *t : blocks[l]->parameters_mut()) p.push_back(t);
    }
    p.push_back(&norm_f);
    return p;
}

}  // namespace helix

// ============================================================================================ C handles

namespace {
hx_status fail_from(const helix::TensorError &e) { return hx::fail(e.code, "%s", e.message.c_str()); }
helix::Device dev_of(int device_id) { return helix::Device::cuda(device_id); }
}  // namespace

#define HX_RETURN_IF_ERR(res)                   \
    do {                                        \
        if (!(res).ok()) return fail_from((res).error()); \
    } while (0)

extern "C" {

void hx_manual_seed(uint64_t seed) { helix::manual_seed(seed); }

hx_status hx_tensor_from_host(const float *data, const int64_t *dims, int32_t ndim, int32_t dtype, int32_t device_id,
                              hx_tensor **out) {
    HX_REQUIRE(out && (dims || ndim == 0) && ndim >= 0 && ndim <= 8, HX_ERR_INVALID_INPUT, "hx_tensor_from_host: bad arguments");
    HX_REQUIRE(dtype == HX_F32 || dtype == HX_BF16, HX_ERR_DTYPE_MISMATCH, "hx_tensor_from_host: dtype must be F32 or BF16");
    helix::Shape shape(std::vector<int64_t>(dims, dims + ndim));
    auto r = helix::DeviceTensor::from_host_f32(data, shape, (helix::DType)dtype, dev_of(device_id));
    HX_RETURN_IF_ERR(r);
    *out = new hx_tensor{std::move(r.value())};
    return HX_OK;
}

hx_status hx_tensor_from_host_u8(const uint8_t *data, const int64_t *dims, int32_t ndim, int32_t device_id, hx_tensor **out) {
    HX_REQUIRE(out && (dims || ndim == 0) && ndim >= 0 && ndim <= 8, HX_ERR_INVALID_INPUT, "hx_tensor_from_host_u8: bad arguments");
    helix::Shape shape(std::vector<int64_t>(dims, dims + ndim));
    auto r = helix::DeviceTensor::from_host_u8(data, shape, dev_of(device_id));
    HX_RETURN_IF_ERR(r);
    *out = new hx_tensor{std::move(r.value())};
    return HX_OK;
}

hx_status hx_tensor_to_host(const hx_tensor *t, float *out, int64_t n) {
    HX_REQUIRE(t != nullptr, HX_ERR_INVALID_INPUT, "hx_tensor_to_host: tensor is NULL");
    auto r = t->t.to_host_f32(out, n);
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

hx_status hx_tensor_copy_from_host(hx_tensor *t, const float *data, int64_t n) {
    HX_REQUIRE(t != nullptr, HX_ERR_INVALID_INPUT, "hx_tensor_copy_from_host: tensor is NULL");
    auto r = t->t.copy_from_host_f32(data, n);
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

hx_status hx_tensor_info(const hx_tensor *t, int32_t *ndim, int64_t *dims8, int32_t *dtype, int32_t *device_id) {
    HX_REQUIRE(t != nullptr, HX_ERR_INVALID_INPUT, "hx_tensor_info: tensor is NULL");
    if (ndim) *ndim = (int32_t)t->t.ndim();
    if (dims8)
        for (size_t i = 0; i < t->t.ndim() && i < 8; ++i) dims8[i] = t->t.shape().dim(i);
    if (dtype) *dtype = (int32_t)t->t.dtype();
    if (device_id) *device_id = t->t.device().id;
    return HX_OK;
}

void *hx_tensor_data(const hx_tensor *t) { return t ? t->t.data() : nullptr; }

void hx_tensor_free(hx_tensor *t) { delete t; }

hx_status hx_mamba_block_new(int64_t d_model, int64_t d_state, int64_t d_conv, int64_t expand, int32_t dtype,
                             int32_t device_id, hx_module **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_mamba_block_new: out is NULL");
    auto r = helix::MambaBlock::create(d_model, d_state, d_conv, expand, (helix::DType)dtype, dev_of(device_id));
    HX_RETURN_IF_ERR(r);
    *out = new hx_module{std::move(r.value())};
    return HX_OK;
}

hx_status hx_s4_block_new(int64_t d_model, int64_t d_state, int32_t device_id, hx_module **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_s4_block_new: out is NULL");
    auto r = helix::S4Block::create(d_model, d_state, dev_of(device_id));
    HX_RETURN_IF_ERR(r);
    *out = new hx_module{std::move(r.value())};
    return HX_OK;
}

hx_status hx_linear_new(int64_t in_features, int64_t out_features, int32_t bias, int32_t dtype, int32_t device_id,
                        hx_module **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_linear_new: out is NULL");
    auto r = helix::Linear::create(in_features, out_features, bias != 0, (helix::DType)dtype, dev_of(device_id));
    HX_RETURN_IF_ERR(r);
    *out = new hx_module{std::move(r.value())};
    return HX_OK;
}

hx_status hx_rmsnorm_new(int64_t d_model, float eps, int32_t device_id, hx_module **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_rmsnorm_new: out is NULL");
    auto r = helix::RMSNorm::create(d_model, eps, dev_of(device_id));
    HX_RETURN_IF_ERR(r);
    *out = new hx_module{std::move(r.value())};
    return HX_OK;
}

hx_status hx_byte_lm_new(int64_t n_layer, int64_t d_model, int64_t d_state, int64_t d_conv, int64_t expand, int32_t dtype,
                         int32_t device_id, hx_module **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_new: out is NULL");
    auto r = helix::ByteLM::create(n_layer, d_model, d_state, d_conv, expand, (helix::DType)dtype, dev_of(device_id));
    HX_RETURN_IF_ERR(r);
    *out = new hx_module{std::move(r.value())};
    return HX_OK;
}

hx_status hx_module_forward(const hx_module *m, const hx_tensor *input, hx_tensor **out) {
    HX_REQUIRE(m && input && out, HX_ERR_INVALID_INPUT, "hx_module_forward: NULL argument");
    auto r = m->m->forward(input->t);
    HX_RETURN_IF_ERR(r);
    *out = new hx_tensor{std::move(r.value())};
    return HX_OK;
}

hx_status hx_s4_block_forward_ssm(const hx_module *m, const hx_tensor *input, hx_tensor **out) {
    HX_REQUIRE(m && input && out, HX_ERR_INVALID_INPUT, "hx_s4_block_forward_ssm: NULL argument");
    auto *s4 = dynamic_cast<const helix::S4Block *>(m->m.get());
    HX_REQUIRE(s4 != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "forward_ssm on a module that is not an S4Block");
    auto r = s4->forward_ssm(input->t);
    HX_RETURN_IF_ERR(r);
    *out = new hx_tensor{std::move(r.value())};
    return HX_OK;
}

hx_status hx_byte_lm_forward_host(hx_module *m, const uint8_t *tokens_host, void *logits_host, int64_t batch,
                                  int64_t seq_len, void *stream) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_forward_host: module is NULL");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "forward_host on a module that is not a ByteLM");
    auto r = lm->forward_host(tokens_host, logits_host, batch, seq_len, stream);
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

hx_status hx_byte_lm_forward_device(hx_module *m, const uint8_t *tokens_dev, void *logits_dev, int64_t batch,
                                    int64_t seq_len, void *stream) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_forward_device: module is NULL");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "forward_device on a module that is not a ByteLM");
    auto r = lm->forward_device(tokens_dev, logits_dev, batch, seq_len, stream);
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

hx_status hx_byte_lm_prefill_device(hx_module *m, const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len,
                                    void *stream) {
    HX_REQUIRE(m && tokens_dev && logits_dev, HX_ERR_INVALID_INPUT, "hx_byte_lm_prefill_device: NULL argument");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "prefill on a module that is not a ByteLM");
    auto r = lm->prefill_device(tokens_dev, logits_dev, batch, seq_len, stream);
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

hx_status hx_byte_lm_decode_step_device(hx_module *m, const uint8_t *tokens_dev, void *logits_dev, int64_t batch, void *stream) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_decode_step_device: module is NULL");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "decode step on a module that is not a ByteLM");
    auto r = lm->decode_step_device(tokens_dev, logits_dev, batch, stream);
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

hx_status hx_sequential_new(int32_t device_id, hx_module **out) {
    HX_REQUIRE(out != nullptr, HX_ERR_INVALID_INPUT, "hx_sequential_new: out is NULL");
    *out = new hx_module{std::unique_ptr<helix::Module>(new helix::Sequential(dev_of(device_id)))};
    return HX_OK;
}

hx_status hx_sequential_add(hx_module *seq, hx_module *child) {
    HX_REQUIRE(seq && child && seq != child, HX_ERR_INVALID_INPUT, "hx_sequential_add: bad arguments");
    auto *s = dynamic_cast<helix::Sequential *>(seq->m.get());
    HX_REQUIRE(s != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "hx_sequential_add on a module that is not a Sequential");
    HX_REQUIRE(child->m != nullptr, HX_ERR_INVALID_INPUT, "hx_sequential_add: the child handle is empty");
    HX_REQUIRE(child->m->device() == s->device(), HX_ERR_DEVICE_MISMATCH, "hx_sequential_add: child on another device");
    s->add(std::move(child->m));  // the Sequential owns the module now
    delete child;
    return HX_OK;
}

int32_t hx_sequential_len(const hx_module *seq) {
    auto *s = seq ? dynamic_cast<const helix::Sequential *>(seq->m.get()) : nullptr;
    return s ? (int32_t)s->len() : -1;
}

hx_status hx_byte_lm_forward_graph(hx_module *m, int32_t enable) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_forward_graph: module is NULL");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "forward graph on a module that is not a ByteLM");
    lm->set_forward_graph(enable != 0);
    return HX_OK;
}

hx_status hx_byte_lm_decode_graph(hx_module *m, int32_t enable) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_decode_graph: module is NULL");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "decode graph on a module that is not a ByteLM");
    lm->set_decode_graph(enable != 0);
    return HX_OK;
}

int64_t hx_byte_lm_launches_per_decode_step(const hx_module *m) {
    auto *lm = m ? dynamic_cast<const helix::ByteLM *>(m->m.get()) : nullptr;
    return lm ? lm->launches_per_decode_step() : 0;
}

hx_status hx_byte_lm_profile(hx_module *m, int32_t enable) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_profile: module is NULL");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "profile on a module that is not a ByteLM");
    auto r = lm->set_profile(enable != 0);
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

hx_status hx_byte_lm_profile_read(hx_module *m, float *ms9, int32_t *forwards) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_byte_lm_profile_read: module is NULL");
    auto *lm = dynamic_cast<helix::ByteLM *>(m->m.get());
    HX_REQUIRE(lm != nullptr, HX_ERR_UNSUPPORTED_OPERATION, "profile on a module that is not a ByteLM");
    int n = 0;
    auto r = lm->read_profile(ms9, &n);
    HX_RETURN_IF_ERR(r);
    if (forwards) *forwards = n;
    return HX_OK;
}

int64_t hx_byte_lm_launches_per_forward(const hx_module *m) {
    auto *lm = m ? dynamic_cast<const helix::ByteLM *>(m->m.get()) : nullptr;
    return lm ? lm->launches_per_forward() : 0;
}

int32_t hx_module_num_parameters(const hx_module *m) { return m ? (int32_t)m->m->parameters().size() : 0; }

hx_status hx_module_parameter(hx_module *m, int32_t index, hx_tensor **out) {
    HX_REQUIRE(m && out, HX_ERR_INVALID_INPUT, "hx_module_parameter: NULL argument");
    auto ps = m->m->parameters_mut();
    HX_REQUIRE(index >= 0 && index < (int32_t)ps.size(), HX_ERR_INVALID_DIMENSION, "parameter index %d out of %zu", index,
               ps.size());
    *out = new hx_tensor{*ps[(size_t)index]};  // shares the parameter's storage
    return HX_OK;
}

hx_status hx_module_parameters_updated(hx_module *m) {
    HX_REQUIRE(m != nullptr, HX_ERR_INVALID_INPUT, "hx_module_parameters_updated: module is NULL");
    auto r = m->m->parameters_updated();
    HX_RETURN_IF_ERR(r);
    return HX_OK;
}

const char *hx_module_name(const hx_module *m) { return m ? m->m->name() : ""; }

void hx_module_free(hx_module *m) { delete m; }

}  // extern "C"
