// C++ host layer above the C ABI: the reference's tensor/module interface for the state-space path,
// restated for device-resident tensors.
//
//   reference (Rust)                                         here (C++)
//   tensor_core::Device           device.rs:8-60             helix::Device
//   tensor_core::DType            dtype.rs:8-37              helix::DType (+ BF16)
//   tensor_core::Shape            shape.rs:8-97              helix::Shape
//   tensor_core::TensorError      error.rs:7-37              helix::TensorError (code = hx_status)
//   Result<T>                     error.rs:40                helix::Result<T>
//   Tensor / TensorRandom subset  tensor.rs:7-59,212-233     helix::DeviceTensor
//   nn::Module<T>                 crates/nn/src/lib.rs:20-39 helix::Module
//   nn::Linear / RMSNorm          lib.rs:60-218, 222-327     helix::Linear / helix::RMSNorm
//   nn::ssm::S4Block              crates/nn/src/ssm.rs:14    helix::S4Block
//   nn::MambaBlock                lib.rs:820-971             helix::MambaBlock
//   examples/ssm_byte_lm model    main.rs:104-130            helix::ByteLM
//
// Error behaviour follows the reference: shape/dtype/device problems are returned as errors, never
// thrown across the ABI and never trapped.  forward() takes &self and launches on the tensor's device
// on the current (default) stream; modules are immutable during forward and may be shared by threads.
#pragma once

#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "../../include/helix_b200.h"

namespace helix {

enum class DType : int { F32 = HX_F32, BF16 = HX_BF16, U8 = HX_U8 };
inline size_t dtype_size(DType d) { return d == DType::F32 ? 4 : d == DType::BF16 ? 2 : 1; }

struct Device {
    enum Kind { Cpu, Cuda } kind = Cpu;
    int id = 0;
    static Device cpu() { return {Cpu, 0}; }
    static Device cuda(int id) { return {Cuda, id}; }
    bool is_cpu() const { return kind == Cpu; }
    bool is_cuda() const { return kind == Cuda; }
    bool operator==(const Device &o) const { return kind == o.kind && (kind == Cpu || id == o.id); }
    std::string to_string() const { return kind == Cpu ? "cpu" : "cuda:" + std::to_string(id); }
};

struct TensorError {
    hx_status code = HX_OK;
    std::string message;
};

// Either a value or a TensorError.
template <typename T> class Result {
  public:
    Result(T v) : ok_(true), value_(std::move(v)) {}
    Result(TensorError e) : ok_(false), error_(std::move(e)) {}
    bool ok() const { return ok_; }
    T &value() { return value_; }
    const T &value() const { return value_; }
    const TensorError &error() const { return error_; }

  private:
    bool ok_;
    T value_{};
    TensorError error_;
};
struct Unit {};

class Shape {
  public:
    Shape() = default;
    explicit Shape(std::vector<int64_t> dims) : dims_(std::move(dims)) {}
    size_t ndim() const { return dims_.size(); }
    int64_t dim(size_t i) const { return dims_[i]; }
    int64_t numel() const {
        int64_t n = 1;
        for (auto d : dims_) n *= d;
        return n;
    }
    const std::vector<int64_t> &as_slice() const { return dims_; }
    bool operator==(const Shape &o) const { return dims_ == o.dims_; }

  private:
    std::vector<int64_t> dims_;
};

// A dense, row-major tensor whose storage lives in device memory and is freed with its last owner.
// Copying a DeviceTensor shares the storage; clone() makes a deep copy (the reference's Clone).
class DeviceTensor {
  public:
    DeviceTensor() = default;
    static Result<DeviceTensor> empty(const Shape &shape, DType dtype, const Device &device);
    static Result<DeviceTensor> zeros(const Shape &shape, DType dtype, const Device &device);
    // host data is fp32 (or bytes for U8); it is converted to `dtype` on the way in
    static Result<DeviceTensor> from_host_f32(const float *data, const Shape &shape, DType dtype, const Device &device);
    static Result<DeviceTensor> from_host_u8(const uint8_t *data, const Shape &shape, const Device &device);
    Result<Unit> copy_from_host_f32(const float *data, int64_t n);
    Result<Unit> to_host_f32(float *out, int64_t n) const;  // widens bf16
    Result<DeviceTensor> clone() const;
    Result<DeviceTensor> reshape(const Shape &shape) const;  // shares storage

    const Shape &shape() const { return shape_; }
    DType dtype() const { return dtype_; }
    const Device &device() const { return device_; }
    size_t ndim() const { return shape_.ndim(); }
    int64_t numel() const { return shape_.numel(); }
    void *data() const { return ptr_; }
    bool defined() const { return storage_ != nullptr || shape_.numel() == 0; }

  private:
    std::shared_ptr<void> storage_;
    void *ptr_ = nullptr;
    Shape shape_;
    DType dtype_ = DType::F32;
    Device device_;
};

// crates/nn/src/lib.rs:20-39 (forward_with_autograd is the training path and is not part of this build)
class Module {
  public:
    virtual ~Module() = default;
    virtual Result<DeviceTensor> forward(const DeviceTensor &input) const = 0;
    virtual std::vector<const DeviceTensor *> parameters() const = 0;
    virtual std::vector<DeviceTensor *> parameters_mut() = 0;
    virtual const Device &device() const = 0;
    // Called after parameters were written through parameters_mut(): lets a module refresh what it
    // derives from them (for example whether A is geometric).
    virtual Result<Unit> parameters_updated() { return Unit{}; }
    virtual const char *name() const = 0;
};

// nn::Linear (crates/nn/src/lib.rs:60-134): weight [out, in] ~ N(0, sqrt(2/in)), bias zeros; y = x W^T + b.
class Linear : public Module {
  public:
    static Result<std::unique_ptr<Linear>> create(int64_t in_features, int64_t out_features, bool bias, DType dtype,
                                                  const Device &device);
    Result<DeviceTensor> forward(const DeviceTensor &input) const override;
    std::vector<const DeviceTensor *> parameters() const override;
    std::vector<DeviceTensor *> parameters_mut() override;
    const Device &device() const override { return device_; }
    const char *name() const override { return "Linear"; }
    DeviceTensor weight, bias;  // bias is fp32
    bool has_bias = false;

  private:
    Device device_;
};

// nn::RMSNorm (crates/nn/src/lib.rs:222-285): weight ones [d_model], eps.
class RMSNorm : public Module {
  public:
    static Result<std::unique_ptr<RMSNorm>> create(int64_t d_model, float eps, const Device &device);
    Result<DeviceTensor> forward(const DeviceTensor &input) const override;
    std::vector<const DeviceTensor *> parameters() const override { return {&weight}; }
    std::vector<DeviceTensor *> parameters_mut() override { return {&weight}; }
    const Device &device() const override { return device_; }
    const char *name() const override { return "RMSNorm"; }
    DeviceTensor weight;
    float eps = 1e-5f;

  private:
    Device device_;
};

// nn::ssm::S4Block (crates/nn/src/ssm.rs:14-186).  Parameters, in the reference's order
// (ssm.rs:275-277): A_real [N], A_imag [N], B [N, M], C [M, N], D [M], delta [M], Lambda [N].
//   forward_ssm(u [M, L])  -- the reference's recurrence with dt = 0.1, output buffer [L, M]
//   forward(u [B, L, M] or [L, M]) -- the per-channel diagonal form (abar = exp(delta A), bbar = delta B)
//                                     with A_diag [M, N], B_diag [M, N], C_diag [M, N] as extra parameters.
class S4Block : public Module {
  public:
    static Result<std::unique_ptr<S4Block>> create(int64_t d_model, int64_t d_state, const Device &device);
    Result<DeviceTensor> forward(const DeviceTensor &input) const override;
    Result<DeviceTensor> forward_ssm(const DeviceTensor &input) const;
    std::vector<const DeviceTensor *> parameters() const override;
    std::vector<DeviceTensor *> parameters_mut() override;
    const Device &device() const override { return device_; }
    const char *name() const override { return "S4Block"; }
    DeviceTensor A_real, A_imag, B, C, D, delta, Lambda;  // the reference's seven
    DeviceTensor A_diag, B_diag, C_diag;                   // per-channel diagonal form
    int64_t d_model = 0, d_state = 0;

  private:
    Device device_;
};

// nn::MambaBlock (crates/nn/src/lib.rs:820-971): new(d_model, d_state, d_conv, expand, device), forward.
// The selective-scan block the benchmark configuration describes; parameters, in order:
//   in_proj.weight [2E, M], conv_w [E, K], conv_b [E], x_proj.weight [R+2N, E], dt_proj.weight [E, R],
//   dt_proj.bias [E], A [E, N] (= -exp(A_log), A_log[d,n] = log(n+1)), D [E] (ones), out_proj.weight [M, E]
// with E = expand * d_model, R = ceil(d_model / 16).  The reference's own B_proj / C_proj of shape
// [N*E, E] (lib.rs:864-865) are never read by its forward and are not reproduced.
class MambaBlock : public Module {
  public:
    static Result<std::unique_ptr<MambaBlock>> create(int64_t d_model, int64_t d_state, int64_t d_conv, int64_t expand,
                                                      DType dtype, const Device &device);
    Result<DeviceTensor> forward(const DeviceTensor &input) const override;
    // forward into caller-provided buffers (no allocation): x and out are [batch*seq_len, d_model]
    // h_last [batch, d_inner, d_state] fp32 and conv_state [batch, 3, d_inner] (model dtype), when given, receive
    // the state a decode step continues from.
    // residual [batch*seq_len, d_model] fp32, when given, receives `+= block output` (and `out` is only scratch for
    // the fp32 path).
    Result<Unit> forward_into(const void *x, void *out, int64_t batch, int64_t seq_len, void *workspace,
                              size_t workspace_bytes, void *stream, void **stage_events = nullptr, float *h_last = nullptr,
                              void *conv_state = nullptr, float *residual = nullptr) const;
    size_t workspace_bytes(int64_t batch, int64_t seq_len) const;
    // one decode step: x, out [batch, d_model]; h and conv_state are updated in place
    // With `residual` (fp32 [batch, d_model]) and `norm_w`: the input is rmsnorm(residual) * norm_w and the output
    // is added into residual (x may be NULL, out is scratch for the fp32 path).
    Result<Unit> step_into(const void *x, void *out, int64_t batch, float *h, void *conv_state, void *workspace,
                           size_t workspace_bytes, void *stream, float *residual = nullptr, const float *norm_w = nullptr,
                           float norm_eps = 1e-5f) const;
    // true when a residual-form step runs as four kernels (norm and conv step inside in_proj, add inside out_proj)
    bool step_is_fused(int64_t batch) const { return dtype == DType::BF16 && d_model % 32 == 0 && batch <= 64 && d_inner % 8 == 0; }
    size_t step_workspace_bytes(int64_t batch) const;
    std::vector<const DeviceTensor *> parameters() const override;
    std::vector<DeviceTensor *> parameters_mut() override;
    Result<Unit> parameters_updated() override;
    const Device &device() const override { return device_; }
    const char *name() const override { return "MambaBlock"; }
    DeviceTensor W_in, conv_w, conv_b, W_x, W_dt, b_dt, A, D, W_out;
    int64_t d_model = 0, d_state = 0, d_conv = 0, expand = 0, d_inner = 0, dt_rank = 0;
    DType dtype = DType::F32;
    bool a_geometric = false;

  private:
    Device device_;
};

// nn::Sequential (crates/nn/src/lib.rs:577-661): an ordered list of modules, forward chains them, parameters
// concatenates theirs.  add() takes ownership, like the reference's Box<dyn Module>.
class Sequential : public Module {
  public:
    explicit Sequential(const Device &device) : device_(device) {}
    void add(std::unique_ptr<Module> m) { modules_.push_back(std::move(m)); }
    size_t len() const { return modules_.size(); }
    Result<DeviceTensor> forward(const DeviceTensor &input) const override;
    std::vector<const DeviceTensor *> parameters() const override;
    std::vector<DeviceTensor *> parameters_mut() override;
    Result<Unit> parameters_updated() override;
    const Device &device() const override { return device_; }
    const char *name() const override { return "Sequential"; }

  private:
    std::vector<std::unique_ptr<Module>> modules_;
    Device device_;
};

// Byte-level LM: tied embedding [256, M], n_layer x (RMSNorm -> MambaBlock -> residual add), final
// RMSNorm, logits = h . emb^T.  forward takes U8 tokens [B, L] and returns logits [B, L, 256].
class ByteLM : public Module {
  public:
    static Result<std::unique_ptr<ByteLM>> create(int64_t n_layer, int64_t d_model, int64_t d_state, int64_t d_conv,
                                                  int64_t expand, DType dtype, const Device &device);
    ~ByteLM() override;
    Result<DeviceTensor> forward(const DeviceTensor &tokens) const override;
    // The serving call: tokens from (pinned) host memory, logits back to (pinned) host memory in the
    // model dtype.  Activations live in buffers sized on first use for (batch, seq_len) and kept.
    Result<Unit> forward_host(const uint8_t *tokens_host, void *logits_host, int64_t batch, int64_t seq_len, void *stream);
    // Same on device buffers: tokens_dev [B*L] u8, logits_dev [B*L, 256] model dtype.
    Result<Unit> forward_device(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream);
    int64_t launches_per_forward() const;
    // Serving: prefill_device is forward_device that also keeps, per layer, the scan state and the conv window;
    // decode_step_device then advances every sequence by one token (tokens_dev [batch] u8, logits_dev
    // [batch, 256] model dtype).  From its second call on, a step is one replay of a CUDA graph captured over the
    // module's own step buffers (set_decode_graph(false) keeps plain launches).  One decode stream per module:
    // the state lives in the module.
    Result<Unit> prefill_device(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream);
    Result<Unit> decode_step_device(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, void *stream);
    void set_decode_graph(bool enable) { decode_graph_ = enable; }
    // forward_device / prefill_device / forward_host replay a CUDA graph of the whole forward from the second call
    // with the same (tokens, logits, batch, seq_len) on: 150 to 200 dependent kernels become one launch, which is
    // what a small batch (a few sequences per GPU) is bound by.  Off: plain launches.
    void set_forward_graph(bool enable);
    int64_t launches_per_decode_step() const;
    // per-stage CUDA-event timing (see hx_byte_lm_profile in the C header)
    Result<Unit> set_profile(bool enable);
    Result<Unit> read_profile(float *ms9, int *forwards);
    std::vector<const DeviceTensor *> parameters() const override;
    std::vector<DeviceTensor *> parameters_mut() override;
    Result<Unit> parameters_updated() override;
    const Device &device() const override { return device_; }
    const char *name() const override { return "ByteLM"; }
    DeviceTensor embedding, norm_f;
    std::vector<std::unique_ptr<RMSNorm>> norms;
    std::vector<std::unique_ptr<MambaBlock>> blocks;
    int64_t d_model = 0;
    DType dtype = DType::F32;
    float eps = 1e-5f;

  private:
    Result<Unit> ensure_buffers(int64_t batch, int64_t seq_len);
    Result<Unit> ensure_decode(int64_t batch);
    Result<Unit> enqueue_step(void *stream);
    Result<Unit> run_layers(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream,
                            bool keep_state);
    Device device_;
    struct Buffers;
    Buffers *buf_ = nullptr;
    struct Decode;
    Decode *dec_ = nullptr;
    bool decode_graph_ = true;
    struct FwdGraphs;
    FwdGraphs *fwd_ = nullptr;
    bool forward_graph_ = true;
    Result<Unit> run_layers_plain(const uint8_t *tokens_dev, void *logits_dev, int64_t batch, int64_t seq_len, void *stream,
                                  bool keep_state);
    struct Profile;
    Profile *prof_ = nullptr;
    // The activation buffers, the decode state and the profile belong to the module: every call that touches them
    // holds this lock while it queues its work (forward() until its result is complete), so threads that share one
    // handle are serialised.  Their work must go to ONE stream: stream order is what keeps a later call from
    // overwriting buffers an earlier one still reads.
    mutable std::recursive_mutex mu_;
};

// Seed of the parameter initialisers (the reference draws from an unseeded thread_rng,
// crates/backend-cpu/src/lib.rs:1209; here initialisation is reproducible).
void manual_seed(uint64_t seed);

// TensorRandom::{random_normal, random_uniform, random_bernoulli} (crates/tensor-core/src/tensor.rs:212-221)
Result<DeviceTensor> init_normal(const Shape &shape, double stddev, DType dtype, const Device &device, double mean = 0.0);
Result<DeviceTensor> init_uniform(const Shape &shape, double lo, double hi, DType dtype, const Device &device);
Result<DeviceTensor> init_bernoulli(const Shape &shape, double p, DType dtype, const Device &device);

// The tensor primitives the reference's generic blocks call on T (csrc/tensor_ops.cu): TensorOps
// (tensor.rs:62-134), TensorBroadcast (:137-149), TensorActivation (:191-209), TensorMixedPrecision::cast (:238),
// Tensor::{transpose, slice, cat, stack} (:37-46), TensorRandom::{zeros, ones, eye, arange} (:223-232).
// `op` is an hx_binary_op / hx_unary_op code.
namespace tops {
Result<DeviceTensor> binary(int op, const DeviceTensor &a, const DeviceTensor &b);
Result<DeviceTensor> unary(int op, const DeviceTensor &a, float p0 = 0.f, float p1 = 0.f);
Result<DeviceTensor> matmul(const DeviceTensor &a, const DeviceTensor &b);
Result<DeviceTensor> transpose(const DeviceTensor &a, int64_t dim0, int64_t dim1);
Result<DeviceTensor> slice(const DeviceTensor &a, const std::vector<int64_t> &start, const std::vector<int64_t> &end);
Result<DeviceTensor> cat(const std::vector<const DeviceTensor *> &tensors, int64_t dim);
Result<DeviceTensor> stack(const std::vector<const DeviceTensor *> &tensors, int64_t dim);
Result<DeviceTensor> broadcast_to(const DeviceTensor &a, const Shape &shape);
Result<DeviceTensor> cast(const DeviceTensor &a, DType dtype);
Result<float> to_scalar(const DeviceTensor &a);
Result<DeviceTensor> full(float value, const Shape &shape, DType dtype, const Device &device);
Result<DeviceTensor> eye(int64_t n, DType dtype, const Device &device);
Result<DeviceTensor> arange(float start, float end, float step, DType dtype, const Device &device);
}  // namespace tops

}  // namespace helix

// The opaque handles of the C ABI (include/helix_b200.h) wrap these.
struct hx_tensor { helix::DeviceTensor t; };
struct hx_module { std::unique_ptr<helix::Module> m; };
