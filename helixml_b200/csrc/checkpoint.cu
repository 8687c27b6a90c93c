// Checkpoints in the reference's on-disk layout, so that a file written here loads in the reference and the
// other way round (crates/training/src/checkpoint.rs:136-197):
//   u32 big-endian  length of the metadata JSON          (tokio's write_u32)
//   bytes           serde_json of CheckpointData          (checkpoint.rs:246-266; timestamp as seconds, :268-288)
//   rest            bincode 1.3 (default options: little-endian, fixed-width integers, u64 lengths, u32 enum
//                   variants) of Vec<CpuTensor>
// A CpuTensor (crates/backend-cpu/src/lib.rs:23-29) serialises field by field:
//   data   ndarray 0.15 ArrayD<f32> with its serde feature: u8 version = 1, the dimensions as a sequence of
//          usize, the elements in logical (row-major) order as a sequence of f32
//   shape  Shape { dims: Vec<usize> }                     (crates/tensor-core/src/shape.rs:7-10)
//   dtype  DType variant index, F32 = 9                   (crates/tensor-core/src/dtype.rs:8-37)
//   device Device variant index, Cpu = 0, Cuda(id) = 1 followed by the id (crates/tensor-core/src/device.rs:8-25)
// The reference stores f32 whatever the dtype label says, so bf16 parameters are widened on the way out and
// rounded on the way in; tensors are written with the labels F32 / Cpu.  bincode and ndarray are not part of
// the reference tree; the layouts above are their published formats for the versions its manifests pin
// (crates/training/Cargo.toml:30, crates/backend-cpu/Cargo.toml:13).
#include <cinttypes>
#include <cmath>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "helix_host.hpp"
#include "hx_common.cuh"

struct hx_checkpoint {
    hx_checkpoint_meta meta;
    std::vector<std::vector<int64_t>> dims;
    std::vector<std::vector<float>> data;
};

namespace {

constexpr uint32_t kDTypeF32 = 9, kDeviceCpu = 0;
constexpr uint32_t kDeviceIdVariants[] = {1, 4, 5, 6};  // Cuda, Qpu, Npu, Tpu carry a usize

void put_u64(std::string &b, uint64_t v) { b.append(reinterpret_cast<const char *>(&v), 8); }
void put_u32(std::string &b, uint32_t v) { b.append(reinterpret_cast<const char *>(&v), 4); }

std::string json_number(double v) {
    if (!std::isfinite(v)) return "null";  // serde_json writes non-finite floats as null
    char buf[40];
    snprintf(buf, sizeof(buf), "%.17g", v);
    std::string s(buf);
    if (s.find_first_of(".eE") == std::string::npos) s += ".0";
    return s;
}

std::string meta_json(const hx_checkpoint_meta &m, int64_t n_params) {
    std::string j = "{";
    j += "\"epoch\":" + std::to_string(m.epoch);
    j += ",\"step\":" + std::to_string(m.step);
    j += ",\"training_loss\":" + json_number(m.training_loss);
    j += ",\"validation_loss\":" + json_number(m.validation_loss);
    j += ",\"learning_rate\":" + json_number(m.learning_rate);
    j += ",\"timestamp\":" + std::to_string(m.timestamp_secs);
    j += ",\"model_params_count\":" + std::to_string(n_params);
    // Metrics (crates/training/src/metrics.rs:11-53): the durations and instants are #[serde(skip)]
    j += ",\"metrics\":{";
    j += "\"training_loss\":" + json_number(m.training_loss);
    j += ",\"validation_loss\":" + json_number(m.validation_loss);
    j += ",\"epoch\":" + std::to_string(m.epoch);
    j += ",\"step\":" + std::to_string(m.step);
    j += ",\"learning_rate\":" + json_number(m.learning_rate);
    j += ",\"custom_metrics\":{}";
    j += ",\"history\":{\"training_losses\":[],\"validation_losses\":[],\"learning_rates\":[],\"epochs\":[],\"steps\":[],"
         "\"custom_metrics_history\":{}}";
    j += "}}";
    return j;
}

// First occurrence of "key": in serde_json's output is the top-level field (the nested Metrics comes last).
bool json_field(const std::string &j, const char *key, double *out) {
    const std::string pat = std::string("\"") + key + "\":";
    const size_t p = j.find(pat);
    if (p == std::string::npos) return false;
    const char *s = j.c_str() + p + pat.size();
    if (strncmp(s, "null", 4) == 0) {
        *out = NAN;
        return true;
    }
    char *end = nullptr;
    *out = strtod(s, &end);
    return end != s;
}

struct Reader {
    const unsigned char *p, *end;
    bool ok = true;
    bool take(void *dst, size_t n) {
        if (!ok || (size_t)(end - p) < n) return ok = false;
        memcpy(dst, p, n);
        p += n;
        return true;
    }
    uint64_t u64() { uint64_t v = 0; take(&v, 8); return v; }
    uint32_t u32() { uint32_t v = 0; take(&v, 4); return v; }
    uint8_t u8() { uint8_t v = 0; take(&v, 1); return v; }
};

hx_status write_file(const char *path, const hx_checkpoint_meta *meta, int32_t n, const float *const *data,
                     const int64_t *const *dims, const int32_t *ndims) {
    HX_REQUIRE(path && meta && n >= 0 && (n == 0 || (data && dims && ndims)), HX_ERR_INVALID_INPUT,
               "hx_checkpoint_write: bad arguments");
    const std::string json = meta_json(*meta, n);
    std::string body;
    put_u64(body, (uint64_t)n);
    for (int32_t i = 0; i < n; ++i) {
        HX_REQUIRE(ndims[i] >= 0 && ndims[i] <= 8 && data[i] && (dims[i] || ndims[i] == 0), HX_ERR_INVALID_INPUT,
                   "hx_checkpoint_write: tensor %d is malformed", i);
        uint64_t numel = 1;
        for (int k = 0; k < ndims[i]; ++k) {
            HX_REQUIRE(dims[i][k] >= 0, HX_ERR_INVALID_DIMENSION, "hx_checkpoint_write: negative dimension in tensor %d", i);
            numel *= (uint64_t)dims[i][k];
        }
        body.push_back((char)1);                                 // ndarray format version
        put_u64(body, (uint64_t)ndims[i]);                       // dim: IxDyn as a sequence
        for (int k = 0; k < ndims[i]; ++k) put_u64(body, (uint64_t)dims[i][k]);
        put_u64(body, numel);                                    // data: sequence of f32
        body.append(reinterpret_cast<const char *>(data[i]), numel * sizeof(float));
        put_u64(body, (uint64_t)ndims[i]);                       // shape.dims
        for (int k = 0; k < ndims[i]; ++k) put_u64(body, (uint64_t)dims[i][k]);
        put_u32(body, kDTypeF32);
        put_u32(body, kDeviceCpu);
    }
    FILE *f = fopen(path, "wb");
    HX_REQUIRE(f != nullptr, HX_ERR_SERIALIZATION, "hx_checkpoint_write: cannot create %s", path);
    const uint32_t len = (uint32_t)json.size();
    const unsigned char be[4] = {(unsigned char)(len >> 24), (unsigned char)(len >> 16), (unsigned char)(len >> 8), (unsigned char)len};
    bool ok = fwrite(be, 1, 4, f) == 4 && fwrite(json.data(), 1, json.size(), f) == json.size() &&
              fwrite(body.data(), 1, body.size(), f) == body.size();
    ok = (fclose(f) == 0) && ok;
    HX_REQUIRE(ok, HX_ERR_SERIALIZATION, "hx_checkpoint_write: short write to %s", path);
    return HX_OK;
}

hx_status read_file_impl(const char *path, hx_checkpoint *ck) {
    FILE *f = fopen(path, "rb");
    HX_REQUIRE(f != nullptr, HX_ERR_SERIALIZATION, "hx_checkpoint_open: cannot open %s", path);
    std::vector<unsigned char> buf;
    unsigned char chunk[1 << 16];
    size_t got;
    while ((got = fread(chunk, 1, sizeof(chunk), f)) > 0) buf.insert(buf.end(), chunk, chunk + got);
    fclose(f);
    HX_REQUIRE(buf.size() >= 4, HX_ERR_SERIALIZATION, "hx_checkpoint_open: %s is shorter than its header", path);
    const uint32_t len = ((uint32_t)buf[0] << 24) | ((uint32_t)buf[1] << 16) | ((uint32_t)buf[2] << 8) | buf[3];
    HX_REQUIRE((size_t)len + 4 <= buf.size(), HX_ERR_SERIALIZATION, "hx_checkpoint_open: metadata length %u exceeds the file", len);
    const std::string json(reinterpret_cast<const char *>(buf.data()) + 4, len);
    double v = 0;
    memset(&ck->meta, 0, sizeof(ck->meta));
    HX_REQUIRE(json_field(json, "epoch", &v), HX_ERR_SERIALIZATION, "hx_checkpoint_open: metadata has no epoch");
    ck->meta.epoch = (uint64_t)v;
    HX_REQUIRE(json_field(json, "step", &v), HX_ERR_SERIALIZATION, "hx_checkpoint_open: metadata has no step");
    ck->meta.step = (uint64_t)v;
    if (json_field(json, "training_loss", &v)) ck->meta.training_loss = v;
    if (json_field(json, "validation_loss", &v)) ck->meta.validation_loss = v;
    if (json_field(json, "learning_rate", &v)) ck->meta.learning_rate = v;
    if (json_field(json, "timestamp", &v)) ck->meta.timestamp_secs = (uint64_t)v;
    double declared = -1;
    json_field(json, "model_params_count", &declared);

    Reader r{buf.data() + 4 + len, buf.data() + buf.size()};
    const uint64_t n = r.u64();
    HX_REQUIRE(r.ok && n <= (1u << 20), HX_ERR_SERIALIZATION, "hx_checkpoint_open: implausible tensor count");
    if (declared >= 0 && (uint64_t)declared != n)
        return hx::fail(HX_ERR_INVALID_CHECKPOINT, "metadata declares %" PRIu64 " parameters, the file holds %" PRIu64,
                        (uint64_t)declared, n);
    for (uint64_t i = 0; i < n; ++i) {
        const uint8_t ver = r.u8();
        HX_REQUIRE(r.ok && ver == 1, HX_ERR_SERIALIZATION, "hx_checkpoint_open: tensor %" PRIu64 " has array format version %u", i, ver);
        const uint64_t nd = r.u64();
        HX_REQUIRE(r.ok && nd <= 8, HX_ERR_SERIALIZATION, "hx_checkpoint_open: tensor %" PRIu64 " has %" PRIu64 " dimensions", i, nd);
        std::vector<int64_t> dims(nd);
        uint64_t numel = 1;
        bool wrapped = false;
        for (auto &d : dims) {
            const uint64_t dv = r.u64();
            d = (int64_t)dv;
            // sizes come from the file: a product that wraps, or a dimension beyond int64, is a malformed file
            if (dv > (uint64_t)INT64_MAX || (dv != 0 && numel > UINT64_MAX / dv)) wrapped = true;
            else numel *= dv;
        }
        HX_REQUIRE(r.ok && !wrapped, HX_ERR_SERIALIZATION, "hx_checkpoint_open: tensor %" PRIu64 " has an implausible shape", i);
        const uint64_t cnt = r.u64();
        HX_REQUIRE(r.ok && cnt == numel && cnt <= (uint64_t)(r.end - r.p) / 4, HX_ERR_SERIALIZATION,
                   "hx_checkpoint_open: tensor %" PRIu64 " holds %" PRIu64 " elements for a shape of %" PRIu64, i, cnt, numel);
        std::vector<float> data(cnt);
        r.take(data.data(), cnt * 4);
        const uint64_t snd = r.u64();
        HX_REQUIRE(r.ok && snd == nd, HX_ERR_SERIALIZATION, "hx_checkpoint_open: tensor %" PRIu64 ": shape and array disagree", i);
        for (uint64_t k = 0; k < snd; ++k) {
            const uint64_t d = r.u64();
            HX_REQUIRE(r.ok && (int64_t)d == dims[k], HX_ERR_SERIALIZATION, "hx_checkpoint_open: tensor %" PRIu64 ": shape and array disagree", i);
        }
        r.u32();  // dtype label: the storage is f32 whatever it says
        const uint32_t dev = r.u32();
        for (uint32_t with_id : kDeviceIdVariants)
            if (dev == with_id) r.u64();
        HX_REQUIRE(r.ok && dev != 7, HX_ERR_SERIALIZATION, "hx_checkpoint_open: tensor %" PRIu64 " is truncated or on a custom device", i);
        ck->dims.push_back(std::move(dims));
        ck->data.push_back(std::move(data));
    }
    HX_REQUIRE(r.p == r.end, HX_ERR_SERIALIZATION, "hx_checkpoint_open: %zu trailing bytes", (size_t)(r.end - r.p));
    return HX_OK;
}

// No C++ exception crosses the C ABI: a file whose sizes ask for more memory than there is becomes a status.
hx_status read_file(const char *path, hx_checkpoint *ck) {
    try {
        return read_file_impl(path, ck);
    } catch (const std::bad_alloc &) {
        return hx::fail(HX_ERR_ALLOCATION_FAILED, "hx_checkpoint_open: out of host memory while reading %s", path);
    } catch (const std::exception &e) {
        return hx::fail(HX_ERR_SERIALIZATION, "hx_checkpoint_open: %s", e.what());
    }
}

}  // namespace

extern "C" {

hx_status hx_checkpoint_write(const char *path, const hx_checkpoint_meta *meta, int32_t n_tensors, const float *const *data,
                              const int64_t *const *dims, const int32_t *ndims) {
    return write_file(path, meta, n_tensors, data, dims, ndims);
}

hx_status hx_checkpoint_open(const char *path, hx_checkpoint **out) {
    HX_REQUIRE(path && out, HX_ERR_INVALID_INPUT, "hx_checkpoint_open: NULL argument");
    auto ck = std::unique_ptr<hx_checkpoint>(new hx_checkpoint());
    const hx_status s = read_file(path, ck.get());
    if (s != HX_OK) return s;
    *out = ck.release();
    return HX_OK;
}

void hx_checkpoint_close(hx_checkpoint *ck) { delete ck; }

int32_t hx_checkpoint_num_tensors(const hx_checkpoint *ck) { return ck ? (int32_t)ck->data.size() : 0; }

hx_status hx_checkpoint_meta_get(const hx_checkpoint *ck, hx_checkpoint_meta *meta) {
    HX_REQUIRE(ck && meta, HX_ERR_INVALID_INPUT, "hx_checkpoint_meta_get: NULL argument");
    *meta = ck->meta;
    return HX_OK;
}

hx_status hx_checkpoint_tensor(const hx_checkpoint *ck, int32_t index, const float **data, const int64_t **dims, int32_t *ndim) {
    HX_REQUIRE(ck && data && dims && ndim, HX_ERR_INVALID_INPUT, "hx_checkpoint_tensor: NULL argument");
    HX_REQUIRE(index >= 0 && index < (int32_t)ck->data.size(), HX_ERR_INVALID_DIMENSION, "tensor index %d out of %zu", index,
               ck->data.size());
    *data = ck->data[(size_t)index].data();
    *dims = ck->dims[(size_t)index].data();
    *ndim = (int32_t)ck->dims[(size_t)index].size();
    return HX_OK;
}

// CheckpointableModule::checkpoint (crates/nn/src/lib.rs:50-52) + CheckpointManager::save_checkpoint_to_file
hx_status hx_module_save_checkpoint(const hx_module *m, const char *path, const hx_checkpoint_meta *meta) {
    HX_REQUIRE(m && path && meta, HX_ERR_INVALID_INPUT, "hx_module_save_checkpoint: NULL argument");
    const auto ps = m->m->parameters();
    std::vector<std::vector<float>> host(ps.size());
    std::vector<const float *> data(ps.size());
    std::vector<const int64_t *> dims(ps.size());
    std::vector<int32_t> ndims(ps.size());
    for (size_t i = 0; i < ps.size(); ++i) {
        host[i].resize((size_t)ps[i]->numel());
        auto r = ps[i]->to_host_f32(host[i].data(), ps[i]->numel());
        if (!r.ok()) return hx::fail(r.error().code, "%s", r.error().message.c_str());
        data[i] = host[i].data();
        dims[i] = ps[i]->shape().as_slice().data();
        ndims[i] = (int32_t)ps[i]->ndim();
    }
    return write_file(path, meta, (int32_t)ps.size(), data.data(), dims.data(), ndims.data());
}

// CheckpointManager::load_checkpoint_from_file + CheckpointableModule::restore (crates/nn/src/lib.rs:54-55)
hx_status hx_module_load_checkpoint(hx_module *m, const char *path, hx_checkpoint_meta *meta_out) {
    HX_REQUIRE(m && path, HX_ERR_INVALID_INPUT, "hx_module_load_checkpoint: NULL argument");
    hx_checkpoint ck;
    hx_status s = read_file(path, &ck);
    if (s != HX_OK) return s;
    auto ps = m->m->parameters_mut();
    if (ck.data.size() != ps.size())
        return hx::fail(HX_ERR_INVALID_CHECKPOINT, "the module has %zu parameters, the checkpoint %zu", ps.size(), ck.data.size());
    for (size_t i = 0; i < ps.size(); ++i) {
        const auto &want = ps[i]->shape().as_slice();
        if (want != ck.dims[i]) return hx::fail(HX_ERR_SHAPE_MISMATCH, "parameter %zu: checkpoint shape differs from the module's", i);
    }
    for (size_t i = 0; i < ps.size(); ++i) {
        auto r = ps[i]->copy_from_host_f32(ck.data[i].data(), (int64_t)ck.data[i].size());
        if (!r.ok()) return hx::fail(r.error().code, "%s", r.error().message.c_str());
    }
    auto r = m->m->parameters_updated();
    if (!r.ok()) return hx::fail(r.error().code, "%s", r.error().message.c_str());
    if (meta_out) *meta_out = ck.meta;
    return HX_OK;
}

}  // extern "C"
