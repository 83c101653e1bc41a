// Checkpoint boundary of the quantized Linear: a safetensors reader and the rule that turns one layer's tensors into
// a QuantWeight with device pointers.
//
// The rule is `quant()` of the reference's loader (src/dit/transformer_load.cpp:585-659), format decided from the file
// itself, in this order:
//   1. `<layer>.comfy_quant` (rank-1 U8 JSON) or the header's `_quantization_metadata` says "asym_w4a8_int8" /
//      "w6a8_int8"  -> W4A8 / W6A8 with `.weight_s_rel` (e4m3 group scales), `.weight_s_channel`, `.weight_codebook`;
//      group 16 for W4, a multiple of 16 for W6, ConvRot 256 (read_packed_int8_state, src/core/w4a8.cpp:95-125);
//   2. `<layer>.weight.quant_state.bitsandbytes__nf4` exists -> NF4 with double-quantized block scales
//      (read_nf4_state, src/core/nf4.cpp:21-70: blocksize 64, nested 256, fp32 nested, bf16 source);
//   3. U8 `.weight` beside an e4m3 `.weight_scale` of shape [*, in/16] -> NVFP4; `.weight_scale_2` is mandatory
//      (is_nvfp4, src/dit/transformer_support.h:150-160);
//   4. otherwise the tensor's dtype (F32 / BF16 / F16 / F8_E4M3 with `.weight_scale` / I8 with per-channel
//      `.weight_scale`), and the comfy_quant tag may switch on ConvRot for int8 (read_comfy_quant,
//      src/dit/weight_metadata.cpp:13-52).
// Tensors are uploaded once per checkpoint handle (verbatim bytes, or converted to fp32 where the runner wants
// fp32) and freed when the handle is closed. safetensors layout: u64 little-endian header length, a JSON header
// {name: {dtype, shape, data_offsets}, "__metadata__": {...}}, then the tensor bytes.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/sfq.h"
#include "json_min.h"

namespace sfq_capi {
int run_guarded(void (*fn)(void*), void* ctx);
}

namespace {

struct Tensor {
  std::string name;
  int dtype = SFQ_DT_UNKNOWN;
  std::vector<int64_t> shape;
  const uint8_t* data = nullptr;
  size_t nbytes = 0;
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
  }
};

int dtype_from(const std::string& s) {
  static const std::pair<const char*, int> table[] = {
      {"BOOL", SFQ_DT_BOOL}, {"U8", SFQ_DT_U8},   {"I8", SFQ_DT_I8},     {"I16", SFQ_DT_I16},         {"I32", SFQ_DT_I32},
      {"I64", SFQ_DT_I64},   {"F16", SFQ_DT_F16}, {"BF16", SFQ_DT_BF16}, {"F32", SFQ_DT_F32},         {"F64", SFQ_DT_F64},
      {"F8_E4M3", SFQ_DT_F8E4M3},                  {"F8_E5M2", SFQ_DT_F8E5M2}};
  for (const auto& e : table)
    if (s == e.first) return e.second;
  return SFQ_DT_UNKNOWN;
}

size_t dtype_bytes(int dt) {
  switch (dt) {
    case SFQ_DT_BOOL: case SFQ_DT_U8: case SFQ_DT_I8: case SFQ_DT_F8E4M3: case SFQ_DT_F8E5M2: return 1;
    case SFQ_DT_I16: case SFQ_DT_F16: case SFQ_DT_BF16: return 2;
    case SFQ_DT_I32: case SFQ_DT_F32: return 4;
    case SFQ_DT_I64: case SFQ_DT_F64: return 8;
    default: return 0;
  }
}

float half_to_float(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 31u, man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      bits = sign | uint32_t(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | man << 13;
  } else {
    bits = sign | (exp + 127 - 15) << 23 | man << 13;
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("checkpoint: ") + what + ": " + cudaGetErrorString(e));
}

}  // namespace

struct sfq_checkpoint {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t map_bytes = 0;
  std::vector<Tensor> tensors;
  std::unordered_map<std::string, size_t> index;
  std::vector<std::pair<std::string, std::string>> metadata;
  std::unordered_map<std::string, void*> device;      // verbatim uploads, by tensor name
  std::unordered_map<std::string, void*> device_f32;  // fp32 conversions, by tensor name
  std::unordered_map<std::string, std::vector<float>> host_f32;  // the same conversions for the host view
  bool host_view = false;  // linear() hands out host pointers (into the mapping / host_f32) instead of uploading
  std::mutex mutex;        // serialises linear(): the flag above and the caches are per handle
  int upload_device = -1;  // the device the caches' pointers live on (set by the first upload)

  // Uploads are cached by tensor name, so every pointer handed out belongs to one device: the one that was current at
  // the first upload. Asking from another device is refused instead of returning foreign pointers.
  void bind_device() {
    int dev = -1;
    check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (upload_device < 0) upload_device = dev;
    if (dev != upload_device)
      throw std::runtime_error("checkpoint: this handle uploaded its tensors to device " + std::to_string(upload_device) +
                               "; open the file again for device " + std::to_string(dev));
  }

  ~sfq_checkpoint() {
    for (auto& kv : device) cudaFree(kv.second);
    for (auto& kv : device_f32) cudaFree(kv.second);
    if (map != nullptr) munmap(map, map_bytes);
    if (fd >= 0) close(fd);
  }
  const Tensor* find(const std::string& name) const {
    const auto it = index.find(name);
    return it == index.end() ? nullptr : &tensors[it->second];
  }
  const Tensor& at(const std::string& name) const {
    const Tensor* t = find(name);
    if (t == nullptr) throw std::runtime_error("checkpoint: tensor '" + name + "' is missing");
    return *t;
  }
  const std::string* meta(const std::string& key) const {
    for (const auto& kv : metadata)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }

  void open(const char* path) {
    fd = ::open(path, O_RDONLY);
    if (fd < 0) throw std::runtime_error(std::string("checkpoint: cannot open '") + path + "'");
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) throw std::runtime_error(std::string("checkpoint: '") + path + "' is too short");
    map_bytes = size_t(st.st_size);
    void* p = mmap(nullptr, map_bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    if (p == MAP_FAILED) throw std::runtime_error(std::string("checkpoint: cannot map '") + path + "'");
    map = static_cast<uint8_t*>(p);
    uint64_t header_len = 0;
    for (int i = 7; i >= 0; --i) header_len = (header_len << 8) | map[i];
    if (header_len > map_bytes - 8) throw std::runtime_error("checkpoint: header length exceeds the file");
    const std::string header(reinterpret_cast<const char*>(map + 8), size_t(header_len));
    const sfq::json::Value root = sfq::json::parse(header);
    if (!root.is_object()) throw std::runtime_error("checkpoint: header is not a JSON object");
    const uint8_t* data0 = map + 8 + header_len;
    const size_t data_bytes = map_bytes - 8 - size_t(header_len);
    for (const auto& kv : root.object) {
      if (kv.first == "__metadata__") {
        if (kv.second.is_object())
          for (const auto& m : kv.second.object)
            if (m.second.kind == sfq::json::Value::kString) metadata.emplace_back(m.first, m.second.string);
        continue;
      }
      const sfq::json::Value* dt = kv.second.find("dtype");
      const sfq::json::Value* shape = kv.second.find("shape");
      const sfq::json::Value* off = kv.second.find("data_offsets");
      if (dt == nullptr || shape == nullptr || off == nullptr || off->array.size() != 2)
        throw std::runtime_error("checkpoint: malformed entry for '" + kv.first + "'");
      Tensor t;
      t.name = kv.first;
      t.dtype = dtype_from(dt->as_string());
      for (const auto& d : shape->array) {
        const int64_t v = d.as_int();
        if (v < 0) throw std::runtime_error("checkpoint: negative dimension in '" + kv.first + "'");
        t.shape.push_back(v);
      }
      {  // the element count must not wrap: a wrapped product could agree with the byte count checked below
        int64_t n = 1;
        for (int64_t d : t.shape) {
          if (d != 0 && n > INT64_MAX / d) throw std::runtime_error("checkpoint: the shape of '" + kv.first + "' overflows");
          n *= d;
        }
      }
      const int64_t b = off->array[0].as_int(), e = off->array[1].as_int();
      if (b < 0 || e < b || size_t(e) > data_bytes) throw std::runtime_error("checkpoint: offsets of '" + kv.first + "' leave the file");
      t.data = data0 + b;
      t.nbytes = size_t(e - b);
      const size_t width = dtype_bytes(t.dtype);
      if (width != 0 && size_t(t.numel()) * width != t.nbytes)
        throw std::runtime_error("checkpoint: '" + kv.first + "' has " + std::to_string(t.nbytes) + " bytes for its shape and dtype");
      index.emplace(t.name, tensors.size());
      tensors.push_back(std::move(t));
    }
  }

  // ---- uploads ("ptr" and "f32" of the reference's loader)
  const void* upload(const std::string& name) {
    if (host_view) return at(name).data;
    bind_device();
    const auto it = device.find(name);
    if (it != device.end()) return it->second;
    const Tensor& t = at(name);
    void* d = nullptr;
    check_cuda(cudaMalloc(&d, t.nbytes > 0 ? t.nbytes : 16), "cudaMalloc");
    if (t.nbytes > 0) {
      const cudaError_t e = cudaMemcpy(d, t.data, t.nbytes, cudaMemcpyHostToDevice);
      if (e != cudaSuccess) {
        cudaFree(d);
        check_cuda(e, "upload");
      }
    }
    device.emplace(name, d);
    return d;
  }
  std::vector<float> to_f32(const Tensor& t) const {
    std::vector<float> out(size_t(t.numel()));
    switch (t.dtype) {
      case SFQ_DT_F32: std::memcpy(out.data(), t.data, t.nbytes); break;
      case SFQ_DT_BF16:
        for (size_t i = 0; i < out.size(); ++i) {
          const uint32_t bits = uint32_t(reinterpret_cast<const uint16_t*>(t.data)[i]) << 16;
          std::memcpy(&out[i], &bits, 4);
        }
        break;
      case SFQ_DT_F16:
        for (size_t i = 0; i < out.size(); ++i) out[i] = half_to_float(reinterpret_cast<const uint16_t*>(t.data)[i]);
        break;
      case SFQ_DT_F64:
        for (size_t i = 0; i < out.size(); ++i) out[i] = float(reinterpret_cast<const double*>(t.data)[i]);
        break;
      default: throw std::runtime_error("checkpoint: '" + t.name + "' cannot be read as floating point");
    }
    return out;
  }
  const float* upload_f32(const std::string& name) {  // null when the tensor is absent
    const Tensor* t = find(name);
    if (t == nullptr) return nullptr;
    if (host_view) {
      auto hit = host_f32.find(name);
      if (hit == host_f32.end()) hit = host_f32.emplace(name, to_f32(*t)).first;
      return hit->second.data();
    }
    bind_device();
    const auto it = device_f32.find(name);
    if (it != device_f32.end()) return static_cast<const float*>(it->second);
    const std::vector<float> host = to_f32(*t);
    void* d = nullptr;
    check_cuda(cudaMalloc(&d, host.empty() ? 16 : host.size() * sizeof(float)), "cudaMalloc");
    if (!host.empty()) {
      const cudaError_t e = cudaMemcpy(d, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice);
      if (e != cudaSuccess) {
        cudaFree(d);
        check_cuda(e, "upload");
      }
    }
    device_f32.emplace(name, d);
    return static_cast<const float*>(d);
  }
  float host_scalar(const std::string& name) const {  // 0 when absent, as the reference
    const Tensor* t = find(name);
    if (t == nullptr) return 0.0f;
    const std::vector<float> v = to_f32(*t);
    return v.empty() ? 0.0f : v[0];
  }

  // ---- quantization_state (src/core/w4a8.cpp:47-70): the layer's own tag, else the header's table
  sfq::json::Value quant_state(const std::string& layer) const {
    if (const Tensor* local = find(layer + ".comfy_quant")) {
      if (local->dtype != SFQ_DT_U8 || local->shape.size() != 1)
        throw std::runtime_error("quantization: '" + layer + ".comfy_quant' is not rank-1 U8 JSON");
      std::string text(reinterpret_cast<const char*>(local->data), local->nbytes);
      while (!text.empty() && (text.back() == '\0' || text.back() == ' ' || text.back() == '\n')) text.pop_back();
      return text.empty() ? sfq::json::Value() : sfq::json::parse(text);
    }
    const std::string* table = meta("_quantization_metadata");
    if (table == nullptr) return {};
    const sfq::json::Value root = sfq::json::parse(*table);
    const sfq::json::Value* version = root.find("format_version");
    if (version == nullptr || version->as_string() != "1.0")
      throw std::runtime_error("unsupported checkpoint quantization metadata version");
    const sfq::json::Value* layers = root.find("layers");
    if (layers == nullptr || !layers->is_object()) throw std::runtime_error("invalid quantization layers metadata");
    const sfq::json::Value* entry = layers->find(layer);
    return entry != nullptr ? *entry : sfq::json::Value();
  }

  void linear(const std::string& name, int out_features, int in_features, sfq_quant_weight* w) {
    if (out_features <= 0 || in_features <= 0) throw std::invalid_argument("checkpoint: layer dimensions must be positive");
    sfq_quant_weight_init(w);
    const Tensor& v = at(name + ".weight");
    const size_t n = size_t(out_features) * size_t(in_features);
    w->out_features = out_features;
    w->in_features = in_features;
    const sfq::json::Value state = quant_state(name);
    const sfq::json::Value* fmt = state.find("format");
    const std::string format = fmt != nullptr ? fmt->as_string() : std::string();
    auto param = [&](const char* key) -> const sfq::json::Value* {  // top level, or under "params"
      if (const sfq::json::Value* x = state.find(key)) return x;
      if (const sfq::json::Value* p = state.find("params")) return p->find(key);
      return nullptr;
    };
    auto need_bytes = [&](const Tensor& t, size_t bytes) {
      if (t.nbytes != bytes)
        throw std::runtime_error("checkpoint: '" + t.name + "' has " + std::to_string(t.nbytes) + " bytes, the layer needs " +
                                 std::to_string(bytes));
    };

    if (format == "asym_w4a8_int8" || format == "w6a8_int8") {
      const sfq::json::Value* group = param("group_size");
      const sfq::json::Value* rotation = param("convrot_groupsize");
      if (group == nullptr || rotation == nullptr) throw std::runtime_error("checkpoint: incomplete packed INT8 state for '" + name + "'");
      if (const sfq::json::Value* enabled = param("convrot"); enabled != nullptr && !enabled->as_bool())
        throw std::runtime_error("W4A8/W6A8 requires ConvRot");
      const int bits = format == "w6a8_int8" ? 6 : 4;
      const int64_t g = group->as_int(), rot = rotation->as_int();
      if ((bits == 4 ? g != 16 : (g < 16 || g > 131072 || g % 16)) || rot != 256)
        throw std::runtime_error("checkpoint: unsupported packed INT8 layout for '" + name +
                                 "' (requires W4 group 16 or W6 group divisible by 16, and ConvRot 256)");
      if (size_t(in_features) % size_t(g) != 0) throw std::runtime_error("checkpoint: '" + name + "' rows are not whole groups");
      need_bytes(v, n * size_t(bits) / 8);
      need_bytes(at(name + ".weight_s_rel"), n / size_t(g));
      if (at(name + ".weight_s_channel").numel() != out_features)
        throw std::runtime_error("checkpoint: '" + name + ".weight_s_channel' needs one scale per output channel");
      w->format = bits == 6 ? SFQ_W6A8 : SFQ_W4A8;
      w->packed_group_size = uint32_t(g);
      w->data = upload(name + ".weight");
      w->block_scale = static_cast<const uint8_t*>(upload(name + ".weight_s_rel"));
      w->weight_scale = upload_f32(name + ".weight_s_channel");
      w->w4_codebook = upload_f32(name + ".weight_codebook");
      if (bits == 4 && (w->w4_codebook == nullptr || at(name + ".weight_codebook").numel() != 16))
        throw std::runtime_error("checkpoint: '" + name + "' is W4A8 and needs a 16-entry codebook");
      if (bits == 6 && w->w4_codebook != nullptr) throw std::runtime_error("checkpoint: '" + name + "' is W6A8 and must not ship a codebook");
      w->per_channel_scale = 1;
      w->convrot = 1;
      w->convrot_group = 256;
    } else if (find(name + ".weight.quant_state.bitsandbytes__nf4") != nullptr) {
      const Tensor& st = at(name + ".weight.quant_state.bitsandbytes__nf4");
      if (st.dtype != SFQ_DT_U8 || st.shape.size() != 1) throw std::runtime_error("checkpoint: '" + st.name + "' is not rank-1 U8 JSON");
      const sfq::json::Value nf4 = sfq::json::parse(std::string(reinterpret_cast<const char*>(st.data), st.nbytes));
      auto get = [&](const char* key) -> const sfq::json::Value& {
        const sfq::json::Value* x = nf4.find(key);
        if (x == nullptr) throw std::runtime_error(std::string("checkpoint: NF4 state missing '") + key + "'");
        return *x;
      };
      if (get("quant_type").as_string() != "nf4" || get("nested_dtype").as_string() != "float32")
        throw std::runtime_error("checkpoint: unsupported NF4 contract for '" + name + ".weight'");
      if (const sfq::json::Value* dt = nf4.find("dtype"); dt == nullptr || dt->as_string() != "bfloat16")
        throw std::runtime_error("checkpoint: NF4 source dtype must be bfloat16 for '" + name + ".weight'");
      const int64_t block = get("blocksize").as_int(), nested = get("nested_blocksize").as_int();
      const double offset = get("nested_offset").as_number();
      if (block != 64 || nested != 256 || !std::isfinite(offset))
        throw std::runtime_error("checkpoint: unsupported NF4 block layout for '" + name + ".weight'");
      need_bytes(v, (n + 1) / 2);
      need_bytes(at(name + ".weight.absmax"), (n + size_t(block) - 1) / size_t(block));
      w->format = SFQ_NF4;
      w->data = upload(name + ".weight");
      w->nf4_absmax = static_cast<const uint8_t*>(upload(name + ".weight.absmax"));
      w->nf4_quant_map = upload_f32(name + ".weight.quant_map");
      w->nf4_nested_absmax = upload_f32(name + ".weight.nested_absmax");
      w->nf4_nested_quant_map = upload_f32(name + ".weight.nested_quant_map");
      if (w->nf4_quant_map == nullptr || w->nf4_nested_absmax == nullptr || w->nf4_nested_quant_map == nullptr)
        throw std::runtime_error("checkpoint: '" + name + "' is NF4 without its complete double-quant state");
      w->nf4_block_size = int32_t(block);
      w->nf4_nested_block_size = int32_t(nested);
      w->nf4_nested_offset = float(offset);
    } else if (const Tensor* s = find(name + ".weight_scale");
               v.dtype == SFQ_DT_U8 && s != nullptr && s->dtype == SFQ_DT_F8E4M3 && s->shape.size() == 2 &&
               s->shape[1] == in_features / 16) {
      if (find(name + ".weight_scale_2") == nullptr)
        throw std::runtime_error("checkpoint: '" + name + ".weight' is nvfp4 but ships no weight_scale_2; the default 1.0 "
                                 "would be wrong by about 700x rather than visibly broken");
      need_bytes(v, n / 2);
      need_bytes(*s, n / 16);
      w->format = SFQ_NVFP4;
      w->data = upload(name + ".weight");
      w->block_scale = static_cast<const uint8_t*>(upload(name + ".weight_scale"));  // raw e4m3 bytes, 128x4 tiling
      w->global_scale = host_scalar(name + ".weight_scale_2");
    } else {
      switch (v.dtype) {
        case SFQ_DT_F32: w->format = SFQ_F32; break;
        case SFQ_DT_BF16: w->format = SFQ_BF16; break;
        case SFQ_DT_F16: w->format = SFQ_F16; break;
        case SFQ_DT_F8E4M3: w->format = SFQ_F8E4M3; break;
        case SFQ_DT_I8: w->format = SFQ_I8; break;
        default: throw std::runtime_error("checkpoint: tensor '" + name + ".weight' has a dtype no linear layer can consume");
      }
      need_bytes(v, n * dtype_bytes(v.dtype));
      w->data = upload(name + ".weight");
      w->weight_scale = upload_f32(name + ".weight_scale");
      if (w->format == SFQ_F8E4M3 && w->weight_scale == nullptr)
        throw std::runtime_error("checkpoint: '" + name + ".weight' is fp8 but ships no weight_scale");
      if (w->format == SFQ_I8 && (w->weight_scale == nullptr || at(name + ".weight_scale").numel() != out_features))
        throw std::runtime_error("checkpoint: '" + name + ".weight' is int8 but ships no per-channel weight_scale");
      w->per_channel_scale = w->format == SFQ_I8 ? 1 : 0;
    }
    w->input_scale = host_scalar(name + ".input_scale");

    // read_comfy_quant: what the file says about matrix-multiply precision and the rotation
    if (!state.is_null()) {
      if (format != "nvfp4" && format != "float8_e4m3fn" && format != "int8_tensorwise" && format != "asym_w4a8_int8" &&
          format != "w6a8_int8")
        throw std::runtime_error("checkpoint: '" + name + "' declares quant format '" + format + "', which is not implemented");
      if (const sfq::json::Value* p = state.find("full_precision_matrix_mult")) w->full_precision = p->as_bool() ? 1 : 0;
      bool rotate = false;
      int rotation_group = 256;
      if (const sfq::json::Value* c = state.find("convrot")) rotate = c->as_bool();
      if (const sfq::json::Value* g = state.find("convrot_groupsize")) {
        const int64_t value = g->as_int();
        if (value <= 0 || value > 256) throw std::runtime_error("checkpoint: '" + name + ".comfy_quant' has invalid convrot_groupsize");
        rotation_group = int(value);
      }
      if (rotate) {
        int power = 1;
        while (power < rotation_group) power *= 4;
        const bool compatible = (format == "int8_tensorwise" && w->format == SFQ_I8) ||
                                (format == "asym_w4a8_int8" && w->format == SFQ_W4A8) ||
                                (format == "w6a8_int8" && w->format == SFQ_W6A8);
        if (!compatible || power != rotation_group) throw std::runtime_error("checkpoint: '" + name + "' has incompatible ConvRot metadata");
        // the quantizer leaves a contraction axis that is not a multiple of the group unrotated: same rule here
        w->convrot = in_features % rotation_group == 0 ? 1 : 0;
        w->convrot_group = rotation_group;
      }
    }
  }
};

namespace {
template <class F> int guarded(F&& f) {
  return sfq_capi::run_guarded([](void* p) { (*static_cast<F*>(p))(); }, &f);
}
}  // namespace

extern "C" {

int sfq_checkpoint_open(const char* path, sfq_checkpoint** out) {
  return guarded([&] {
    if (path == nullptr || out == nullptr) throw std::invalid_argument("sfq_checkpoint_open: null argument");
    *out = nullptr;
    auto* c = new sfq_checkpoint();
    try {
      c->open(path);
    } catch (...) {
      delete c;
      throw;
    }
    *out = c;
  });
}

void sfq_checkpoint_close(sfq_checkpoint* c) { delete c; }

int sfq_checkpoint_count(const sfq_checkpoint* c) { return c != nullptr ? int(c->tensors.size()) : 0; }

int sfq_checkpoint_tensor(const sfq_checkpoint* c, const char* name, int32_t* dtype, int32_t* rank, int64_t* shape8,
                          const void** h_data, size_t* nbytes) {
  return guarded([&] {
    if (c == nullptr || name == nullptr) throw std::invalid_argument("sfq_checkpoint_tensor: null argument");
    const Tensor& t = c->at(name);
    if (t.shape.size() > 8) throw std::runtime_error("checkpoint: more than 8 dimensions");
    if (dtype) *dtype = t.dtype;
    if (rank) *rank = int32_t(t.shape.size());
    if (shape8)
      for (size_t i = 0; i < t.shape.size(); ++i) shape8[i] = t.shape[i];
    if (h_data) *h_data = t.data;
    if (nbytes) *nbytes = t.nbytes;
  });
}

int sfq_checkpoint_metadata(const sfq_checkpoint* c, const char* key, char* buffer, size_t capacity, size_t* length) {
  return guarded([&] {
    if (c == nullptr || key == nullptr) throw std::invalid_argument("sfq_checkpoint_metadata: null argument");
    const std::string* v = c->meta(key);
    if (v == nullptr) throw std::runtime_error(std::string("checkpoint: no metadata entry '") + key + "'");
    if (length) *length = v->size();
    if (buffer != nullptr && capacity > 0) {
      const size_t k = v->size() < capacity - 1 ? v->size() : capacity - 1;
      std::memcpy(buffer, v->data(), k);
      buffer[k] = '\0';
    }
  });
}

int sfq_checkpoint_linear(sfq_checkpoint* c, const char* name, int out_features, int in_features, sfq_quant_weight* out) {
  return guarded([&] {
    if (c == nullptr || name == nullptr || out == nullptr) throw std::invalid_argument("sfq_checkpoint_linear: null argument");
    std::lock_guard<std::mutex> lock(c->mutex);
    c->host_view = false;
    c->linear(name, out_features, in_features, out);
  });
}

int sfq_checkpoint_linear_host(sfq_checkpoint* c, const char* name, int out_features, int in_features, sfq_quant_weight* out) {
  return guarded([&] {
    if (c == nullptr || name == nullptr || out == nullptr) throw std::invalid_argument("sfq_checkpoint_linear_host: null argument");
    std::lock_guard<std::mutex> lock(c->mutex);
    c->host_view = true;
    c->linear(name, out_features, in_features, out);
  });
}

}  // extern "C"
