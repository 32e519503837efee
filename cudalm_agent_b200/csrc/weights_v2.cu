// Reader of CUDALM's `.cudalm` v2 weight container (normative layout:
// CUDALM include/cudalm/weight_format_v2.h:35-190; reference reader
// src/runtime/weight_loader_v2.cpp:49-242).  Host code: parse, validate, look
// tensors up by name, upload a tensor to device memory.  Every rule the
// reference's reader enforces is enforced here, so a file one accepts the other
// accepts too:
//
//   header (88 bytes, little endian): magic "CUDLMW02", version 2, flags 0,
//   num_tensors <= 100000, num_metadata <= 256, pad 0, then offset/size pairs of
//   the config (size exactly 88), metadata, tensor-table and payload sections.
//   Sections lie inside the file and do not overlap; the payload starts on a
//   16-byte boundary.  The config blob's reserved word is 0 and its fields pass
//   the model-configuration checks.  Metadata and table are consumed exactly
//   (no trailing bytes).  Tensor names are 1..255 characters of [A-Za-z0-9._-],
//   unique; dtype 1..5; 1..8 dims, each in 1..1e8, unused dims 0; pads 0; align
//   a power of two <= 16 that the tensor's file position honours; the tensor
//   lies inside the payload and its byte size equals what dtype and dims imply
//   (int4_packed dims are in packed bytes).
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace {

constexpr std::size_t kHeader = 88, kConfig = 88, kEntryTail = 1 + 1 + 2 + 64 + 8 + 8 + 1 + 1;

std::uint16_t u16_at(const std::uint8_t* p) { std::uint16_t v; std::memcpy(&v, p, 2); return v; }
std::uint32_t u32_at(const std::uint8_t* p) { std::uint32_t v; std::memcpy(&v, p, 4); return v; }
std::uint64_t u64_at(const std::uint8_t* p) { std::uint64_t v; std::memcpy(&v, p, 8); return v; }
std::int32_t i32_at(const std::uint8_t* p) { std::int32_t v; std::memcpy(&v, p, 4); return v; }
float f32_at(const std::uint8_t* p) { float v; std::memcpy(&v, p, 4); return v; }

int element_bytes(int dtype) {  // CUDALM include/cudalm/weight_format.h: Dtype
  switch (dtype) {
    case CUDALM_B200_V2_FP16: return 2;
    case CUDALM_B200_V2_INT4_PACKED: return 1;
    case CUDALM_B200_V2_FP16_SCALE: return 2;
    case CUDALM_B200_V2_FP32: return 4;
    case CUDALM_B200_V2_BF16: return 2;
    default: return 0;
  }
}

// The model-configuration checks of CUDALM include/cudalm/qwen35_config.h:90-116.
bool config_ok(const std::uint8_t* c) {
  const int hidden = i32_at(c + 0), layers = i32_at(c + 4), inter = i32_at(c + 8);
  const int heads = i32_at(c + 16), kv_heads = i32_at(c + 20), head_dim = i32_at(c + 24);
  const int lin_k = i32_at(c + 28), lin_v = i32_at(c + 32), lin_kd = i32_at(c + 36), lin_vd = i32_at(c + 40);
  const int conv = i32_at(c + 44), interval = i32_at(c + 48), group = i32_at(c + 52), max_seq = i32_at(c + 56);
  const float eps = f32_at(c + 60), theta = f32_at(c + 64), rotary = f32_at(c + 68);
  const int sections = i32_at(c + 72) + i32_at(c + 76) + i32_at(c + 80);
  if (hidden <= 0 || layers <= 0 || inter <= 0) return false;
  if (heads <= 0 || kv_heads <= 0 || head_dim <= 0 || heads % kv_heads != 0) return false;
  if (lin_k <= 0 || lin_v <= 0 || lin_v % lin_k != 0 || lin_kd <= 0 || lin_vd <= 0) return false;
  if (conv < 2 || interval < 2 || group <= 0 || max_seq <= 0) return false;
  if (!(eps > 0.0f) || !(theta > 0.0f)) return false;
  const int rotary_dim = static_cast<int>(head_dim * rotary + 0.5f);
  if (rotary_dim <= 0 || rotary_dim > head_dim || rotary_dim % 2 != 0) return false;
  if (sections != rotary_dim / 2) return false;
  if (hidden % group != 0 || (heads * head_dim) % group != 0 || inter % group != 0) return false;
  if ((lin_v * lin_vd) % group != 0) return false;
  return true;
}

struct Entry {
  std::string name;
  int dtype = 0, ndim = 0, align = 0;
  long long dims[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  std::uint64_t offset = 0, byte_size = 0;
};

}  // namespace

struct cudalm_b200_v2_file {
  std::vector<std::uint8_t> bytes;
  std::uint64_t payload_offset = 0, payload_size = 0, config_offset = 0;
  std::vector<Entry> tensors;
  std::unordered_map<std::string, int> by_name;
  std::vector<std::pair<std::string, std::string>> metadata;
};

namespace {

// Parses `f->bytes`; on failure returns false with the reason in `why`.
bool parse(cudalm_b200_v2_file* f, std::string* why) {
  auto fail = [&](const std::string& m) {
    *why = m;
    return false;
  };
  const std::uint8_t* p = f->bytes.data();
  const std::uint64_t n = f->bytes.size();
  if (n < kHeader) return fail("file too small for the header");
  if (std::memcmp(p, "CUDLMW02", 8) != 0) return fail("bad magic");
  if (u32_at(p + 8) != 2) return fail("unsupported version");
  if (u32_at(p + 12) != 0) return fail("reserved flags must be 0");
  const std::uint32_t n_tensors = u32_at(p + 16);
  const std::uint16_t n_meta = u16_at(p + 20);
  if (u16_at(p + 22) != 0) return fail("reserved pad must be 0");
  std::uint64_t sec[4][2];  // config, metadata, table, payload: {offset, size}
  for (int s = 0; s < 4; ++s) {
    sec[s][0] = u64_at(p + 24 + 16 * s);
    sec[s][1] = u64_at(p + 32 + 16 * s);
  }
  if (n_tensors > 100000) return fail("num_tensors exceeds limit");
  if (n_meta > 256) return fail("num_metadata exceeds limit");
  if (sec[0][1] != kConfig) return fail("config_size must be 88");
  static const char* const kSection[4] = {"config", "metadata", "tensor table", "payload"};
  for (int s = 0; s < 4; ++s)
    if (sec[s][0] > n || sec[s][1] > n - sec[s][0]) return fail(std::string(kSection[s]) + " section out of bounds");
  if (sec[3][0] % 16 != 0) return fail("payload_offset must be 16-byte aligned");
  for (int a = 0; a < 4; ++a)
    for (int b = a + 1; b < 4; ++b)
      if (sec[a][0] < sec[b][0] + sec[b][1] && sec[b][0] < sec[a][0] + sec[a][1]) return fail("sections overlap");

  const std::uint8_t* cfg = p + sec[0][0];
  if (u32_at(cfg + 84) != 0) return fail("config blob reserved word must be 0");
  if (!config_ok(cfg)) return fail("config blob failed validation");
  f->config_offset = sec[0][0];

  {
    std::uint64_t pos = sec[1][0];
    const std::uint64_t end = sec[1][0] + sec[1][1];
    for (int i = 0; i < n_meta; ++i) {
      if (pos + 1 > end) return fail("metadata: key length out of bounds");
      const std::uint64_t klen = p[pos++];
      if (pos + klen + 2 > end) return fail("metadata: key out of bounds");
      std::string key(reinterpret_cast<const char*>(p + pos), klen);
      pos += klen;
      const std::uint64_t vlen = u16_at(p + pos);
      pos += 2;
      if (vlen > 4096) return fail("metadata: value too long for '" + key + "'");
      if (pos + vlen > end) return fail("metadata: value out of bounds for '" + key + "'");
      f->metadata.emplace_back(std::move(key), std::string(reinterpret_cast<const char*>(p + pos), vlen));
      pos += vlen;
    }
    if (pos != end) return fail("metadata: trailing bytes");
  }

  f->payload_offset = sec[3][0];
  f->payload_size = sec[3][1];
  std::uint64_t pos = sec[2][0];
  const std::uint64_t end = sec[2][0] + sec[2][1];
  for (std::uint32_t i = 0; i < n_tensors; ++i) {
    Entry e;
    if (pos + 1 > end) return fail("tensor table: name length out of bounds");
    const std::uint64_t nlen = p[pos++];
    if (nlen == 0) return fail("tensor table: empty name");
    if (pos + nlen + kEntryTail > end) return fail("tensor table: entry out of bounds");
    e.name.assign(reinterpret_cast<const char*>(p + pos), nlen);
    pos += nlen;
    for (char ch : e.name) {
      const bool ok = (ch >= 'A' && ch <= 'Z') || (ch >= 'a' && ch <= 'z') || (ch >= '0' && ch <= '9') ||
                      ch == '.' || ch == '_' || ch == '-';
      if (!ok) return fail("tensor table: bad character in name '" + e.name + "'");
    }
    if (f->by_name.count(e.name)) return fail("duplicate tensor name '" + e.name + "'");
    e.dtype = p[pos++];
    if (element_bytes(e.dtype) == 0) return fail("bad dtype in tensor '" + e.name + "'");
    e.ndim = p[pos++];
    if (e.ndim < 1 || e.ndim > 8) return fail("bad ndim in tensor '" + e.name + "'");
    if (u16_at(p + pos) != 0) return fail("tensor '" + e.name + "': reserved pad must be 0");
    pos += 2;
    std::uint64_t expect = static_cast<std::uint64_t>(element_bytes(e.dtype));
    for (int d = 0; d < 8; ++d) {
      const long long v = static_cast<long long>(u64_at(p + pos + 8 * d));
      if (d < e.ndim) {
        if (v <= 0 || v > 100000000ll) return fail("bad dim in tensor '" + e.name + "'");
        e.dims[d] = v;
        // dims <= 1e8 and the running product is checked against the payload below
        if (expect > (~0ull) / static_cast<std::uint64_t>(v)) return fail("tensor '" + e.name + "': size overflows");
        expect *= static_cast<std::uint64_t>(v);
      } else if (v != 0) {
        return fail("tensor '" + e.name + "': unused dim must be 0");
      }
    }
    pos += 64;
    e.offset = u64_at(p + pos);
    e.byte_size = u64_at(p + pos + 8);
    pos += 16;
    e.align = p[pos++];
    if (p[pos++] != 0) return fail("tensor '" + e.name + "': reserved pad must be 0");
    if (!(e.align == 1 || e.align == 2 || e.align == 4 || e.align == 8 || e.align == 16))
      return fail("tensor '" + e.name + "': bad align");
    if (e.offset > f->payload_size || e.byte_size > f->payload_size - e.offset)
      return fail("tensor '" + e.name + "' out of payload bounds");
    if ((f->payload_offset + e.offset) % static_cast<std::uint64_t>(e.align) != 0)
      return fail("tensor '" + e.name + "' misses its alignment");
    if (e.byte_size != expect) return fail("tensor '" + e.name + "': byte_size does not match dtype and dims");
    f->by_name.emplace(e.name, static_cast<int>(f->tensors.size()));
    f->tensors.push_back(std::move(e));
  }
  if (pos != end) return fail("tensor table: trailing bytes");
  return true;
}

void put_error(char* err, size_t cap, const std::string& m) {
  if (!err || cap == 0) return;
  const size_t k = m.size() < cap - 1 ? m.size() : cap - 1;
  std::memcpy(err, m.data(), k);
  err[k] = 0;
}

}  // namespace

extern "C" {

int cudalm_b200_v2_open(const char* path, cudalm_b200_v2_file** out, char* err, size_t err_cap) {
  if (!path || !out) return CUDALM_B200_ERR_NULL;
  *out = nullptr;
  std::FILE* fp = std::fopen(path, "rb");
  if (!fp) {
    put_error(err, err_cap, std::string("cannot open ") + path);
    return CUDALM_B200_ERR_FILE;
  }
  cudalm_b200_v2_file* f = new cudalm_b200_v2_file();
  bool ok = std::fseek(fp, 0, SEEK_END) == 0;
  const long sz = ok ? std::ftell(fp) : -1;
  ok = ok && sz >= 0;
  if (ok) {
    std::rewind(fp);
    f->bytes.resize(static_cast<size_t>(sz));
    ok = sz == 0 || std::fread(f->bytes.data(), 1, f->bytes.size(), fp) == f->bytes.size();
  }
  std::fclose(fp);
  std::string why = "read failed";
  if (!ok || !parse(f, &why)) {
    put_error(err, err_cap, why);
    delete f;
    return CUDALM_B200_ERR_FILE;
  }
  *out = f;
  return CUDALM_B200_OK;
}

void cudalm_b200_v2_close(cudalm_b200_v2_file* f) { delete f; }

int cudalm_b200_v2_num_tensors(const cudalm_b200_v2_file* f) { return f ? static_cast<int>(f->tensors.size()) : -1; }
int cudalm_b200_v2_num_metadata(const cudalm_b200_v2_file* f) { return f ? static_cast<int>(f->metadata.size()) : -1; }

int cudalm_b200_v2_tensor_at(const cudalm_b200_v2_file* f, int i, cudalm_b200_v2_tensor* t) {
  if (!f || !t) return CUDALM_B200_ERR_NULL;
  if (i < 0 || i >= static_cast<int>(f->tensors.size())) return CUDALM_B200_ERR_BAD_SHAPE;
  const Entry& e = f->tensors[static_cast<size_t>(i)];
  t->name = e.name.c_str();
  t->dtype = e.dtype;
  t->ndim = e.ndim;
  for (int d = 0; d < 8; ++d) t->dims[d] = e.dims[d];
  t->offset = e.offset;
  t->byte_size = e.byte_size;
  t->align = e.align;
  t->reserved = 0;
  t->host_bytes = f->bytes.data() + f->payload_offset + e.offset;
  return CUDALM_B200_OK;
}

int cudalm_b200_v2_find(const cudalm_b200_v2_file* f, const char* name) {
  if (!f || !name) return -1;
  const auto it = f->by_name.find(name);
  return it == f->by_name.end() ? -1 : it->second;
}

int cudalm_b200_v2_config_blob(const cudalm_b200_v2_file* f, uint8_t* out88) {
  if (!f || !out88) return CUDALM_B200_ERR_NULL;
  std::memcpy(out88, f->bytes.data() + f->config_offset, kConfig);
  return CUDALM_B200_OK;
}

int cudalm_b200_v2_metadata_at(const cudalm_b200_v2_file* f, int i, const char** key, const char** value) {
  if (!f || !key || !value) return CUDALM_B200_ERR_NULL;
  if (i < 0 || i >= static_cast<int>(f->metadata.size())) return CUDALM_B200_ERR_BAD_SHAPE;
  *key = f->metadata[static_cast<size_t>(i)].first.c_str();
  *value = f->metadata[static_cast<size_t>(i)].second.c_str();
  return CUDALM_B200_OK;
}

int cudalm_b200_v2_upload(const cudalm_b200_v2_file* f, int i, void* device_dst, size_t capacity,
                          void* stream) {
  if (!f || !device_dst) return CUDALM_B200_ERR_NULL;
  if (i < 0 || i >= static_cast<int>(f->tensors.size())) return CUDALM_B200_ERR_BAD_SHAPE;
  const Entry& e = f->tensors[static_cast<size_t>(i)];
  if (capacity < e.byte_size) return CUDALM_B200_ERR_TOO_LARGE;
  using namespace cb200;
  CB200_CUDA_TRY(cudaMemcpyAsync(device_dst, f->bytes.data() + f->payload_offset + e.offset, e.byte_size,
                                 cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  return CUDALM_B200_OK;
}

int cudalm_b200_v2_linear(const cudalm_b200_v2_file* f, const char* weight_name, const char* scale_name,
                          int* weight_index, int* scale_index, int* N, int* K) {
  if (!f || !weight_name || !scale_name) return CUDALM_B200_ERR_NULL;
  const int wi = cudalm_b200_v2_find(f, weight_name), si = cudalm_b200_v2_find(f, scale_name);
  if (wi < 0 || si < 0) return CUDALM_B200_ERR_FILE;
  const Entry& w = f->tensors[static_cast<size_t>(wi)];
  const Entry& s = f->tensors[static_cast<size_t>(si)];
  // weight [N, K/2] packed bytes, scale [N, K/128] (CUDALM include/cudalm/weight_loader.h:58-63)
  if (w.dtype != CUDALM_B200_V2_INT4_PACKED || s.dtype != CUDALM_B200_V2_FP16_SCALE) return CUDALM_B200_ERR_FILE;
  if (w.ndim != 2 || s.ndim != 2 || w.dims[0] != s.dims[0]) return CUDALM_B200_ERR_FILE;
  if (w.dims[1] % 64 != 0 || s.dims[1] * 64 != w.dims[1]) return CUDALM_B200_ERR_FILE;
  if (weight_index) *weight_index = wi;
  if (scale_index) *scale_index = si;
  if (N) *N = static_cast<int>(w.dims[0]);
  if (K) *K = static_cast<int>(w.dims[1] * 2);
  return CUDALM_B200_OK;
}

// ---------------------------------------------------------------------------
// Model-level loading: the tensor set of one decoder layer, checked against the
// file's configuration and uploaded (CUDALM src/runtime/weight_loader_v2.cpp:
// validate_layer 273-372, validate_full_model 383-408, Qwen35LayerWeights::load
// 416-499).
// ---------------------------------------------------------------------------
}  // extern "C"

namespace {

struct ModelConfig {
  int hidden, layers, inter, vocab, heads, kv_heads, head_dim;
  int lin_k_heads, lin_v_heads, lin_kd, lin_vd, conv, interval, group;
};

ModelConfig read_config(const cudalm_b200_v2_file* f) {
  const std::uint8_t* c = f->bytes.data() + f->config_offset;
  ModelConfig m;
  m.hidden = i32_at(c + 0);
  m.layers = i32_at(c + 4);
  m.inter = i32_at(c + 8);
  m.vocab = i32_at(c + 12);
  m.heads = i32_at(c + 16);
  m.kv_heads = i32_at(c + 20);
  m.head_dim = i32_at(c + 24);
  m.lin_k_heads = i32_at(c + 28);
  m.lin_v_heads = i32_at(c + 32);
  m.lin_kd = i32_at(c + 36);
  m.lin_vd = i32_at(c + 40);
  m.conv = i32_at(c + 44);
  m.interval = i32_at(c + 48);
  m.group = i32_at(c + 52);
  return m;
}

// CUDALM include/cudalm/qwen35_config.h:82-85
bool is_full_attention(const ModelConfig& c, int i) {
  return i >= 0 && i < c.layers && c.interval > 0 && (i + 1) % c.interval == 0;
}

const char* dtype_name(int dtype) {
  switch (dtype) {
    case CUDALM_B200_V2_FP16: return "fp16";
    case CUDALM_B200_V2_INT4_PACKED: return "int4_packed";
    case CUDALM_B200_V2_FP16_SCALE: return "fp16_scale";
    case CUDALM_B200_V2_FP32: return "fp32";
    case CUDALM_B200_V2_BF16: return "bf16";
    default: return "?";
  }
}

// One tensor a layer must hold.  `proj` >= 0: the weight (part 0) or scale (part 1)
// of that projection; else `aux` >= 0: one of the layer's other tensors.
struct Expect {
  std::string name;
  int dtype;
  std::vector<long long> dims;
  int proj, part, aux;
};

// The layer's tensors in the order the reference checks them, so that the first
// fault found is the one it reports.
std::vector<Expect> layer_expectations(const ModelConfig& c, int layer) {
  const std::string L = "layers." + std::to_string(layer) + ".";
  const long long H = c.hidden, G = c.group;
  std::vector<Expect> out;
  auto aux = [&](const char* n, int dtype, std::vector<long long> dims, int slot) {
    out.push_back(Expect{L + n, dtype, std::move(dims), -1, 0, slot});
  };
  auto weight = [&](const char* n, long long N, long long K, int proj) {
    out.push_back(Expect{L + n + ".weight", CUDALM_B200_V2_INT4_PACKED, {N, K / 2}, proj, 0, -1});
  };
  auto scale = [&](const char* n, long long N, long long K, int proj) {
    out.push_back(Expect{L + n + ".scale", CUDALM_B200_V2_FP16_SCALE, {N, K / G}, proj, 1, -1});
  };
  aux("input_layernorm.weight", CUDALM_B200_V2_BF16, {H}, CUDALM_B200_AUX_INPUT_LAYERNORM);
  aux("post_attention_layernorm.weight", CUDALM_B200_V2_BF16, {H}, CUDALM_B200_AUX_POST_ATTENTION_LAYERNORM);
  weight("mlp.gate_proj", c.inter, H, CUDALM_B200_PROJ_GATE);
  weight("mlp.up_proj", c.inter, H, CUDALM_B200_PROJ_UP);
  scale("mlp.gate_proj", c.inter, H, CUDALM_B200_PROJ_GATE);
  scale("mlp.up_proj", c.inter, H, CUDALM_B200_PROJ_UP);
  weight("mlp.down_proj", H, c.inter, CUDALM_B200_PROJ_DOWN);
  scale("mlp.down_proj", H, c.inter, CUDALM_B200_PROJ_DOWN);
  if (is_full_attention(c, layer)) {
    const long long qo = 2ll * c.heads * c.head_dim, kvo = 1ll * c.kv_heads * c.head_dim;
    const long long oin = 1ll * c.heads * c.head_dim;
    weight("self_attn.q_proj", qo, H, CUDALM_B200_PROJ_Q);
    scale("self_attn.q_proj", qo, H, CUDALM_B200_PROJ_Q);
    weight("self_attn.k_proj", kvo, H, CUDALM_B200_PROJ_K);
    scale("self_attn.k_proj", kvo, H, CUDALM_B200_PROJ_K);
    weight("self_attn.v_proj", kvo, H, CUDALM_B200_PROJ_V);
    scale("self_attn.v_proj", kvo, H, CUDALM_B200_PROJ_V);
    weight("self_attn.o_proj", H, oin, CUDALM_B200_PROJ_O);
    scale("self_attn.o_proj", H, oin, CUDALM_B200_PROJ_O);
    aux("self_attn.q_norm.weight", CUDALM_B200_V2_BF16, {c.head_dim}, CUDALM_B200_AUX_Q_NORM);
    aux("self_attn.k_norm.weight", CUDALM_B200_V2_BF16, {c.head_dim}, CUDALM_B200_AUX_K_NORM);
  } else {
    const long long cv = 1ll * c.lin_v_heads * c.lin_vd;
    const long long cd = 2ll * c.lin_k_heads * c.lin_kd + cv;
    weight("linear_attn.in_proj_qkv", cd, H, CUDALM_B200_PROJ_IN_QKV);
    scale("linear_attn.in_proj_qkv", cd, H, CUDALM_B200_PROJ_IN_QKV);
    weight("linear_attn.in_proj_z", cv, H, CUDALM_B200_PROJ_IN_Z);
    scale("linear_attn.in_proj_z", cv, H, CUDALM_B200_PROJ_IN_Z);
    weight("linear_attn.in_proj_b", c.lin_v_heads, H, CUDALM_B200_PROJ_IN_B);
    scale("linear_attn.in_proj_b", c.lin_v_heads, H, CUDALM_B200_PROJ_IN_B);
    weight("linear_attn.in_proj_a", c.lin_v_heads, H, CUDALM_B200_PROJ_IN_A);
    scale("linear_attn.in_proj_a", c.lin_v_heads, H, CUDALM_B200_PROJ_IN_A);
    weight("linear_attn.out_proj", H, cv, CUDALM_B200_PROJ_OUT);
    scale("linear_attn.out_proj", H, cv, CUDALM_B200_PROJ_OUT);
    aux("linear_attn.conv1d.weight", CUDALM_B200_V2_BF16, {cd, 1, c.conv}, CUDALM_B200_AUX_CONV1D);
    aux("linear_attn.dt_bias", CUDALM_B200_V2_BF16, {c.lin_v_heads}, CUDALM_B200_AUX_DT_BIAS);
    aux("linear_attn.A_log", CUDALM_B200_V2_FP32, {c.lin_v_heads}, CUDALM_B200_AUX_A_LOG);
    aux("linear_attn.norm.weight", CUDALM_B200_V2_FP32, {c.lin_vd}, CUDALM_B200_AUX_LINEAR_NORM);
  }
  return out;
}

// The reference's expect_tensor: empty string when the tensor is as expected.
std::string check_tensor(const cudalm_b200_v2_file* f, const std::string& name, int dtype,
                         const std::vector<long long>& dims, int* index) {
  const auto it = f->by_name.find(name);
  if (it == f->by_name.end()) return "missing tensor '" + name + "'";
  const Entry& e = f->tensors[static_cast<size_t>(it->second)];
  if (e.dtype != dtype) return "dtype mismatch for '" + name + "' (expected " + dtype_name(dtype) + ")";
  bool same = e.ndim == static_cast<int>(dims.size());
  for (int d = 0; same && d < e.ndim; ++d) same = e.dims[d] == dims[static_cast<size_t>(d)];
  if (!same) return "shape mismatch for '" + name + "' (expected " + std::to_string(dims.size()) + "-D)";
  if (index) *index = it->second;
  return std::string();
}

std::string validate_layer_impl(const cudalm_b200_v2_file* f, int layer, std::vector<int>* indices) {
  const ModelConfig c = read_config(f);
  if (layer < 0 || layer >= c.layers) return "layer_idx out of range";
  const std::vector<Expect> want = layer_expectations(c, layer);
  if (indices) indices->assign(want.size(), -1);
  for (size_t i = 0; i < want.size(); ++i) {
    const std::string why =
        check_tensor(f, want[i].name, want[i].dtype, want[i].dims, indices ? &(*indices)[i] : nullptr);
    if (!why.empty()) return why;
  }
  return std::string();
}

constexpr std::uint64_t kSlotAlign = 256;  // as CUDALM's DeviceBuffer (include/cudalm/device_buffer.h:17-68)
std::uint64_t slot_bytes(std::uint64_t n) { return (n + kSlotAlign - 1) / kSlotAlign * kSlotAlign; }

}  // namespace

extern "C" {

int cudalm_b200_v2_validate_layer(const cudalm_b200_v2_file* f, int layer_idx, char* err, size_t err_cap) {
  if (!f) return CUDALM_B200_ERR_NULL;
  const std::string why = validate_layer_impl(f, layer_idx, nullptr);
  if (why.empty()) return CUDALM_B200_OK;
  put_error(err, err_cap, why);
  return CUDALM_B200_ERR_FILE;
}

int cudalm_b200_v2_validate_full_model(const cudalm_b200_v2_file* f, char* err, size_t err_cap) {
  if (!f) return CUDALM_B200_ERR_NULL;
  const ModelConfig c = read_config(f);
  std::string why = check_tensor(f, "embed_tokens.weight", CUDALM_B200_V2_BF16, {c.vocab, c.hidden}, nullptr);
  if (why.empty()) why = check_tensor(f, "norm.weight", CUDALM_B200_V2_BF16, {c.hidden}, nullptr);
  for (int i = 0; why.empty() && i < c.layers; ++i) {
    why = validate_layer_impl(f, i, nullptr);
    if (!why.empty()) why = "layer " + std::to_string(i) + ": " + why;
  }
  if (why.empty()) {
    // the vocabulary projection is tied to the embedding in the model this format carries
    bool tied = false;
    for (const auto& kv : f->metadata) tied |= kv.first == "tie_word_embeddings" && kv.second == "true";
    if (!tied) why = "full model: tie_word_embeddings metadata must be \"true\"";
  }
  if (why.empty()) return CUDALM_B200_OK;
  put_error(err, err_cap, why);
  return CUDALM_B200_ERR_FILE;
}

size_t cudalm_b200_v2_layer_device_bytes(const cudalm_b200_v2_file* f, int layer_idx) {
  if (!f) return 0;
  std::vector<int> idx;
  if (!validate_layer_impl(f, layer_idx, &idx).empty()) return 0;
  std::uint64_t total = 0;
  for (int i : idx) total += slot_bytes(f->tensors[static_cast<size_t>(i)].byte_size);
  return static_cast<size_t>(total);
}

int cudalm_b200_v2_load_layer(const cudalm_b200_v2_file* f, int layer_idx, void* device_dst, size_t capacity,
                              void* stream, cudalm_b200_v2_layer* out, char* err, size_t err_cap) {
  if (!f || !device_dst || !out) return CUDALM_B200_ERR_NULL;
  std::vector<int> idx;
  const std::string why = validate_layer_impl(f, layer_idx, &idx);
  if (!why.empty()) {
    put_error(err, err_cap, why);
    return CUDALM_B200_ERR_FILE;
  }
  if ((reinterpret_cast<std::uintptr_t>(device_dst) & (kSlotAlign - 1)) != 0) return CUDALM_B200_ERR_MISALIGNED;
  const ModelConfig c = read_config(f);
  const std::vector<Expect> want = layer_expectations(c, layer_idx);
  std::uint64_t total = 0;
  for (int i : idx) total += slot_bytes(f->tensors[static_cast<size_t>(i)].byte_size);
  if (capacity < total) return CUDALM_B200_ERR_TOO_LARGE;
  std::memset(out, 0, sizeof(*out));
  out->layer_idx = layer_idx;
  out->full_attention = is_full_attention(c, layer_idx) ? 1 : 0;
  std::uint8_t* dst = static_cast<std::uint8_t*>(device_dst);
  std::uint64_t off = 0;
  using namespace cb200;
  for (size_t i = 0; i < want.size(); ++i) {
    const Entry& e = f->tensors[static_cast<size_t>(idx[i])];
    CB200_CUDA_TRY(cudaMemcpyAsync(dst + off, f->bytes.data() + f->payload_offset + e.offset, e.byte_size,
                                   cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    if (want[i].proj >= 0) {
      cudalm_b200_linear& l = out->proj[want[i].proj];
      if (want[i].part == 0) {
        l.weight = dst + off;
        // CUDALM src/runtime/weight_loader_v2.cpp:479-482: N = dim 0, K = 2 * dim 1
        l.N = static_cast<int32_t>(e.dims[0]);
        l.K = static_cast<int32_t>(2 * e.dims[1]);
      } else {
        l.scales = reinterpret_cast<const uint16_t*>(dst + off);
      }
    } else {
      out->aux[want[i].aux] = dst + off;
      out->aux_dtype[want[i].aux] = e.dtype;
      out->aux_bytes[want[i].aux] = e.byte_size;
    }
    off += slot_bytes(e.byte_size);
  }
  return CUDALM_B200_OK;
}

}  // extern "C"
