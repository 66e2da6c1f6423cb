// files.cu -- expert tensors straight from the engine's model files (host code only).
//
// hgn ("HGN1", the engine's own container; layout read by Checkpoint::map_file,
// src/hgn.h:48-62, 295-363): a 104-byte header {magic, version, tensor_count, reserved,
// records_offset, data_offset, file_size, model_name[64]}, then tensor_count records of 160
// bytes {name[96], dtype, ndims, dims[4], data_offset (from the start of the file), data_size,
// extra}. dtype 5 = q4cp blob, dtype 0 = bf16. The MoE tensors of layer L are
//   layers.L.mlp.experts.gate_up_proj.weight [E*2*mid, d], ...down_proj.weight [E*d, mid],
//   layers.L.mlp.gate.weight [E, d] (router), and with a shared expert
//   layers.L.mlp.shared_expert.{gate_proj,up_proj,down_proj}.weight, ...shared_expert_gate.weight
// (src/ref.cpp:566-633).
//
// GGUF v2/v3 (layout facts in src/gguf.h:1-11, parser src/gguf.h:136-314): header {magic,
// version, tensor_count, kv_count}, kv_count typed key/value pairs, tensor_count tensor infos
// {name, n_dims, dims, type, offset}, then the data section at the next multiple of
// general.alignment (default 32); offsets are relative to it. Sharded models are named
// NAME-0000i-of-0000n.gguf and hold disjoint tensor sets. The expert tensors of layer L are
// blk.L.ffn_gate_exps.weight, blk.L.ffn_up_exps.weight, blk.L.ffn_down_exps.weight with
// ne = [K, N, E] (src/gpu/parts/30_host_util.inc:384-412).
//
// Files are mapped read-only; the loaders hand the mapped bytes to b200moe_load_q4cp /
// b200moe_load_gguf (which stage host memory to the device) and unmap afterwards.
#include "../../include/b200moe.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Mapping {
  const uint8_t* p = nullptr;
  size_t len = 0;
  bool open(const char* path) {
    int fd = ::open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return false;
    struct stat st;
    if (fstat(fd, &st) < 0) {
      ::close(fd);
      return false;
    }
    len = (size_t)st.st_size;
    void* m = len ? mmap(nullptr, len, PROT_READ, MAP_PRIVATE, fd, 0) : MAP_FAILED;
    ::close(fd);
    if (m == MAP_FAILED) return false;
    p = (const uint8_t*)m;
    return true;
  }
  ~Mapping() {
    if (p) munmap((void*)p, len);
  }
};

struct View {
  const uint8_t* data = nullptr;
  uint64_t size = 0, dims[4] = {0, 0, 0, 0};
  uint32_t dtype = 0, ndims = 0;
};

#pragma pack(push, 1)
struct HgnHeader {
  char magic[4];
  uint32_t version, tensor_count, reserved;
  uint64_t records_offset, data_offset, file_size;
  char model_name[64];
};
struct HgnRecord {
  char name[96];
  uint32_t dtype, ndims;
  uint64_t dims[4];
  uint64_t data_offset, data_size, extra;
};
#pragma pack(pop)
static_assert(sizeof(HgnHeader) == 104 && sizeof(HgnRecord) == 160, "hgn records are packed");

// 0 found, 1 not found, 2 malformed file
int hgn_find(const Mapping& m, const std::string& name, View* out) {
  if (m.len < sizeof(HgnHeader)) return 2;
  HgnHeader h;
  memcpy(&h, m.p, sizeof h);
  if (memcmp(h.magic, "HGN1", 4) != 0 || h.file_size != m.len) return 2;
  if (h.records_offset > m.len || (uint64_t)h.tensor_count * sizeof(HgnRecord) > m.len - h.records_offset) return 2;
  for (uint32_t i = 0; i < h.tensor_count; i++) {
    HgnRecord r;
    memcpy(&r, m.p + h.records_offset + (uint64_t)i * sizeof r, sizeof r);
    if (strnlen(r.name, sizeof r.name) != name.size() || memcmp(r.name, name.data(), name.size()) != 0) continue;
    if (r.data_offset > m.len || r.data_size > m.len - r.data_offset) return 2;
    out->data = m.p + r.data_offset;
    out->size = r.data_size;
    out->dtype = r.dtype;
    out->ndims = r.ndims;
    for (int k = 0; k < 4; k++) out->dims[k] = r.dims[k];
    return 0;
  }
  return 1;
}

// ---- GGUF ----
struct Cursor {
  const uint8_t* p;
  size_t len, pos = 0;
  bool ok = true;
  template <typename T>
  T get() {
    T v{};
    if (pos + sizeof(T) > len) {
      ok = false;
      return v;
    }
    memcpy(&v, p + pos, sizeof(T));
    pos += sizeof(T);
    return v;
  }
  std::string str() {
    const uint64_t n = get<uint64_t>();
    if (!ok || n > len - pos) {
      ok = false;
      return std::string();
    }
    std::string s((const char*)p + pos, (size_t)n);
    pos += (size_t)n;
    return s;
  }
  void skip(uint64_t n) {
    if (n > len - pos) ok = false;
    else pos += (size_t)n;
  }
};

// size of a scalar GGUF value type, 0 = not a scalar (string 8, array 9)
size_t gguf_scalar(uint32_t t) {
  switch (t) {
    case 0: case 1: case 7: return 1;   // u8, i8, bool
    case 2: case 3: return 2;           // u16, i16
    case 4: case 5: case 6: return 4;   // u32, i32, f32
    case 10: case 11: case 12: return 8;  // u64, i64, f64
    default: return 0;
  }
}

void gguf_skip_value(Cursor& c, uint32_t t, uint64_t* u_out) {
  if (size_t n = gguf_scalar(t)) {
    if (u_out && (t == 4 || t == 5)) {
      size_t save = c.pos;
      *u_out = c.get<uint32_t>();
      c.pos = save;
    }
    c.skip(n);
  } else if (t == 8) {
    c.str();
  } else if (t == 9) {
    const uint32_t et = c.get<uint32_t>();
    const uint64_t cnt = c.get<uint64_t>();
    if (size_t n = gguf_scalar(et)) {
      if (cnt > (c.len - c.pos) / n) c.ok = false;
      else c.skip(cnt * n);
    } else if (et == 8) {
      for (uint64_t i = 0; i < cnt && c.ok; i++) c.str();
    } else {
      c.ok = false;  // nested arrays do not occur in model files
    }
  } else {
    c.ok = false;
  }
}

// 0 found, 1 not found, 2 malformed, 3 found with a block type this library does not read
int gguf_find(const Mapping& m, const std::string& name, View* out) {
  Cursor c{m.p, m.len};
  if (c.get<uint32_t>() != 0x46554747u) return 2;  // "GGUF"
  const uint32_t version = c.get<uint32_t>();
  if (version < 2 || version > 3) return 2;
  const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
  uint64_t alignment = 32;
  for (uint64_t i = 0; i < n_kv && c.ok; i++) {
    const std::string key = c.str();
    const uint32_t t = c.get<uint32_t>();
    uint64_t u = 0;
    gguf_skip_value(c, t, key == "general.alignment" ? &u : nullptr);
    if (key == "general.alignment" && u) alignment = u;
  }
  if (!c.ok) return 2;
  bool found = false;
  uint64_t off = 0;
  for (uint64_t i = 0; i < n_tensors && c.ok; i++) {
    const std::string tn = c.str();
    const uint32_t nd = c.get<uint32_t>();
    if (nd > 4) return 2;
    uint64_t dims[4] = {1, 1, 1, 1};
    for (uint32_t k = 0; k < nd; k++) dims[k] = c.get<uint64_t>();
    const uint32_t type = c.get<uint32_t>();
    const uint64_t o = c.get<uint64_t>();
    if (c.ok && tn == name) {
      found = true;
      off = o;
      out->dtype = type;
      out->ndims = nd;
      for (int k = 0; k < 4; k++) out->dims[k] = dims[k];
    }
  }
  if (!c.ok) return 2;
  if (!found) return 1;
  const uint64_t data0 = (c.pos + alignment - 1) / alignment * alignment;
  // bytes per row: Q4_K 144 per 256 elements, Q5_K 176 per 256, Q5_1 24 per 32, Q8_0 34 per 32, IQ4_NL 18 per 32, IQ4_XS 136 per 256
  uint64_t row = 0;
  if (out->dtype == B200MOE_GGML_Q4_K && out->dims[0] % 256 == 0) row = out->dims[0] / 256 * 144;
  else if (out->dtype == B200MOE_GGML_Q5_K && out->dims[0] % 256 == 0) row = out->dims[0] / 256 * 176;
  else if (out->dtype == B200MOE_GGML_Q5_1 && out->dims[0] % 32 == 0) row = out->dims[0] / 32 * 24;
  else if (out->dtype == B200MOE_GGML_Q8_0 && out->dims[0] % 32 == 0) row = out->dims[0] / 32 * 34;
  else if (out->dtype == B200MOE_GGML_IQ4_NL && out->dims[0] % 32 == 0) row = out->dims[0] / 32 * 18;
  else if (out->dtype == B200MOE_GGML_IQ4_XS && out->dims[0] % 256 == 0) row = out->dims[0] / 256 * 136;
  else return 3;
  out->size = row * out->dims[1] * out->dims[2] * out->dims[3];
  if (data0 > m.len || off > m.len - data0 || out->size > m.len - data0 - off) return 2;
  out->data = m.p + data0 + off;
  return 0;
}

// Five decimal digits at s[pos..pos+4] as a number; -1 when one of them is not a digit.
int five_digits(const std::string& s, size_t pos) {
  int v = 0;
  for (size_t i = pos; i < pos + 5; i++) {
    if (s[i] < '0' || s[i] > '9') return -1;
    v = v * 10 + (s[i] - '0');
  }
  return v;
}

// A sharded model is a set of files STEM-<i>-of-<n>.gguf, i and n written with five digits,
// i = 1..n. Given any member, returns the n member names in order; a path that does not end in
// such a suffix (or whose numbers are inconsistent) is a single file.
std::vector<std::string> gguf_shards(const std::string& path) {
  constexpr size_t kTail = 5 + 4 + 5 + 5;  // "00001" "-of-" "00003" ".gguf"
  if (path.size() > kTail) {
    const size_t t = path.size() - kTail;  // where the shard number starts
    const int i = five_digits(path, t), n = five_digits(path, t + 9);
    if (path[t - 1] == '-' && path.compare(t + 5, 4, "-of-") == 0 && path.compare(t + 14, 5, ".gguf") == 0 &&
        i >= 1 && n >= 1 && i <= n) {
      std::vector<std::string> all;
      const std::string stem = path.substr(0, t);
      for (int k = 1; k <= n; k++) {
        char tail[24];
        snprintf(tail, sizeof tail, "%05d-of-%05d.gguf", k, n);
        all.push_back(stem + tail);
      }
      return all;
    }
  }
  return std::vector<std::string>{path};
}

// bytes of a q4cp blob [rows, cols]: code book, codes, per-row scale records padded to 16 bytes (src/hgn.h:219-238)
uint64_t q4cp_blob_bytes(uint64_t rows, uint64_t cols) {
  return 64 + rows * cols / 2 + rows * (((cols / 32 * 2) + 15) & ~(uint64_t)15);
}

std::string layer_name(const char* fmt, int layer) {
  char buf[128];
  snprintf(buf, sizeof buf, fmt, layer);
  return buf;
}

}  // namespace

extern "C" int b200moe_load_hgn_file(b200moe_handle h, int layer, const char* path, int model_layer) {
  if (!h || !path) return B200MOE_ERR_BAD_ARG;
  b200moe_config cfg;
  if (int s = b200moe_get_config(h, &cfg)) return s;
  Mapping m;
  if (!m.open(path)) return B200MOE_ERR_BAD_ARG;
  const uint64_t E = cfg.experts, d = cfg.d_model, mid = cfg.d_mid;
  View gu, dn;
  if (hgn_find(m, layer_name("layers.%d.mlp.experts.gate_up_proj.weight", model_layer), &gu) ||
      hgn_find(m, layer_name("layers.%d.mlp.experts.down_proj.weight", model_layer), &dn))
    return B200MOE_ERR_BAD_ARG;
  if (gu.dtype == 23 && dn.dtype == 23) {
    // hgn v2 i4r experts: [E, O, K] (or flat [E*O, K]) with fp16 sign-scale planes as separate
    // tensors <base>.suh [K] (gate_up: else the shared input plane experts.su) and <base>.svh [O]
    // (src/gpu/parts/30_host_util.inc:840-858 of the reference)
    auto shape_ok = [&](const View& v, uint64_t O, uint64_t K) {
      if (v.ndims == 3) return v.dims[0] == E && v.dims[1] == O && v.dims[2] == K;
      return v.ndims == 2 && v.dims[0] == E * O && v.dims[1] == K;
    };
    if (!shape_ok(gu, 2 * mid, d) || !shape_ok(dn, d, mid)) return B200MOE_ERR_UNSUPPORTED;
    auto plane = [&](const std::string& name, uint64_t n, View* out) {
      const int r = hgn_find(m, name, out);
      if (r != 0) return r;
      return out->dtype == 2 && out->size == n * 2 ? 0 : 2;
    };
    const std::string ex = layer_name("layers.%d.mlp.experts", model_layer);
    View p[4];
    int r = plane(ex + ".gate_up_proj.suh", d, &p[0]);
    if (r == 1) r = plane(ex + ".su", d, &p[0]);
    if (r || plane(ex + ".gate_up_proj.svh", 2 * mid, &p[1]) || plane(ex + ".down_proj.suh", mid, &p[2]) ||
        plane(ex + ".down_proj.svh", d, &p[3]))
      return B200MOE_ERR_BAD_ARG;
    if (int s = b200moe_load_i4r(h, layer, gu.data, gu.size, dn.data, dn.size, p[0].data, p[1].data, p[2].data, p[3].data))
      return s;
    View rw;
    const int rr = hgn_find(m, layer_name("layers.%d.mlp.gate.weight", model_layer), &rw);
    if (rr == 2) return B200MOE_ERR_BAD_ARG;
    if (rr == 0 && rw.dtype == 0 && rw.size >= E * d * 2 && E <= 512 && d % 64 == 0)
      if (int s = b200moe_load_router(h, layer, rw.data)) return s;
    return B200MOE_OK;
  }
  if (gu.dtype != 5 || dn.dtype != 5 || gu.ndims != 2 || dn.ndims != 2 || gu.dims[0] != E * 2 * mid || gu.dims[1] != d ||
      dn.dims[0] != E * d || dn.dims[1] != mid)
    return B200MOE_ERR_UNSUPPORTED;
  if (int s = b200moe_load_q4cp(h, layer, gu.data, gu.size, dn.data, dn.size)) return s;
  if (cfg.has_shared) {
    View sg, su, sd, sw;
    if (hgn_find(m, layer_name("layers.%d.mlp.shared_expert.gate_proj.weight", model_layer), &sg) ||
        hgn_find(m, layer_name("layers.%d.mlp.shared_expert.up_proj.weight", model_layer), &su) ||
        hgn_find(m, layer_name("layers.%d.mlp.shared_expert.down_proj.weight", model_layer), &sd) ||
        hgn_find(m, layer_name("layers.%d.mlp.shared_expert_gate.weight", model_layer), &sw))
      return B200MOE_ERR_BAD_ARG;
    if (sg.dtype != 5 || su.dtype != 5 || sd.dtype != 5 || sw.dtype != 0 || sw.size < d * 2) return B200MOE_ERR_UNSUPPORTED;
    // b200moe_load_shared_q4cp takes no sizes and reads whole [mid,d] / [d,mid] blobs: the
    // mapped tensors must have exactly that shape and size
    const uint64_t gu_b = q4cp_blob_bytes(mid, d), dn_b = q4cp_blob_bytes(d, mid);
    if (sg.ndims != 2 || su.ndims != 2 || sd.ndims != 2 || sg.dims[0] != mid || sg.dims[1] != d || su.dims[0] != mid ||
        su.dims[1] != d || sd.dims[0] != d || sd.dims[1] != mid)
      return B200MOE_ERR_UNSUPPORTED;
    if (sg.size != gu_b || su.size != gu_b || sd.size != dn_b) return B200MOE_ERR_BAD_ARG;
    if (((uintptr_t)sg.data | (uintptr_t)su.data | (uintptr_t)sd.data) & 15) return B200MOE_ERR_BAD_ARG;
    if (int s = b200moe_load_shared_q4cp(h, layer, sg.data, su.data, sd.data, sw.data)) return s;
  }
  View rw;
  const int r = hgn_find(m, layer_name("layers.%d.mlp.gate.weight", model_layer), &rw);
  if (r == 2) return B200MOE_ERR_BAD_ARG;
  if (r == 0 && rw.dtype == 0 && rw.size >= E * d * 2 && E <= 512 && d % 64 == 0)
    if (int s = b200moe_load_router(h, layer, rw.data)) return s;
  return B200MOE_OK;
}

extern "C" int b200moe_load_gguf_file(b200moe_handle h, int layer, const char* path, int model_layer) {
  if (!h || !path) return B200MOE_ERR_BAD_ARG;
  b200moe_config cfg;
  if (int s = b200moe_get_config(h, &cfg)) return s;
  const uint64_t E = cfg.experts, d = cfg.d_model, mid = cfg.d_mid;
  const std::string names[3] = {layer_name("blk.%d.ffn_gate_exps.weight", model_layer),
                                layer_name("blk.%d.ffn_up_exps.weight", model_layer),
                                layer_name("blk.%d.ffn_down_exps.weight", model_layer)};
  const std::vector<std::string> files = gguf_shards(path);
  std::vector<Mapping> maps(files.size());
  View v[3];
  bool have[3] = {false, false, false};
  for (size_t f = 0; f < files.size(); f++) {
    if (!maps[f].open(files[f].c_str())) return B200MOE_ERR_BAD_ARG;
    for (int i = 0; i < 3; i++) {
      if (have[i]) continue;
      const int r = gguf_find(maps[f], names[i], &v[i]);
      if (r == 2) return B200MOE_ERR_BAD_ARG;
      if (r == 3) return B200MOE_ERR_UNSUPPORTED;
      have[i] = r == 0;
    }
  }
  if (!have[0] || !have[1] || !have[2]) return B200MOE_ERR_BAD_ARG;
  // ne = [K, N, E]
  for (int i = 0; i < 2; i++)
    if (v[i].dims[0] != d || v[i].dims[1] != mid || v[i].dims[2] != E) return B200MOE_ERR_UNSUPPORTED;
  if (v[2].dims[0] != mid || v[2].dims[1] != d || v[2].dims[2] != E || v[0].dtype != v[1].dtype) return B200MOE_ERR_UNSUPPORTED;
  return b200moe_load_gguf(h, layer, v[0].data, v[1].data, v[2].data, (int)v[0].dtype, (int)v[2].dtype);
}
