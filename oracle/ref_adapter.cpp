// ref_adapter.cpp -- TEST INFRASTRUCTURE ONLY. Not part of the product library.
//
// Compiles the reference's own CPU forward (src/ref.cpp with src/hgn.h, src/rope.h and
// src/gguf.h) from the sources where they lie -- nothing is copied -- and exposes the
// three reference functions the MoE path is checked against through a C ABI:
//   * Model::moe                      src/ref.cpp:563-637   (unmodified, called as is)
//   * hgn::Checkpoint::q4cp_row       src/hgn.h:249-261
//   * gguf::dequant_row               src/gguf.h:339-443
//   * hgn::Checkpoint(path), gguf::File(path)   src/hgn.h:295-363, src/gguf.h:136-314
//     (the reference's file readers: prove that the files the loader tests write are files
//     the reference itself accepts, and that it sees the same tensor bytes)
// The reference's `main` is renamed so that the file can be included as a library
// (the reference's own kernel test does the same to its engine, tools/ktest.cu:1-5).
//
// Built by oracle/Makefile into oracle/_ref/libref.so, only where the reference tree
// is present; the restated oracle (moe_oracle.cpp) is what runs everywhere else.
#define main ref_cli_main
#include "ref.cpp"
#undef main
#include "gguf.h"

#include <memory>
#include <omp.h>

namespace {

hgn::Tensor make_tensor(const char* name, uint32_t dtype, std::initializer_list<uint64_t> dims,
                        const void* data, uint64_t size) {
  hgn::Tensor t;
  t.name = name;
  t.dtype = dtype;
  t.ndims = (uint32_t)dims.size();
  int i = 0;
  for (uint64_t v : dims) t.dims[i++] = v;
  t.data = (const uint8_t*)data;
  t.data_size = size;
  return t;
}

uint64_t q4cp_bytes(uint64_t rows, uint64_t cols) {
  return 64 + rows * cols / 2 + rows * (((cols / 32 * 2) + 15) & ~15ull);
}

}  // namespace

extern "C" {

// Runs the reference Model::moe on T tokens. Blobs are in the on-disk layouts of the
// reference (bf16 router weight [E][d]; q4cp tensors). The shared expert is always
// present in the reference; pass all-zero down-projection scales to switch it off.
int ref_moe_layer(int d, int E, int k, int mid, const uint16_t* router_w, const uint8_t* gate_up,
                  const uint8_t* down, const uint16_t* sh_gate_w, const uint8_t* sh_gate,
                  const uint8_t* sh_up, const uint8_t* sh_down, const float* x, int T, float* y,
                  int threads) {
  try {
    g_cfg.d = d;
    g_cfg.experts = E;
    g_cfg.topk = k;
    g_cfg.moe_mid = mid;
    g_cfg.layers = 1;
    hgn::Checkpoint ck;
    // The Model constructor insists on the n-gram layer's tensors; minimal stand-ins.
    static const uint16_t zero2[2] = {0, 0};
    static int64_t ones3[3] = {1, 1, 1}, ones16[16], zeros16[16];
    static uint8_t table[164];
    for (int i = 0; i < 16; i++) ones16[i] = 1, zeros16[i] = 0;
    memset(table, 0, sizeof table);
    float one = 1.f;
    memcpy(table + 160, &one, 4);
    ck.add_view(make_tensor("layers.1.ple.key_proj.weight", 0, {1, 2}, zero2, 4));
    ck.add_view(make_tensor("layers.1.ple.value_proj.weight", 0, {1, 2}, zero2, 4));
    ck.add_view(make_tensor("layers.1.ple.conv1d.weight", 0, {1, 2}, zero2, 4));
    ck.add_view(make_tensor("layers.1.ple.norm_key.weight", 0, {2}, zero2, 4));
    ck.add_view(make_tensor("layers.1.ple.norm_query.weight", 0, {2}, zero2, 4));
    ck.add_view(make_tensor("layers.1.ple.norm_conv.weight", 0, {2}, zero2, 4));
    ck.add_view(make_tensor("layers.1.ple.ple_embedding.layer_multipliers", 4, {3}, ones3, 24));
    ck.add_view(make_tensor("layers.1.ple.ple_embedding.ngram_heads_vocab_sizes", 4, {16}, ones16, 128));
    ck.add_view(make_tensor("layers.1.ple.ple_embedding.ngram_heads_offsets", 4, {16}, zeros16, 128));
    ck.add_view(make_tensor("layers.1.ple.ngram_embedding.weight", 10, {1, 160}, table, 164));
    const uint64_t ue = E, ud = d, um = mid;
    ck.add_view(make_tensor("layers.0.mlp.gate.weight", 0, {ue, ud}, router_w, ue * ud * 2));
    ck.add_view(make_tensor("layers.0.mlp.experts.gate_up_proj.weight", 5, {ue, 2 * um, ud}, gate_up,
                            q4cp_bytes(ue * 2 * um, ud)));
    ck.add_view(make_tensor("layers.0.mlp.experts.down_proj.weight", 5, {ue, ud, um}, down,
                            q4cp_bytes(ue * ud, um)));
    ck.add_view(make_tensor("layers.0.mlp.shared_expert_gate.weight", 0, {1, ud}, sh_gate_w, ud * 2));
    ck.add_view(make_tensor("layers.0.mlp.shared_expert.gate_proj.weight", 5, {um, ud}, sh_gate,
                            q4cp_bytes(um, ud)));
    ck.add_view(make_tensor("layers.0.mlp.shared_expert.up_proj.weight", 5, {um, ud}, sh_up,
                            q4cp_bytes(um, ud)));
    ck.add_view(make_tensor("layers.0.mlp.shared_expert.down_proj.weight", 5, {ud, um}, sh_down,
                            q4cp_bytes(ud, um)));
    Model model(ck);
    if (threads > 0) omp_set_num_threads(threads);
#pragma omp parallel for schedule(dynamic, 1)
    for (int t = 0; t < T; t++) model.moe(0, x + (size_t)t * d, y + (size_t)t * d);
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_moe_layer: %s\n", e.what());
    return -1;
  }
}

int ref_q4cp_rows(const uint8_t* blob, uint64_t rows, uint64_t cols, uint64_t row0, uint64_t n,
                  float* out) {
  try {
    hgn::Tensor t = make_tensor("t", 5, {rows, cols}, blob, q4cp_bytes(rows, cols));
    auto q = hgn::Checkpoint::q4cp_parse(t);
    for (uint64_t r = 0; r < n; r++) hgn::Checkpoint::q4cp_row(q, row0 + r, out + r * cols);
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_q4cp_rows: %s\n", e.what());
    return -1;
  }
}

int ref_gguf_rows(uint32_t type, const uint8_t* src, uint64_t k, uint64_t n, float* out) {
  try {
    uint32_t be, bb;
    gguf::block_info(type, be, bb);
    if (!be) return -1;
    for (uint64_t r = 0; r < n; r++) gguf::dequant_row(type, src + r * (k / be * bb), out + r * k, k);
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_gguf_rows: %s\n", e.what());
    return -1;
  }
}

}  // extern "C"

namespace {
// CRC-32 (IEEE, the polynomial of zlib.crc32) of a byte range
uint32_t crc32_bytes(const uint8_t* p, uint64_t n) {
  static uint32_t table[256];
  static bool init = false;
  if (!init) {
    for (uint32_t i = 0; i < 256; i++) {
      uint32_t c = i;
      for (int k = 0; k < 8; k++) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
      table[i] = c;
    }
    init = true;
  }
  uint32_t c = 0xFFFFFFFFu;
  for (uint64_t i = 0; i < n; i++) c = table[(c ^ p[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}
}  // namespace

extern "C" {

// Opens `path` with the reference's hgn::Checkpoint and reports tensor `name`:
// meta = {dtype, ndims, dims[0..3], data_size, crc32 of the data}. 0 ok, 1 no such tensor, -1 the
// reference refused the file.
int ref_hgn_tensor(const char* path, const char* name, uint64_t* meta8) {
  try {
    hgn::Checkpoint ck(path);
    const hgn::Tensor* t = ck.find(name);
    if (!t) return 1;
    meta8[0] = t->dtype;
    meta8[1] = t->ndims;
    for (int i = 0; i < 4; i++) meta8[2 + i] = t->dims[i];
    meta8[6] = t->data_size;
    meta8[7] = crc32_bytes(t->data, t->data_size);
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_hgn_tensor: %s\n", e.what());
    return -1;
  }
}

// The same through the reference's gguf::File (all shards of a sharded model are opened):
// meta = {type, nd, ne[0..3], nbytes, crc32 of the data}.
int ref_gguf_tensor(const char* path, const char* name, uint64_t* meta8) {
  try {
    gguf::File f{std::string(path)};
    const gguf::Tensor* t = f.find(name);
    if (!t) return 1;
    meta8[0] = t->type;
    meta8[1] = t->nd;
    for (int i = 0; i < 4; i++) meta8[2 + i] = t->ne[i];
    meta8[6] = t->nbytes;
    meta8[7] = crc32_bytes(t->data, t->nbytes);
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "ref_gguf_tensor: %s\n", e.what());
    return -1;
  }
}

}  // extern "C"
