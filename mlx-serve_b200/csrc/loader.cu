// Checkpoint -> device loader for MLX-format quantized checkpoints: safetensors files whose quantized linears are
// stored as `<name>.weight` (uint32 packed codes), `<name>.scales`, `<name>.biases`, next to a config.json with a
// top-level "quantization": {bits, group_size, mode}.
//
// What it restates from mlx-serve (host code only; the device side is a plain copy because the kernels consume the
// checkpoint's own layout):
//   * config.json quantization parse and the affine bit-width check   src/model.zig:1480-1505
//   * per-weight geometry: bits = w_cols * 32 / in_dim, group = in_dim / s_cols   src/transformer.zig:16763-16790
//   * which loaded f16 tensors are narrowed to bf16 (quant scales/biases by suffix, any 1-D table)   src/model.zig:3030-3061
// The safetensors container itself (8-byte little-endian header length, a JSON header of
// name -> {dtype, shape, data_offsets}, then the raw tensor bytes) is read with a small JSON reader written here.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "kernels.h"

struct qb200_checkpoint {
  int fd = -1;
  const unsigned char* map = nullptr;
  size_t size = 0, data0 = 0;
  struct Entry {
    std::string name;
    int dtype = -1, ndim = 0;
    int64_t shape[QB200_MAX_DIMS] = {};
    size_t begin = 0, end = 0;
  };
  std::vector<Entry> entries;
};

namespace {

using Entry = qb200_checkpoint::Entry;

int ld_fail(int status, const std::string& msg) { return qb::report_error(status, msg.c_str()); }

// ---- a JSON reader for what the two files hold: objects, arrays, strings, numbers, literals ----
struct Json {
  const char* p; const char* end; bool ok = true;
  void ws() { while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
  bool peek(char c) { ws(); return p < end && *p == c; }
  std::string str() {
    std::string out;
    ws();
    if (p >= end || *p != '"') { ok = false; return out; }
    ++p;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'u': out += '?'; p += (end - p > 4 ? 4 : 0); break;   // names in these files are ASCII
          default: out += *p;
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= end) { ok = false; return out; }
    ++p;
    return out;
  }
  double num() {
    ws();
    char* e = nullptr;
    const double v = strtod(p, &e);
    if (e == p) ok = false;
    p = e;
    return v;
  }
  void skip() {   // any value
    ws();
    if (p >= end) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{') {
      ++p;
      if (eat('}')) return;
      do { str(); if (!eat(':')) { ok = false; return; } skip(); } while (ok && eat(','));
      if (!eat('}')) ok = false;
      return;
    }
    if (*p == '[') {
      ++p;
      if (eat(']')) return;
      do { skip(); } while (ok && eat(','));
      if (!eat(']')) ok = false;
      return;
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']' && *p != ' ' && *p != '\n') ++p;   // number or literal
  }
};

int dtype_of(const std::string& s) {
  static const struct { const char* n; int d; } tab[] = {
      {"F32", QB200_FLOAT32}, {"F16", QB200_FLOAT16}, {"BF16", QB200_BFLOAT16}, {"F64", QB200_FLOAT64}, {"U32", QB200_UINT32},
      {"I32", QB200_INT32}, {"I64", QB200_INT64}, {"U64", QB200_UINT64}, {"U8", QB200_UINT8}, {"I8", QB200_INT8},
      {"U16", QB200_UINT16}, {"I16", QB200_INT16}, {"BOOL", QB200_BOOL}};
  for (const auto& t : tab)
    if (s == t.n) return t.d;
  return -1;
}
int size_of(int dt) {
  switch (dt) {
    case QB200_BOOL: case QB200_UINT8: case QB200_INT8: return 1;
    case QB200_UINT16: case QB200_INT16: case QB200_FLOAT16: case QB200_BFLOAT16: return 2;
    case QB200_UINT32: case QB200_INT32: case QB200_FLOAT32: return 4;
    case QB200_UINT64: case QB200_INT64: case QB200_FLOAT64: return 8;
    default: return 0;
  }
}
bool ends_with(const char* s, const char* suf) {
  const size_t n = strlen(s), m = strlen(suf);
  return n >= m && memcmp(s + n - m, suf, m) == 0;
}
const Entry* find(const qb200_checkpoint* ck, const char* name) {
  for (const auto& e : ck->entries)
    if (e.name == name) return &e;
  return nullptr;
}
float half_to_float(uint16_t h) {
  const uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1F, m = h & 0x3FF;
  uint32_t u;
  if (e == 0) {
    if (m == 0) u = s;
    else {   // subnormal: renormalise
      int sh = 0;
      uint32_t mm = m;
      while (!(mm & 0x400)) { mm <<= 1; ++sh; }
      u = s | ((uint32_t)(127 - 15 - sh + 1) << 23) | ((mm & 0x3FF) << 13);
    }
  } else if (e == 31) u = s | 0x7F800000u | (m << 13);
  else u = s | ((e + 112) << 23) | (m << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t float_to_bf16(float f) {   // round to nearest even; NaN stays NaN
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x7FFFFFu)) return (uint16_t)((u >> 16) | 0x40);
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

}  // namespace

extern "C" {

QB200_API bool qb200_narrows_loaded_f16(const char* name, int ndim, int dtype) {
  if (dtype != QB200_FLOAT16 || name == nullptr) return false;
  if (ends_with(name, ".scales") || ends_with(name, ".biases")) return true;
  return ndim == 1;
}

QB200_API int qb200_affine_params_from_geometry(int64_t w_cols, int64_t s_cols, int64_t in_dim, int* bits, int* group_size) {
  if (w_cols <= 0 || s_cols <= 0 || in_dim <= 0 || !bits || !group_size) return ld_fail(QB200_ERR_BAD_ARG, "affine_params_from_geometry: bad argument");
  if ((w_cols * 32) % in_dim != 0 || in_dim % s_cols != 0)
    return ld_fail(QB200_ERR_BAD_SHAPE, "affine_params_from_geometry: the packed width or the scale count does not divide the input dimension");
  const int64_t b = (w_cols * 32) / in_dim, g = in_dim / s_cols;
  if (!(b == 2 || b == 3 || b == 4 || b == 5 || b == 6 || b == 8) || !(g == 32 || g == 64 || g == 128))
    return ld_fail(QB200_ERR_UNSUPPORTED, "affine_params_from_geometry: not an affine geometry MLX produces");
  *bits = (int)b;
  *group_size = (int)g;
  return QB200_OK;
}

QB200_API int qb200_config_quantization(const char* json_text, int* bits, int* group_size, char* mode, size_t mode_cap) {
  if (!json_text || !bits || !group_size) return ld_fail(QB200_ERR_BAD_ARG, "config_quantization: null argument");
  *bits = 0; *group_size = 0;
  if (mode && mode_cap) snprintf(mode, mode_cap, "affine");
  Json j{json_text, json_text + strlen(json_text)};
  if (!j.eat('{')) return ld_fail(QB200_ERR_BAD_ARG, "config_quantization: not a JSON object");
  bool found = false;
  if (!j.peek('}')) {
    do {
      const std::string key = j.str();
      if (!j.ok || !j.eat(':')) return ld_fail(QB200_ERR_BAD_ARG, "config_quantization: malformed JSON");
      if (key == "quantization" && j.peek('{')) {
        found = true;
        j.eat('{');
        if (!j.peek('}')) {
          do {
            const std::string k2 = j.str();
            if (!j.ok || !j.eat(':')) return ld_fail(QB200_ERR_BAD_ARG, "config_quantization: malformed quantization object");
            if (k2 == "bits") *bits = (int)j.num();
            else if (k2 == "group_size") *group_size = (int)j.num();
            else if (k2 == "mode" && j.peek('"')) { const std::string m = j.str(); if (mode && mode_cap) snprintf(mode, mode_cap, "%s", m.c_str()); }
            else j.skip();   // per-layer overrides and the like
          } while (j.ok && j.eat(','));
        }
        if (!j.eat('}')) return ld_fail(QB200_ERR_BAD_ARG, "config_quantization: malformed quantization object");
      } else {
        j.skip();
      }
    } while (j.ok && j.eat(','));
  }
  if (!j.ok) return ld_fail(QB200_ERR_BAD_ARG, "config_quantization: malformed JSON");
  if (!found) return ld_fail(QB200_ERR_UNSUPPORTED, "config_quantization: no \"quantization\" object (a dense checkpoint)");
  // MLX ships affine kernels only for these widths; anything else is refused at parse time (src/model.zig:1492-1505)
  if (mode && strcmp(mode, "affine") == 0 && *bits != 0) {
    const int b = *bits;
    if (!(b == 2 || b == 3 || b == 4 || b == 5 || b == 6 || b == 8)) return ld_fail(QB200_ERR_UNSUPPORTED, "config_quantization: unsupported affine bit width");
  }
  return QB200_OK;
}

QB200_API int qb200_checkpoint_open(qb200_checkpoint** out, const char* path) {
  if (!out || !path) return ld_fail(QB200_ERR_BAD_ARG, "checkpoint_open: null argument");
  *out = nullptr;
  const int fd = open(path, O_RDONLY);
  if (fd < 0) return ld_fail(QB200_ERR_BAD_ARG, std::string("checkpoint_open: cannot open ") + path);
  struct stat st;
  if (fstat(fd, &st) != 0 || st.st_size < 8) { close(fd); return ld_fail(QB200_ERR_BAD_ARG, "checkpoint_open: file shorter than a safetensors header"); }
  void* m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  if (m == MAP_FAILED) { close(fd); return ld_fail(QB200_ERR_BAD_ARG, "checkpoint_open: mmap failed"); }
  auto* ck = new qb200_checkpoint;
  ck->fd = fd; ck->map = (const unsigned char*)m; ck->size = (size_t)st.st_size;
  uint64_t hlen = 0;
  memcpy(&hlen, ck->map, 8);
  auto bail = [&](const char* why) { munmap((void*)ck->map, ck->size); close(fd); delete ck; return ld_fail(QB200_ERR_BAD_ARG, std::string("checkpoint_open: ") + why); };
  if (hlen > ck->size - 8) return bail("header length beyond the end of the file (an interrupted download?)");
  ck->data0 = 8 + (size_t)hlen;
  Json j{(const char*)ck->map + 8, (const char*)ck->map + 8 + hlen};
  if (!j.eat('{')) return bail("the header is not a JSON object");
  if (!j.peek('}')) {
    do {
      Entry e;
      e.name = j.str();
      if (!j.ok || !j.eat(':')) return bail("malformed header");
      if (e.name == "__metadata__") { j.skip(); continue; }
      if (!j.eat('{')) return bail("malformed tensor entry");
      do {
        const std::string k = j.str();
        if (!j.ok || !j.eat(':')) return bail("malformed tensor entry");
        if (k == "dtype") e.dtype = dtype_of(j.str());
        else if (k == "shape") {
          if (!j.eat('[')) return bail("malformed shape");
          if (!j.eat(']')) {
            do { if (e.ndim >= QB200_MAX_DIMS) return bail("more than 8 dims"); e.shape[e.ndim++] = (int64_t)j.num(); } while (j.ok && j.eat(','));
            if (!j.eat(']')) return bail("malformed shape");
          }
        } else if (k == "data_offsets") {
          if (!j.eat('[')) return bail("malformed data_offsets");
          e.begin = (size_t)j.num();
          if (!j.eat(',')) return bail("malformed data_offsets");
          e.end = (size_t)j.num();
          if (!j.eat(']')) return bail("malformed data_offsets");
        } else j.skip();
      } while (j.ok && j.eat(','));
      if (!j.eat('}')) return bail("malformed tensor entry");
      int64_t n = 1;
      for (int d = 0; d < e.ndim; ++d) n *= e.shape[d];
      if (e.dtype < 0 || e.end < e.begin || ck->data0 + e.end > ck->size || (size_t)n * size_of(e.dtype) != e.end - e.begin)
        return bail("a tensor's dtype, shape and byte range disagree (or run past the end of the file)");
      ck->entries.push_back(e);
    } while (j.ok && j.eat(','));
  }
  if (!j.ok) return bail("malformed header");
  if (ck->entries.empty()) return bail("no tensors in the file");
  *out = ck;
  return QB200_OK;
}

QB200_API void qb200_checkpoint_close(qb200_checkpoint* ck) {
  if (!ck) return;
  if (ck->map) munmap((void*)ck->map, ck->size);
  if (ck->fd >= 0) close(ck->fd);
  delete ck;
}

QB200_API int qb200_checkpoint_num_tensors(const qb200_checkpoint* ck) { return ck ? (int)ck->entries.size() : 0; }
QB200_API const char* qb200_checkpoint_tensor_name(const qb200_checkpoint* ck, int i) {
  return (ck && i >= 0 && i < (int)ck->entries.size()) ? ck->entries[i].name.c_str() : nullptr;
}

// Shape and dtype AFTER loading (an f16 tensor that the narrowing rule covers reports bf16); desc->data stays null.
QB200_API int qb200_checkpoint_tensor_info(const qb200_checkpoint* ck, const char* name, qb200_tensor* desc, size_t* nbytes) {
  if (!ck || !name || !desc) return ld_fail(QB200_ERR_BAD_ARG, "checkpoint_tensor_info: null argument");
  const Entry* e = find(ck, name);
  if (!e) return ld_fail(QB200_ERR_BAD_ARG, std::string("checkpoint_tensor_info: no tensor named ") + name);
  memset(desc, 0, sizeof(*desc));
  desc->dtype = qb200_narrows_loaded_f16(name, e->ndim, e->dtype) ? QB200_BFLOAT16 : e->dtype;
  desc->ndim = e->ndim;
  int64_t st = 1;
  for (int d = e->ndim - 1; d >= 0; --d) { desc->shape[d] = e->shape[d]; desc->stride[d] = st; st *= e->shape[d]; }
  if (nbytes) *nbytes = e->end - e->begin;
  return QB200_OK;
}

// Copies a tensor into caller-allocated device memory (narrowed to bf16 where the rule says so).  Synchronous.
QB200_API int qb200_checkpoint_load_tensor(const qb200_checkpoint* ck, const char* name, void* device_dst, size_t dst_bytes) {
  if (!ck || !name || !device_dst) return ld_fail(QB200_ERR_BAD_ARG, "checkpoint_load_tensor: null argument");
  const Entry* e = find(ck, name);
  if (!e) return ld_fail(QB200_ERR_BAD_ARG, std::string("checkpoint_load_tensor: no tensor named ") + name);
  const size_t n = e->end - e->begin;
  if (dst_bytes < n) return ld_fail(QB200_ERR_WORKSPACE, "checkpoint_load_tensor: destination too small");
  const unsigned char* src = ck->map + ck->data0 + e->begin;
  cudaError_t err;
  if (qb200_narrows_loaded_f16(name, e->ndim, e->dtype)) {
    std::vector<uint16_t> tmp(n / 2);
    for (size_t i = 0; i < n / 2; ++i) {
      uint16_t h;
      memcpy(&h, src + 2 * i, 2);
      tmp[i] = float_to_bf16(half_to_float(h));
    }
    err = cudaMemcpy(device_dst, tmp.data(), n, cudaMemcpyHostToDevice);
  } else {
    err = cudaMemcpy(device_dst, src, n, cudaMemcpyHostToDevice);
  }
  if (err != cudaSuccess) return ld_fail(QB200_ERR_CUDA, std::string("checkpoint_load_tensor: ") + cudaGetErrorString(err));
  return QB200_OK;
}

// The host bytes of a tensor as the loader would upload them (for hosts that stage their own copies, and for tests
// without a GPU): writes min(cap, size) bytes, returns the tensor's size through *nbytes.
QB200_API int qb200_checkpoint_read_tensor(const qb200_checkpoint* ck, const char* name, void* host_dst, size_t cap, size_t* nbytes) {
  if (!ck || !name) return ld_fail(QB200_ERR_BAD_ARG, "checkpoint_read_tensor: null argument");
  const Entry* e = find(ck, name);
  if (!e) return ld_fail(QB200_ERR_BAD_ARG, std::string("checkpoint_read_tensor: no tensor named ") + name);
  const size_t n = e->end - e->begin;
  if (nbytes) *nbytes = n;
  if (!host_dst) return QB200_OK;
  const unsigned char* src = ck->map + ck->data0 + e->begin;
  const size_t m = cap < n ? cap : n;
  if (qb200_narrows_loaded_f16(name, e->ndim, e->dtype)) {
    for (size_t i = 0; i < m / 2; ++i) {
      uint16_t h;
      memcpy(&h, src + 2 * i, 2);
      const uint16_t b = float_to_bf16(half_to_float(h));
      memcpy((unsigned char*)host_dst + 2 * i, &b, 2);
    }
  } else {
    memcpy(host_dst, src, m);
  }
  return QB200_OK;
}

}  // extern "C"
