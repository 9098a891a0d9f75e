// Chunked persistence of the affine-quantized KV cache: the on-disk format of mlx-serve's SSD tier for its prefix
// cache (src/kv_disk_cache.zig:1-48), the data-format half of it.  A chunk file is a safetensors container holding,
// for every layer that has a KV cache, the token slice [pos0, pos1) of the layer's six capacity buffers under the
// keys "l{i}.k", "l{i}.v", "l{i}.ks", "l{i}.kb", "l{i}.vs", "l{i}.vb" (src/kv_disk_cache.zig:1062-1074), each of shape
// [1, Hkv, pos1 - pos0, cols].  Restoring follows restoreKvInto (src/kv_disk_cache.zig:320-440): a layer whose "l{i}.k"
// is absent is skipped (hybrid architectures keep no KV for some layers), any other missing key, a rank other than
// four or fewer stored positions than asked for is a corrupt chunk, and a chunk that holds MORE positions than asked
// for is sliced down, never trusted.  The index around the chunks (meta.json, tokens.bin, the longest-prefix
// lookup, eviction) is host policy and is not restated here.
//
// Host code plus strided copies: the token slice of a capacity buffer [1, Hkv, cap, cols] is Hkv runs of
// (pos1 - pos0) * cols contiguous elements, one 2-D copy per buffer.
#include <fcntl.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <set>
#include <string>
#include <vector>

#include "kernels.h"

namespace {

int kc_fail(int status, const std::string& msg) { return qb::report_error(status, msg.c_str()); }

const char* const kKinds[6] = {"k", "ks", "kb", "v", "vs", "vb"};   // order of the fields of qb200_kv_layer

const qb200_tensor* field(const qb200_kv_layer& l, int k) {
  switch (k) {
    case 0: return &l.k_q;
    case 1: return &l.k_scales;
    case 2: return &l.k_biases;
    case 3: return &l.v_q;
    case 4: return &l.v_scales;
    default: return &l.v_biases;
  }
}

int elem_bytes(int dtype) { return dtype == QB200_UINT32 || dtype == QB200_FLOAT32 ? 4 : 2; }
const char* st_dtype(int dtype) {
  switch (dtype) {
    case QB200_UINT32: return "U32";
    case QB200_FLOAT32: return "F32";
    case QB200_FLOAT16: return "F16";
    default: return "BF16";
  }
}

// [1, Hkv, cap, cols] with contiguous rows: the only layout the cache's capacity buffers take
int check_buffer(const qb200_tensor* t, const char* what, int64_t pos_end) {
  if (!t->data) return kc_fail(QB200_ERR_BAD_ARG, std::string("kv_chunk: missing buffer ") + what);
  if (t->ndim != 4 || t->shape[0] != 1) return kc_fail(QB200_ERR_BAD_SHAPE, std::string("kv_chunk: ") + what + " must be [1, Hkv, cap, cols]");
  if (t->stride[3] != 1 || t->stride[2] != t->shape[3]) return kc_fail(QB200_ERR_BAD_STRIDE, std::string("kv_chunk: rows of ") + what + " must be contiguous");
  if (pos_end > t->shape[2]) return kc_fail(QB200_ERR_BAD_SHAPE, std::string("kv_chunk: positions beyond the capacity of ") + what);
  return QB200_OK;
}

}  // namespace

extern "C" {

QB200_API int qb200_kv_chunk_save(const char* path, const qb200_kv_layer* layers, int n_layers, int64_t pos0, int64_t pos1,
                                  qb200_stream s) {
  if (!path || !layers || n_layers <= 0) return kc_fail(QB200_ERR_BAD_ARG, "kv_chunk_save: null argument");
  if (pos0 < 0 || pos1 <= pos0) return kc_fail(QB200_ERR_BAD_SHAPE, "kv_chunk_save: empty position range");
  const int64_t n = pos1 - pos0;
  struct Item { std::string key; const qb200_tensor* t; size_t begin, bytes; };
  std::vector<Item> items;
  size_t total = 0;
  for (int li = 0; li < n_layers; ++li) {
    if (!layers[li].k_q.data) continue;   // a layer without a KV cache is absent from the chunk
    for (int k = 0; k < 6; ++k) {
      const qb200_tensor* t = field(layers[li], k);
      const std::string key = "l" + std::to_string(li) + "." + kKinds[k];
      if (int st = check_buffer(t, key.c_str(), pos1)) return st;
      const size_t bytes = (size_t)t->shape[1] * (size_t)n * (size_t)t->shape[3] * elem_bytes(t->dtype);
      items.push_back({key, t, total, bytes});
      total += bytes;
    }
  }
  if (items.empty()) return kc_fail(QB200_ERR_BAD_ARG, "kv_chunk_save: no layer has a cache");
  std::string hdr = "{";
  for (size_t i = 0; i < items.size(); ++i) {
    const qb200_tensor* t = items[i].t;
    char buf[256];
    snprintf(buf, sizeof(buf), "%s\"%s\":{\"dtype\":\"%s\",\"shape\":[1,%lld,%lld,%lld],\"data_offsets\":[%zu,%zu]}", i ? "," : "",
             items[i].key.c_str(), st_dtype(t->dtype), (long long)t->shape[1], (long long)n, (long long)t->shape[3],
             items[i].begin, items[i].begin + items[i].bytes);
    hdr += buf;
  }
  hdr += "}";
  while (hdr.size() % 8) hdr += ' ';
  std::vector<unsigned char> host(total);
  for (const Item& it : items) {   // Hkv runs of n * cols elements, head stride apart
    const qb200_tensor* t = it.t;
    const size_t eb = elem_bytes(t->dtype), run = (size_t)n * t->shape[3] * eb;
    const unsigned char* src = (const unsigned char*)t->data + (size_t)pos0 * t->stride[2] * eb;
    const cudaError_t e = cudaMemcpy2DAsync(host.data() + it.begin, run, src, (size_t)t->stride[1] * eb, run, (size_t)t->shape[1],
                                            cudaMemcpyDeviceToHost, (cudaStream_t)s);
    if (e != cudaSuccess) return kc_fail(QB200_ERR_CUDA, std::string("kv_chunk_save: ") + cudaGetErrorString(e));
  }
  const cudaError_t e = cudaStreamSynchronize((cudaStream_t)s);
  if (e != cudaSuccess) return kc_fail(QB200_ERR_CUDA, std::string("kv_chunk_save: ") + cudaGetErrorString(e));
  // written under a temporary name and renamed, so that a reader never sees half a chunk
  const std::string tmp = std::string(path) + ".tmp";
  FILE* f = fopen(tmp.c_str(), "wb");
  if (!f) return kc_fail(QB200_ERR_BAD_ARG, std::string("kv_chunk_save: cannot create ") + tmp);
  const uint64_t hl = hdr.size();
  bool ok = fwrite(&hl, 8, 1, f) == 1 && fwrite(hdr.data(), 1, hdr.size(), f) == hdr.size() &&
            (total == 0 || fwrite(host.data(), 1, total, f) == total);
  ok = (fclose(f) == 0) && ok;
  if (!ok || rename(tmp.c_str(), path) != 0) {
    remove(tmp.c_str());
    return kc_fail(QB200_ERR_BAD_ARG, std::string("kv_chunk_save: cannot write ") + path);
  }
  return QB200_OK;
}

QB200_API int qb200_kv_chunk_restore(const char* path, const qb200_kv_layer* layers, int n_layers, int64_t pos0, int64_t need,
                                     qb200_stream s) {
  if (!path || !layers || n_layers <= 0) return kc_fail(QB200_ERR_BAD_ARG, "kv_chunk_restore: null argument");
  if (pos0 < 0 || need <= 0) return kc_fail(QB200_ERR_BAD_SHAPE, "kv_chunk_restore: empty position range");
  qb200_checkpoint* ck = nullptr;
  if (int st = qb200_checkpoint_open(&ck, path)) return st;
  int status = QB200_OK;
  std::set<std::string> names;
  for (int i = 0; i < qb200_checkpoint_num_tensors(ck); ++i) names.insert(qb200_checkpoint_tensor_name(ck, i));
  std::vector<std::vector<unsigned char>> staged;   // host copies stay alive until the stream has consumed them
  for (int li = 0; li < n_layers && status == QB200_OK; ++li) {
    for (int k = 0; k < 6 && status == QB200_OK; ++k) {
      const std::string key = "l" + std::to_string(li) + "." + kKinds[k];
      if (!names.count(key)) {
        if (k == 0) break;   // layer absent from this chunk
        status = kc_fail(QB200_ERR_BAD_SHAPE, "kv_chunk_restore: corrupt chunk, missing " + key);
        break;
      }
      qb200_tensor d;
      size_t bytes = 0;
      if ((status = qb200_checkpoint_tensor_info(ck, key.c_str(), &d, &bytes))) break;
      const qb200_tensor* t = field(layers[li], k);
      if (!layers[li].k_q.data) { status = kc_fail(QB200_ERR_BAD_ARG, "kv_chunk_restore: the chunk holds layer " + std::to_string(li) + ", the cache does not"); break; }
      if ((status = check_buffer(t, key.c_str(), pos0 + need))) break;
      if (d.ndim != 4 || d.shape[0] != 1 || d.shape[2] < need || d.shape[1] != t->shape[1] || d.shape[3] != t->shape[3] ||
          d.dtype != t->dtype) {
        status = kc_fail(QB200_ERR_BAD_SHAPE, "kv_chunk_restore: corrupt chunk or another cache geometry at " + key);
        break;
      }
      staged.emplace_back(bytes);
      if ((status = qb200_checkpoint_read_tensor(ck, key.c_str(), staged.back().data(), bytes, nullptr))) break;
      // the first `need` of the stored positions of every head -> positions [pos0, pos0 + need) of the buffer
      const size_t eb = elem_bytes(t->dtype), run = (size_t)need * t->shape[3] * eb;
      unsigned char* dst = (unsigned char*)t->data + (size_t)pos0 * t->stride[2] * eb;
      const cudaError_t e = cudaMemcpy2DAsync(dst, (size_t)t->stride[1] * eb, staged.back().data(), (size_t)d.shape[2] * d.shape[3] * eb, run,
                                              (size_t)t->shape[1], cudaMemcpyHostToDevice, (cudaStream_t)s);
      if (e != cudaSuccess) status = kc_fail(QB200_ERR_CUDA, std::string("kv_chunk_restore: ") + cudaGetErrorString(e));
    }
  }
  const cudaError_t e = cudaStreamSynchronize((cudaStream_t)s);
  if (status == QB200_OK && e != cudaSuccess) status = kc_fail(QB200_ERR_CUDA, std::string("kv_chunk_restore: ") + cudaGetErrorString(e));
  qb200_checkpoint_close(ck);
  return status;
}

}  // extern "C"
