// Decode attention over the packed KV cache for callers that cannot allocate device memory.
//
// qb200_kv_decode_attention needs a scratch buffer for its split-KV partials and asks the caller
// for it.  Some callers have no way to provide one: a host runtime whose device heap is fixed at
// start-up and fully handed out to model weights and the KV cache, or code running inside a
// region where cudaMalloc is forbidden (it synchronises the device and is illegal while a stream
// is being captured).  For them this file keeps one scratch array inside the library image.
//
// The array lives in device memory of every GPU that loads the library, from load until exit
// (kStaticScratchBytes per GPU).  Its name is only a host-side handle; the device address is
// looked up once per device with cudaGetSymbolAddress while that device is current, and that
// address is what the kernels receive.
#include <cstdio>

#include "kernels.h"

namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB: e.g. 16 sequences x 32 heads x 128 dims up to 12 splits
static __device__ __align__(256) unsigned char g_kv_static_scratch[kStaticScratchBytes];

// Device address of the scratch array on the current device (resolved on first use per device).
cudaError_t static_scratch_address(void** out) {
  static void* addr[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> setup_lk(qb::setup_mutex());
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_kv_static_scratch);
    if (e != cudaSuccess) return e;
    addr[dev] = p;
  }
  *out = addr[dev];
  return cudaSuccess;
}

}  // namespace

extern "C" {

QB200_API size_t qb200_kv_decode_attention_noalloc_max_scratch(void) { return kStaticScratchBytes; }

QB200_API int qb200_kv_decode_attention_noalloc(qb200_tensor* res, const qb200_tensor* q, const qb200_tensor* k_q,
                                                const qb200_tensor* k_scales, const qb200_tensor* k_biases,
                                                const qb200_tensor* v_q, const qb200_tensor* v_scales,
                                                const qb200_tensor* v_biases, int bits, int group_size, float scale,
                                                const char* mask_mode, const qb200_tensor* mask_arr,
                                                const qb200_tensor* kv_lens, qb200_stream s) {
  // Size check first, from the shapes alone, so that an oversized request never reaches a kernel.
  if (q == nullptr || k_q == nullptr || v_q == nullptr || q->ndim != 4 || k_q->ndim != 4 || v_q->ndim != 4 ||
      (bits != 4 && bits != 8))
    return qb200_kv_decode_attention(res, q, k_q, k_scales, k_biases, v_q, v_scales, v_biases, bits, group_size, scale,
                                     mask_mode, mask_arr, kv_lens, nullptr, 0, s);  // reports the shape/argument error
  const int64_t B = q->shape[0], Hq = q->shape[1], Hkv = k_q->shape[1], T = k_q->shape[2];
  const int64_t Dv = v_q->shape[3] * (32 / bits);
  const size_t need = qb200_kv_decode_attention_workspace_size(B, Hq, Hkv, T, Dv);
  if (need == 0)   // an empty batch, head list or cache view: the main entry answers it (OK or a shape error) without a launch
    return qb200_kv_decode_attention(res, q, k_q, k_scales, k_biases, v_q, v_scales, v_biases, bits, group_size, scale,
                                     mask_mode, mask_arr, kv_lens, nullptr, 0, s);
  if (need > kStaticScratchBytes) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "kv_decode_attention_noalloc: this shape needs %zu bytes of scratch, the built-in array holds %zu; "
             "use qb200_kv_decode_attention with a caller-provided workspace",
             need, kStaticScratchBytes);
    return qb::report_error(QB200_ERR_WORKSPACE, msg);
  }
  void* scratch = nullptr;
  if (static_scratch_address(&scratch) != cudaSuccess)
    return qb::report_error(QB200_ERR_CUDA, "kv_decode_attention_noalloc: cudaGetSymbolAddress failed for the scratch array");
  return qb200_kv_decode_attention(res, q, k_q, k_scales, k_biases, v_q, v_scales, v_biases, bits, group_size, scale,
                                   mask_mode, mask_arr, kv_lens, scratch, kStaticScratchBytes, s);
}

}  // extern "C"
