// C++ host-side mirror of the wrappers through which mlx-serve's Zig code reaches the quantized-inference
// path, on top of libqb200's C ABI (include/qb200.h).  Same names, argument meaning and error behaviour as the
// reference's wrappers, so that a call site reads the same after the switch:
//
//   quantizeAffine / dequantizeAffine        src/kv_quant.zig:126-162, :407-430
//   QuantizedKV, quantAttention              src/kv_quant.zig:102-124, :478-687
//   qmatmulBits                              src/transformer.zig:20894-20983
//   gatherExpertMm                           src/transformer.zig:20763-20784
//   gatherExpertGateUpSwiGLU                 src/transformer.zig:15007-15035 with fusedSwiGLU, :19925-19931
//   KVCacheEntry, KVCache::updateAffine      src/transformer.zig:2777-2858, :3224-3337
//   moeSortByExpert (argsort chain of moeMLP2) src/transformer.zig:14961-15006
//   quantAttentionBatched (per-slot caches)  src/transformer.zig:9742-9792, :10165-10249
//   rmsNorm, addRmsNorm, ropeDynamic, computeGeglu, updateAffineBatched   src/transformer.zig:7770-7779, :9678, :8220-8243, :9738-9756
//   rotateLastDim, quantizeTurbo, dequantizeTurbo   src/kv_quant.zig:362-403
//   saveChunk / restoreChunk (chunk files of the prefix cache's SSD tier)   src/kv_disk_cache.zig:320-440, :1062-1074
//   Checkpoint (safetensors triples, f16 narrowing, geometry)   src/model.zig:3030-3061, :3241-3256; src/transformer.zig:16763-16790
//   moeBlockEp (moeMLP2 over several GPUs; define QB200_HOST_WITH_EP and link libqb200_ep)   src/transformer.zig:14945-15140
//
// Differences that follow from the eager ABI: arrays are caller-owned device buffers described by `Array`
// (no refcounted handles), results are allocated by the caller, and every call takes the CUDA stream (as the ABI's `qb200_stream`, a `cudaStream_t`).  A
// request the library declines surfaces as `Declined` (the reference's wrappers treat a declined fast lane as
// fall-through, src/transformer.zig:20463-20475); every other failure as `Error` with the library's message.
// Header only; needs nothing but the C ABI.
#pragma once
#include <cstdint>
#include <initializer_list>
#include <stdexcept>
#include <string>
#include <vector>

#include "qb200.h"

namespace qb200h {

struct Error : std::runtime_error {
  int status;
  Error(int st, const std::string& msg) : std::runtime_error(msg), status(st) {}
};
struct Declined : Error {
  using Error::Error;
};

// 0 -> ok; QB200_ERR_UNSUPPORTED (1) -> Declined; anything else -> Error (src/mlx.zig:547-550 maps non-zero to
// error.MlxError).
inline void check(int rc) {
  if (rc == 0) return;
  const char* m = qb200_last_error();
  if (rc == 1) throw Declined(rc, m ? m : "declined");
  throw Error(rc, m ? m : "qb200 error");
}

// A device buffer seen as a tensor: the caller owns `data`.
struct Array {
  qb200_tensor t{};
  Array() = default;
  // contiguous row-major view
  Array(void* data, qb200_dtype dtype, std::initializer_list<int64_t> shape) {
    t.data = data;
    t.dtype = dtype;
    t.ndim = (int32_t)shape.size();
    int i = 0;
    for (int64_t d : shape) t.shape[i++] = d;
    int64_t run = 1;
    for (int d = t.ndim - 1; d >= 0; --d) { t.stride[d] = run; run *= t.shape[d]; }
  }
  bool empty() const { return t.data == nullptr; }
  int64_t dim(int i) const { return t.shape[i < 0 ? t.ndim + i : i]; }
  // view of `len` entries starting at `start` along axis `axis` (strides kept: cache views are strided slices,
  // src/transformer.zig:3472-3495)
  Array slice(int axis, int64_t start, int64_t len, size_t elem_bytes) const {
    Array r = *this;
    r.t.data = (char*)t.data + (size_t)(start * t.stride[axis]) * elem_bytes;
    r.t.shape[axis] = len;
    return r;
  }
};

inline qb200_optional_int some(int v) { return qb200_optional_int{v, true}; }

// One quantized weight (or expert bank): the triple the loader keeps per tensor (src/transformer.zig:18085).
struct QWeight {
  Array q, scales, biases;
  int group_size = 64, bits = 4;
};

// kv_quant.QuantizedKV (src/kv_quant.zig:102-124): packed codes + scales + biases, quantised along the last axis.
struct QuantizedKV {
  Array q, scales, biases;
  int group_size = 64, bits = 4;
};

// quantizeAffine (src/kv_quant.zig:126-162): x [..., D] -> triple, all three caller-allocated.
inline void quantizeAffine(QuantizedKV& out, const Array& x, qb200_stream s) {
  check(qb200_quantize(&out.q.t, &out.scales.t, &out.biases.t, &x.t, some(out.group_size), some(out.bits), "affine",
                       nullptr, s));
}

// dequantizeAffine (src/kv_quant.zig:407-430): triple -> dense [..., D] in res's dtype.
inline void dequantizeAffine(Array& res, const QuantizedKV& kv, qb200_stream s) {
  qb200_optional_dtype dt{(qb200_dtype)res.t.dtype, true};
  check(qb200_dequantize(&res.t, &kv.q.t, &kv.scales.t, &kv.biases.t, some(kv.group_size), some(kv.bits), "affine", nullptr,
                         dt, s));
}

// qmatmulBits (src/transformer.zig:20894-20983): res = x . dequant(w)^T.
inline void qmatmulBits(Array& res, const Array& x, const QWeight& w, qb200_stream s) {
  check(qb200_quantized_matmul(&res.t, &x.t, &w.q.t, &w.scales.t, &w.biases.t, true, some(w.group_size), some(w.bits),
                               "affine", s));
}

// The projections that share their input (q,k,v / gate,up: src/transformer.zig:9202-9207, :9452-9454) in one call.
inline void qmatmulBitsBatch(Array* const* res, const Array& x, const QWeight* const* w, int count, qb200_stream s) {
  if (count < 1 || count > 8) throw Error(2, "qmatmulBitsBatch: count must be 1..8");
  qb200_tensor* r[8];
  const qb200_tensor *q[8], *sc[8], *bi[8];
  for (int i = 0; i < count; ++i) { r[i] = &res[i]->t; q[i] = &w[i]->q.t; sc[i] = &w[i]->scales.t; bi[i] = &w[i]->biases.t; }
  check(qb200_quantized_matmul_batch(r, &x.t, q, sc, bi, count, true, some(w[0]->group_size), some(w[0]->bits), "affine",
                                     s));
}

// gatherExpertMm (src/transformer.zig:20763-20784): res[i] = x[lhs(i)] . dequant(bank[rhs[i]])^T; lhs may be null.
inline void gatherExpertMm(Array& res, const Array& x, const QWeight& bank, const Array* lhs_indices, const Array& rhs_indices,
                           bool sorted_indices, qb200_stream s) {
  check(qb200_gather_qmm(&res.t, &x.t, &bank.q.t, &bank.scales.t, &bank.biases.t, lhs_indices ? &lhs_indices->t : nullptr,
                         &rhs_indices.t, true, some(bank.group_size), some(bank.bits), "affine", sorted_indices,
                         s));
}

// The gate and up projections of the routed-expert block with fusedSwiGLU applied (src/transformer.zig:15007-15035,
// :19925-19931): res[i] = silu(x[lhs(i)] . gate[rhs[i]]^T) * (x[lhs(i)] . up[rhs[i]]^T).  Throws Declined for shapes the
// fused kernel does not serve; the caller then keeps two gatherExpertMm calls and its own SwiGLU, as the reference's
// fusedSwiGLU returns null to its caller.
inline void gatherExpertGateUpSwiGLU(Array& res, const Array& x, const QWeight& gate, const QWeight& up, const Array* lhs_indices,
                                     const Array& rhs_indices, bool sorted_indices, qb200_stream s) {
  check(qb200_gather_qmm_swiglu(&res.t, &x.t, &gate.q.t, &gate.scales.t, &gate.biases.t, &up.q.t, &up.scales.t, &up.biases.t,
                                lhs_indices ? &lhs_indices->t : nullptr, &rhs_indices.t, some(gate.group_size), some(gate.bits),
                                "affine", sorted_indices, s));
}

// gatherQmvDownReduce (src/transformer.zig:20559-20623, :20675-20761): the single-token tail of the routed-expert block,
// res[t, n] = sum_j round(round(act[t, j] . down[inds[t, j]][n]) * scores[t, j]).  Throws Declined beyond a few tokens.
inline void gatherQmvDownReduce(Array& res, const Array& act, const QWeight& down, const Array& inds, const Array& scores,
                                qb200_stream s) {
  check(qb200_moe_down_reduce(&res.t, &act.t, &down.q.t, &down.scales.t, &down.biases.t, &inds.t, &scores.t,
                              some(down.group_size), some(down.bits), "affine", s));
}

// moeRoutingChain (src/transformer.zig:17022-17063): the k largest logits per row and their renormalised softmax scores.
inline void moeRoutingChain(Array& inds, Array& norm_scores, const Array& router_logits, int k, qb200_stream s) {
  check(qb200_moe_route(&inds.t, &norm_scores.t, &router_logits.t, k, s));
}

// The tail of moeMLP2 (src/transformer.zig:15036-15042, :15127-15140): rows of the down projection back to token
// order, times norm_scores, summed over top-k.  inv_order may be null (rows already in token order).
inline void moeWeightedSum(Array& res, const Array& down_sorted, const Array& norm_scores, const Array* inv_order, qb200_stream s) {
  check(qb200_moe_weighted_sum(&res.t, &down_sorted.t, &norm_scores.t, inv_order ? &inv_order->t : nullptr, s));
}

// KVCacheEntry (src/transformer.zig:2777-2858): six capacity buffers [B, Hkv, cap, *] per layer and the fill level.
struct KVCacheEntry {
  QuantizedKV keys, values;   // capacity buffers
  int64_t offset = 0;         // tokens stored so far
  int64_t capacity() const { return keys.q.dim(2); }
  // views of the first `offset` tokens, with the capacity buffers' strides
  QuantizedKV view(const QuantizedKV& c) const {
    QuantizedKV v = c;
    v.q = c.q.slice(2, 0, offset, 4);
    v.scales = c.scales.slice(2, 0, offset, 2);
    v.biases = c.biases.slice(2, 0, offset, 2);
    return v;
  }
};

// KVCache.updateAffine (src/transformer.zig:3224-3337): quantise the new K and V rows [B, Hkv, S, D] and write
// them at `offset`; the caller grows the capacity buffers (the reference grows them by 25 %, :3116-3146).
inline void updateAffine(KVCacheEntry& e, const Array& k_new, const Array& v_new, qb200_stream s) {
  const int64_t S = k_new.dim(2);
  if (e.offset + S > e.capacity()) throw Error(2, "updateAffine: capacity exceeded; grow the cache first");
  check(qb200_kv_append(&e.keys.q.t, &e.keys.scales.t, &e.keys.biases.t, &k_new.t, e.offset, e.keys.bits, e.keys.group_size,
                        s));
  check(qb200_kv_append(&e.values.q.t, &e.values.scales.t, &e.values.biases.t, &v_new.t, e.offset, e.values.bits,
                        e.values.group_size, s));
  e.offset += S;
}

// quantAttention (src/kv_quant.zig:478-687) for T_q == 1: out [B, Hq, 1, Dv] = softmax(q K^T * scale) V over the
// packed cache views.  `mask` is an optional additive row (mask mode "array"), `kv_lens` optional int32 [B].
inline size_t quantAttentionWorkspace(int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t Dv) {
  return qb200_kv_decode_attention_workspace_size(B, Hq, Hkv, T, Dv);
}
inline void quantAttention(Array& out, const Array& q, const QuantizedKV& k, const QuantizedKV& v, float scale, const Array* mask,
                           const Array* kv_lens, void* workspace, size_t workspace_bytes, qb200_stream s) {
  check(qb200_kv_decode_attention(&out.t, &q.t, &k.q.t, &k.scales.t, &k.biases.t, &v.q.t, &v.scales.t, &v.biases.t, k.bits,
                                  k.group_size, scale, mask ? "array" : "", mask ? &mask->t : nullptr,
                                  kv_lens ? &kv_lens->t : nullptr, workspace, workspace_bytes, s));
}

// The sort step of moeMLP2 (src/transformer.zig:14961-15006): order = argsort(flat_inds), inv_order = argsort(order),
// sorted_inds = flat_inds[order], lhs_idx = order / k, and the row range of every expert.  Any output may be null.
inline void moeSortByExpert(Array* order, Array* inv_order, Array* sorted_inds, Array* lhs_idx, Array* expert_offsets,
                            const Array& inds, int num_experts, qb200_stream s) {
  check(qb200_moe_sort_by_expert(order ? &order->t : nullptr, inv_order ? &inv_order->t : nullptr, sorted_inds ? &sorted_inds->t : nullptr,
                                 lhs_idx ? &lhs_idx->t : nullptr, expert_offsets ? &expert_offsets->t : nullptr, &inds.t, num_experts, s));
}

// The KV read of forwardBatchedDecode (src/transformer.zig:9742-9792): every slot owns a B = 1 cache with its own
// capacity and length.  The reference dequantises, pads to the longest and concatenates; here the packed views are
// read in place.  `entries[n]` is slot n's cache of this layer (views of its first `offset` tokens are taken here).
inline size_t quantAttentionBatchedWorkspace(int64_t slots, int64_t Hq, int64_t Hkv, int64_t T_max, int64_t Dv) {
  return qb200_kv_decode_attention_ptrs_workspace_size(slots, Hq, Hkv, T_max, Dv);
}
inline void quantAttentionBatched(Array& out, const Array& q, const KVCacheEntry* const* entries, int slots, float scale,
                                  void* workspace, size_t workspace_bytes, qb200_stream s) {
  if (slots < 1 || slots > 4096) throw Error(2, "quantAttentionBatched: 1..4096 slots");
  std::vector<QuantizedKV> kv(2 * (size_t)slots);
  std::vector<const qb200_tensor*> p(6 * (size_t)slots);
  for (int n = 0; n < slots; ++n) {
    kv[2 * n] = entries[n]->view(entries[n]->keys);
    kv[2 * n + 1] = entries[n]->view(entries[n]->values);
    p[0 * slots + n] = &kv[2 * n].q.t; p[1 * slots + n] = &kv[2 * n].scales.t; p[2 * slots + n] = &kv[2 * n].biases.t;
    p[3 * slots + n] = &kv[2 * n + 1].q.t; p[4 * slots + n] = &kv[2 * n + 1].scales.t; p[5 * slots + n] = &kv[2 * n + 1].biases.t;
  }
  check(qb200_kv_decode_attention_ptrs(&out.t, &q.t, &p[0], &p[slots], &p[2 * slots], &p[3 * slots], &p[4 * slots], &p[5 * slots], slots,
                                       entries[0]->keys.bits, entries[0]->keys.group_size, scale, "", nullptr, nullptr, workspace,
                                       workspace_bytes, s));
}

// The per-slot cache update loop of forwardBatchedDecode (src/transformer.zig:9738-9756) as one launch: the new K and V
// rows [slots, Hkv, 1, D] go to each slot's own cache at its own offset, which then advances.
inline void updateAffineBatched(KVCacheEntry* const* entries, int slots, const Array& k_new, const Array& v_new, qb200_stream s) {
  if (slots < 1 || slots > 4096) throw Error(2, "updateAffineBatched: 1..4096 slots");
  std::vector<qb200_tensor*> p(6 * (size_t)slots);
  std::vector<int64_t> offs((size_t)slots);
  for (int n = 0; n < slots; ++n) {
    KVCacheEntry& e = *entries[n];
    if (e.offset + 1 > e.capacity()) throw Error(2, "updateAffineBatched: capacity exceeded; grow the cache first");
    p[0 * slots + n] = &e.keys.q.t; p[1 * slots + n] = &e.keys.scales.t; p[2 * slots + n] = &e.keys.biases.t;
    p[3 * slots + n] = &e.values.q.t; p[4 * slots + n] = &e.values.scales.t; p[5 * slots + n] = &e.values.biases.t;
    offs[n] = e.offset;
  }
  check(qb200_kv_append_seqs(&p[0], &p[slots], &p[2 * slots], &p[3 * slots], &p[4 * slots], &p[5 * slots], &k_new.t, &v_new.t, offs.data(),
                             slots, entries[0]->keys.bits, entries[0]->keys.group_size, s));
  for (int n = 0; n < slots; ++n) entries[n]->offset += 1;
}

// The same with the rotary embedding of the decode step folded in (mlx_fast_rope_dynamic on q and k, src/transformer.zig:9678,
// :9735, then the per-slot update): q [slots, Hq, 1, D] is rotated in place, k_new on its way into the caches, every
// slot at its own offset.
inline void ropeUpdateAffineBatched(Array& q, int dims, float base, float scale, KVCacheEntry* const* entries, int slots,
                                    const Array& k_new, const Array& v_new, qb200_stream s) {
  if (slots < 1 || slots > 4096) throw Error(2, "ropeUpdateAffineBatched: 1..4096 slots");
  std::vector<qb200_tensor*> p(6 * (size_t)slots);
  std::vector<int64_t> offs((size_t)slots);
  for (int n = 0; n < slots; ++n) {
    KVCacheEntry& e = *entries[n];
    if (e.offset + 1 > e.capacity()) throw Error(2, "ropeUpdateAffineBatched: capacity exceeded; grow the cache first");
    p[0 * slots + n] = &e.keys.q.t; p[1 * slots + n] = &e.keys.scales.t; p[2 * slots + n] = &e.keys.biases.t;
    p[3 * slots + n] = &e.values.q.t; p[4 * slots + n] = &e.values.scales.t; p[5 * slots + n] = &e.values.biases.t;
    offs[n] = e.offset;
  }
  check(qb200_rope_kv_append_seqs(&q.t, dims, base, scale, &p[0], &p[slots], &p[2 * slots], &p[3 * slots], &p[4 * slots], &p[5 * slots],
                                  &k_new.t, &v_new.t, offs.data(), slots, entries[0]->keys.bits, entries[0]->keys.group_size, s));
  for (int n = 0; n < slots; ++n) entries[n]->offset += 1;
}

// rmsNorm / rmsNormEps (src/transformer.zig:7770-7779) and the mlx_add that precedes the post-attention and the next
// layer's input norm (:9836-9843, :9856-9859) fused with it.
inline void rmsNorm(Array& res, const Array& x, const Array& weight, float eps, qb200_stream s) {
  check(qb200_rms_norm(&res.t, &x.t, &weight.t, eps, s));
}
inline void addRmsNorm(Array& sum, Array* normed, const Array& a, const Array& b, const Array* weight, float eps, qb200_stream s) {
  check(qb200_add_rms_norm(&sum.t, normed ? &normed->t : nullptr, &a.t, &b.t, weight ? &weight->t : nullptr, eps, s));
}
// mlx_fast_rope_dynamic as forwardBatchedDecode calls it (src/transformer.zig:9678, :9735): one position per slot.
inline void ropeDynamic(Array& res, const Array& x, int dims, float base, float scale, const Array& offsets, qb200_stream s) {
  check(qb200_rope(&res.t, &x.t, dims, false, qb200_optional_float{base, true}, scale, &offsets.t, nullptr, s));
}
// computeGeglu with the silu activation (src/transformer.zig:8220-8243): the reference's bit-exact fused SwiGLU.
inline void computeGeglu(Array& res, const Array& gate, const Array& up, qb200_stream s) { check(qb200_swiglu(&res.t, &gate.t, &up.t, s)); }

// One opened .safetensors file.  `loadTriple` is what the reference's loader does per quantized linear
// (src/model.zig:3241-3256 narrows f16 scales and biases to bf16; src/transformer.zig:16763-16790 solves bits and
// group size from the packed geometry): the three tensors go to caller-allocated device memory and the QWeight
// describes them.
class Checkpoint {
 public:
  explicit Checkpoint(const std::string& path) { check(qb200_checkpoint_open(&ck_, path.c_str())); }
  ~Checkpoint() { qb200_checkpoint_close(ck_); }
  Checkpoint(const Checkpoint&) = delete;
  Checkpoint& operator=(const Checkpoint&) = delete;
  int size() const { return qb200_checkpoint_num_tensors(ck_); }
  std::string name(int i) const { const char* n = qb200_checkpoint_tensor_name(ck_, i); return n ? n : ""; }
  // shape and dtype as loaded (data stays null) and the bytes to allocate
  Array info(const std::string& name, size_t* nbytes) const {
    Array a;
    check(qb200_checkpoint_tensor_info(ck_, name.c_str(), &a.t, nbytes));
    return a;
  }
  void load(const std::string& name, void* device_dst, size_t bytes) const {
    check(qb200_checkpoint_load_tensor(ck_, name.c_str(), device_dst, bytes));
  }
  // <prefix>.weight / .scales / .biases into the three buffers (sizes from info()); in_dim is the layer's input width
  QWeight loadTriple(const std::string& prefix, int64_t in_dim, void* q, void* scales, void* biases) const {
    QWeight w;
    size_t nq = 0, ns = 0, nb = 0;
    w.q = info(prefix + ".weight", &nq);
    w.scales = info(prefix + ".scales", &ns);
    w.biases = info(prefix + ".biases", &nb);
    check(qb200_affine_params_from_geometry(w.q.dim(-1), w.scales.dim(-1), in_dim, &w.bits, &w.group_size));
    load(prefix + ".weight", q, nq);
    load(prefix + ".scales", scales, ns);
    load(prefix + ".biases", biases, nb);
    w.q.t.data = q;
    w.scales.t.data = scales;
    w.biases.t.data = biases;
    return w;
  }

 private:
  qb200_checkpoint* ck_ = nullptr;
};

// The TurboQuant cache schemes (src/kv_quant.zig:164-403): a Hadamard rotation of the last axis before the affine
// quantiser and after the dequantiser; `seed` names the rotation (TurboState: 0x9E37 ^ layer for K, 0x85EB ^ layer for V).
inline void rotateLastDim(Array& res, const Array& x, uint64_t seed, qb200_stream s) { check(qb200_turbo_rotate(&res.t, &x.t, seed, s)); }
inline void quantizeTurbo(QuantizedKV& out, Array& rotated_scratch, const Array& x, uint64_t seed, qb200_stream s) {
  rotateLastDim(rotated_scratch, x, seed, s);
  quantizeAffine(out, rotated_scratch, s);
}
inline void dequantizeTurbo(Array& res, const QuantizedKV& kv, uint64_t seed, qb200_stream s) {
  dequantizeAffine(res, kv, s);
  rotateLastDim(res, res, seed, s);   // R is its own inverse
}

// The chunk files of kv_disk_cache.zig's SSD tier (src/kv_disk_cache.zig:1-48): positions [pos0, pos1) of every
// layer's six buffers as "l{i}.k" ... "l{i}.vb" in one safetensors file; an entry whose buffers are empty stands for
// a layer without a KV cache.  restoreChunk slices an over-long chunk down to `need` positions and throws on a
// corrupt one (the caller then resets the cache and prefills, as DiskTier's callers do).
inline std::vector<qb200_kv_layer> chunkLayers(const KVCacheEntry* const* entries, int n) {
  std::vector<qb200_kv_layer> v((size_t)n);
  for (int i = 0; i < n; ++i) {
    if (!entries[i]) { v[(size_t)i] = qb200_kv_layer{}; continue; }
    const KVCacheEntry& e = *entries[i];
    v[(size_t)i] = qb200_kv_layer{e.keys.q.t, e.keys.scales.t, e.keys.biases.t, e.values.q.t, e.values.scales.t, e.values.biases.t};
  }
  return v;
}
inline void saveChunk(const std::string& path, const KVCacheEntry* const* entries, int n, int64_t pos0, int64_t pos1, qb200_stream s) {
  const std::vector<qb200_kv_layer> v = chunkLayers(entries, n);
  check(qb200_kv_chunk_save(path.c_str(), v.data(), n, pos0, pos1, s));
}
inline void restoreChunk(const std::string& path, KVCacheEntry* const* entries, int n, int64_t pos0, int64_t need, qb200_stream s) {
  const std::vector<qb200_kv_layer> v = chunkLayers(entries, n);
  check(qb200_kv_chunk_restore(path.c_str(), v.data(), n, pos0, need, s));
}

#ifdef QB200_HOST_WITH_EP
}  // namespace qb200h
#include "qb200_ep.h"
namespace qb200h {
// moeMLP2 (src/transformer.zig:14945-15140) with the experts spread over `world` GPUs: this rank's tokens x [T, H]
// with their routing (inds, scores [T, k]), this rank's slice of the three expert banks, an NCCL communicator made
// with qb200_ep_comm_create.  `overflow` (device int, may be null) counts routed rows beyond the per-peer capacity.
inline void moeBlockEp(Array& res, const Array& x, const Array& inds, const Array& scores, const QWeight& gate,
                       const QWeight& up, const QWeight& down, int num_experts, int world, int rank, void* comm,
                       int64_t capacity, int* overflow, void* workspace, size_t workspace_bytes, qb200_stream s) {
  check(qb200_moe_block_ep(&res.t, &x.t, &inds.t, &scores.t, &gate.q.t, &gate.scales.t, &gate.biases.t, &up.q.t,
                           &up.scales.t, &up.biases.t, &down.q.t, &down.scales.t, &down.biases.t, num_experts, world,
                           rank, comm, capacity, gate.group_size, gate.bits, overflow, workspace, workspace_bytes, s));
}
#endif

}  // namespace qb200h
