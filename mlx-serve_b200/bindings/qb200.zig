//! Zig externs for libqb200 (include/qb200.h).  Text only: Zig is not installed where this
//! library is built, so this file has not been compiled; it restates the C declarations one
//! for one, next to the mlx-c externs of mlx-serve's src/mlx.zig that they replace.
const std = @import("std");

pub const MAX_DIMS = 8;

/// qb200_tensor: device pointer + dtype (same numbers as mlx_dtype, src/mlx.zig:20-35) + shape
/// and strides in elements.  `.{}` (null data, ndim 0) stands for mlx-c's empty handle.
pub const Tensor = extern struct {
    data: ?*anyopaque = null,
    dtype: i32 = 0,
    ndim: i32 = 0,
    shape: [MAX_DIMS]i64 = [_]i64{0} ** MAX_DIMS,
    stride: [MAX_DIMS]i64 = [_]i64{0} ** MAX_DIMS,
};
pub const OptionalInt = extern struct { value: c_int = 0, has_value: bool = false };
pub const OptionalDtype = extern struct { value: c_int = 0, has_value: bool = false };
pub const OptionalFloat = extern struct { value: f32 = 0, has_value: bool = false };
pub const Stream = ?*anyopaque; // cudaStream_t

pub const ErrorHandler = ?*const fn ([*:0]const u8, ?*anyopaque) callconv(.c) void;
pub extern "c" fn qb200_set_error_handler(handler: ErrorHandler, data: ?*anyopaque, dtor: ?*const fn (?*anyopaque) callconv(.c) void) void;
pub extern "c" fn qb200_last_error() [*:0]const u8;

// replaces mlx_quantized_matmul (src/mlx.zig:262)
pub extern "c" fn qb200_quantized_matmul(res: *Tensor, x: *const Tensor, w: *const Tensor, scales: *const Tensor, biases: *const Tensor, transpose_w: bool, group_size: OptionalInt, bits: OptionalInt, mode: [*:0]const u8, s: Stream) c_int;
pub extern "c" fn qb200_quantized_matmul_batch(res: [*]const *Tensor, x: *const Tensor, w: [*]const *const Tensor, scales: [*]const *const Tensor, biases: [*]const *const Tensor, count: c_int, transpose_w: bool, group_size: OptionalInt, bits: OptionalInt, mode: [*:0]const u8, s: Stream) c_int;
pub extern "c" fn qb200_quantized_matmul_shape(x: *const Tensor, w: *const Tensor, scales: *const Tensor, transpose_w: bool, group_size: OptionalInt, bits: OptionalInt, out_shape: [*]i64, out_ndim: *i32) c_int;
// replaces mlx_gather_qmm (src/mlx.zig:265)
pub extern "c" fn qb200_gather_qmm(res: *Tensor, x: *const Tensor, w: *const Tensor, scales: *const Tensor, biases: *const Tensor, lhs_indices: *const Tensor, rhs_indices: *const Tensor, transpose_w: bool, group_size: OptionalInt, bits: OptionalInt, mode: [*:0]const u8, sorted_indices: bool, s: Stream) c_int;
// replaces the two gatherExpertMm calls + fusedSwiGLU of moeMLP2 (src/transformer.zig:15007-15035, :19925-19931);
// returns 1 (declined) for shapes it does not serve: keep the unfused chain then
pub extern "c" fn qb200_gather_qmm_swiglu(res: *Tensor, x: *const Tensor, w_gate: *const Tensor, scales_gate: *const Tensor, biases_gate: *const Tensor, w_up: *const Tensor, scales_up: *const Tensor, biases_up: *const Tensor, lhs_indices: *const Tensor, rhs_indices: *const Tensor, group_size: OptionalInt, bits: OptionalInt, mode: [*:0]const u8, sorted_indices: bool, s: Stream) c_int;
// replaces mlx_take_axis(inv_order) + mlx_multiply(norm_scores) + mlx_sum_axis(-2) at the end of moeMLP2 (src/transformer.zig:15036-15042, :15127-15140)
pub extern "c" fn qb200_moe_weighted_sum(res: *Tensor, y: *const Tensor, scores: *const Tensor, inv_order: *const Tensor, s: Stream) c_int;
// replaces moeRoutingChain (src/transformer.zig:17022-17063): argpartition, softmax, take_along_axis, sum, divide
pub extern "c" fn qb200_moe_route(inds: *Tensor, norm_scores: *Tensor, logits: *const Tensor, k: c_int, s: Stream) c_int;
// replaces gatherQmvDownReduce (src/transformer.zig:20559-20623, :20675-20761); returns 1 (declined) beyond 4 tokens: keep qb200_gather_qmm + qb200_moe_weighted_sum then
pub extern "c" fn qb200_moe_down_reduce(res: *Tensor, act: *const Tensor, w: *const Tensor, scales: *const Tensor, biases: *const Tensor, inds: *const Tensor, scores: *const Tensor, group_size: OptionalInt, bits: OptionalInt, mode: [*:0]const u8, s: Stream) c_int;
// replaces mlx_dequantize (src/mlx.zig:271)
pub extern "c" fn qb200_dequantize(res: *Tensor, w: *const Tensor, scales: *const Tensor, biases: *const Tensor, group_size: OptionalInt, bits: OptionalInt, mode: [*:0]const u8, global_scale: *const Tensor, dtype: OptionalDtype, s: Stream) c_int;
// replaces mlx_quantize (src/mlx.zig:275); results in mlx-c's vector order [q, scales, biases]
pub extern "c" fn qb200_quantize(res_q: *Tensor, res_scales: *Tensor, res_biases: *Tensor, w: *const Tensor, group_size: OptionalInt, bits: OptionalInt, mode: [*:0]const u8, global_scale: *const Tensor, s: Stream) c_int;
// replaces kv_quant.quantAttention / qkvAttnDecodeKernel + qkvMergePartials at T_q = 1
pub extern "c" fn qb200_kv_decode_attention(res: *Tensor, q: *const Tensor, k_q: *const Tensor, k_scales: *const Tensor, k_biases: *const Tensor, v_q: *const Tensor, v_scales: *const Tensor, v_biases: *const Tensor, bits: c_int, group_size: c_int, scale: f32, mask_mode: [*:0]const u8, mask_arr: *const Tensor, kv_lens: *const Tensor, workspace: ?*anyopaque, workspace_bytes: usize, s: Stream) c_int;
pub extern "c" fn qb200_kv_decode_attention_workspace_size(B: i64, Hq: i64, Hkv: i64, T: i64, Dv: i64) usize;
// no counterpart in mlx-c: the same attention with scratch from an 8 MiB array inside the library
pub extern "c" fn qb200_kv_decode_attention_noalloc(res: *Tensor, q: *const Tensor, k_q: *const Tensor, k_scales: *const Tensor, k_biases: *const Tensor, v_q: *const Tensor, v_scales: *const Tensor, v_biases: *const Tensor, bits: c_int, group_size: c_int, scale: f32, mask_mode: [*:0]const u8, mask_arr: *const Tensor, kv_lens: *const Tensor, s: Stream) c_int;
pub extern "c" fn qb200_kv_decode_attention_noalloc_max_scratch() usize;
// replaces steps 2 and 5 of KVCache.updateAffine (src/transformer.zig:3224-3337)
pub extern "c" fn qb200_kv_append(cache_q: *Tensor, cache_scales: *Tensor, cache_biases: *Tensor, dense: *const Tensor, offset: i64, bits: c_int, group_size: c_int, s: Stream) c_int;

// replaces the argsort chain of moeMLP2 (src/transformer.zig:14961-15006): order, inv_order, sorted_inds, order / k, expert row ranges
pub extern "c" fn qb200_moe_sort_by_expert(order: ?*Tensor, inv_order: ?*Tensor, sorted_inds: ?*Tensor, token_rows: ?*Tensor, expert_offsets: ?*Tensor, inds: *const Tensor, num_experts: c_int, s: Stream) c_int;
// replaces the dequantise / pad / concat / mask / SDPA read of forwardBatchedDecode (src/transformer.zig:9742-9792): per-slot cache views in place
pub extern "c" fn qb200_kv_decode_attention_ptrs(res: *Tensor, q: *const Tensor, k_q: [*]const *const Tensor, k_scales: [*]const *const Tensor, k_biases: [*]const *const Tensor, v_q: [*]const *const Tensor, v_scales: [*]const *const Tensor, v_biases: [*]const *const Tensor, num_seqs: c_int, bits: c_int, group_size: c_int, scale: f32, mask_mode: [*:0]const u8, mask_arr: ?*const Tensor, kv_lens: ?*const Tensor, workspace: ?*anyopaque, workspace_bytes: usize, s: Stream) c_int;
pub extern "c" fn qb200_kv_decode_attention_ptrs_workspace_size(num_seqs: i64, Hq: i64, Hkv: i64, T_max: i64, Dv: i64) usize;
// replaces the per-slot cache.update loop of forwardBatchedDecode (src/transformer.zig:9738-9756)
pub extern "c" fn qb200_kv_append_seqs(k_q: [*]const *Tensor, k_scales: [*]const *Tensor, k_biases: [*]const *Tensor, v_q: [*]const *Tensor, v_scales: [*]const *Tensor, v_biases: [*]const *Tensor, dense_k: *const Tensor, dense_v: *const Tensor, offsets: [*]const i64, num_seqs: c_int, bits: c_int, group_size: c_int, s: Stream) c_int;
// replace mlx_fast_rms_norm (src/mlx.zig:319), mlx_add + rmsNorm, mlx_fast_rope_dynamic (src/mlx.zig:324), fusedSwiGLU
pub extern "c" fn qb200_rms_norm(res: *Tensor, x: *const Tensor, weight: *const Tensor, eps: f32, s: Stream) c_int;
pub extern "c" fn qb200_add_rms_norm(sum_res: ?*Tensor, norm_res: ?*Tensor, a: *const Tensor, b: ?*const Tensor, weight: ?*const Tensor, eps: f32, s: Stream) c_int;
pub extern "c" fn qb200_rope(res: *Tensor, x: *const Tensor, dims: c_int, traditional: bool, base: OptionalFloat, scale: f32, offsets: *const Tensor, freqs: ?*const Tensor, s: Stream) c_int;
pub extern "c" fn qb200_swiglu(res: *Tensor, gate: *const Tensor, up: *const Tensor, s: Stream) c_int;
// checkpoint loader (src/model.zig loadWeights; narrowsLoadedF16 :3030-3061; affineParamsFromGeometry src/transformer.zig:16763-16790)
pub const Checkpoint = opaque {};
pub extern "c" fn qb200_checkpoint_open(out: *?*Checkpoint, path: [*:0]const u8) c_int;
pub extern "c" fn qb200_checkpoint_close(ck: ?*Checkpoint) void;
pub extern "c" fn qb200_checkpoint_num_tensors(ck: ?*const Checkpoint) c_int;
pub extern "c" fn qb200_checkpoint_tensor_name(ck: ?*const Checkpoint, i: c_int) ?[*:0]const u8;
pub extern "c" fn qb200_checkpoint_tensor_info(ck: ?*const Checkpoint, name: [*:0]const u8, desc: *Tensor, nbytes: ?*usize) c_int;
pub extern "c" fn qb200_checkpoint_load_tensor(ck: ?*const Checkpoint, name: [*:0]const u8, device_dst: ?*anyopaque, dst_bytes: usize) c_int;
pub extern "c" fn qb200_checkpoint_read_tensor(ck: ?*const Checkpoint, name: [*:0]const u8, host_dst: ?*anyopaque, cap: usize, nbytes: ?*usize) c_int;
pub extern "c" fn qb200_narrows_loaded_f16(name: [*:0]const u8, ndim: c_int, dtype: c_int) bool;
pub extern "c" fn qb200_affine_params_from_geometry(w_cols: i64, s_cols: i64, in_dim: i64, bits: *c_int, group_size: *c_int) c_int;
pub extern "c" fn qb200_config_quantization(json_text: [*:0]const u8, bits: *c_int, group_size: *c_int, mode: ?[*]u8, mode_cap: usize) c_int;
// status of the bounded waits inside the tensor-core and wide streaming kernels: poll once per step after the stream sync
pub extern "c" fn qb200_debug_tc_status() c_int;
pub extern "c" fn qb200_debug_tc_reset() void;
// expert-parallel routed-expert block (include/qb200_ep.h, libqb200_ep.so: links NCCL)
pub extern "c" fn qb200_moe_block_ep(res: *Tensor, x: *const Tensor, inds: *const Tensor, scores: *const Tensor, w_gate: *const Tensor, s_gate: *const Tensor, b_gate: *const Tensor, w_up: *const Tensor, s_up: *const Tensor, b_up: *const Tensor, w_down: *const Tensor, s_down: *const Tensor, b_down: *const Tensor, num_experts: c_int, world: c_int, rank: c_int, comm: ?*anyopaque, capacity: i64, group_size: c_int, bits: c_int, overflow: ?*c_int, workspace: ?*anyopaque, workspace_bytes: usize, s: Stream) c_int;
pub extern "c" fn qb200_moe_block_ep_capacity(T: i64, topk: c_int, world: c_int) i64;
pub extern "c" fn qb200_moe_block_ep_workspace_size(T: i64, topk: c_int, H: i64, I: i64, num_experts: c_int, world: c_int, capacity: i64) usize;

/// Same convention as mlx.check (src/mlx.zig:547-550): 0 is success.  UNSUPPORTED (1) means
/// "declined": the caller keeps its existing mlx-c path for that call.
pub fn check(ret: c_int) !void {
    if (ret == 1) return error.Qb200Declined;
    if (ret != 0) return error.Qb200Error;
}

// chunk files of the quantized KV cache: the slice writes and reads of kv_disk_cache.zig (appendCommit's chunk write,
// src/kv_disk_cache.zig:1062-1074; restoreKvInto, :320-440).  k_q.data == null: the layer keeps no KV cache.
pub const KvLayer = extern struct { k_q: Tensor, k_scales: Tensor, k_biases: Tensor, v_q: Tensor, v_scales: Tensor, v_biases: Tensor };
pub extern "c" fn qb200_kv_chunk_save(path: [*:0]const u8, layers: [*]const KvLayer, n_layers: c_int, pos0: i64, pos1: i64, s: Stream) c_int;
pub extern "c" fn qb200_kv_chunk_restore(path: [*:0]const u8, layers: [*]const KvLayer, n_layers: c_int, pos0: i64, need: i64, s: Stream) c_int;

// mlx_fast_rope_dynamic on q and k followed by the per-slot updateAffine (src/transformer.zig:9678, :9735, :9738-9756): one launch
pub extern "c" fn qb200_rope_kv_append_seqs(q: *Tensor, dims: c_int, base: f32, scale: f32, k_q: [*]const *Tensor, k_scales: [*]const *Tensor, k_biases: [*]const *Tensor, v_q: [*]const *Tensor, v_scales: [*]const *Tensor, v_biases: [*]const *Tensor, dense_k: *const Tensor, dense_v: *const Tensor, offsets: [*]const i64, num_seqs: c_int, bits: c_int, group_size: c_int, s: Stream) c_int;

// rotateLastDim of the TurboQuant schemes (src/kv_quant.zig:362-372; quantizeTurbo / dequantizeTurbo around it): res = x @ R with
// TurboState's Hadamard rotation of the given seed (0x9E37 ^ layer for K, 0x85EB ^ layer for V) instead of an mlx_matmul by the [D, D] matrix
pub extern "c" fn qb200_turbo_rotate(res: *Tensor, x: *const Tensor, seed: u64, s: Stream) c_int;
pub extern "c" fn qb200_turbo_signs(seed: u64, n: c_int, bits: [*]u32) c_int;
