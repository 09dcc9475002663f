//! Raw bindings to libstrix_cuda.so. GENERATED from include/*.h by strix.rs_b200/rust/gen_ffi.py: do not edit.
//! Not compiled in the repository's build image (no Rust toolchain there); the C ABI itself is compiled and
//! tested, and tests/test_abi.py checks that this file declares every exported entry point.
#![allow(non_camel_case_types, clippy::too_many_arguments)]
use std::os::raw::{c_char, c_int, c_longlong, c_void};

#[repr(C)]
pub struct StrixCuda { _private: [u8; 0] }
#[repr(C)]
pub struct StrixGguf { _private: [u8; 0] }

/// strix_cuda_opts
#[repr(C)]
#[derive(Default, Clone, Copy)]
pub struct StrixCudaOpts { pub rank: c_int, pub world: c_int, pub profile: c_int, pub reserved: [c_int; 5] }

/// strix_gpu_layer_cfg: plain-data mirror of strix_core::accel::GpuLayerCfg (accel.rs:19-40)
#[repr(C)]
#[derive(Default, Clone, Copy)]
pub struct StrixGpuLayerCfg {
    pub head_dim: u32, pub n_kv: u32, pub k_eq_v: c_int, pub rope_theta: f32, pub is_local: c_int,
    pub output_scale: f32, pub no_rope: c_int, pub rope_norm: c_int,
}

/// strix_gpu_decode_config: plain-data mirror of GpuDecodeConfig (accel.rs:42-72) plus the two fields the
/// reference does not have (attn_standin_q, act)
#[repr(C)]
#[derive(Clone, Copy)]
pub struct StrixGpuDecodeConfig {
    pub hidden: u32, pub n_heads: u32, pub ffn: u32, pub vocab: u32, pub n_layers: u32,
    pub eps: f32, pub final_softcap: f32,
    pub attn_rsqrt: c_int, pub norm_v: c_int, pub qk_norm: c_int, pub post_norm: c_int, pub act_gelu: c_int,
    pub gpu_prefill: c_int,
    pub n_swa: u32, pub max_seq: u32,
    pub layers: *const StrixGpuLayerCfg,
    pub attn_standin_q: c_int, pub act: c_int,
}

/// strix_gguf_tensor
#[repr(C)]
pub struct StrixGgufTensor {
    pub name: *const c_char, pub n_dims: u32, pub dims: [u64; 4], pub ggml_type: u32, pub offset: u64,
    pub data: *const u8, pub nbytes: usize,
}

/// strix_spec_gate
#[repr(C)]
#[derive(Default, Clone, Copy)]
pub struct StrixSpecGate { pub zero_rounds: u32, pub plain_left: u32 }

pub type StrixEmbedFn = Option<unsafe extern "C" fn(user: *mut c_void, token: u32, hidden_out: *mut f32)>;

pub const ACT_F32: c_int = 0;
pub const ACT_Q8DOT: c_int = 1;
pub const PRE_NONE: c_int = 0;
pub const PRE_RMSNORM: c_int = 1;
pub const PRE_SWIGLU: c_int = 2;
pub const PRE_GEGLU: c_int = 3;

#[link(name = "strix_cuda")]
extern "C" {
    // ---- include/strix_cuda.h
    pub fn strix_cuda_profile_dump(h: *mut StrixCuda, buf: *mut c_char, cap: usize) -> usize;
    pub fn strix_cuda_create(device: c_int, opts: *const StrixCudaOpts, out: *mut *mut StrixCuda) -> c_int;
    pub fn strix_cuda_destroy(h: *mut StrixCuda);
    pub fn strix_cuda_last_error(h: *mut StrixCuda) -> *const c_char;
    pub fn strix_cuda_create_error() -> *const c_char;
    pub fn strix_cuda_name(h: *mut StrixCuda) -> *const c_char;
    pub fn strix_cuda_resident_count(h: *mut StrixCuda) -> usize;
    pub fn strix_cuda_upload_q4_0(h: *mut StrixCuda, key: *const c_char, bytes: *const u8, len: usize, in_dim: usize, out_dim: usize) -> c_int;
    pub fn strix_cuda_upload_q8_0(h: *mut StrixCuda, key: *const c_char, bytes: *const u8, len: usize, in_dim: usize, out_dim: usize) -> c_int;
    pub fn strix_cuda_upload_q6_k(h: *mut StrixCuda, key: *const c_char, bytes: *const u8, len: usize, in_dim: usize, out_dim: usize) -> c_int;
    pub fn strix_cuda_upload_q4_1(h: *mut StrixCuda, key: *const c_char, bytes: *const u8, len: usize, in_dim: usize, out_dim: usize) -> c_int;
    pub fn strix_cuda_upload_f32(h: *mut StrixCuda, key: *const c_char, data: *const f32, n: usize) -> c_int;
    pub fn strix_cuda_weight_info(h: *mut StrixCuda, key: *const c_char, in_dim: *mut usize, out_dim_total: *mut usize, shard_row0: *mut usize, shard_rows: *mut usize, ggml_type: *mut c_int) -> c_int;
    pub fn strix_cuda_gemv(h: *mut StrixCuda, key: *const c_char, x: *const f32, k: usize, y: *mut f32, y_cap: usize, act: c_int) -> c_int;
    pub fn strix_cuda_gemv_batch(h: *mut StrixCuda, n: usize, keys: *const *const c_char, xs: *const *const f32, ks: *const usize, ys: *const *mut f32, y_caps: *const usize, act: c_int, status: *mut c_int) -> c_int;
    pub fn strix_cuda_gemv_dev(h: *mut StrixCuda, nmat: c_int, keys: *const *const c_char, d_a: *const f32, d_b: *const f32, eps: f32, pre: c_int, act: c_int, d_ys: *const *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_gemv_res_dev(h: *mut StrixCuda, nmat: c_int, keys: *const *const c_char, d_a: *const f32, d_b: *const f32, eps: f32, pre: c_int, act: c_int, d_ys: *const *mut f32, d_res: *const *const f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_gemv_peers_dev(h: *mut StrixCuda, nmat: c_int, keys: *const *const c_char, d_a: *const f32, d_b: *const f32, eps: f32, pre: c_int, act: c_int, d_res: *const *const f32, n_peers: c_int, peer_ys: *const *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_enable_peer_access(h: *mut StrixCuda, peer_device: c_int) -> c_int;
    pub fn strix_cuda_ipc_open(h: *mut StrixCuda, handle: *const c_void, handle_len: usize, out: *mut *mut c_void) -> c_int;
    pub fn strix_cuda_ipc_close(h: *mut StrixCuda, p: *mut c_void) -> c_int;
    pub fn strix_cuda_ipc_export(h: *mut StrixCuda, d_ptr: *const c_void, handle: *mut c_void, handle_cap: usize) -> c_int;
    pub fn strix_cuda_peek_u32(h: *mut StrixCuda, d_ptr: *const c_void, out: *mut u32) -> c_int;
    pub fn strix_cuda_poke_u32(h: *mut StrixCuda, d_ptr: *mut c_void, value: u32) -> c_int;
    pub fn strix_cuda_peer_barrier_dev(h: *mut StrixCuda, d_epoch: *mut u32, d_local_flags: *mut u32, peer_flags: *const *mut u32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_gemv_batch_dev(h: *mut StrixCuda, n: usize, keys: *const *const c_char, d_xs: *const *const f32, d_ys: *const *mut f32, act: c_int, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_gemv_batch_peers_dev(h: *mut StrixCuda, n: usize, keys: *const *const c_char, d_xs: *const *const f32, n_peers: c_int, peer_ys: *const *mut f32, act: c_int, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_prefill_q8_gemm(h: *mut StrixCuda, key: *const c_char, xs: *const f32, m: usize, y: *mut f32, y_cap: usize) -> c_int;
    pub fn strix_cuda_prefill_q8_gemm_dev(h: *mut StrixCuda, key: *const c_char, d_xs: *const f32, m: usize, d_y: *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_prefill_q4_gemm(h: *mut StrixCuda, key: *const c_char, xs: *const f32, m: usize, y: *mut f32, y_cap: usize) -> c_int;
    pub fn strix_cuda_prefill_q4_gemm_dev(h: *mut StrixCuda, key: *const c_char, d_xs: *const f32, m: usize, d_y: *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_prefill_q8_gemm_noalloc(h: *mut StrixCuda, key: *const c_char, d_xs: *const f32, m: usize, d_y: *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_noalloc_scratch_bytes() -> usize;
    pub fn strix_cuda_upload_moe_q8(h: *mut StrixCuda, layer: usize, gate: *const u8, gate_len: usize, up: *const u8, up_len: usize, down: *const u8, down_len: usize, hidden: usize, eff: usize, ne: usize) -> c_int;
    pub fn strix_cuda_upload_moe_q6(h: *mut StrixCuda, layer: usize, gate: *const u8, gate_len: usize, up: *const u8, up_len: usize, down: *const u8, down_len: usize, hidden: usize, eff: usize, ne: usize) -> c_int;
    pub fn strix_cuda_moe_ffn(h: *mut StrixCuda, layer: usize, ids: *const c_int, wexp: *const f32, k: usize, x: *const f32, x_len: usize, sgate: f32, act: c_int, y: *mut f32, y_cap: usize) -> c_int;
    pub fn strix_cuda_moe_ffn_dev(h: *mut StrixCuda, layer: usize, d_ids: *const c_int, d_wexp: *const f32, k: usize, d_x: *const f32, sgate: f32, act: c_int, d_y: *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_moe_expert_ffn(h: *mut StrixCuda, layer: usize, e: usize, xs: *const f32, m: usize, act: c_int, y: *mut f32, y_cap: usize) -> c_int;
    pub fn strix_cuda_moe_layer_ffn(h: *mut StrixCuda, layer: usize, plan: *const c_int, n_plan: usize, xs: *const f32, rows: usize, act: c_int, y: *mut f32, y_cap: usize) -> c_int;
    pub fn strix_cuda_topk_router(h: *mut StrixCuda, logits: *const f32, ne: usize, k: usize, ids: *mut c_int, w: *mut f32) -> c_int;
    pub fn strix_cuda_topk_router_dev(h: *mut StrixCuda, d_logits: *const f32, ne: usize, k: usize, d_ids: *mut c_int, d_w: *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_configure_decode(h: *mut StrixCuda, cfg: *const StrixGpuDecodeConfig) -> c_int;
    pub fn strix_cuda_decode_step(h: *mut StrixCuda, hvec: *const f32, pos: usize, logits: *mut f32, logits_cap: usize) -> c_int;
    pub fn strix_cuda_decode_step_argmax(h: *mut StrixCuda, hvec: *const f32, pos: usize, id: *mut u32) -> c_int;
    pub fn strix_cuda_lm_head_argmax_rows(h: *mut StrixCuda, key: *const c_char, xs: *const f32, xs_len: usize, m: usize, act: c_int, ids: *mut u32, vals: *mut f32) -> c_int;
    pub fn strix_cuda_fold_argmax_shards(n_shards: usize, m: usize, ids: *const u32, vals: *const f32, out_ids: *mut u32, out_vals: *mut f32);
    pub fn strix_cuda_argmax_dev(h: *mut StrixCuda, d_x: *const f32, n: usize, stride: usize, rows: usize, d_ids: *mut u32, d_vals: *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_prefill(h: *mut StrixCuda, hs: *const f32, start_pos: usize, m: usize, logits: *mut f32, logits_cap: usize) -> c_int;
    pub fn strix_cuda_verify(h: *mut StrixCuda, hs: *const f32, start_pos: usize, m: usize, logits: *mut f32, logits_cap: usize) -> c_int;
    pub fn strix_cuda_verify_argmax(h: *mut StrixCuda, hs: *const f32, start_pos: usize, m: usize, ids: *mut u32) -> c_int;
    pub fn strix_cuda_prefill_max(h: *mut StrixCuda) -> usize;
    pub fn strix_cuda_seed_decode_kv(h: *mut StrixCuda, il: usize, k: *const f32, v: *const f32, tokens: usize) -> c_int;
    pub fn strix_cuda_decode_exchange_info(h: *mut StrixCuda, base: *mut *mut c_void, bytes: *mut usize) -> c_int;
    pub fn strix_cuda_decode_set_peers(h: *mut StrixCuda, n: c_int, blocks: *const *mut c_void) -> c_int;
    pub fn strix_cuda_decode_chain_dev(h: *mut StrixCuda, d_h: *mut f32, d_logits: *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_gemv_rows(h: *mut StrixCuda, key: *const c_char, xs: *const f32, b: usize, y: *mut f32, y_cap: usize, act: c_int) -> c_int;
    pub fn strix_cuda_gemv_rows_dev(h: *mut StrixCuda, nmat: c_int, keys: *const *const c_char, d_xs: *const f32, b: usize, act: c_int, d_ys: *const *mut f32, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_device_status(h: *mut StrixCuda, stream: *mut c_void, status: *mut u32) -> c_int;
    pub fn strix_cuda_clear_device_status(h: *mut StrixCuda, stream: *mut c_void) -> c_int;
    pub fn strix_cuda_set_option(h: *mut StrixCuda, name: *const c_char, value: c_longlong) -> c_int;
    pub fn strix_cuda_decode_trace(h: *mut StrixCuda, out: *mut u64, cap_words: usize) -> c_int;
    pub fn strix_cuda_dequant_to_f32(h: *mut StrixCuda, key: *const c_char, out: *mut f32, out_cap: usize) -> c_int;
    pub fn strix_cuda_xquant8(h: *mut StrixCuda, x: *const f32, n: usize, q: *mut i8, d: *mut f32) -> c_int;
    pub fn strix_cuda_debug_block_isums(h: *mut StrixCuda, key: *const c_char, xs: *const f32, m: usize, out: *mut i32, out_cap: usize) -> c_int;
    pub fn strix_cuda_debug_gemm_isums(h: *mut StrixCuda, key: *const c_char, xs: *const f32, m: usize, splits: u32, out: *mut i32, out_cap: usize) -> c_int;
    pub fn strix_cuda_debug_gemm_mode_dev(h: *mut StrixCuda, key: *const c_char, d_xs: *const f32, m: usize, d_y: *mut f32, mode: c_int, reps: c_int, stream: *mut c_void) -> c_int;
    // ---- include/strix_gguf.h
    pub fn strix_gguf_open(path: *const c_char, out: *mut *mut StrixGguf) -> c_int;
    pub fn strix_gguf_open_memory(bytes: *const u8, len: usize, out: *mut *mut StrixGguf) -> c_int;
    pub fn strix_gguf_close(g: *mut StrixGguf);
    pub fn strix_gguf_last_error() -> *const c_char;
    pub fn strix_gguf_version(g: *const StrixGguf) -> u32;
    pub fn strix_gguf_alignment(g: *const StrixGguf) -> usize;
    pub fn strix_gguf_data_offset(g: *const StrixGguf) -> usize;
    pub fn strix_gguf_tensor_count(g: *const StrixGguf) -> usize;
    pub fn strix_gguf_meta_count(g: *const StrixGguf) -> usize;
    pub fn strix_gguf_tensor_at(g: *const StrixGguf, i: usize, out: *mut StrixGgufTensor) -> c_int;
    pub fn strix_gguf_find_tensor(g: *const StrixGguf, name: *const c_char, out: *mut StrixGgufTensor) -> c_int;
    pub fn strix_gguf_meta_u64(g: *const StrixGguf, key: *const c_char, out: *mut u64) -> c_int;
    pub fn strix_gguf_meta_f32(g: *const StrixGguf, key: *const c_char, out: *mut f32) -> c_int;
    pub fn strix_gguf_meta_str(g: *const StrixGguf, key: *const c_char, out: *mut *const c_char, len: *mut usize) -> c_int;
    pub fn strix_gguf_meta_array_len(g: *const StrixGguf, key: *const c_char, len: *mut u64, elem_type: *mut u32) -> c_int;
    pub fn strix_gguf_meta_key_at(g: *const StrixGguf, i: usize, key: *mut *const c_char, value_type: *mut u32) -> c_int;
    pub fn strix_gguf_advise_dontneed(g: *const StrixGguf, name: *const c_char);
    pub fn strix_ggml_block_elems(ggml_type: u32) -> usize;
    pub fn strix_ggml_block_bytes(ggml_type: u32) -> usize;
    pub fn strix_cuda_upload_gguf_tensor(h: *mut StrixCuda, g: *const StrixGguf, name: *const c_char, drop_pages: c_int) -> c_int;
    pub fn strix_cuda_upload_gguf(h: *mut StrixCuda, g: *const StrixGguf, drop_pages: c_int, adopted: *mut usize, declined: *mut usize) -> c_int;
    // ---- include/strix_spec.h
    pub fn strix_spec_propose_ngram(ctx: *const u32, n_ctx: usize, gamma: usize, out: *mut u32) -> usize;
    pub fn strix_spec_accept(proposal: *const u32, n_prop: usize, argmax: *const u32, room: usize, next: *mut u32) -> usize;
    pub fn strix_spec_gate_plain(g: *mut StrixSpecGate) -> c_int;
    pub fn strix_spec_gate_round(g: *mut StrixSpecGate, accepted: usize);
    pub fn strix_cuda_spec_round(target: *mut StrixCuda, draft: *mut StrixCuda, embed_target: StrixEmbedFn, user_target: *mut c_void, embed_draft: StrixEmbedFn, user_draft: *mut c_void, hidden_target: usize, hidden_draft: usize, cur: u32, pos: usize, gamma: usize, out_tokens: *mut u32, next: *mut u32) -> c_int;
}
