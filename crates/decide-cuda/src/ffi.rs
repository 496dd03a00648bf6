//! Raw bindings of libdecide_cuda.so: GENERATED from include/decide_cuda.h by gen_ffi.py; do not edit.
//! Not compiled in the image this crate was written in (no Rust toolchain there): unverified.
#![allow(clippy::too_many_arguments)]
use std::os::raw::{c_char, c_void};

#[repr(C)] pub struct DcCtx { _private: [u8; 0] }
#[repr(C)] pub struct DcModel { _private: [u8; 0] }

/// dc_convert_report: the converter's fp16 precision-loss counters.
#[repr(C)] #[derive(Clone, Copy, Debug, Default, PartialEq, Eq)]
pub struct DcConvertReport { pub values: u64, pub f16_subnormal: u64, pub f16_flushed_to_zero: u64, pub f16_overflow: u64 }

/// dc_dims: the model's dims, compile-time constants in the reference (config.rs:4-37).
#[repr(C)] #[derive(Clone, Copy, Debug, PartialEq)]
pub struct DcDims {
    pub hidden: u32, pub n_layers: u32, pub nq: u32, pub nkv: u32, pub head_dim: u32, pub rot_dim: u32,
    pub gdn_nk: u32, pub gdn_nv: u32, pub gdn_dk: u32, pub gdn_dv: u32, pub inter: u32, pub vocab: u32,
    pub full_attn_interval: u32, pub attn_gate: u32, pub swiglu_block: u32, pub eps: f32, pub rope_theta: f32,
}

/// dc_layer_weights: one layer's device pointers in the fused layouts (convert.rs:204-245); unused members null.
#[repr(C)] #[derive(Clone, Copy, Debug)]
pub struct DcLayerWeights {
    pub in_norm: *const f32, pub w_in: *const c_void, pub w_out: *const c_void, pub post_norm: *const f32,
    pub w_gu: *const c_void, pub w_down: *const c_void, pub conv_w: *const f32, pub a_log: *const f32, pub dt_bias: *const f32,
    pub gnorm: *const f32, pub q_norm: *const f32, pub k_norm: *const f32,
}

pub const DC_OK: i32 = 0;
pub const DC_INVALID_ARG: i32 = 1;
pub const DC_CUDA_ERROR: i32 = 2;
pub const DC_UNSUPPORTED: i32 = 3;
pub const DC_TIMEOUT: i32 = 4;
pub const DC_NOALLOC_MAX_VALUES: u64 = 1 << 32;
pub const DC_GEMM_SMALL_MAX_M: u32 = 16;

#[link(name = "decide_cuda")]
extern "C" {
    pub fn dc_open(device: i32, err: *mut c_char, err_len: usize) -> *mut DcCtx;
    pub fn dc_close(ctx: *mut DcCtx);
    pub fn dc_last_error(ctx: *mut DcCtx, buf: *mut c_char, len: usize) -> usize;
    pub fn dc_set_impl(ctx: *mut DcCtx, family: u32, impl_: u32) -> i32;
    pub fn dc_get_impl(ctx: *mut DcCtx, family: u32) -> u32;
    pub fn dc_set_activation_dtype(ctx: *mut DcCtx, act: u32) -> i32;
    pub fn dc_get_activation_dtype(ctx: *mut DcCtx) -> u32;
    pub fn dc_set_delta_split(ctx: *mut DcCtx, split: u32) -> i32;
    pub fn dc_set_engine(ctx: *mut DcCtx, family: u32, engine: u32) -> i32;
    pub fn dc_check_status(ctx: *mut DcCtx, stream: *mut c_void) -> i32;
    pub fn dc_selftest_wait_timeout(ctx: *mut DcCtx, stream: *mut c_void) -> i32;
    pub fn dc_launch_count(ctx: *mut DcCtx) -> u64;
    pub fn dc_reserve_workspace(ctx: *mut DcCtx, bytes: usize) -> i32;
    pub fn dc_set_workspace_frozen(ctx: *mut DcCtx, on: u32) -> i32;
    pub fn dc_workspace_bytes(ctx: *mut DcCtx) -> usize;
    pub fn dc_warm_up(ctx: *mut DcCtx) -> i32;
    pub fn dc_alloc_count(ctx: *mut DcCtx) -> u64;
    pub fn dc_tmap_encode_count(ctx: *mut DcCtx) -> u64;
    pub fn dc_tmap_cache_size(ctx: *mut DcCtx) -> usize;
    pub fn dc_sm_count(ctx: *mut DcCtx) -> i32;
    pub fn dc_source_hash() -> *const c_char;
    pub fn dc_convert_bf16_to_f16(ctx: *mut DcCtx, stream: *mut c_void, src: *const c_void, dst: *mut c_void, n: usize, report: *mut DcConvertReport) -> i32;
    pub fn dc_convert_bf16_to_f16_noalloc(stream: *mut c_void, src: *const c_void, dst: *mut c_void, n: usize, report: *mut DcConvertReport, err: *mut c_char, err_len: usize) -> i32;
    pub fn dc_gemm(ctx: *mut DcCtx, stream: *mut c_void, x: *const c_void, w: *const c_void, y: *mut c_void, m: u32, n: u32, k: u32, ldx: u32, ldw: u32, ldy: u32, epilogue: u32, swiglu_block: u32) -> i32;
    pub fn dc_gemm_tile(ctx: *mut DcCtx, stream: *mut c_void, x: *const c_void, w: *const c_void, y: *mut c_void, m: u32, n: u32, k: u32, ldx: u32, ldw: u32, ldy: u32, epilogue: u32, bn: u32) -> i32;
    pub fn dc_gemm_plan_for(ctx: *mut DcCtx, m: u32, n: u32, k: u32, epilogue: u32, bn: u32, tail_split: *mut u32) -> u32;
    pub fn dc_gemm_plan(ctx: *mut DcCtx, m: u32, n: u32) -> u32;
    pub fn dc_gemm_plan_k(ctx: *mut DcCtx, m: u32, n: u32, k: u32, tail_split: *mut u32) -> u32;
    pub fn dc_rmsnorm(ctx: *mut DcCtx, stream: *mut c_void, x: *const f32, w: *const f32, y: *mut c_void, rowmap: *const u32, rows: u32, h: u32, ld_in: u32, ld_out: u32, eps: f32, add_one: u32) -> i32;
    pub fn dc_add_rmsnorm(ctx: *mut DcCtx, stream: *mut c_void, x: *mut f32, add: *const f32, w: *const f32, y: *mut c_void, rows: u32, h: u32, eps: f32, add_one: u32) -> i32;
    pub fn dc_add16_rmsnorm(ctx: *mut DcCtx, stream: *mut c_void, x: *mut f32, add16: *const c_void, w: *const f32, y: *mut c_void, rows: u32, h: u32, eps: f32, add_one: u32) -> i32;
    pub fn dc_tp_unique_id(id128: *mut c_void, err: *mut c_char, err_len: usize) -> i32;
    pub fn dc_tp_init(ctx: *mut DcCtx, id128: *const c_void, world: u32, rank: u32) -> i32;
    pub fn dc_tp_all_reduce_f32(ctx: *mut DcCtx, stream: *mut c_void, buf: *mut f32, n: usize) -> i32;
    pub fn dc_tp_all_reduce_16(ctx: *mut DcCtx, stream: *mut c_void, buf: *mut c_void, n: usize) -> i32;
    pub fn dc_tp_set_exchange_16bit(ctx: *mut DcCtx, on: u32) -> i32;
    pub fn dc_tp_world(ctx: *mut DcCtx) -> u32;
    pub fn dc_tp_rank(ctx: *mut DcCtx) -> u32;
    pub fn dc_tp_destroy(ctx: *mut DcCtx);
    pub fn dc_embed(ctx: *mut DcCtx, stream: *mut c_void, ids: *const u32, table: *const c_void, out: *mut f32, t: u32, h: u32) -> i32;
    pub fn dc_gather_rows_f32(ctx: *mut DcCtx, stream: *mut c_void, x: *const f32, rowmap: *const u32, out: *mut f32, rows: u32, h: u32) -> i32;
    pub fn dc_gather_rows_bf16(ctx: *mut DcCtx, stream: *mut c_void, x: *const c_void, rowmap: *const u32, out: *mut c_void, rows: u32, h: u32) -> i32;
    pub fn dc_final_head(ctx: *mut DcCtx, stream: *mut c_void, x: *const f32, w: *const f32, table: *const c_void, cand: *const u32, ncand: *const u32, logits: *mut f32, rows: u32, h: u32, max_cand: u32, eps: f32) -> i32;
    pub fn dc_gated_rmsnorm_silu(ctx: *mut DcCtx, stream: *mut c_void, o: *const f32, z: *const f32, w: *const f32, y: *mut c_void, t: u32, nv: u32, dv: u32, ldz: u32, eps: f32) -> i32;
    pub fn dc_q_norm_rope(ctx: *mut DcCtx, stream: *mut c_void, pq: *const f32, qw: *const f32, inv_freq: *const f32, qpos: *const u32, qo: *mut c_void, rows: u32, ldq: u32, nq: u32, hd: u32, rot: u32, eps: f32) -> i32;
    pub fn dc_kv_norm_rope(ctx: *mut DcCtx, stream: *mut c_void, pkv: *const f32, kw: *const f32, inv_freq: *const f32, kc: *mut c_void, vc: *mut c_void, rows: u32, ldkv: u32, kcol: u32, vcol: u32, pos0: u32, pos: *const u32, cache_rows: u32, nkv: u32, hd: u32, rot: u32, eps: f32) -> i32;
    pub fn dc_attention(ctx: *mut DcCtx, stream: *mut c_void, q: *const c_void, kc: *const c_void, vc: *const c_void, gate: *const f32, qpos: *const u32, y: *mut c_void, rows: u32, ldg: u32, nq: u32, nkv: u32, hd: u32, seq_start: *const u32, n_seq: u32, max_len: u32) -> i32;
    pub fn dc_attention_rows(ctx: *mut DcCtx, stream: *mut c_void, q: *const c_void, kc: *const c_void, vc: *const c_void, gate: *const f32, qpos: *const u32, kv_start: *const u32, y: *mut c_void, rows: u32, ldg: u32, nq: u32, nkv: u32, hd: u32) -> i32;
    pub fn dc_attention_rows_scratch_bytes(ctx: *mut DcCtx, rows: u32, nq: u32, nkv: u32) -> usize;
    pub fn dc_conv_silu_l2(ctx: *mut DcCtx, stream: *mut c_void, p: *const f32, prev: *const f32, w: *const f32, q: *mut f32, k: *mut f32, v: *mut f32, t: u32, ldp: u32, nk: u32, nv: u32, dk: u32, dv: u32, seq_start: *const u32, n_seq: u32, max_len: u32) -> i32;
    pub fn dc_conv_state_update(ctx: *mut DcCtx, stream: *mut c_void, p: *const f32, prev_in: *const f32, prev_out: *mut f32, t: u32, ldp: u32, conv_dim: u32) -> i32;
    pub fn dc_gated_delta(ctx: *mut DcCtx, stream: *mut c_void, q: *const f32, k: *const f32, v: *const f32, a: *const f32, b: *const f32, a_log: *const f32, dt_bias: *const f32, state_in: *const f32, state_out: *mut f32, o: *mut f32, t: u32, ldab: u32, write_state: u32, nk: u32, nv: u32, dk: u32, dv: u32, seq_start: *const u32, n_seq: u32, max_len: u32) -> i32;
    pub fn dc_gated_delta_scratch_bytes(t: u32, n_seq: u32, nv: u32) -> usize;
    pub fn dc_attention_scratch_bytes(rows: u32, n_seq: u32, nkv: u32) -> usize;
    pub fn dc_conv_gated_delta(ctx: *mut DcCtx, stream: *mut c_void, p: *const f32, prev: *const f32, w: *const f32, a: *const f32, b: *const f32, a_log: *const f32, dt_bias: *const f32, state_in: *const f32, state_out: *mut f32, o: *mut f32, t: u32, ldp: u32, write_state: u32, nk: u32, nv: u32, dk: u32, dv: u32, seq_start: *const u32, n_seq: u32, max_len: u32) -> i32;
    pub fn dc_conv_gated_delta_supported(ctx: *mut DcCtx) -> i32;
    pub fn dc_model_create(ctx: *mut DcCtx, dims: *const DcDims, layers: *const DcLayerWeights, embed: *const c_void, final_norm: *const f32, max_rows: u32, max_seqs: u32, max_answers: u32, max_cand: u32) -> *mut DcModel;
    pub fn dc_model_destroy(m: *mut DcModel);
    pub fn dc_model_activation_bytes(m: *mut DcModel) -> usize;
    pub fn dc_model_prefill(m: *mut DcModel, stream: *mut c_void, ids: *const u32, seq_start: *const u32, n_seq: u32, ans_rows: *const u32, cand: *const u32, ncand: *const u32, n_ans: u32, logits: *mut f32) -> i32;
    pub fn dc_model_forward_resident(m: *mut DcModel, stream: *mut c_void, seq_start: *const u32, n_seq: u32, n_ans: u32) -> i32;
    pub fn dc_model_set_graphs(m: *mut DcModel, on: u32) -> i32;
    pub fn dc_model_graph_count(m: *mut DcModel) -> usize;
    pub fn dc_model_set_pruning(m: *mut DcModel, on: u32) -> i32;
    pub fn dc_model_set_truncation(m: *mut DcModel, on: u32) -> i32;
    pub fn dc_model_resident_rows(m: *mut DcModel) -> u32;
    pub fn dc_model_set_chunk(m: *mut DcModel, rows: u32) -> i32;
    pub fn dc_model_build_snapshot(m: *mut DcModel, stream: *mut c_void, prefix_ids: *const u32, n: u32) -> i32;
    pub fn dc_model_last_route(m: *mut DcModel) -> u32;
    pub fn dc_model_last_start(m: *mut DcModel) -> u32;
    pub fn dc_model_set_state_cache(m: *mut DcModel, entries: u32) -> i32;
    pub fn dc_model_forget_states(m: *mut DcModel);
    pub fn dc_model_state_cache_capacity(m: *mut DcModel) -> u32;
    pub fn dc_model_cached_states(m: *mut DcModel, lens: *mut u32, cap: u32) -> u32;
    pub fn dc_model_set_state_marker(m: *mut DcModel, ids: *const u32, n: u32) -> i32;
    pub fn dc_model_set_layer_limit(m: *mut DcModel, n: u32) -> i32;
    pub fn dc_model_buffer(m: *mut DcModel, name: *const c_char) -> *mut c_void;
    pub fn dc_model_read_buffer(m: *mut DcModel, name: *const c_char, dst: *mut c_void, bytes: usize) -> i32;
    pub fn dc_model_set_profiling(m: *mut DcModel, on: u32) -> i32;
    pub fn dc_model_profile(m: *mut DcModel, buf: *mut c_char, len: usize) -> usize;
}
