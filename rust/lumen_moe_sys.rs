//! Raw bindings of `liblumen_moe_b200.so` (C ABI: `include/lumen_moe.h`) for
//! `crates/lumen-runtime/src/cuda/`. NOT COMPILED HERE: the image this library is built in has
//! no Rust toolchain. The same symbols with the same argument lists are bound and exercised by
//! the Python ctypes harness (`lumen_b200/_lib.py`), and `tests/test_abi.py` checks this file's
//! function names against the header, so the two cannot drift apart silently.
//!
//! Where each call goes in the reference (call-site map in INTEGRATION.md):
//!   allocate_moe_scratch              cuda/moe.rs:968   -> lumen_moe_create
//!   build_moe_meta + build_batched_offsets + build_repacked_down
//!                                     cuda/moe.rs:223,272,337 -> lumen_moe_layer_prepare
//!   ensure_prefill_grouped            cuda/moe.rs:1015  -> lumen_moe_ensure_prefill
//!   encode_moe_ffn_decode             cuda/moe.rs:1119  -> lumen_moe_decode
//!   encode_moe_ffn_decode_fused_norm  cuda/moe.rs:3184  -> lumen_moe_decode_fused_norm
//!   encode_moe_ffn_prefill_grouped    cuda/moe.rs:1900  -> lumen_moe_prefill
//!   encode_shared_expert_ffn_*        cuda/moe.rs:5494,2788 -> lumen_moe_shared_expert_*
//!   Result<(), RuntimeError>          error.rs:6-31     -> status code + lumen_moe_last_error,
//!                                                          lumen_moe_poll_status for failures
//!                                                          that happen on the device
#![allow(non_camel_case_types, dead_code)]

use std::os::raw::{c_char, c_void};

pub const LUMEN_MOE_OK: i32 = 0;
pub const LUMEN_MOE_INVALID_ARG: i32 = 1;
pub const LUMEN_MOE_UNSUPPORTED: i32 = 2;
pub const LUMEN_MOE_CUDA_ERROR: i32 = 3;
pub const LUMEN_MOE_TIMEOUT: i32 = 4;
pub const LUMEN_MOE_NCCL_ERROR: i32 = 5;

/// lumen_moe_quant_t: QuantScheme::Q8_0 -> 0, Q4_0 -> 1, Bf16 -> 2 (cuda/moe.rs:1185-1191).
pub const LUMEN_MOE_Q8_0: i32 = 0;
pub const LUMEN_MOE_Q4_0: i32 = 1;
pub const LUMEN_MOE_BF16: i32 = 2;

/// lumen_moe_gating_t
pub const LUMEN_MOE_SOFTMAX_RENORM: i32 = 0;
pub const LUMEN_MOE_SIGMOID_RENORM: i32 = 1;
pub const LUMEN_MOE_SIGMOID_GATE: i32 = 2;
pub const LUMEN_MOE_UNIT_WEIGHT: i32 = 3;

/// lumen_moe_act_t
pub const LUMEN_MOE_ACT_F32: i32 = 0;
pub const LUMEN_MOE_ACT_BF16: i32 = 1;
pub const LUMEN_MOE_ACT_F16: i32 = 2;

/// lumen_moe_config.flags
pub const LUMEN_MOE_FLAG_DECODE_SPLIT: i32 = 0x1;
pub const LUMEN_MOE_FLAG_PREFILL_MMA: i32 = 0x2;
pub const LUMEN_MOE_FLAG_SHORT_WAITS: i32 = 0x4;
pub const LUMEN_MOE_FLAG_PREFILL_F16_WEIGHTS: i32 = 0x8;
pub const fn lumen_moe_flag_tc_ctas(n: i32) -> i32 { (n & 0xff) << 8 }

pub const LUMEN_MOE_EP_HANDLE_BYTES: usize = 64;

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct LumenMoeConfig {
    pub hidden_dim: i32,
    pub inter_dim: i32,
    pub num_experts: i32,
    pub top_k: i32,
    pub max_tokens: i32,
    pub gating_mode: i32,
    pub device: i32,
    pub flags: i32,
}

#[repr(C)] pub struct LumenMoeCtx { _private: [u8; 0] }
#[repr(C)] pub struct LumenMoeLayer { _private: [u8; 0] }

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct LumenLbcSlice { pub offset: u64, pub length: u64, pub quant: u32, pub present: u32 }

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct LumenLbcHeader {
    pub version: u32, pub num_layers: u32, pub num_heads: u32, pub num_kv_heads: u32, pub head_dim: u32,
    pub hidden_dim: u32, pub intermediate_dim: u32, pub vocab_size: u32, pub max_seq_len: u32,
    pub num_experts: u32, pub num_active_experts: u32, pub norm_eps: f32, pub primary_quant: u32,
    pub has_expert_index: u32, pub alignment: u64, pub layer_index_offset: u64, pub payload_offset: u64,
    pub header_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct LumenLbcMoeLayer {
    pub layer_offset_bytes: u64, pub layer_length_bytes: u64, pub is_moe: u32, pub num_experts: u32,
    pub expert_gate_quant: u32, pub expert_down_quant: u32, pub expert_gate_bytes: u64, pub expert_down_bytes: u64,
    pub router_weight: LumenLbcSlice, pub ffn_norm: LumenLbcSlice,
    pub shared_expert_gate: LumenLbcSlice, pub shared_expert_up: LumenLbcSlice, pub shared_expert_down: LumenLbcSlice,
    pub ffn_gate_inp_shexp: LumenLbcSlice, pub has_layer_type: u32, pub layer_type: u32,
}

/// Every pointer named d_* is a device pointer (`CudaSlice::device_ptr()`); `stream` is the
/// backend's `CudaDevice::cu_stream()` (cuda/ffi.rs:81-87). All calls are asynchronous on that
/// stream unless the header says otherwise.
#[link(name = "lumen_moe_b200")]
extern "C" {
    // -- context and layers ------------------------------------------------------------------
    pub fn lumen_moe_create(cfg: *const LumenMoeConfig, out_ctx: *mut *mut LumenMoeCtx) -> i32;
    pub fn lumen_moe_destroy(ctx: *mut LumenMoeCtx);
    pub fn lumen_moe_ensure_prefill(ctx: *mut LumenMoeCtx, tokens: i32) -> i32;
    pub fn lumen_moe_layer_prepare(ctx: *mut LumenMoeCtx, d_layer_blob: *const c_void, blob_bytes: usize,
        router_off: u64, gate_offs: *const u64, up_offs: *const u64, down_offs: *const u64, quant: i32,
        stream: *mut c_void, out_layer: *mut *mut LumenMoeLayer) -> i32;
    pub fn lumen_moe_layer_destroy(layer: *mut LumenMoeLayer);
    pub fn lumen_moe_layer_bytes(layer: *const LumenMoeLayer) -> usize;

    // -- the operator ------------------------------------------------------------------------
    pub fn lumen_moe_decode(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_normed: *const f32,
        d_residual: *const f32, d_out: *mut f32, tokens: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_decode_fused_norm(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_x: *const f32,
        d_gamma: *const f32, d_normed_out: *mut f32, d_out: *mut f32, eps: f32, tokens: i32,
        stream: *mut c_void) -> i32;
    pub fn lumen_moe_prefill(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_normed: *const c_void,
        d_residual: *const f32, d_out: *mut f32, tokens: i32, act_dtype: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_prefill_routed(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_normed: *const c_void,
        d_ids: *const u32, d_weights: *const f32, d_residual: *const f32, d_out: *mut f32, tokens: i32,
        act_dtype: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_shared_expert_decode(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_normed: *const f32,
        d_out: *mut f32, tokens: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_shared_expert_prefill(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer,
        d_normed: *const c_void, d_out: *mut f32, tokens: i32, act_dtype: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_stack_decode(ctx: *mut LumenMoeCtx, layers: *const *const LumenMoeLayer,
        d_gammas: *const *const f32, n_layers: i32, d_x: *mut f32, eps: f32, tokens: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_stack_prefill(ctx: *mut LumenMoeCtx, layers: *const *const LumenMoeLayer,
        d_gammas: *const *const f32, n_layers: i32, d_x: *mut f32, d_normed: *mut f32, eps: f32, tokens: i32,
        stream: *mut c_void) -> i32;

    // -- routing only ------------------------------------------------------------------------
    pub fn lumen_moe_route_only(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_normed: *const f32,
        tokens: i32, d_ids: *mut u32, d_weights: *mut f32, d_logits_out: *mut f32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_topk_from_logits(ctx: *mut LumenMoeCtx, d_logits: *const f32, tokens: i32, d_ids: *mut u32,
        d_weights: *mut f32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_route_small_static(d_logits: *const f32, tokens: i32, num_experts: i32, top_k: i32,
        gating_mode: i32, d_ids: *mut u32, d_weights: *mut f32, d_dst_to_col: *mut i32,
        d_expert_bounds: *mut i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_set_logits_override(ctx: *mut LumenMoeCtx, d_logits: *const f32) -> i32;
    pub fn lumen_moe_get_routing(ctx: *mut LumenMoeCtx, tokens: i32, ids: *mut u32, weights: *mut f32,
        dst_to_col: *mut i32, col_src_tok: *mut i32, expert_bounds: *mut i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_get_routing_ids_stride_e(ctx: *mut LumenMoeCtx, tokens: i32, ids_stride_e: *mut u32,
        stream: *mut c_void) -> i32;
    pub fn lumen_moe_get_routing_device(ctx: *mut LumenMoeCtx, tokens: i32, d_dst_to_col: *mut i32,
        d_col_src_tok: *mut i32, d_col_expert: *mut i32, d_expert_bounds: *mut i32, stream: *mut c_void) -> i32;

    // -- error state of a context (failures that happen on the device) -------------------------
    pub fn lumen_moe_poll_status(ctx: *const LumenMoeCtx) -> i32;
    pub fn lumen_moe_clear_status(ctx: *mut LumenMoeCtx, stream: *mut c_void) -> i32;
    pub fn lumen_moe_last_error() -> *const c_char;
    pub fn lumen_moe_version() -> *const c_char;

    // -- expert parallelism over several GPUs (one process per GPU) ----------------------------
    pub fn lumen_moe_ep_create(ctx: *mut LumenMoeCtx, rank: i32, world: i32, max_tokens: i32, recv_rows: i32,
        handle_out: *mut c_void /* 64 bytes */) -> i32;
    pub fn lumen_moe_ep_attach(ctx: *mut LumenMoeCtx, handles: *const c_void /* world * 64 bytes */, rank: i32,
        world: i32) -> i32;
    pub fn lumen_moe_ep_layer_prepare(ctx: *mut LumenMoeCtx, d_layer_blob: *const c_void, blob_bytes: usize,
        router_off: u64, gate_offs: *const u64, up_offs: *const u64, down_offs: *const u64, quant: i32,
        stream: *mut c_void, out_layer: *mut *mut LumenMoeLayer) -> i32;
    pub fn lumen_moe_prefill_ep(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_normed: *const c_void,
        d_residual: *const f32, d_out: *mut f32, tokens: i32, act_dtype: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_stack_prefill_ep(ctx: *mut LumenMoeCtx, layers: *const *const LumenMoeLayer,
        d_gammas: *const *const f32, n_layers: i32, d_x: *mut f32, d_normed: *mut f32, eps: f32, tokens: i32,
        stream: *mut c_void) -> i32;
    pub fn lumen_moe_ep_profile(ctx: *mut LumenMoeCtx, enable: i32) -> i32;
    pub fn lumen_moe_ep_phase_ms(ctx: *mut LumenMoeCtx, out_ms6: *mut f32) -> i32;
    // building blocks of the collective-library form (NCCL all-to-all driven by the host)
    pub fn lumen_moe_ep_prepare(ctx: *mut LumenMoeCtx, d_normed: *const c_void, act_dtype: i32, tokens: i32,
        experts_per_rank: i32, d_rows16: *mut c_void, d_local_ids: *mut i32, d_send_counts: *mut i64,
        stream: *mut c_void) -> i32;
    pub fn lumen_moe_experts_routed_f16(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_rows: *const c_void,
        d_ids: *const u32, d_out16: *mut c_void, rows: i32, act_dtype: i32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_combine_f16(d_d16: *const c_void, d_residual: *const f32, d_weights: *const f32,
        d_dst_to_col: *const i32, d_out: *mut f32, tokens: i32, hidden_dim: i32, top_k: i32,
        stream: *mut c_void) -> i32;

    // -- LBC container index (host only) -------------------------------------------------------
    pub fn lumen_lbc_read_header(data: *const c_void, bytes: usize, out: *mut LumenLbcHeader) -> i32;
    pub fn lumen_lbc_read_moe_layer(data: *const c_void, bytes: usize, layer: u32, out: *mut LumenLbcMoeLayer,
        gate_offs: *mut u64, up_offs: *mut u64, down_offs: *mut u64, capacity: u32) -> i32;
    pub fn lumen_lbc_quant_to_moe(lbc_tag: u32) -> i32;

    // -- helpers, instrumentation --------------------------------------------------------------
    pub fn lumen_moe_quantize(d_src: *const f32, n_elements: i64, quant: i32, d_dst: *mut c_void,
        stream: *mut c_void) -> i32;
    pub fn lumen_moe_rmsnorm(d_x: *const f32, d_gamma: *const f32, d_out: *mut f32, tokens: i32, hidden_dim: i32,
        eps: f32, stream: *mut c_void) -> i32;
    pub fn lumen_moe_debug_expf(d_in: *const f32, d_out: *mut f32, n: i64, stream: *mut c_void) -> i32;
    pub fn lumen_moe_debug_decode_phase(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, phase: i32,
        stream: *mut c_void) -> i32;
    pub fn lumen_moe_debug_decode_trace(ctx: *mut LumenMoeCtx, layer: *const LumenMoeLayer, d_trace: *mut u64,
        stream: *mut c_void) -> i32;
    pub fn lumen_moe_debug_expire_next_wait(ctx: *mut LumenMoeCtx, which: i32) -> i32;
    pub fn lumen_moe_launch_count(reset: i32) -> i64;
}

/// `Result<(), RuntimeError>` from a status code, as the call sites in cuda/moe.rs expect it
/// (error.rs:6-31). `RuntimeError` is the reference crate's own type.
#[cfg(feature = "lumen_runtime_types")]
pub fn check(status: i32) -> Result<(), crate::error::RuntimeError> {
    use crate::error::RuntimeError;
    if status == LUMEN_MOE_OK {
        return Ok(());
    }
    let msg = unsafe { std::ffi::CStr::from_ptr(lumen_moe_last_error()) }.to_string_lossy().into_owned();
    if status == LUMEN_MOE_UNSUPPORTED { Err(RuntimeError::Unsupported(msg)) } else { Err(RuntimeError::Compute(msg)) }
}
