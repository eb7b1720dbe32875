//! `extern "C"` declarations of libhanzoquant_b200 (include/hanzoquant_b200.h, ABI version 3).
//! NOT COMPILED in this repository (no Rust toolchain in the build image).  Field order and widths follow the C
//! header exactly; every pointer is a device pointer unless its name ends in `_host`.
#![allow(non_camel_case_types, dead_code)]
use std::ffi::c_void;

pub const HQ_OK: i32 = 0;
pub const HQ_FMT_Q8_0: i32 = 0;
pub const HQ_FMT_Q4_K: i32 = 1;
pub const HQ_FMT_FP8_BLOCK: i32 = 2;
pub const HQ_FMT_MXFP4: i32 = 3;
pub const HQ_FMT_Q6_K: i32 = 4;
pub const HQ_FMT_Q5_K: i32 = 5;
pub const HQ_FMT_Q4_0: i32 = 6;
pub const HQ_FMT_Q5_0: i32 = 7;
pub const HQ_FMT_Q4_1: i32 = 8;
pub const HQ_FMT_Q5_1: i32 = 9;
pub const HQ_FMT_Q2_K: i32 = 10;
pub const HQ_FMT_Q3_K: i32 = 11;
pub const HQ_DT_F32: i32 = 0;
pub const HQ_DT_F16: i32 = 1;
pub const HQ_DT_BF16: i32 = 2;
pub const HQ_ACT_NONE: i32 = 0;
pub const HQ_ACT_SWIGLU: i32 = 1;
pub const HQ_ACT_GPTOSS: i32 = 2;
pub const HQ_ROWS_PER_TOKEN: i32 = 0;
pub const HQ_ROWS_PER_SLOT: i32 = 1;
pub const HQ_ROWS_SORTED: i32 = 2;

#[repr(C)]
#[derive(Clone, Copy)]
pub struct hq_weight {
    pub format: i32,
    pub n_experts: i32,
    pub n: i64,
    pub k: i64,
    pub data: *const c_void,
    pub scales: *const c_void,
    pub bias: *const c_void,
    pub bias_dtype: i32,
    pub reserved: i32,
    pub fp8_tile_scale: *const c_void,
    pub fp8_rel_scale: *const c_void,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct hq_router_args {
    pub n_experts: i32,
    pub top_k: i32,
    pub score_mode: i32,
    pub weight_mode: i32,
    pub renormalize: i32,
    pub clamp_logits: i32,
    pub clamp_min: f32,
    pub clamp_max: f32,
    pub norm_min: f32,
    pub output_scale: f32,
    pub selection_bias: *const f32,
    pub expert_scale: *const f32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct hq_act_args {
    pub act: i32,
    pub has_limit: i32,
    pub limit: f32,
    pub alpha: f32,
}

#[repr(C)]
pub struct hq_moe_layer {
    pub gate: *const hq_weight,
    pub up: *const hq_weight,
    pub down: *const hq_weight,
    pub act: hq_act_args,
    pub router: hq_router_args,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct hq_ep_layout {
    pub world: i32,
    pub top_k: i32,
    pub experts_per_rank: i32,
    pub capacity: i32,
    pub pad_rows: i32,
    pub rows_per_peer: i32,
    pub fp8: i32,
    pub wire_dtype: i32,
    pub hidden: i64,
    pub row_bytes: i64,
    pub message_bytes: i64,
}

extern "C" {
    pub fn hq_abi_version() -> i32;
    pub fn hq_error_string(code: i32) -> *const std::os::raw::c_char;
    pub fn hq_status_read(status_dev: *const i32, out_host: *mut i32, stream: *mut c_void) -> i32;
    pub fn hq_config_set(key: i32, value: i64) -> i32;
    pub fn hq_config_get(key: i32) -> i64;

    pub fn hq_linear_workspace_bytes(w: *const hq_weight, m: i64) -> i64;
    pub fn hq_linear_forward_ws(
        w: *const hq_weight, x: *const c_void, x_dtype: i32, x_stride: i64, y: *mut c_void, y_dtype: i32,
        y_stride: i64, m: i64, workspace: *mut c_void, workspace_bytes: i64, status_dev: *mut i32,
        stream: *mut c_void,
    ) -> i32;
    pub fn hq_linear_glu_forward(
        w_gate: *const hq_weight, w_up: *const hq_weight, act: *const hq_act_args, x: *const c_void, x_dtype: i32,
        x_stride: i64, y: *mut c_void, y_dtype: i32, y_stride: i64, m: i64, status_dev: *mut i32,
        stream: *mut c_void,
    ) -> i32;

    pub fn hq_router_topk(
        logits: *const c_void, logits_dtype: i32, n_rows: i64, args: *const hq_router_args, ids_out: *mut u32,
        weights_out: *mut f32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_dispatch_workspace_bytes(n_tokens: i64, top_k: i32, n_experts: i32) -> i64;
    pub fn hq_moe_dispatch_build(
        ids: *const u32, n_tokens: i64, top_k: i32, n_experts: i32, expert_bounds: *mut i32,
        sorted_assign: *mut i32, sorted_token: *mut i32, inv_perm: *mut i32, workspace: *mut c_void,
        workspace_bytes: i64, stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_gather_forward(
        w: *const hq_weight, w_up: *const hq_weight, act: *const hq_act_args, x: *const c_void, x_dtype: i32,
        x_layout: i32, n_tokens: i64, top_k: i32, expert_bounds: *const i32, sorted_assign: *const i32,
        sorted_token: *const i32, workspace: *const c_void, out: *mut c_void, out_dtype: i32, out_layout: i32,
        status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_weighted_reduce(
        y: *const c_void, y_dtype: i32, w: *const f32, row_map: *const i32, addend: *const c_void,
        out: *mut c_void, out_dtype: i32, n_tokens: i64, top_k: i32, hidden: i64, stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_layer_workspace_bytes(layer: *const hq_moe_layer, n_tokens: i64, x_dtype: i32) -> i64;
    pub fn hq_moe_layer_forward(
        layer: *const hq_moe_layer, logits: *const c_void, logits_dtype: i32, x: *const c_void, x_dtype: i32,
        n_tokens: i64, shared_addend: *const c_void, out: *mut c_void, out_dtype: i32, workspace: *mut c_void,
        workspace_bytes: i64, status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;

    pub fn hq_fp8_scale_prepare(
        scales: *const f32, n_experts: i32, n: i64, k: i64, tile_scale_out: *mut f32, rel_scale_out: *mut f32,
        stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_quant_rows_n(
        x: *const c_void, x_dtype: i32, x_stride: i64, row_map: *const i32, n_valid_dev: *const i32, n_rows: i64,
        k: i64, codes: *mut u8, scales: *mut f32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_gather_rows(
        src_codes: *const u8, src_code_stride: i64, src_scales: *const f32, src_scale_stride_bytes: i64,
        row_map: *const i32, n_valid_dev: *const i32, n_rows: i64, k: i64, codes: *mut u8, scales: *mut f32,
        stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_fp8_gate_up_forward(
        w_gate: *const hq_weight, w_up: *const hq_weight, act: *const hq_act_args, x_codes: *const u8,
        x_scales: *const f32, n_tokens: i64, top_k: i32, expert_bounds: *const i32, h_codes: *mut u8,
        h_scales: *mut f32, status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_fp8_gather_forward(
        w: *const hq_weight, x_codes: *const u8, x_scales: *const f32, n_tokens: i64, top_k: i32,
        expert_bounds: *const i32, sorted_assign: *const i32, workspace: *const c_void, out: *mut c_void,
        out_dtype: i32, out_stride: i64, out_layout: i32, status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;

    pub fn hq_ep_layout_init(
        layout: *mut hq_ep_layout, world: i32, top_k: i32, experts_per_rank: i32, capacity: i32, hidden: i64,
        wire_dtype: i32, fp8: i32,
    ) -> i32;
    pub fn hq_ep_pack(
        layout: *const hq_ep_layout, x: *const c_void, x_dtype: i32, ids: *const u32, weights: *const f32,
        n_tokens: i64, send: *mut c_void, back_map: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_ep_unpack_meta(
        layout: *const hq_ep_layout, recv: *const c_void, ids_out: *mut u32, weights_out: *mut f32,
        stream: *mut c_void,
    ) -> i32;

    pub fn hq_convert_status(
        src: *const c_void, src_dtype: i32, dst: *mut c_void, dst_dtype: i32, n_elems: i64, status_dev: *mut i32,
        stream: *mut c_void,
    ) -> i32;
    pub fn hq_gated_act(
        gate: *const c_void, up: *const c_void, dtype: i32, n_elems: i64, interleaved: i32,
        act: *const hq_act_args, out: *mut c_void, stream: *mut c_void,
    ) -> i32;

    // ---- the remaining entry points of the header ----
    pub fn hq_linear_forward(
        w: *const hq_weight, x: *const c_void, x_dtype: i32, x_stride: i64, y: *mut c_void, y_dtype: i32,
        y_stride: i64, m: i64, status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_linear_qkv_forward(
        w_q: *const hq_weight, w_k: *const hq_weight, w_v: *const hq_weight, x: *const c_void, x_dtype: i32,
        x_stride: i64, q: *mut c_void, k: *mut c_void, v: *mut c_void, y_dtype: i32, m: i64,
        status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_dense_gemv(
        w: *const c_void, w_dtype: i32, n: i64, k: i64, bias: *const c_void, bias_dtype: i32, x: *const c_void,
        x_dtype: i32, x_stride: i64, y: *mut c_void, y_dtype: i32, y_stride: i64, m: i64, stream: *mut c_void,
    ) -> i32;
    pub fn hq_router_topk_grouped(
        logits: *const c_void, logits_dtype: i32, n_rows: i64, args: *const hq_router_args, n_group: i32,
        topk_group: i32, group_score_mode: i32, ids_out: *mut u32, weights_out: *mut f32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_dispatch_build_noalloc(
        ids: *const u32, n_tokens: i64, top_k: i32, n_experts: i32, expert_bounds: *mut i32,
        sorted_assign: *mut i32, sorted_token: *mut i32, inv_perm: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_quant_rows(
        x: *const c_void, x_dtype: i32, x_stride: i64, row_map: *const i32, n_rows: i64, k: i64, codes: *mut u8,
        scales: *mut f32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_gated_quant_rows(
        gate_up: *const c_void, dtype: i32, n_rows: i64, width: i64, act: *const hq_act_args, codes: *mut u8,
        scales: *mut f32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_linear_forward(
        w: *const hq_weight, x_codes: *const u8, x_scales: *const f32, m: i64, y: *mut c_void, y_dtype: i32,
        y_stride: i64, status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_vector_quant(
        x: *const c_void, x_dtype: i32, n_elems: i64, codes: *mut u8, scales: *mut f32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_vector_dequant(
        codes: *const u8, scales: *const f32, n_elems: i64, out: *mut c_void, out_dtype: i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_block_quant(
        w: *const c_void, w_dtype: i32, rows: i64, cols: i64, by: i32, bx: i32, codes: *mut u8, scales: *mut f32,
        stream: *mut c_void,
    ) -> i32;
    pub fn hq_fp8_block_dequant(
        codes: *const u8, scales: *const f32, rows: i64, cols: i64, by: i32, bx: i32, out: *mut c_void,
        out_dtype: i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_convert(
        src: *const c_void, src_dtype: i32, dst: *mut c_void, dst_dtype: i32, n_elems: i64, stream: *mut c_void,
    ) -> i32;
    pub fn hq_probe_tensor_peak(
        kind: i32, n: i32, iters: i32, status_dev: *mut i32, flops_host: *mut f64, stream: *mut c_void,
    ) -> i32;
    // MXFP4 layers with MXFP8 activations (block-scaled tensor-core MMA)
    pub fn hq_mxfp8_quant_rows(
        x: *const c_void, x_dtype: i32, x_stride: i64, row_map: *const i32, n_valid_dev: *const i32, n_rows: i64,
        k: i64, codes: *mut u8, scales: *mut u8, stream: *mut c_void,
    ) -> i32;
    pub fn hq_mx_linear_forward(
        w: *const hq_weight, x_codes: *const u8, x_scales: *const u8, m: i64, y: *mut c_void, y_dtype: i32,
        y_stride: i64, status_dev: *mut i32, stream: *mut c_void,
    ) -> i32;
    pub fn hq_moe_mx_gather_forward(
        w: *const hq_weight, act: *const hq_act_args, x_codes: *const u8, x_scales: *const u8, n_tokens: i64,
        top_k: i32, expert_bounds: *const i32, sorted_assign: *const i32, out: *mut c_void, out_dtype: i32,
        out_stride: i64, out_layout: i32, h_codes: *mut u8, h_scales: *mut u8, status_dev: *mut i32,
        stream: *mut c_void,
    ) -> i32;
}
