// GENERATED from include/mcb.h by include/gen_rust_binding.py -- do not edit by hand.
// Raw FFI of libmcb.so: one declaration per function of the C ABI, argument for argument.
// Place in crates/modern-chainer-cuda/src/ and link with `cargo:rustc-link-lib=dylib=mcb`.
#![allow(non_camel_case_types, dead_code)]
use core::ffi::{c_char, c_void};

pub type Status = i32;
#[repr(C)]
pub struct McbAdam {
    _private: [u8; 0],
}
#[repr(C)]
pub struct McbArena {
    _private: [u8; 0],
}
#[repr(C)]
pub struct McbCtx {
    _private: [u8; 0],
}
#[repr(C)]
pub struct McbDpSim {
    _private: [u8; 0],
}
#[repr(C)]
pub struct McbModel {
    _private: [u8; 0],
}
#[repr(C)]
pub struct McbScaler {
    _private: [u8; 0],
}
#[repr(C)]
pub struct McbStaticStep {
    _private: [u8; 0],
}
#[repr(C)]
pub struct McbVar {
    _private: [u8; 0],
}

pub const MCB_OK: i32 = 0;
pub const MCB_SHAPE_MISMATCH: i32 = 1;
pub const MCB_BROADCAST: i32 = 2;
pub const MCB_DTYPE_MISMATCH: i32 = 3;
pub const MCB_UNSUPPORTED_DTYPE: i32 = 4;
pub const MCB_INVALID_ARGUMENT: i32 = 5;
pub const MCB_OUT_OF_BOUNDS: i32 = 6;
pub const MCB_UNSUPPORTED: i32 = 7;
pub const MCB_BACKEND: i32 = 8;
pub const MCB_IO: i32 = 9;
pub const MCB_F32: i32 = 0;
pub const MCB_I64: i32 = 1;
pub const MCB_I32: i32 = 2;
pub const MCB_U8: i32 = 3;
pub const MCB_F16: i32 = 4;
pub const MCB_BF16: i32 = 5;
pub const MCB_COMPUTE_F32: i32 = 0;
pub const MCB_COMPUTE_BF16: i32 = 1;
pub const MCB_COMPUTE_F16: i32 = 2;
pub const MCB_ADD: i32 = 0;
pub const MCB_SUB: i32 = 1;
pub const MCB_MUL: i32 = 2;
pub const MCB_DIV: i32 = 3;
pub const MCB_EXP: i32 = 0;
pub const MCB_LOG: i32 = 1;
pub const MCB_SIGMOID: i32 = 2;
pub const MCB_SQRT: i32 = 3;
pub const MCB_SILU: i32 = 4;
pub const MCB_ABS: i32 = 5;
pub const MCB_NEG: i32 = 6;
pub const MCB_ACT_NONE: i32 = 0;
pub const MCB_ACT_RELU: i32 = 1;
pub const MCB_ACT_GELU: i32 = 2;
pub const MCB_PROF_GEMM_TC: i32 = 0;
pub const MCB_PROF_GEMM_F32: i32 = 1;
pub const MCB_PROF_ATTENTION: i32 = 2;
pub const MCB_PROF_OPTIMIZER: i32 = 3;
pub const MCB_PROF_NORM: i32 = 4;
pub const MCB_PROF_LOSS: i32 = 5;
pub const MCB_PROF_ELEMENTWISE: i32 = 6;
pub const MCB_PROF_REDUCE: i32 = 7;
pub const MCB_PROF_EMBEDDING: i32 = 8;
pub const MCB_PROF_CONV: i32 = 9;
pub const MCB_PROF_CLASSES: i32 = 10;
pub const MCB_OPT_ADAM: i32 = 0;
pub const MCB_OPT_ADAMW: i32 = 1;
pub const MCB_OPT_SGD: i32 = 2;
pub const MCB_OPT_MOMENTUM_SGD: i32 = 3;

#[link(name = "mcb")]
unsafe extern "C" {
    pub fn mcb_ctx_create(ordinal: i32, out: *mut *mut McbCtx) -> Status;
    pub fn mcb_ctx_destroy(ctx: *mut McbCtx);
    pub fn mcb_set_knob(ctx: *mut McbCtx, name: *const c_char, value: i32) -> Status;
    pub fn mcb_last_error(ctx: *mut McbCtx) -> *const c_char;
    pub fn mcb_device_count() -> i32;
    pub fn mcb_alloc(ctx: *mut McbCtx, bytes: usize, out: *mut *mut c_void) -> Status;
    pub fn mcb_free(ctx: *mut McbCtx, ptr: *mut c_void) -> Status;
    pub fn mcb_host_alloc(bytes: usize, host_out: *mut *mut c_void) -> Status;
    pub fn mcb_host_free(host_ptr: *mut c_void) -> Status;
    pub fn mcb_memcpy_h2d(ctx: *mut McbCtx, dst: *mut c_void, host_src: *const c_void, bytes: usize) -> Status;
    pub fn mcb_memcpy_d2h(ctx: *mut McbCtx, host_dst: *mut c_void, src: *const c_void, bytes: usize) -> Status;
    pub fn mcb_memcpy_d2h_async(ctx: *mut McbCtx, host_dst: *mut c_void, src: *const c_void, bytes: usize) -> Status;
    pub fn mcb_memcpy_d2d(ctx: *mut McbCtx, dst: *mut c_void, src: *const c_void, bytes: usize) -> Status;
    pub fn mcb_memset(ctx: *mut McbCtx, dst: *mut c_void, byte: i32, bytes: usize) -> Status;
    pub fn mcb_sync(ctx: *mut McbCtx) -> Status;
    pub fn mcb_stream(ctx: *mut McbCtx) -> *mut c_void;
    pub fn mcb_launch_count(ctx: *mut McbCtx) -> i64;
    pub fn mcb_allocated_bytes(ctx: *mut McbCtx) -> i64;
    pub fn mcb_event_create(ctx: *mut McbCtx, event_out: *mut *mut c_void) -> Status;
    pub fn mcb_event_record(ctx: *mut McbCtx, event: *mut c_void) -> Status;
    pub fn mcb_event_elapsed_ms(ctx: *mut McbCtx, start: *mut c_void, stop: *mut c_void, ms_out: *mut f32) -> Status;
    pub fn mcb_event_destroy(ctx: *mut McbCtx, event: *mut c_void) -> Status;
    pub fn mcb_prof_enable(ctx: *mut McbCtx, on: i32) -> Status;
    pub fn mcb_prof_read(ctx: *mut McbCtx, klass: i32, launches_out: *mut i64, ms_out: *mut f64, flops_out: *mut f64, bytes_out: *mut f64) -> Status;
    pub fn mcb_clock_trace_start(ctx: *mut McbCtx, duration_us: i32, interval_us: i32) -> Status;
    pub fn mcb_clock_trace_read(ctx: *mut McbCtx, mhz_out: *mut f64, max_out: i32, n_out: *mut i32) -> Status;
    pub fn mcb_set_compute_type(ctx: *mut McbCtx, compute: i32) -> Status;
    pub fn mcb_binary(ctx: *mut McbCtx, op: i32, a: *const f32, a_dims: *const i64, a_rank: i32, b: *const f32, b_dims: *const i64, b_rank: i32, out: *mut f32) -> Status;
    pub fn mcb_add_inplace(ctx: *mut McbCtx, dst: *mut c_void, src: *const c_void, n: i64, dt: i32) -> Status;
    pub fn mcb_scale(ctx: *mut McbCtx, x: *const f32, factor: f64, out: *mut f32, n: i64) -> Status;
    pub fn mcb_fill(ctx: *mut McbCtx, out: *mut f32, value: f32, n: i64) -> Status;
    pub fn mcb_unary(ctx: *mut McbCtx, op: i32, x: *const f32, out: *mut f32, n: i64) -> Status;
    pub fn mcb_relu(ctx: *mut McbCtx, x: *const c_void, out: *mut c_void, n: i64, dt: i32) -> Status;
    pub fn mcb_relu_backward(ctx: *mut McbCtx, x: *const c_void, g: *const c_void, out: *mut c_void, n: i64, dt: i32) -> Status;
    pub fn mcb_gelu(ctx: *mut McbCtx, x: *const c_void, out: *mut c_void, n: i64, dt: i32) -> Status;
    pub fn mcb_gelu_backward(ctx: *mut McbCtx, x: *const c_void, g: *const c_void, out: *mut c_void, n: i64, dt: i32) -> Status;
    pub fn mcb_cast(ctx: *mut McbCtx, src: *const c_void, src_dt: i32, dst: *mut c_void, dst_dt: i32, n: i64) -> Status;
    pub fn mcb_transpose2d(ctx: *mut McbCtx, a: *const f32, out: *mut f32, rows: i64, cols: i64) -> Status;
    pub fn mcb_permute(ctx: *mut McbCtx, a: *const f32, dims: *const i64, rank: i32, axes: *const i32, out: *mut f32) -> Status;
    pub fn mcb_sum_all(ctx: *mut McbCtx, x: *const f32, n: i64, out: *mut f32) -> Status;
    pub fn mcb_sum_to(ctx: *mut McbCtx, a: *const f32, a_dims: *const i64, a_rank: i32, t_dims: *const i64, t_rank: i32, out: *mut f32) -> Status;
    pub fn mcb_col_sum(ctx: *mut McbCtx, a: *const c_void, dt: i32, rows: i64, cols: i64, out: *mut f32) -> Status;
    pub fn mcb_softmax(ctx: *mut McbCtx, x: *const f32, out: *mut f32, rows: i64, cols: i64) -> Status;
    pub fn mcb_softmax_backward(ctx: *mut McbCtx, x: *const f32, g: *const f32, out: *mut f32, rows: i64, cols: i64) -> Status;
    pub fn mcb_softmax_backward_from_output(ctx: *mut McbCtx, y: *const f32, g: *const f32, out: *mut f32, rows: i64, cols: i64) -> Status;
    pub fn mcb_layer_norm(ctx: *mut McbCtx, x: *const f32, gamma: *const f32, beta: *const f32, eps: f64, out: *mut c_void, out_dt: i32, mean: *mut f32, rstd: *mut f32, rows: i64, dim: i64) -> Status;
    pub fn mcb_layer_norm_backward(ctx: *mut McbCtx, x: *const f32, gamma: *const f32, g: *const c_void, g_dt: i32, eps: f64, mean: *const f32, rstd: *const f32, dx: *mut f32, dgamma: *mut f32, dbeta: *mut f32, rows: i64, dim: i64) -> Status;
    pub fn mcb_layer_norm_backward_noalloc(stream: *mut c_void, x: *const f32, gamma: *const f32, g: *const c_void, g_dt: i32, eps: f64, mean: *const f32, rstd: *const f32, dx: *mut f32, dgamma: *mut f32, dbeta: *mut f32, rows: i64, dim: i64) -> Status;
    pub fn mcb_noalloc_last_error() -> *const c_char;
    pub fn mcb_softmax_cross_entropy(ctx: *mut McbCtx, logits: *const f32, labels: *const c_void, label_dt: i32, n: i64, c: i64, loss_out: *mut f32) -> Status;
    pub fn mcb_softmax_cross_entropy_backward(ctx: *mut McbCtx, logits: *const f32, labels: *const c_void, label_dt: i32, n: i64, c: i64, out: *mut f32) -> Status;
    pub fn mcb_softmax_ce_fused(ctx: *mut McbCtx, logits: *mut c_void, logits_dt: i32, labels: *const c_void, label_dt: i32, n: i64, c: i64, loss_out: *mut f32, upstream: *const f32) -> Status;
    pub fn mcb_embedding(ctx: *mut McbCtx, ids: *const c_void, id_dt: i32, n: i64, weight: *const f32, vocab: i64, dim: i64, out: *mut f32) -> Status;
    pub fn mcb_embedding_backward(ctx: *mut McbCtx, ids: *const c_void, id_dt: i32, n: i64, g: *const c_void, g_dt: i32, vocab: i64, dim: i64, out: *mut f32, accumulate: i32) -> Status;
    pub fn mcb_matmul(ctx: *mut McbCtx, a: *const f32, b: *const f32, c: *mut f32, m: i64, k: i64, n: i64) -> Status;
    pub fn mcb_linear(ctx: *mut McbCtx, x: *const f32, w: *const f32, bias: *const f32, y: *mut f32, m: i64, k: i64, n: i64, act: i32) -> Status;
    pub fn mcb_linear_backward(ctx: *mut McbCtx, g: *const f32, x: *const f32, w: *const f32, dx: *mut f32, dw: *mut f32, db: *mut f32, m: i64, k: i64, n: i64) -> Status;
    pub fn mcb_gemm_bf16(ctx: *mut McbCtx, a: *const c_void, a_mn_major: i32, b: *const c_void, b_mn_major: i32, d: *mut c_void, out_dt: i32, bias: *const f32, m: i64, n: i64, k: i64, accumulate: i32, split_k: i32) -> Status;
    pub fn mcb_gemm_lowp(ctx: *mut McbCtx, in_dt: i32, a: *const c_void, a_mn_major: i32, b: *const c_void, b_mn_major: i32, d: *mut c_void, out_dt: i32, bias: *const f32, m: i64, n: i64, k: i64, accumulate: i32, split_k: i32) -> Status;
    pub fn mcb_attention(ctx: *mut McbCtx, q: *const c_void, k: *const c_void, v: *const c_void, out: *mut c_void, lse: *mut f32, n: i64, seq: i64, dim: i64, heads: i64, causal: i32, dt: i32) -> Status;
    pub fn mcb_attention_backward(ctx: *mut McbCtx, q: *const c_void, k: *const c_void, v: *const c_void, out: *const c_void, gout: *const c_void, lse: *const f32, dq: *mut c_void, dk: *mut c_void, dv: *mut c_void, n: i64, seq: i64, dim: i64, heads: i64, causal: i32, dt: i32) -> Status;
    pub fn mcb_conv2d(ctx: *mut McbCtx, x: *const f32, w: *const f32, bias: *const f32, out: *mut f32, n: i64, c: i64, h: i64, wd: i64, o: i64, kh: i64, kw: i64, stride: i64, pad: i64) -> Status;
    pub fn mcb_conv2d_backward(ctx: *mut McbCtx, x: *const f32, w: *const f32, g: *const f32, dx: *mut f32, dw: *mut f32, db: *mut f32, n: i64, c: i64, h: i64, wd: i64, o: i64, kh: i64, kw: i64, stride: i64, pad: i64) -> Status;
    pub fn mcb_max_pool2d(ctx: *mut McbCtx, x: *const f32, out: *mut f32, n: i64, c: i64, h: i64, w: i64, kernel: i64, stride: i64, pad: i64) -> Status;
    pub fn mcb_max_pool2d_backward(ctx: *mut McbCtx, x: *const f32, g: *const f32, dx: *mut f32, n: i64, c: i64, h: i64, w: i64, kernel: i64, stride: i64, pad: i64) -> Status;
    pub fn mcb_adam_update(ctx: *mut McbCtx, p: *const f32, g: *const f32, m: *const f32, v: *const f32, new_p: *mut f32, new_m: *mut f32, new_v: *mut f32, n: i64, lr: f64, beta1: f64, beta2: f64, eps: f64, step: i32) -> Status;
    pub fn mcb_adam_flat(ctx: *mut McbCtx, p: *mut f32, g: *const c_void, g_dt: i32, m: *mut f32, v: *mut f32, p_bf16: *mut c_void, n: i64, lr: f64, beta1: f64, beta2: f64, eps: f64, step: i32, inv_scale: f64, skip_flag: *const i32) -> Status;
    pub fn mcb_check_finite(ctx: *mut McbCtx, g: *const c_void, g_dt: i32, n: i64, flag: *mut i32) -> Status;
    pub fn mcb_var_new(ctx: *mut McbCtx, host_data: *const c_void, dtype: i32, dims: *const i64, rank: i32, requires_grad: i32, out: *mut *mut McbVar) -> Status;
    pub fn mcb_var_release(v: *mut McbVar);
    pub fn mcb_var_rank(v: *mut McbVar, rank_out: *mut i32) -> Status;
    pub fn mcb_var_dims(v: *mut McbVar, dims_out: *mut i64) -> Status;
    pub fn mcb_var_dtype(v: *mut McbVar, dtype_out: *mut i32) -> Status;
    pub fn mcb_var_data(v: *mut McbVar, host_out: *mut c_void) -> Status;
    pub fn mcb_var_grad(v: *mut McbVar, host_out: *mut f32, has_grad: *mut i32) -> Status;
    pub fn mcb_var_set_data(v: *mut McbVar, host_data: *const c_void) -> Status;
    pub fn mcb_var_set_grad(v: *mut McbVar, host_grad: *const f32) -> Status;
    pub fn mcb_var_cleargrad(v: *mut McbVar) -> Status;
    pub fn mcb_var_requires_grad(v: *mut McbVar, out: *mut i32) -> Status;
    pub fn mcb_var_is_leaf(v: *mut McbVar, out: *mut i32) -> Status;
    pub fn mcb_var_unchain_backward(v: *mut McbVar) -> Status;
    pub fn mcb_var_backward(v: *mut McbVar) -> Status;
    pub fn mcb_set_grad_enabled(enabled: i32);
    pub fn mcb_is_grad_enabled() -> i32;
    pub fn mcb_set_autocast(dtype_or_minus1: i32);
    pub fn mcb_get_autocast() -> i32;
    pub fn mcb_f_binary(op: i32, a: *mut McbVar, b: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_scale(x: *mut McbVar, factor: f64, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_unary(op: i32, x: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_relu(x: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_gelu(x: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_sum(x: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_mean(x: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_matmul(a: *mut McbVar, b: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_linear(x: *mut McbVar, w: *mut McbVar, bias_or_null: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_linear_activation(x: *mut McbVar, w: *mut McbVar, bias_or_null: *mut McbVar, act: i32, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_softmax(x: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_layer_norm(x: *mut McbVar, gamma: *mut McbVar, beta: *mut McbVar, eps: f64, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_softmax_cross_entropy(logits: *mut McbVar, target: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_embedding(ids: *mut McbVar, weight: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_reshape(x: *mut McbVar, dims: *const i64, rank: i32, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_transpose(x: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_permute(x: *mut McbVar, axes: *const i32, rank: i32, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_multi_head_attention(q: *mut McbVar, k: *mut McbVar, v: *mut McbVar, heads: i64, causal: i32, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_conv2d(x: *mut McbVar, w: *mut McbVar, bias_or_null: *mut McbVar, stride: i64, pad: i64, out: *mut *mut McbVar) -> Status;
    pub fn mcb_f_max_pool2d(x: *mut McbVar, kernel: i64, stride: i64, pad: i64, out: *mut *mut McbVar) -> Status;
    pub fn mcb_arena_create(ctx: *mut McbCtx, params: *mut *mut McbVar, n: i32, out: *mut *mut McbArena) -> Status;
    pub fn mcb_arena_release(a: *mut McbArena);
    pub fn mcb_arena_numel(a: *mut McbArena, out: *mut i64) -> Status;
    pub fn mcb_zero_grad(params: *mut *mut McbVar, n: i32) -> Status;
    pub fn mcb_adam_create(ctx: *mut McbCtx, lr: f64, beta1: f64, beta2: f64, eps: f64, out: *mut *mut McbAdam) -> Status;
    pub fn mcb_adam_release(opt: *mut McbAdam);
    pub fn mcb_adam_step(opt: *mut McbAdam, params: *mut *mut McbVar, n: i32) -> Status;
    pub fn mcb_scaler_create(ctx: *mut McbCtx, init_scale: f64, growth_factor: f64, backoff_factor: f64, growth_interval: i32, out: *mut *mut McbScaler) -> Status;
    pub fn mcb_scaler_release(s: *mut McbScaler);
    pub fn mcb_scaler_scale_loss(s: *mut McbScaler, loss: *mut McbVar, out: *mut *mut McbVar) -> Status;
    pub fn mcb_scaler_step(s: *mut McbScaler, opt: *mut McbAdam, params: *mut *mut McbVar, n: i32, applied: *mut i32) -> Status;
    pub fn mcb_scaler_step_async(s: *mut McbScaler, opt: *mut McbAdam, params: *mut *mut McbVar, n: i32) -> Status;
    pub fn mcb_scaler_state(s: *mut McbScaler, scale_out: *mut f64, growth_tracker_out: *mut i32, last_found_inf: *mut i32) -> Status;
    pub fn mcb_opt_create(ctx: *mut McbCtx, kind: i32, lr: f64, beta1: f64, beta2: f64, eps: f64, weight_decay: f64, out: *mut *mut McbAdam) -> Status;
    pub fn mcb_opt_set_lr(opt: *mut McbAdam, lr: f64) -> Status;
    pub fn mcb_opt_get_lr(opt: *mut McbAdam, lr_out: *mut f64) -> Status;
    pub fn mcb_clip_grad_norm(params: *mut *mut McbVar, n: i32, max_norm: f64, norm_out: *mut f64) -> Status;
    pub fn mcb_lr_linear_warmup_cosine(step: u64, warmup_steps: u64, total_steps: u64, base_lr: f64, min_lr: f64) -> f64;
    pub fn mcb_lr_step(step: u64, base_lr: f64, step_size: u64, gamma: f64) -> f64;
    pub fn mcb_lr_polynomial(step: u64, base_lr: f64, total_steps: u64, power: f64, min_lr: f64) -> f64;
    pub fn mcb_he_normal(host_out: *mut f32, n: i64, fan_in: i64, seed: u64) -> Status;
    pub fn mcb_checkpoint_save(ctx: *mut McbCtx, path: *const c_char, names: *const *const c_char, params: *mut *mut McbVar, n: i32, opt_or_null: *mut McbAdam, scaler_or_null: *mut McbScaler) -> Status;
    pub fn mcb_checkpoint_load(ctx: *mut McbCtx, path: *const c_char, names: *const *const c_char, params: *mut *mut McbVar, n: i32, opt_or_null: *mut McbAdam, scaler_or_null: *mut McbScaler) -> Status;
    pub fn mcb_model_create(ctx: *mut McbCtx, kind: i32, cfg: *const i64, n_cfg: i32, out: *mut *mut McbModel) -> Status;
    pub fn mcb_model_release(m: *mut McbModel);
    pub fn mcb_model_num_params(m: *mut McbModel, out: *mut i32) -> Status;
    pub fn mcb_model_param(m: *mut McbModel, index: i32, out: *mut *mut McbVar) -> Status;
    pub fn mcb_model_loss(m: *mut McbModel, input: *mut McbVar, target: *mut McbVar, loss_out: *mut *mut McbVar) -> Status;
    pub fn mcb_static_step_create(model: *mut McbModel, opt: *mut McbAdam, scaler_or_null: *mut McbScaler, autocast_dt: i32, x_dims: *const i64, x_rank: i32, x_dt: i32, y_dims: *const i64, y_rank: i32, y_dt: i32, out: *mut *mut McbStaticStep) -> Status;
    pub fn mcb_static_step_inputs(s: *mut McbStaticStep, x_dev_out: *mut *mut c_void, y_dev_out: *mut *mut c_void) -> Status;
    pub fn mcb_static_step_run(s: *mut McbStaticStep, host_x_or_null: *const c_void, host_y_or_null: *const c_void) -> Status;
    pub fn mcb_static_step_loss(s: *mut McbStaticStep, loss_out: *mut f32) -> Status;
    pub fn mcb_static_step_run_pipelined(s: *mut McbStaticStep, host_x_or_null: *const c_void, host_y_or_null: *const c_void, prev_loss_out: *mut f32, have_prev_out: *mut i32) -> Status;
    pub fn mcb_static_step_drain(s: *mut McbStaticStep, loss_out: *mut f32, have_out: *mut i32) -> Status;
    pub fn mcb_static_step_launches(s: *mut McbStaticStep, kernels_per_step_out: *mut i64) -> Status;
    pub fn mcb_static_step_release(s: *mut McbStaticStep);
    pub fn mcb_dp_unique_id(host_id_out_128: *mut c_void) -> Status;
    pub fn mcb_dp_init(ctx: *mut McbCtx, rank: i32, world: i32, host_id_128: *const c_void) -> Status;
    pub fn mcb_dp_set_timeout_ms(ctx: *mut McbCtx, timeout_ms: i64) -> Status;
    pub fn mcb_dp_attach(ctx: *mut McbCtx, arena: *mut McbArena, bucket_bytes: i64) -> Status;
    pub fn mcb_dp_allreduce_f32(ctx: *mut McbCtx, buf: *mut f32, n: i64, op_max: i32) -> Status;
    pub fn mcb_dp_shutdown(ctx: *mut McbCtx) -> Status;
    pub fn mcb_dp_plan_buckets(sizes: *const i64, n: i32, bucket_elems: i64, bucket_of: *mut i32, n_buckets_out: *mut i32) -> Status;
    pub fn mcb_dp_check_plan_checksums(checksums: *const u64, world: i32) -> Status;
    pub fn mcb_dp_sim_create(slot_sizes: *const i64, n: i32, bucket_elems: i64, world: i32, out: *mut *mut McbDpSim) -> Status;
    pub fn mcb_dp_sim_release(s: *mut McbDpSim);
    pub fn mcb_dp_sim_backward_begin(s: *mut McbDpSim) -> Status;
    pub fn mcb_dp_sim_grad_ready(s: *mut McbDpSim, param: i32) -> Status;
    pub fn mcb_dp_sim_finish(s: *mut McbDpSim) -> Status;
    pub fn mcb_dp_sim_zero_grad(s: *mut McbDpSim) -> Status;
    pub fn mcb_dp_sim_host_wait(s: *mut McbDpSim, timeout_ms: i32) -> Status;
    pub fn mcb_dp_sim_inject(s: *mut McbDpSim, what: i32, value: i32);
    pub fn mcb_dp_sim_log(s: *mut McbDpSim, buckets_out: *mut i32, max: i32) -> i32;
    pub fn mcb_dp_sim_bucket_of(s: *mut McbDpSim, param: i32) -> i32;
    pub fn mcb_dp_sim_buckets(s: *mut McbDpSim) -> i32;
    pub fn mcb_dp_sim_joins(s: *mut McbDpSim) -> i32;
    pub fn mcb_dp_sim_aborted(s: *mut McbDpSim) -> i32;
    pub fn mcb_dp_sim_plan_checksum(s: *mut McbDpSim) -> u64;
    pub fn mcb_dp_sim_last_error(s: *mut McbDpSim) -> *const c_char;
}
