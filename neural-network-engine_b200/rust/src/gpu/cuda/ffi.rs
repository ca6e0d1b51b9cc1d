//! Raw bindings of `include/nne_cuda.h`.  One declaration per exported symbol, nothing else.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_int, c_void};

#[repr(C)]
pub struct nne_ctx {
    _private: [u8; 0],
}
#[repr(C)]
pub struct nne_plan {
    _private: [u8; 0],
}
#[repr(C)]
pub struct nne_qlinear {
    _private: [u8; 0],
}

pub const NNE_OK: c_int = 0;
pub const NNE_ERR_INVALID_ARGUMENT: c_int = 1;
pub const NNE_ERR_SHAPE_MISMATCH: c_int = 2;

extern "C" {
    pub fn nne_status_string(status: c_int) -> *const c_char;
    pub fn nne_last_error(buf: *mut c_char, n: usize) -> c_int;

    pub fn nne_cuda_ctx_create(device: c_int, out: *mut *mut nne_ctx) -> c_int;
    pub fn nne_cuda_ctx_destroy(ctx: *mut nne_ctx) -> c_int;
    pub fn nne_cuda_ctx_check(ctx: *mut nne_ctx) -> c_int;
    pub fn nne_cuda_ctx_info(
        ctx: *const nne_ctx,
        device: *mut c_int,
        sm_count: *mut c_int,
        cc_major: *mut c_int,
        cc_minor: *mut c_int,
        total_mem_bytes: *mut usize,
    ) -> c_int;

    pub fn nne_quantize_rows(
        ctx: *mut nne_ctx,
        w_host: *const f32,
        rows: usize,
        cols: usize,
        q_host: *mut i8,
        scales_host: *mut f32,
    ) -> c_int;
    pub fn nne_quantize_tensor(
        ctx: *mut nne_ctx,
        v_host: *const f32,
        n: usize,
        q_host: *mut i8,
        scale_out: *mut f32,
    ) -> c_int;
    pub fn nne_dequantize_rows(
        ctx: *mut nne_ctx,
        q_host: *const i8,
        scales_host: *const f32,
        rows: usize,
        cols: usize,
        out_host: *mut f32,
    ) -> c_int;

    pub fn nne_qlinear_create_from_f32(
        ctx: *mut nne_ctx,
        w_host: *const f32,
        bias_host_or_null: *const f32,
        n: usize,
        k: usize,
        out: *mut *mut nne_qlinear,
    ) -> c_int;
    pub fn nne_qlinear_create_from_i8(
        ctx: *mut nne_ctx,
        q_host: *const i8,
        scales_host: *const f32,
        bias_host_or_null: *const f32,
        n: usize,
        k: usize,
        out: *mut *mut nne_qlinear,
    ) -> c_int;
    pub fn nne_qlinear_destroy(ql: *mut nne_qlinear) -> c_int;
    pub fn nne_qlinear_download(ql: *const nne_qlinear, q_host: *mut i8, scales_host: *mut f32) -> c_int;
    pub fn nne_qlinear_memory_bytes(ql: *const nne_qlinear) -> usize;
    pub fn nne_qlinear_forward_host(
        ql: *mut nne_qlinear,
        x_host: *const f32,
        m: usize,
        k: usize,
        y_host: *mut f32,
    ) -> c_int;
    pub fn nne_qlinear_forward_dev(
        ql: *mut nne_qlinear,
        x_dev: *const f32,
        m: usize,
        k: usize,
        y_dev: *mut f32,
        stream: *mut c_void,
    ) -> c_int;
    pub fn nne_qlinear_forward_dev_strided(
        ql: *mut nne_qlinear,
        x_dev: *const f32,
        m: usize,
        k: usize,
        y_dev: *mut f32,
        ldy: usize,
        stream: *mut c_void,
    ) -> c_int;
    pub fn nne_qlinear_kernel_for(ql: *const nne_qlinear, m: usize) -> c_int;
    pub fn nne_cuda_ctx_reserve_sms(ctx: *mut nne_ctx, count: c_int) -> c_int;

    // Several independent projections (q/k/v at src/models/llama.rs:226-228) as one launch.
    pub fn nne_qlinear_plan_create(
        ctx: *mut nne_ctx,
        count: usize,
        layers: *const *mut nne_qlinear,
        x_dev: *const *const f32,
        y_dev: *const *mut f32,
        m: usize,
        out: *mut *mut nne_plan,
    ) -> c_int;
    pub fn nne_qlinear_plan_run(plan: *mut nne_plan, stream: *mut c_void) -> c_int;
    pub fn nne_qlinear_plan_run_host(plan: *mut nne_plan, x_all_host: *const f32, y_all_host: *mut f32) -> c_int;
    pub fn nne_qlinear_plan_launches(plan: *const nne_plan) -> c_int;
    pub fn nne_qlinear_plan_destroy(plan: *mut nne_plan) -> c_int;
}
