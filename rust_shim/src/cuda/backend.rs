//! The shared backend: one context on device 0, created on first use
//! (stands in for src/cuda/backend.rs:17-42: CudaContext::new(0) + default_stream + NVRTC compile cache).
use super::sys;
use std::ffi::CStr;
use std::sync::OnceLock;

struct Ctx(*mut sys::nrs_ctx);
unsafe impl Send for Ctx {}
unsafe impl Sync for Ctx {}

static CTX: OnceLock<Ctx> = OnceLock::new();

/// The global context.  Panics like the reference's `.expect("no CUDA device")` when no sm_100 device exists.
pub fn ctx() -> *mut sys::nrs_ctx {
    CTX.get_or_init(|| {
        let mut c: *mut sys::nrs_ctx = std::ptr::null_mut();
        let st = unsafe { sys::nrs_init(0, &mut c) };
        if st != sys::NRS_OK {
            panic!("nrs-b200: {}", last_error(std::ptr::null()));
        }
        Ctx(c)
    })
    .0
}

pub fn last_error(ctx: *const sys::nrs_ctx) -> String {
    unsafe { CStr::from_ptr(sys::nrs_last_error(ctx)) }.to_string_lossy().into_owned()
}

/// Every reference call site ends in `.expect(..)`: a failure is a panic carrying the library's message.
pub fn check(status: i32) {
    if status != sys::NRS_OK {
        panic!("nrs-b200: {}", last_error(ctx()));
    }
}

/// Contraction precision: 3xTF32 (default, <= 1e-4 vs the CPU path), TF32 (opt-in, <= 1e-2) or FP32.
pub fn set_math_mode(mode: i32) {
    check(unsafe { sys::nrs_set_math_mode(ctx(), mode) });
}
