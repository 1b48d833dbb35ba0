//! AdamW — src/cuda/optim/adamw.rs:43-143.
use super::backend::{check, ctx};
use super::runtime::handle;
use super::sys;
use crate::autograd::node::Node;
use std::cell::RefCell;
use std::rc::Rc;

pub struct AdamW { h: *mut sys::nrs_adamw }

impl AdamW {
    /// :56-63.
    pub fn new(lr: f32, beta1: f32, beta2: f32, epsilon: f32, weight_decay: f32) -> Self {
        let mut h = std::ptr::null_mut();
        check(unsafe { sys::nrs_adamw_new(ctx(), lr, beta1, beta2, epsilon, weight_decay, &mut h) });
        AdamW { h }
    }
    /// :65-110.  One launch over the whole model when the parameters share a flat block
    /// (`nrs_flatten_params`), one per parameter otherwise.
    pub fn step(&mut self, params: &[Rc<RefCell<Node>>]) {
        let hs: Vec<*mut sys::nrs_node> = params.iter().map(|p| handle(p, "adamw: param")).collect();
        check(unsafe { sys::nrs_adamw_step_nodes(self.h, hs.as_ptr(), hs.len() as i32) });
    }
    /// :116-128: (t, all first moments in parameter order, then all second moments).
    pub fn export_state(&self) -> (usize, Vec<Vec<f32>>) {
        let n = unsafe { sys::nrs_adamw_state_count(self.h) };
        let mut out = Vec::with_capacity(n as usize);
        for i in 0..n {
            let mut v = vec![0.0f32; unsafe { sys::nrs_adamw_state_len(self.h, i) } as usize];
            check(unsafe { sys::nrs_adamw_state_get(self.h, i, v.as_mut_ptr()) });
            out.push(v);
        }
        (unsafe { sys::nrs_adamw_t(self.h) } as usize, out)
    }
    /// :130-143.
    pub fn import_state(&mut self, t: usize, moments: &[Vec<f32>]) {
        let ptrs: Vec<*const f32> = moments.iter().map(|m| m.as_ptr()).collect();
        let lens: Vec<i64> = moments.iter().map(|m| m.len() as i64).collect();
        check(unsafe { sys::nrs_adamw_import_state(self.h, t as i64, ptrs.as_ptr(), lens.as_ptr(), moments.len() as i32) });
    }
}
impl Drop for AdamW { fn drop(&mut self) { unsafe { sys::nrs_adamw_free(self.h); } } }
