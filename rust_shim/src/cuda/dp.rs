//! Data-parallel gradient exchange for a loop over nodes (examples/cifar_cuda.rs:267-286 on several
//! GPUs, one process per GPU).  No reference counterpart: the reference is single-GPU.
//!
//!     let dp = DataParallel::new(rank, world, &id, global_batch, &params, 32 << 20);
//!     // per step: zero_grad, forward, cross-entropy backward dividing by the GLOBAL batch, then
//!     dp.backward_graph(&logits);      // instead of autograd::node::backward_graph
//!     optimizer.step(&params);         // on the summed gradients
use super::backend::{check, ctx};
use super::runtime::handle;
use super::sys;
use crate::autograd::node::Node;
use std::cell::RefCell;
use std::rc::Rc;

type N = Rc<RefCell<Node>>;

/// 128-byte rendezvous id, made by rank 0 and handed to every rank by the launcher.
pub fn unique_id() -> [u8; 128] {
    let mut id = [0u8; 128];
    check(unsafe { sys::nrs_dp_unique_id(id.as_mut_ptr() as *mut std::os::raw::c_void) });
    id
}

/// (begin, end) of this rank's contiguous shard of the global batch.
pub fn shard_range(global_batch: usize, rank: usize, world: usize) -> (usize, usize) {
    let (mut b, mut e) = (0i32, 0i32);
    check(unsafe { sys::nrs_dp_shard_range(global_batch as i32, rank as i32, world as i32, &mut b, &mut e) });
    (b as usize, e as usize)
}

pub struct DataParallel { h: *mut sys::nrs_dp }

impl DataParallel {
    pub fn new(rank: usize, world: usize, id: &[u8; 128], global_batch: usize, params: &[N], bucket_bytes: usize) -> Self {
        let mut h = std::ptr::null_mut();
        check(unsafe {
            sys::nrs_dp_create(ctx(), rank as i32, world as i32, id.as_ptr() as *const std::os::raw::c_void,
                               global_batch as i32, 0.0, &mut h)
        });
        let hs: Vec<*mut sys::nrs_node> = params.iter().map(|p| handle(p, "data parallel: param")).collect();
        check(unsafe { sys::nrs_bucket_register(h, hs.as_ptr(), hs.len() as i32, bucket_bytes) });
        DataParallel { h }
    }
    /// backward_graph that all-reduces each gradient bucket as soon as backward has produced it.
    pub fn backward_graph(&self, root: &N) {
        check(unsafe { sys::nrs_backward_graph_dp(handle(root, "backward_graph: root"), self.h) });
    }
    /// The same in pieces, for a caller that drives its own backward calls.
    pub fn begin_step(&self) { check(unsafe { sys::nrs_dp_begin_step(self.h) }); }
    pub fn grad_ready(&self, param: &N) { check(unsafe { sys::nrs_grad_ready(self.h, handle(param, "nrs_grad_ready: param")) }); }
    pub fn allreduce_wait(&self) { check(unsafe { sys::nrs_allreduce_wait(self.h) }); }
    /// Host-side wait under the group's deadline: a rank that never arrives panics here instead of hanging.
    pub fn host_wait(&self) { check(unsafe { sys::nrs_dp_host_wait(self.h) }); }
}
impl Drop for DataParallel { fn drop(&mut self) { unsafe { sys::nrs_dp_free(self.h); } } }
