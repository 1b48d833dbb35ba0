//! Residency helpers — src/cuda/runtime.rs:39-124 with the same names and meaning.
use super::backend::{check, ctx};
use super::sys;
use crate::autograd::node::{GpuBuffers, Node};
use std::cell::RefCell;
use std::rc::Rc;

type N = Rc<RefCell<Node>>;

/// `GpuBuffers` (src/autograd/node.rs:49-53) for this backend: a node owned by the library.
/// `impl Drop for GpuBuffers { fn drop(&mut self) { unsafe { sys::nrs_node_release(self.handle); } } }`
pub(crate) fn handle(node: &N, what: &str) -> *mut sys::nrs_node {
    node.borrow().gpu.as_ref().unwrap_or_else(|| panic!("{what}: not on GPU")).handle
}

/// A Rust node standing for a library-side result: data stays on the device (`data` is empty until
/// `to_host`), `backward_fn` runs the library node's own closure.
pub(crate) fn resident(h: *mut sys::nrs_node, parents: Vec<N>) -> N {
    let ndim = unsafe { sys::nrs_node_ndim(h) } as usize;
    let mut shape = vec![0i64; ndim];
    check(unsafe { sys::nrs_node_shape(h, shape.as_mut_ptr(), ndim as i32) });
    let node = Node::new(Vec::new(), shape.iter().map(|&d| d as usize).collect());
    {
        let mut n = node.borrow_mut();
        n.parents = parents;
        n.gpu = Some(GpuBuffers { handle: h });
        n.backward_fn = Some(Box::new(move |_grad: &Vec<f32>| check(unsafe { sys::nrs_node_backward(h) })));
    }
    node
}

/// src/cuda/runtime.rs:39-51.
pub fn to_cuda(node: &N) {
    let mut n = node.borrow_mut();
    if n.gpu.is_none() {
        let shape: Vec<i64> = n.shape.iter().map(|&d| d as i64).collect();
        let mut h: *mut sys::nrs_node = std::ptr::null_mut();
        check(unsafe { sys::nrs_node_new(ctx(), n.data.as_ptr(), shape.as_ptr(), shape.len() as i32, &mut h) });
        check(unsafe { sys::nrs_node_set_requires_grad(h, n.requires_grad as i32) });
        n.gpu = Some(GpuBuffers { handle: h });
    } else {
        // a second upload of changed host data into the same device buffer
        check(unsafe { sys::nrs_node_set_data(n.gpu.as_ref().unwrap().handle, n.data.as_ptr()) });
    }
    check(unsafe { sys::nrs_to_cuda(n.gpu.as_ref().unwrap().handle) });
}

/// src/cuda/runtime.rs:57-62.
pub fn to_host(node: &N) -> Vec<f32> {
    let h = handle(node, "to_host: node");
    let mut out = vec![0.0f32; unsafe { sys::nrs_node_len(h) } as usize];
    check(unsafe { sys::nrs_to_host(h, out.as_mut_ptr()) });
    out
}

/// src/cuda/runtime.rs:87-94.
pub fn set_grad(node: &N, grad: &[f32]) {
    let h = handle(node, "set_grad: node");
    assert_eq!(grad.len(), unsafe { sys::nrs_node_len(h) } as usize, "set_grad: length mismatch");
    check(unsafe { sys::nrs_set_grad(h, grad.as_ptr()) });
}

/// src/cuda/runtime.rs:96-106.
pub fn read_grad(node: &N) -> Vec<f32> {
    let h = handle(node, "read_grad: node");
    let mut out = vec![0.0f32; unsafe { sys::nrs_node_len(h) } as usize];
    check(unsafe { sys::nrs_read_grad(h, out.as_mut_ptr()) });
    out
}

/// src/cuda/runtime.rs:108-120.  No memset: the next writer of each gradient overwrites it.
pub fn zero_grad(params: &[N]) {
    let hs: Vec<*mut sys::nrs_node> = params.iter().map(|p| handle(p, "zero_grad: node")).collect();
    check(unsafe { sys::nrs_zero_grad(hs.as_ptr(), hs.len() as i32) });
}

/// src/cuda/runtime.rs:122-124.
pub fn synchronize() {
    check(unsafe { sys::nrs_sync(ctx()) });
}
