//! Graph operators — src/cuda/graph/{matmul,add,relu,gelu,reshape,softmax,bmm,transpose,scale,
//! slice_cols,concat_cols}.rs, same signatures.
use super::backend::check;
use super::runtime::{handle, resident};
use super::sys;
use crate::autograd::node::Node;
use std::cell::RefCell;
use std::rc::Rc;

type N = Rc<RefCell<Node>>;

fn unary(x: &N, what: &str, op: unsafe extern "C" fn(*mut sys::nrs_node, *mut *mut sys::nrs_node) -> i32) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe { op(handle(x, what), &mut out) });
    resident(out, vec![x.clone()])
}

fn binary(a: &N, b: &N, what: &str,
          op: unsafe extern "C" fn(*mut sys::nrs_node, *mut sys::nrs_node, *mut *mut sys::nrs_node) -> i32) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe { op(handle(a, what), handle(b, what), &mut out) });
    resident(out, vec![a.clone(), b.clone()])
}

/// src/cuda/graph/matmul.rs:386.
pub fn matmul(a: &N, b: &N) -> N { binary(a, b, "cuda matmul: operand", sys::nrs_op_matmul) }
/// src/cuda/graph/add.rs:41 (same shape, or [r,c] + [c]).
pub fn add(a: &N, b: &N) -> N { binary(a, b, "cuda add: operand", sys::nrs_op_add) }
/// src/cuda/graph/bmm.rs:65.
pub fn bmm(a: &N, b: &N) -> N { binary(a, b, "cuda bmm: operand", sys::nrs_op_bmm) }
/// src/cuda/graph/relu.rs:63.
pub fn relu(x: &N) -> N { unary(x, "cuda relu: input", sys::nrs_op_relu) }
/// src/cuda/graph/gelu.rs:37.
pub fn gelu(a: &N) -> N { unary(a, "cuda gelu: input", sys::nrs_op_gelu) }
/// src/cuda/graph/softmax.rs:43.
pub fn softmax(a: &N) -> N { unary(a, "cuda softmax: input", sys::nrs_op_softmax) }
/// src/cuda/graph/transpose.rs:31.
pub fn transpose(a: &N) -> N { unary(a, "cuda transpose: input", sys::nrs_op_transpose) }

/// src/cuda/graph/reshape.rs:31 (a view here: no copy, the gradient buffer is shared).
pub fn reshape(x: &N, new_shape: Vec<usize>) -> N {
    let shape: Vec<i64> = new_shape.iter().map(|&d| d as i64).collect();
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_reshape(handle(x, "cuda reshape: input"), shape.as_ptr(), shape.len() as i32, &mut out) });
    resident(out, vec![x.clone()])
}

/// src/cuda/graph/scale.rs:27.
pub fn scale(a: &N, s: f32) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_scale(handle(a, "cuda scale: input"), s, &mut out) });
    resident(out, vec![a.clone()])
}

/// src/cuda/graph/slice_cols.rs:37.
pub fn slice_cols(a: &N, col_start: usize, col_end: usize) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_slice_cols(handle(a, "cuda slice_cols: input"), col_start as i64, col_end as i64, &mut out) });
    resident(out, vec![a.clone()])
}

/// src/cuda/graph/concat_cols.rs:38.
pub fn concat_cols(parts: &[N]) -> N {
    let hs: Vec<*mut sys::nrs_node> = parts.iter().map(|p| handle(p, "cuda concat_cols: part")).collect();
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_concat_cols(hs.as_ptr(), hs.len() as i32, &mut out) });
    resident(out, parts.to_vec())
}
