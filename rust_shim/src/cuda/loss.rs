//! Cross-entropy on raw logits with one-hot targets — src/cuda/loss/cross_entropy.rs:74-128.
use super::backend::check;
use super::runtime::handle;
use super::sys;
use crate::autograd::node::Node;
use std::cell::RefCell;
use std::rc::Rc;

type N = Rc<RefCell<Node>>;

/// :74-98.  The batch mean is reduced on the device; one float comes back.
pub fn cross_entropy(pred: &N, target: &N) -> f32 {
    let mut loss = 0.0f32;
    check(unsafe { sys::nrs_cross_entropy(handle(pred, "cuda ce: logits"), handle(target, "cuda ce: target"), &mut loss) });
    loss
}

/// :107-128.  Overwrites the logits' gradient with (softmax - target) / batch.
pub fn cross_entropy_backward(pred: &N, target: &N) {
    check(unsafe { sys::nrs_cross_entropy_backward(handle(pred, "cuda ce: logits"), handle(target, "cuda ce: target")) });
}
