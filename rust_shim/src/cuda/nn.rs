//! Layers — src/cuda/nn/*.rs, same names, argument meaning and panics.
use super::backend::{check, ctx};
use super::graph::{add, matmul};
use super::runtime::{handle, resident};
use super::sys;
use crate::autograd::node::Node;
use std::cell::RefCell;
use std::rc::Rc;

type N = Rc<RefCell<Node>>;

/// src/cuda/nn/conv.rs:244-250.  The input gradient is skipped when `input.requires_grad` is false (:304).
pub fn conv2d(input: &N, weight: &N, bias: &N, stride: usize, pad: usize) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe {
        sys::nrs_op_conv2d(handle(input, "cuda conv2d: input"), handle(weight, "cuda conv2d: weight"),
                           handle(bias, "cuda conv2d: bias"), stride as i64, pad as i64, &mut out)
    });
    resident(out, vec![input.clone(), weight.clone(), bias.clone()])
}

/// conv2d followed by ReLU in one kernel (no reference counterpart; same values as relu(conv2d(..))).
pub fn conv2d_relu(input: &N, weight: &N, bias: &N, stride: usize, pad: usize) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe {
        sys::nrs_op_conv2d_act(handle(input, "cuda conv2d: input"), handle(weight, "cuda conv2d: weight"),
                               handle(bias, "cuda conv2d: bias"), stride as i64, pad as i64, sys::NRS_ACT_RELU, &mut out)
    });
    resident(out, vec![input.clone(), weight.clone(), bias.clone()])
}

/// src/cuda/nn/maxpool.rs:66.
pub fn maxpool2d(input: &N, kernel: usize, stride: usize) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_maxpool2d(handle(input, "cuda maxpool: input"), kernel as i64, stride as i64, &mut out) });
    resident(out, vec![input.clone()])
}

/// src/cuda/nn/flatten.rs:11.
pub fn flatten(x: &N) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_flatten(handle(x, "cuda flatten: input"), &mut out) });
    resident(out, vec![x.clone()])
}

/// src/cuda/nn/normalization.rs:87.
pub fn layernorm(x: &N, gamma: &N, beta: &N, eps: f32) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe {
        sys::nrs_op_layernorm(handle(x, "cuda layernorm: input"), handle(gamma, "cuda layernorm: gamma"),
                              handle(beta, "cuda layernorm: beta"), eps, &mut out)
    });
    resident(out, vec![x.clone(), gamma.clone(), beta.clone()])
}

/// src/cuda/nn/normalization.rs:168-183.
pub struct LayerNorm { pub gamma: N, pub beta: N, pub eps: f32 }
impl LayerNorm {
    pub fn new(gamma: N, beta: N, eps: f32) -> Self { LayerNorm { gamma, beta, eps } }
    pub fn forward(&self, x: &N) -> N { layernorm(x, &self.gamma, &self.beta, self.eps) }
}

/// src/cuda/nn/linear.rs:11-26: matmul + broadcast add.
pub struct Linear { pub weights: N, pub bias: N }
impl Linear {
    pub fn new(weights: N, bias: N) -> Self { Linear { weights, bias } }
    pub fn forward(&self, input: &N) -> N { add(&matmul(input, &self.weights), &self.bias) }
}

/// src/cuda/nn/batchnorm.rs:118 ([batch, features]).
pub fn batchnorm(x: &N, gamma: &N, beta: &N, running_mean: &N, running_var: &N, momentum: f32, eps: f32, training: bool) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe {
        sys::nrs_op_batchnorm(handle(x, "cuda bn: input"), handle(gamma, "cuda bn: gamma"), handle(beta, "cuda bn: beta"),
                              handle(running_mean, "cuda bn: running_mean"), handle(running_var, "cuda bn: running_var"),
                              momentum, eps, training as i32, &mut out)
    });
    resident(out, vec![x.clone(), gamma.clone(), beta.clone()])
}

/// src/cuda/nn/batchnorm2d.rs:131 ([batch, channels, h, w]).
pub fn batchnorm2d(x: &N, gamma: &N, beta: &N, running_mean: &N, running_var: &N, momentum: f32, eps: f32, training: bool) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe {
        sys::nrs_op_batchnorm2d(handle(x, "cuda bn2d: input"), handle(gamma, "cuda bn2d: gamma"), handle(beta, "cuda bn2d: beta"),
                                handle(running_mean, "cuda bn2d: running_mean"), handle(running_var, "cuda bn2d: running_var"),
                                momentum, eps, training as i32, &mut out)
    });
    resident(out, vec![x.clone(), gamma.clone(), beta.clone()])
}

/// src/cuda/nn/dropout.rs:32.  The mask is drawn on the device (seeded, `nrs_rng_seed`), not on the host.
pub fn dropout(input: &N, p: f32, training: bool) -> N {
    if !training { return input.clone(); }
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_dropout(handle(input, "cuda dropout: input"), p, 1, std::ptr::null_mut(), &mut out) });
    resident(out, vec![input.clone()])
}

/// src/cuda/nn/dropout2d.rs:38.
pub fn dropout2d(input: &N, p: f32, training: bool) -> N {
    if !training { return input.clone(); }
    let mut out = std::ptr::null_mut();
    check(unsafe { sys::nrs_op_dropout2d(handle(input, "cuda dropout2d: input"), p, 1, std::ptr::null_mut(), &mut out) });
    resident(out, vec![input.clone()])
}

/// src/cuda/nn/embedding.rs:35-100.
pub struct Embedding { pub weight: N, pub vocab_size: usize, pub embedding_dim: usize }
impl Embedding {
    pub fn new(weight: N, vocab_size: usize, embedding_dim: usize) -> Self { Embedding { weight, vocab_size, embedding_dim } }
    pub fn forward(&self, indices: &[usize]) -> N {
        for &i in indices { assert!(i < self.vocab_size, "token index out of vocab range"); }
        let idx: Vec<i32> = indices.iter().map(|&i| i as i32).collect();
        let mut out = std::ptr::null_mut();
        check(unsafe { sys::nrs_op_embedding(handle(&self.weight, "cuda embedding: weight"), idx.as_ptr(), idx.len() as i64, &mut out) });
        resident(out, vec![self.weight.clone()])
    }
    /// The batched form the reference has on its CPU path (src/nn/embedding.rs:60-113).
    pub fn forward_batch(&self, batch_indices: &[Vec<usize>]) -> N {
        let seq = batch_indices.first().map_or(0, |r| r.len());
        let mut idx = Vec::with_capacity(batch_indices.len() * seq);
        for row in batch_indices {
            assert_eq!(row.len(), seq, "embedding: ragged batch");
            for &i in row { assert!(i < self.vocab_size, "token index out of vocab range"); idx.push(i as i32); }
        }
        let mut out = std::ptr::null_mut();
        check(unsafe {
            sys::nrs_op_embedding_batch(handle(&self.weight, "cuda embedding: weight"), idx.as_ptr(), batch_indices.len() as i64,
                                        seq as i64, &mut out)
        });
        resident(out, vec![self.weight.clone()])
    }
}

/// src/cuda/nn/positional.rs:12-44: the sinusoidal table is made once and stays resident.
pub struct PositionalEncoding { pub d_model: usize, pub max_len: usize, table: *mut sys::nrs_node }
impl PositionalEncoding {
    pub fn new(d_model: usize, max_len: usize) -> Self {
        let mut table = std::ptr::null_mut();
        check(unsafe { sys::nrs_positional_new(ctx(), d_model as i64, max_len as i64, &mut table) });
        PositionalEncoding { d_model, max_len, table }
    }
    pub fn forward(&self, x: &N) -> N {
        let mut out = std::ptr::null_mut();
        check(unsafe { sys::nrs_op_positional(handle(x, "cuda positional: input"), self.table, &mut out) });
        resident(out, vec![x.clone()])
    }
}
impl Drop for PositionalEncoding { fn drop(&mut self) { unsafe { sys::nrs_node_release(self.table); } } }

/// src/cuda/nn/attention.rs:23-32: softmax(Q K^T / sqrt(d_head)) V on [batch, seq, d_head].
pub fn attention_batch(q: &N, k: &N, v: &N) -> N {
    let mut out = std::ptr::null_mut();
    check(unsafe {
        sys::nrs_op_attention_batch(handle(q, "cuda attention: q"), handle(k, "cuda attention: k"), handle(v, "cuda attention: v"),
                                    0, &mut out)
    });
    resident(out, vec![q.clone(), k.clone(), v.clone()])
}

/// src/cuda/nn/multihead.rs:14-85 (weights [d_model, d_model], no biases).
pub struct MultiHeadAttention { pub w_q: N, pub w_k: N, pub w_v: N, pub w_o: N, pub d_model: usize, pub num_heads: usize }
impl MultiHeadAttention {
    pub fn new(w_q: N, w_k: N, w_v: N, w_o: N, d_model: usize, num_heads: usize) -> Self {
        assert!(d_model % num_heads == 0, "d_model must be divisible by num_heads");
        MultiHeadAttention { w_q, w_k, w_v, w_o, d_model, num_heads }
    }
    pub fn forward_batch(&self, x: &N) -> N {
        let mut out = std::ptr::null_mut();
        check(unsafe {
            sys::nrs_op_mha(handle(x, "cuda mha: input"), handle(&self.w_q, "cuda mha: w_q"), handle(&self.w_k, "cuda mha: w_k"),
                            handle(&self.w_v, "cuda mha: w_v"), handle(&self.w_o, "cuda mha: w_o"), self.num_heads as i64, 0, &mut out)
        });
        resident(out, vec![x.clone(), self.w_q.clone(), self.w_k.clone(), self.w_v.clone(), self.w_o.clone()])
    }
}

/// src/cuda/nn/transformer_block.rs:16-60: post-LN block with a ReLU feed-forward.
pub struct TransformerBlock {
    pub mha: MultiHeadAttention, pub norm1: LayerNorm, pub norm2: LayerNorm, pub ff1: Linear, pub ff2: Linear,
    pub d_model: usize, pub d_ff: usize,
}
impl TransformerBlock {
    fn run(&self, x: &N, final_norm: bool) -> N {
        // parameters() order of src/nn/transformer_block.rs:58-66
        let ps = [&self.mha.w_q, &self.mha.w_k, &self.mha.w_v, &self.mha.w_o, &self.norm1.gamma, &self.norm1.beta,
                  &self.norm2.gamma, &self.norm2.beta, &self.ff1.weights, &self.ff1.bias, &self.ff2.weights, &self.ff2.bias];
        let hs: Vec<*mut sys::nrs_node> = ps.iter().map(|p| handle(p, "cuda transformer block: parameter")).collect();
        let mut out = std::ptr::null_mut();
        check(unsafe {
            sys::nrs_op_transformer_block(handle(x, "cuda transformer block: input"), hs.as_ptr(), self.mha.num_heads as i64,
                                          self.norm1.eps, sys::NRS_ACT_RELU, 0, final_norm as i32, &mut out)
        });
        let mut parents = vec![x.clone()];
        parents.extend(ps.iter().map(|p| (*p).clone()));
        resident(out, parents)
    }
    pub fn forward(&self, x: &N) -> N { self.run(x, true) }
    pub fn forward_no_final_norm(&self, x: &N) -> N { self.run(x, false) }
}
