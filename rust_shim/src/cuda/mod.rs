//! `neuralrs::cuda` over libnrs_b200.so (feature `b200`): same module tree as src/cuda/mod.rs.
pub mod backend;
pub mod dp;
pub mod graph;
pub mod loss;
pub mod nn;
pub mod optim;
pub mod runtime;
pub mod sys;
