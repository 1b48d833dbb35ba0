/* Checkpoint files of the NeuralRs training path: the two formats of the reference's
 * src/serialize.rs, read and written by host code only (no GPU is touched; the
 * trainer-level calls download / upload through the context they belong to).
 *
 *  - text (src/serialize.rs:81-136, save_tensors / load_tensors): "tensors N", then per
 *    tensor "len L" and L lines, one value each, printed as the shortest decimal that
 *    reads back to the same f32 (Rust's `{}`: positional, never an exponent); names and
 *    shapes are dropped, a load synthesises "tensor_{i}" and the flat length (:183-195).
 *  - safetensors (src/serialize.rs:197-238 through the `safetensors` crate, 0.8.0 in the
 *    reference's Cargo.lock): 8-byte little-endian header length, a JSON header
 *    {"name":{"dtype":"F32","shape":[..],"data_offsets":[begin,end]},..} with the tensors
 *    in name order, padded with spaces to a multiple of 8 bytes, then the little-endian
 *    f32 data back to back.  Only F32 tensors are accepted on load (:219-223); a load
 *    returns the tensors sorted by name (:235).
 *
 * Both writers write "<path>.tmp" and rename it into place (:92-101, :214-216), so an
 * interrupted save never truncates an existing checkpoint.  The format is chosen by the
 * extension, ".safetensors" or anything else (:170-177).
 *
 * Every call returns an nrs status (nrs.h); the message of a failure is at
 * nrs_last_error(NULL). */
#ifndef NRS_CHECKPOINT_H
#define NRS_CHECKPOINT_H

#include <stddef.h>
#include <stdint.h>

#include "nrs_graph.h"

#ifdef __cplusplus
extern "C" {
#endif

/* NamedTensor of src/serialize.rs:160: (name, shape, data). */
typedef struct nrs_named_tensor {
  const char* name;
  const int64_t* shape;
  int ndim;
  const float* data;
} nrs_named_tensor;

typedef struct nrs_checkpoint nrs_checkpoint;

/* serialize::save (src/serialize.rs:170-177). */
int nrs_save(const nrs_named_tensor* tensors, int count, const char* path);
/* serialize::load (src/serialize.rs:183-195): the file's tensors, owned by the handle. */
int nrs_load(const char* path, nrs_checkpoint** out);
int nrs_checkpoint_count(const nrs_checkpoint* ck);
const char* nrs_checkpoint_name(const nrs_checkpoint* ck, int i);
int nrs_checkpoint_ndim(const nrs_checkpoint* ck, int i);
int64_t nrs_checkpoint_dim(const nrs_checkpoint* ck, int i, int d);
int64_t nrs_checkpoint_len(const nrs_checkpoint* ck, int i);
const float* nrs_checkpoint_data(const nrs_checkpoint* ck, int i);
/* Index of the tensor called `name`, or -1. */
int nrs_checkpoint_find(const nrs_checkpoint* ck, const char* name);
void nrs_checkpoint_free(nrs_checkpoint* ck);

/* save_checkpoint / load_checkpoint of examples/mnist_cuda_cnn.rs:160-221 for the native
 * trainer: every parameter, then every batchnorm running statistic, under `names`
 * (param_count + buffer_count strings; NULL gives "param.NN" / "buffer.NN"), plus the
 * AdamW state as "optim.t" ([1], the step count as f32), "optim.m.NN" and "optim.v.NN"
 * (flat).  Loading looks everything up by name; tensors of the wrong size or missing
 * parameters are errors, a file without "optim.t" leaves the optimizer as it is.  With
 * the text format (no names) tensors are matched by position. */
int nrs_trainer_save_checkpoint(nrs_trainer* t, const char* const* names, const char* path);
int nrs_trainer_load_checkpoint(nrs_trainer* t, const char* const* names, const char* path);

#ifdef __cplusplus
}
#endif
#endif
