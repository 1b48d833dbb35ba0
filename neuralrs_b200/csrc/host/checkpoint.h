// Host-side reader / writer of the reference's two checkpoint formats (src/serialize.rs): see
// include/nrs_checkpoint.h for the formats.  Errors are thrown as nrs::Error.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace nrs {
namespace checkpoint {

struct Tensor {
  std::string name;
  std::vector<int64_t> shape;
  std::vector<float> data;
};

// serialize::save: ".safetensors" -> binary, anything else -> positional text; atomic (tmp + rename).
void save(const std::vector<Tensor>& tensors, const std::string& path);
// serialize::load: safetensors tensors come back sorted by name; text tensors as "tensor_{i}" with a flat shape.
std::vector<Tensor> load(const std::string& path);

// The shortest decimal that reads back to the same f32, positional like Rust's `{}` (no exponent).
std::string format_f32(float v);

}  // namespace checkpoint
}  // namespace nrs
