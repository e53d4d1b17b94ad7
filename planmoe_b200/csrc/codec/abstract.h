// C++ extension point: user-defined payload codecs.
//
// Subclass AbstractCompressor and register a factory; Python then finds the codec under that name
// (compress_name="mine").  Counterpart of PlanMoE/custom/compressor/abstract.h:11-22 and the factory of
// PlanMoE/custom/custom_kernel.cpp:194-207; the all-to-all itself is not part of the codec here (any
// comm algorithm moves the codec's wire buffer), which removes the reference's per-codec all_to_all
// overrides (int8.cpp:69-74, lz.cpp:68-74).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace planmoe {

class AbstractCompressor {
 public:
  virtual ~AbstractCompressor() = default;
  // Upper bound of the wire size for `bytes` of input split over `parts` destinations; the wire
  // buffer is split evenly over the destinations, so it must be a multiple of `parts`.
  virtual size_t wire_bytes(size_t bytes, int parts) const = 0;
  // elem_size: bytes per element of the payload (2 = bf16/fp16, 4 = fp32); row_elems: last-dim length.
  virtual void compress(const void* in, void* wire, size_t bytes, int parts, int elem_size, size_t row_elems,
                        cudaStream_t stream) = 0;
  virtual void decompress(const void* wire, void* out, size_t bytes, int parts, int elem_size, size_t row_elems,
                          cudaStream_t stream) = 0;
};

using CompressorFactory = std::function<std::unique_ptr<AbstractCompressor>()>;

void register_compressor(const std::string& name, CompressorFactory factory);
bool has_compressor(const std::string& name);
std::unique_ptr<AbstractCompressor> make_compressor(const std::string& name);
std::vector<std::string> compressor_names();

struct CompressorRegistrar {
  CompressorRegistrar(const std::string& name, CompressorFactory f) { register_compressor(name, std::move(f)); }
};

}  // namespace planmoe
