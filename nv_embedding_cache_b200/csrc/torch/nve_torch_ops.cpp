// torch custom ops over the layer registry of libnve_b200: nve_ops::embedding_lookup and
// nve_ops::embedding_lookup_with_pooling, with the reference's schemas
// (python/pynve/torch_bindings/torch_binding.cpp:86-91), so that graphs traced or exported against
// the reference's op library run against this one.  Built as libnve_b200_torch_ops.so; load it
// with torch.ops.load_library (nv_embedding_cache_b200.pynve does so when torch is importable).
//
// Written against torch's stable ABI (torch/csrc/stable): the library does not depend on the ATen
// C++ headers of one torch release.  It holds no kernels; the lookups are
// nve_b200_registry_lookup / nve_b200_registry_lookup_pooled of libnve_b200.so, issued on torch's
// current stream of the keys' device.  The marker's data pointer names the layer
// (python/pynve/torch_bindings/nve_torch_ops.cu:72-146 is the reference counterpart).  Shape
// inference for tracing is registered from Python (torch.library.register_fake), as in the
// reference.
#ifndef USE_CUDA
#define USE_CUDA   // shim.h declares aoti_torch_get_current_cuda_stream only then
#endif
#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/ops.h>
#include <torch/csrc/stable/tensor.h>

#include <array>
#include <optional>
#include <stdexcept>
#include <string>

#include "nve_b200_ops.h"

namespace {

namespace ts = torch::stable;
using torch::headeronly::ScalarType;

[[noreturn]] void fail(const std::string& what) { throw std::runtime_error("nve-torch-ops: " + what); }

void check(nve_status_t st) {
  if (st == NVE_SUCCESS) return;
  const char* message = nullptr;
  nve_get_last_error(&message);
  fail(message ? message : "layer call failed");
}

// Argument rules of the reference ops (python/pynve/torch_bindings/nve_torch_ops_checks.hpp:27-80).
void check_index_tensor(const ts::Tensor& t, const char* name) {
  if (t.scalar_type() != ScalarType::Long) fail(std::string(name) + " must be an int64 tensor");
  if (!t.is_contiguous()) fail(std::string(name) + " must be contiguous");
}

nve_data_type_t check_pooling_weights(const ts::Tensor& weights, int64_t num_keys) {
  if (!weights.is_contiguous()) fail("weights must be contiguous");
  if (weights.numel() != num_keys) fail("weights must have one element per key");
  switch (weights.scalar_type()) {
    case ScalarType::Float: return NVE_DTYPE_FLOAT32;
    case ScalarType::Half: return NVE_DTYPE_FLOAT16;
    default: fail("weights must be a float32 or float16 tensor");
  }
}

struct Registered {
  int64_t dim = 0;
  nve_data_type_t dtype = NVE_DTYPE_UNKNOWN;
  int device = 0;
};

Registered describe(const ts::Tensor& marker, int64_t embedding_size, int64_t dtype_tag) {
  Registered r;
  check(nve_b200_registry_describe(marker.data_ptr(), &r.dim, &r.dtype, &r.device));
  // The two baked arguments exist for shape inference; at run time the registered layer decides,
  // and a graph whose baked values disagree with the layer it was pointed at is refused.
  if (embedding_size != r.dim) {
    fail("the graph was traced for embedding_size " + std::to_string(embedding_size) +
         " but the registered layer has " + std::to_string(r.dim));
  }
  if (dtype_tag != static_cast<int64_t>(r.dtype)) {
    fail("the graph was traced for data type " + std::to_string(dtype_tag) + " but the registered layer holds " +
         std::to_string(static_cast<int>(r.dtype)));
  }
  return r;
}

ScalarType scalar_type_of(nve_data_type_t t) { return t == NVE_DTYPE_FLOAT32 ? ScalarType::Float : ScalarType::Half; }

void* current_stream(const ts::Tensor& on) {
  void* stream = nullptr;
  if (aoti_torch_get_current_cuda_stream(on.get_device_index(), &stream) != AOTI_TORCH_SUCCESS) {
    fail("could not read torch's current CUDA stream");
  }
  return stream;
}

ts::Tensor embedding_lookup_cuda(ts::Tensor marker, ts::Tensor keys, int64_t embedding_size, int64_t dtype) {
  check_index_tensor(keys, "keys");
  const Registered layer = describe(marker, embedding_size, dtype);
  const int64_t num_keys = keys.numel();
  std::array<int64_t, 2> sizes = {num_keys, layer.dim};
  ts::Tensor out = ts::new_empty(keys, torch::headeronly::IntHeaderOnlyArrayRef(sizes.data(), 2),
                                 scalar_type_of(layer.dtype));
  if (num_keys > 0) {
    check(nve_b200_registry_lookup(marker.data_ptr(), num_keys, static_cast<const int64_t*>(keys.data_ptr()),
                                   out.data_ptr(), current_stream(keys)));
  }
  return out;
}

ts::Tensor embedding_lookup_with_pooling_cuda(ts::Tensor marker, ts::Tensor keys, ts::Tensor offsets,
                                              std::optional<ts::Tensor> weights, int64_t pooling_type,
                                              int64_t embedding_size, int64_t dtype) {
  check_index_tensor(keys, "keys");
  check_index_tensor(offsets, "offsets");
  if (offsets.numel() < 2) {
    fail("offsets must have at least two entries (num_bags + 1, include_last_offset=True convention)");
  }
  const Registered layer = describe(marker, embedding_size, dtype);
  const int64_t num_bags = offsets.numel() - 1;
  std::array<int64_t, 2> sizes = {num_bags, layer.dim};
  ts::Tensor out = ts::new_empty(keys, torch::headeronly::IntHeaderOnlyArrayRef(sizes.data(), 2),
                                 scalar_type_of(layer.dtype));
  nve_data_type_t weight_dtype = NVE_DTYPE_UNKNOWN;
  const void* weight_ptr = nullptr;
  if (weights.has_value()) {
    weight_dtype = check_pooling_weights(*weights, keys.numel());
    weight_ptr = weights->data_ptr();
  }
  check(nve_b200_registry_lookup_pooled(marker.data_ptr(), keys.numel(),
                                        static_cast<const int64_t*>(keys.data_ptr()), out.data_ptr(),
                                        static_cast<nve_pooling_type_t>(pooling_type), offsets.numel(),
                                        static_cast<const int64_t*>(offsets.data_ptr()), weight_dtype, weight_ptr,
                                        current_stream(keys)));
  return out;
}

// Host tensors: this library serves GPU layers only (the reference's CPU kernels belong to its
// host layer).
ts::Tensor embedding_lookup_cpu(ts::Tensor, ts::Tensor, int64_t, int64_t) {
  fail("embedding_lookup: keys are on the host; layers of this library live on a GPU");
}
ts::Tensor embedding_lookup_with_pooling_cpu(ts::Tensor, ts::Tensor, ts::Tensor, std::optional<ts::Tensor>, int64_t,
                                             int64_t, int64_t) {
  fail("embedding_lookup_with_pooling: keys are on the host; layers of this library live on a GPU");
}

}  // namespace

STABLE_TORCH_LIBRARY(nve_ops, m) {
  m.def("embedding_lookup(Tensor marker, Tensor keys, int embedding_size, int dtype) -> Tensor");
  m.def(
      "embedding_lookup_with_pooling(Tensor marker, Tensor keys, Tensor offsets, "
      "Tensor? weights, int pooling_type, int embedding_size, int dtype) -> Tensor");
}

STABLE_TORCH_LIBRARY_IMPL(nve_ops, CUDA, m) {
  m.impl("embedding_lookup", TORCH_BOX(&embedding_lookup_cuda));
  m.impl("embedding_lookup_with_pooling", TORCH_BOX(&embedding_lookup_with_pooling_cuda));
}

STABLE_TORCH_LIBRARY_IMPL(nve_ops, CPU, m) {
  m.impl("embedding_lookup", TORCH_BOX(&embedding_lookup_cpu));
  m.impl("embedding_lookup_with_pooling", TORCH_BOX(&embedding_lookup_with_pooling_cpu));
}
