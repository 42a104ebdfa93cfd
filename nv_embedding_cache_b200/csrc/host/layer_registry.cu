// Registry of layers by marker address, and the two lookups that torch custom ops dispatch to.
//
// The reference keeps such a registry inside its torch binding library
// (python/pynve/torch_bindings/nve_registry.hpp:39-60, nve_registry.cu): every torch layer owns a
// one-element "marker" tensor whose data pointer names the layer, a traced or exported graph
// carries that tensor into each op call, and the op finds the layer by the pointer.  Here the
// registry lives behind the C ABI, so the op library (csrc/torch/nve_torch_ops.cpp) and any other
// host that holds only plain pointers use the same entries.
//
// An entry does not own its layer (the binding object that registered it does); it owns the
// execution contexts it creates, one per caller stream, and destroys them when it is unregistered.
#include <map>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <unordered_map>

#include "context.hpp"
#include "nve_b200_ops.h"

namespace nve_b200 {
namespace {

void rethrow(nve_status_t st);

struct RegisteredLayer {
  nve_layer_t layer = nullptr;
  int64_t embedding_dim = 0;
  nve_data_type_t dtype = NVE_DTYPE_UNKNOWN;
  int device = 0;
  int64_t row_bytes = 0;
  std::mutex ctx_mutex;
  std::map<void*, nve_context_t> contexts;   // caller stream -> context

  ~RegisteredLayer() {
    for (auto& kv : contexts) nve_context_destroy(kv.second);
  }

  nve_context_t context_for(void* stream) {
    std::lock_guard<std::mutex> lock(ctx_mutex);
    auto it = contexts.find(stream);
    if (it != contexts.end()) return it->second;
    nve_context_t ctx = nullptr;
    const nve_status_t st =
        nve_layer_create_execution_context(layer, &ctx, stream, stream, nullptr, nullptr);
    if (st != NVE_SUCCESS) rethrow(st);
    contexts.emplace(stream, ctx);
    return ctx;
  }
};

// Lookups take the shared side of the lock (they run concurrently from many threads); register and
// unregister take the exclusive side.  A lookup holds a shared_ptr to its entry, so an entry that
// is unregistered while a lookup runs lives until that lookup returns.
std::shared_mutex g_mutex;
std::unordered_map<const void*, std::shared_ptr<RegisteredLayer>> g_layers;

std::shared_ptr<RegisteredLayer> find_layer(const void* marker) {
  std::shared_lock<std::shared_mutex> lock(g_mutex);
  auto it = g_layers.find(marker);
  if (it == g_layers.end()) {
    throw Error(NVE_ERROR_INVALID_ARGUMENT,
                "no layer is registered under this marker address (was the layer destroyed, or the "
                "marker tensor of a loaded graph not pointed at a live layer?)");
  }
  return it->second;
}

// Re-raises the failure of a nested C ABI call with its own message.
void rethrow(nve_status_t st) {
  const char* message = nullptr;
  nve_get_last_error(&message);
  throw Error(st, message ? std::string(message) : std::string("layer call failed"));
}

int64_t element_bytes(nve_data_type_t dtype) {
  switch (dtype) {
    case NVE_DTYPE_FLOAT32: return 4;
    case NVE_DTYPE_FLOAT16: return 2;
    default: return 0;
  }
}

}  // namespace
}  // namespace nve_b200

using nve_b200::guarded;
using nve_b200::set_last_error;

extern "C" {

nve_status_t nve_b200_registry_register(const void* marker, nve_layer_t layer, int64_t embedding_dim,
                                        nve_data_type_t dtype, int device_id) {
  return guarded([&] {
    NVE_B200_ARG(marker != nullptr, "marker must not be NULL");
    NVE_B200_ARG(layer != nullptr, "layer must not be NULL");
    NVE_B200_ARG(embedding_dim > 0, "embedding_dim must be positive");
    NVE_B200_ARG(nve_b200::element_bytes(dtype) > 0, "registered layers hold float32 or float16 rows");
    auto entry = std::make_shared<nve_b200::RegisteredLayer>();
    entry->layer = layer;
    entry->embedding_dim = embedding_dim;
    entry->dtype = dtype;
    entry->device = device_id;
    entry->row_bytes = embedding_dim * nve_b200::element_bytes(dtype);
    std::unique_lock<std::shared_mutex> lock(nve_b200::g_mutex);
    nve_b200::g_layers[marker] = std::move(entry);   // a marker address that is reused names the new layer
  });
}

nve_status_t nve_b200_registry_unregister(const void* marker) {
  return guarded([&] {
    std::shared_ptr<nve_b200::RegisteredLayer> gone;
    {
      std::unique_lock<std::shared_mutex> lock(nve_b200::g_mutex);
      auto it = nve_b200::g_layers.find(marker);
      if (it == nve_b200::g_layers.end()) return;   // unknown markers are ignored, as in the reference
      gone = std::move(it->second);
      nve_b200::g_layers.erase(it);
    }
    // `gone` is released outside the lock: destroying contexts waits for their streams
  });
}

nve_status_t nve_b200_registry_describe(const void* marker, int64_t* embedding_dim, nve_data_type_t* dtype,
                                        int* device_id) {
  return guarded([&] {
    auto entry = nve_b200::find_layer(marker);
    if (embedding_dim) *embedding_dim = entry->embedding_dim;
    if (dtype) *dtype = entry->dtype;
    if (device_id) *device_id = entry->device;
  });
}

int64_t nve_b200_registry_size(void) {
  std::shared_lock<std::shared_mutex> lock(nve_b200::g_mutex);
  return static_cast<int64_t>(nve_b200::g_layers.size());
}

nve_status_t nve_b200_registry_lookup(const void* marker, int64_t num_keys, const int64_t* keys, void* output,
                                      void* stream) {
  NVE_B200_RANGE();
  return guarded([&] {
    auto entry = nve_b200::find_layer(marker);
    nve_context_t ctx = entry->context_for(stream);
    const nve_status_t st =
        nve_layer_lookup(entry->layer, ctx, num_keys, keys, output, entry->row_bytes, nullptr, nullptr);
    if (st != NVE_SUCCESS) nve_b200::rethrow(st);
  });
}

nve_status_t nve_b200_registry_lookup_pooled(const void* marker, int64_t num_keys, const int64_t* keys,
                                             void* output, nve_pooling_type_t pooling_type,
                                             int64_t num_offsets, const int64_t* offsets,
                                             nve_data_type_t weight_dtype, const void* weights, void* stream) {
  NVE_B200_RANGE();
  return guarded([&] {
    auto entry = nve_b200::find_layer(marker);
    nve_context_t ctx = entry->context_for(stream);
    const nve_status_t st = nve_layer_lookup_pooled(
        entry->layer, ctx, num_keys, keys, output, entry->row_bytes, nullptr, pooling_type, NVE_SPARSE_CSR,
        offsets, num_offsets, 0, weights, weights ? weight_dtype : NVE_DTYPE_FLOAT32, entry->dtype, nullptr);
    if (st != NVE_SUCCESS) nve_b200::rethrow(st);
  });
}

}  // extern "C"
