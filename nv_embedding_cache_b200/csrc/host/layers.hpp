// Host-side embedding layers: the operator interface of the lookup hot path.
//
// EmbeddingLayer mirrors the reference's EmbeddingLayerBase (include/embedding_layer.hpp:34-213):
// same method names, argument meaning and error behaviour, so that a parity test reads like the
// reference's own layer tests.
#pragma once

#include <memory>
#include <string>

#include "context.hpp"

namespace nve_b200 {

// reference include/embedding_layer.hpp:44-64
struct PoolingParams {
  nve_pooling_type_t pooling_type = NVE_POOL_CONCATENATE;
  nve_sparse_type_t sparse_type = NVE_SPARSE_FIXED;
  const void* csr_offsets = nullptr;   // element type == layer key type
  int64_t num_csr_offsets = 0;
  int64_t fixed_hotness = 0;
  const void* weights = nullptr;
  nve_data_type_t weight_type = NVE_DTYPE_UNKNOWN;
  nve_data_type_t output_type = NVE_DTYPE_UNKNOWN;
};

// reference src/layer_utils.cpp:277-328
void validate_pool_params(const PoolingParams& p);
int64_t get_lookup_output_rows(int64_t num_keys, const PoolingParams* p);
// reference src/layer_utils.cpp:526-530
bool is_pooling_raw_concat(const PoolingParams* p, nve_data_type_t value_dtype);

class EmbeddingLayer {
 public:
  virtual ~EmbeddingLayer() = default;
  virtual void lookup(context_ptr_t& ctx, int64_t num_keys, const void* keys, void* output,
                      int64_t output_stride, uint64_t* hitmask, const PoolingParams* pool_params,
                      float* hitrates) = 0;
  virtual void insert(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
                      int64_t value_size, const void* values, int64_t table_id) = 0;
  virtual void update(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
                      int64_t value_size, const void* values, int64_t table_id) = 0;
  virtual void accumulate(context_ptr_t& ctx, int64_t num_keys, const void* keys,
                          int64_t value_stride, int64_t value_size, const void* values,
                          nve_data_type_t value_type, int64_t table_id) = 0;
  virtual void clear(context_ptr_t& ctx) = 0;
  virtual void erase(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t table_id) = 0;
  virtual context_ptr_t create_execution_context(cudaStream_t lookup_stream,
                                                 cudaStream_t modify_stream) = 0;
  virtual int64_t get_num_tables() const = 0;
};

// reference include/gpu_embedding_layer.hpp:29-45
struct GPUEmbeddingLayerConfig {
  std::string layer_name;
  int device_id = 0;
  void* embedding_table = nullptr;
  int64_t num_embeddings = 0;
  int64_t embedding_width_in_bytes = 0;
  nve_data_type_t value_dtype = NVE_DTYPE_UNKNOWN;
  int64_t default_row_index = -1;
};

// Dense table in HBM, no cache (reference GPUEmbeddingLayer<KeyType>,
// src/gpu_embedding_layer.cu:300-627).  Pooled lookups run the fused gather+pool kernel in one
// pass for float AND quantised tables.
class GPUEmbeddingLayer : public EmbeddingLayer {
 public:
  GPUEmbeddingLayer(const GPUEmbeddingLayerConfig& config, nve_key_type_t key_type);
  ~GPUEmbeddingLayer() override;

  void lookup(context_ptr_t& ctx, int64_t num_keys, const void* keys, void* output,
              int64_t output_stride, uint64_t* hitmask, const PoolingParams* pool_params,
              float* hitrates) override;
  void insert(context_ptr_t&, int64_t, const void*, int64_t, int64_t, const void*,
              int64_t) override {}  // no effect for a dense table
  void update(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
              int64_t value_size, const void* values, int64_t table_id) override;
  void accumulate(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
                  int64_t value_size, const void* values, nve_data_type_t value_type,
                  int64_t table_id) override;
  void clear(context_ptr_t&) override {}
  void erase(context_ptr_t&, int64_t, const void*, int64_t) override {}
  context_ptr_t create_execution_context(cudaStream_t lookup_stream,
                                         cudaStream_t modify_stream) override;
  int64_t get_num_tables() const override { return 1; }

 private:
  void modify(context_ptr_t& ctx, int64_t num_keys, const void* keys, int64_t value_stride,
              int64_t value_size, const void* values, bool accumulate, nve_data_type_t value_type);

  GPUEmbeddingLayerConfig config_;
  nve_key_type_t key_type_;
  std::shared_ptr<ContextRegistry> contexts_;
  std::mutex launch_mutex_;
  cudaEvent_t modify_in_progress_ = nullptr;
  cudaStream_t private_modify_stream_ = nullptr;
};

}  // namespace nve_b200
