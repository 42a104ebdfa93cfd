// Table interface behind nve_table_t (reference include/table.hpp:28-181).
#pragma once

#include <vector>

#include "context.hpp"

// Insert heuristic behind nve_heuristic_t: the reference's default heuristic (thresholds per table,
// src/insert_heuristic.cpp:21-35) or the never-insert heuristic.  The cached layer copies it at
// creation, so the handle may be destroyed afterwards.
struct nve_heuristic_s {
  int kind;                       // 0 = default (probabilistic on the hit rate), 1 = never
  std::vector<float> thresholds;  // default kind: one per table
};

namespace nve_b200 {

class Table {
 public:
  virtual ~Table() = default;
  virtual void find(context_ptr_t& ctx, int64_t n, const void* keys, uint64_t* hit_mask,
                    int64_t value_stride, void* values, int64_t* value_sizes) = 0;
  virtual void insert(context_ptr_t& ctx, int64_t n, const void* keys, int64_t value_stride,
                      int64_t value_size, const void* values) = 0;
  virtual void update(context_ptr_t& ctx, int64_t n, const void* keys, int64_t value_stride,
                      int64_t value_size, const void* values) = 0;
  virtual void update_accumulate(context_ptr_t& ctx, int64_t n, const void* keys,
                                 int64_t update_stride, int64_t update_size, const void* updates,
                                 nve_data_type_t update_dtype) = 0;
  virtual void clear(context_ptr_t& ctx) = 0;
  virtual void erase(context_ptr_t& ctx, int64_t n, const void* keys) = 0;
  virtual context_ptr_t create_execution_context(cudaStream_t lookup_stream,
                                                 cudaStream_t modify_stream) = 0;
  virtual int32_t get_device_id() const = 0;
  virtual int64_t get_max_row_size() const = 0;
  virtual int64_t get_key_size() const = 0;
  virtual void reset_lookup_counter(context_ptr_t& ctx) = 0;
  virtual void get_lookup_counter(context_ptr_t& ctx, int64_t* counter) = 0;
};

// Implemented in gpu_table.cu.
void gpu_table_insert_from_backing(Table& table, context_ptr_t& ctx, int64_t n, const void* keys);
void gpu_table_cache_data(Table& table, ExecutionContext& ctx, nve_b200_cache_data_t* out);
void gpu_table_policy_state(Table& table, const float** counters, const int64_t** set_ts);
std::shared_ptr<Table> make_gpu_table(const nve_gpu_table_config_t& config, nve_key_type_t key_type);
// Implemented in linear_uvm_layer.cu.
class EmbeddingLayer;
std::shared_ptr<EmbeddingLayer> make_linear_uvm_layer(const nve_linear_uvm_layer_config_t& config,
                                                      nve_key_type_t key_type,
                                                      std::shared_ptr<Table> gpu_table);

}  // namespace nve_b200
