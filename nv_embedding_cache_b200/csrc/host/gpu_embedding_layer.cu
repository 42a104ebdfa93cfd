#include "layers.hpp"
#include "ops_internal.hpp"

#include <climits>

namespace nve_b200 {

void validate_pool_params(const PoolingParams& p) {
  NVE_B200_ARG(p.output_type != NVE_DTYPE_UNKNOWN, "Unknown output type");
  if (p.pooling_type == NVE_POOL_CONCATENATE) return;  // every other field is ignored
  if (is_weighted(p.pooling_type)) {
    NVE_B200_ARG(p.weights != nullptr, "Sparse weights are required for weighted pooling");
  }
  switch (p.sparse_type) {
    case NVE_SPARSE_FIXED:
      NVE_B200_ARG(p.fixed_hotness > 0, "Invalid fixed hotness");
      break;
    case NVE_SPARSE_CSR:
      NVE_B200_ARG(p.csr_offsets != nullptr, "CSR offsets are required for pooling");
      NVE_B200_ARG(p.num_csr_offsets >= 2, "CSR pooling requires at least two offsets");
      break;
    default:
      throw InvalidArgument(cat("Unsupported sparse type ", static_cast<int>(p.sparse_type)));
  }
}

int64_t get_lookup_output_rows(int64_t num_keys, const PoolingParams* p) {
  NVE_B200_ARG(num_keys >= 0, "Invalid number of keys");
  if (p == nullptr || p->pooling_type == NVE_POOL_CONCATENATE) return num_keys;
  switch (p->sparse_type) {
    case NVE_SPARSE_FIXED:
      NVE_B200_ARG(p->fixed_hotness > 0, "Invalid fixed hotness");
      NVE_B200_ARG(num_keys % p->fixed_hotness == 0,
                   "Number of keys does not divide by fixed hotness");
      return num_keys / p->fixed_hotness;
    case NVE_SPARSE_CSR:
      NVE_B200_ARG(p->csr_offsets != nullptr, "CSR offsets are required for pooling");
      NVE_B200_ARG(p->num_csr_offsets >= 2, "CSR pooling requires at least two offsets");
      return p->num_csr_offsets - 1;
    default:
      throw InvalidArgument(cat("Unsupported sparse type ", static_cast<int>(p->sparse_type)));
  }
}

bool is_pooling_raw_concat(const PoolingParams* p, nve_data_type_t value_dtype) {
  return p && p->pooling_type == NVE_POOL_CONCATENATE && p->output_type == value_dtype;
}

namespace {

int64_t quant_value_count(const GPUEmbeddingLayerConfig& c) {
  const int64_t meta = quant_meta_bytes(c.value_dtype);
  NVE_B200_CHECK(c.embedding_width_in_bytes > meta,
                 "Quantized GPU embedding rows must contain values in addition to metadata");
  return c.embedding_width_in_bytes - meta;  // 1-byte values
}

}  // namespace

GPUEmbeddingLayer::GPUEmbeddingLayer(const GPUEmbeddingLayerConfig& config, nve_key_type_t key_type)
    : config_(config), key_type_(key_type) {
  NVE_B200_CHECK(config_.embedding_table != nullptr, "Invalid embedding table");
  NVE_B200_CHECK(config_.num_embeddings > 0, "Invalid number of embeddings");
  NVE_B200_CHECK(config_.value_dtype == NVE_DTYPE_FLOAT32 ||
                     config_.value_dtype == NVE_DTYPE_FLOAT16 ||
                     is_quant_rowwise(config_.value_dtype),
                 "Unsupported GPU embedding table value type");
  NVE_B200_CHECK(config_.embedding_width_in_bytes > 0, "Invalid embedding width");
  if (is_quant_rowwise(config_.value_dtype)) {
    NVE_B200_CHECK(config_.embedding_width_in_bytes % 2 == 0,
                   "Quantized GPU embedding row width must be even");
    (void)quant_value_count(config_);
  } else {
    NVE_B200_CHECK(config_.embedding_width_in_bytes % dtype_size(config_.value_dtype) == 0,
                   "Embedding width is not a multiple of the value size");
  }
  const uint64_t key_max = key_type_ == NVE_KEY_INT32 ? static_cast<uint64_t>(INT32_MAX)
                                                      : static_cast<uint64_t>(INT64_MAX);
  NVE_B200_CHECK(static_cast<uint64_t>(config_.num_embeddings) <= key_max,
                 "Number of embeddings cannot be represented by the layer key type");
  NVE_B200_CHECK(config_.default_row_index < config_.num_embeddings,
                 "Default row index must be less than num_embeddings");
  contexts_ = std::make_shared<ContextRegistry>();
  ScopedDevice sd(config_.device_id);
  NVE_B200_CUDA(cudaEventCreateWithFlags(&modify_in_progress_, cudaEventDisableTiming));
  NVE_B200_CUDA(cudaStreamCreateWithFlags(&private_modify_stream_, cudaStreamNonBlocking));
}

GPUEmbeddingLayer::~GPUEmbeddingLayer() {
  if (modify_in_progress_) (void)cudaEventDestroy(modify_in_progress_);
  if (private_modify_stream_) (void)cudaStreamDestroy(private_modify_stream_);
  (void)cudaGetLastError();
}

context_ptr_t GPUEmbeddingLayer::create_execution_context(cudaStream_t lookup_stream,
                                                          cudaStream_t modify_stream) {
  return std::make_shared<ExecutionContext>(config_.device_id, lookup_stream, modify_stream,
                                            contexts_);
}

void GPUEmbeddingLayer::lookup(context_ptr_t& ctx, int64_t num_keys, const void* keys, void* output,
                               int64_t output_stride, uint64_t* hitmask,
                               const PoolingParams* pool_params, float* hitrates) {
  ScopedDevice sd(config_.device_id);
  NVE_B200_ARG(num_keys >= 0, "Invalid num_keys");
  NVE_B200_ARG(keys != nullptr, "Invalid keys buffer");
  NVE_B200_ARG(output != nullptr, "Invalid output buffer");
  NVE_B200_ARG(hitmask == nullptr, "Hitmask is not supported for GPU embedding layer");
  NVE_B200_ARG(ctx != nullptr, "Invalid layer context");
  NVE_B200_ARG(num_keys <= INT_MAX, "Number of keys exceeding max int value is not supported");

  const bool quantized = is_quant_rowwise(config_.value_dtype);
  const bool concatenate = pool_params && pool_params->pooling_type == NVE_POOL_CONCATENATE;
  const bool raw_concat = is_pooling_raw_concat(pool_params, config_.value_dtype);
  const int64_t width_bytes = config_.embedding_width_in_bytes;
  if (pool_params) {
    validate_pool_params(*pool_params);
    if (raw_concat) {
      NVE_B200_ARG(output_stride == width_bytes,
                   "Raw Concatenate output stride must be the same as the stored row width");
    } else if (quantized) {
      const nve_data_type_t required = quant_output_dtype(config_.value_dtype);
      NVE_B200_ARG(pool_params->output_type == required,
                   "Quantized GPU embedding output type must match the quantization metadata "
                   "precision");
      NVE_B200_ARG(output_stride == quant_value_count(config_) * dtype_size(required),
                   "Invalid dequantized output stride for quantized GPU embedding table");
      if (!concatenate && is_weighted(pool_params->pooling_type)) {
        NVE_B200_ARG(pool_params->weight_type == NVE_DTYPE_FLOAT32 ||
                         pool_params->weight_type == NVE_DTYPE_FLOAT16,
                     "Quantized GPU embedding weights must be Float32 or Float16");
      }
    } else {
      NVE_B200_ARG(output_stride == width_bytes,
                   "Output stride must be the same as embedding width");
      NVE_B200_ARG(pool_params->output_type == config_.value_dtype,
                   "GPU embedding layer requires pooled output type to match the table value type");
      if (!concatenate && pool_params->weights != nullptr) {
        NVE_B200_ARG(pool_params->weight_type == config_.value_dtype,
                     "GPU embedding layer requires weight type to match the table value type");
      }
    }
  } else {
    NVE_B200_ARG(output_stride == width_bytes, "Output stride must be the same as embedding width");
  }

  ExecutionContext& c = *ctx;
  const cudaStream_t stream = c.lookup_stream();
  const int kb = key_bytes(key_type_);
  const Staged d_keys =
      stage_in(c, "keys", keys, static_cast<size_t>(num_keys) * kb, true, stream);
  const int64_t out_rows = get_lookup_output_rows(num_keys, pool_params);
  const Staged d_out = stage_in(c, "output", output,
                                static_cast<size_t>(out_rows) * output_stride, false, stream);

  const bool pooled = pool_params && !concatenate;
  if (pooled) {
    nve_b200_pool_args_t a{};
    a.table = config_.embedding_table;
    a.num_rows = config_.num_embeddings;
    a.row_stride = width_bytes;
    a.value_dtype = config_.value_dtype;
    a.row_width = quantized ? quant_value_count(config_)
                            : width_bytes / dtype_size(config_.value_dtype);
    a.default_row_index = config_.default_row_index;
    a.cache = nullptr;
    a.key_type = key_type_;
    a.keys = d_keys.device;
    a.num_keys = num_keys;
    a.pooling_type = pool_params->pooling_type;
    a.sparse_type = pool_params->sparse_type;
    a.offset_bytes = kb;
    a.fixed_hotness = pool_params->fixed_hotness;
    a.num_bags = out_rows;
    Staged d_off, d_w;
    if (pool_params->sparse_type == NVE_SPARSE_CSR) {
      d_off = stage_in(c, "offsets", pool_params->csr_offsets,
                       static_cast<size_t>(pool_params->num_csr_offsets) * kb, true, stream);
      a.csr_offsets = d_off.device;
      // offsets the caller keeps in host memory are checked here, before anything is launched
      if (d_off.staged) validate_csr_offsets_host(pool_params->csr_offsets, kb, pool_params->num_csr_offsets, num_keys);
    }
    if (d_keys.staged && config_.default_row_index < 0 && host_key_checks_enabled()) {
      validate_keys_host(keys, kb, num_keys, config_.num_embeddings);
    }
    if (pool_params->weights != nullptr) {
      d_w = stage_in(c, "weights", pool_params->weights,
                     static_cast<size_t>(num_keys) * dtype_size(pool_params->weight_type), true,
                     stream);
      a.weights = d_w.device;
      a.weight_dtype = pool_params->weight_type;
    }
    a.output = d_out.device;
    a.output_stride = output_stride;
    a.output_dtype = pool_params->output_type;
    std::lock_guard<std::mutex> lock(launch_mutex_);
    NVE_B200_CUDA(cudaStreamWaitEvent(stream, modify_in_progress_, 0));
    lookup_pool(a, -1, stream);
  } else {
    nve_b200_gather_args_t g{};
    g.table = config_.embedding_table;
    g.num_rows = config_.num_embeddings;
    g.row_stride = width_bytes;
    g.value_dtype = config_.value_dtype;
    g.default_row_index = config_.default_row_index;
    g.key_type = key_type_;
    g.keys = d_keys.device;
    g.num_keys = num_keys;
    g.output = d_out.device;
    g.output_stride = output_stride;
    if (pool_params && !raw_concat) {  // quantised Concatenate with dequantisation
      g.output_dtype = pool_params->output_type;
      g.row_width = quant_value_count(config_);
    } else {                           // complete stored rows, metadata included
      g.output_dtype = config_.value_dtype;
      g.row_copy_bytes = width_bytes;
    }
    std::lock_guard<std::mutex> lock(launch_mutex_);
    NVE_B200_CUDA(cudaStreamWaitEvent(stream, modify_in_progress_, 0));
    gather_rows(g, -1, stream);
  }
  d_out.copy_back(stream);
  if (hitrates) hitrates[0] = 1.0f;
}

void GPUEmbeddingLayer::modify(context_ptr_t& ctx, int64_t num_keys, const void* keys,
                               int64_t value_stride, int64_t value_size, const void* values,
                               bool accumulate, nve_data_type_t value_type) {
  ScopedDevice sd(config_.device_id);
  NVE_B200_CHECK(num_keys >= 0, "Invalid num_keys");
  NVE_B200_CHECK(keys != nullptr, "Invalid keys buffer");
  NVE_B200_CHECK(values != nullptr, "Invalid values buffer");
  NVE_B200_CHECK(ctx != nullptr, "Invalid layer context");
  NVE_B200_CHECK(value_size == config_.embedding_width_in_bytes, "Invalid value size");
  if (accumulate) {
    NVE_B200_CHECK(!is_quant_rowwise(config_.value_dtype),
                   "Accumulate is not supported for quantized GPU embedding tables");
    if (value_type != NVE_DTYPE_FLOAT32 && value_type != NVE_DTYPE_FLOAT16) {
      throw InvalidArgument("Unsupported Data type");
    }
  }
  ExecutionContext& c = *ctx;
  const cudaStream_t modify_stream = c.modify_stream();
  // staging buffers of their own: a lookup of the same context may still be reading "keys"
  const Staged d_keys = stage_in(c, "modify_keys", keys,
                                 static_cast<size_t>(num_keys) * key_bytes(key_type_), true,
                                 modify_stream);
  const Staged d_vals = stage_in(c, "modify_values", values,
                                 static_cast<size_t>(num_keys) * value_stride, true, modify_stream);

  std::lock_guard<std::mutex> lock(launch_mutex_);
  // Order: earlier modify, the caller's modify stream, and every lookup already enqueued come
  // before this modify; later lookups wait for modify_in_progress_.
  cudaEvent_t staged;
  NVE_B200_CUDA(cudaEventCreateWithFlags(&staged, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(staged, modify_stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(private_modify_stream_, staged, 0);
  (void)cudaEventDestroy(staged);
  NVE_B200_CUDA(e);
  contexts_->order_after_lookups(private_modify_stream_);
  update_rows(config_.embedding_table, config_.num_embeddings, config_.embedding_width_in_bytes,
              accumulate ? value_type : config_.value_dtype, config_.embedding_width_in_bytes,
              key_type_, d_keys.device, num_keys, d_vals.device, value_stride, accumulate, false,
              private_modify_stream_);
  NVE_B200_CUDA(cudaEventRecord(modify_in_progress_, private_modify_stream_));
  NVE_B200_CUDA(cudaStreamWaitEvent(modify_stream, modify_in_progress_, 0));
}

void GPUEmbeddingLayer::update(context_ptr_t& ctx, int64_t num_keys, const void* keys,
                               int64_t value_stride, int64_t value_size, const void* values,
                               int64_t table_id) {
  NVE_B200_CHECK(table_id < get_num_tables(), "Invalid table_id");
  modify(ctx, num_keys, keys, value_stride, value_size, values, false, config_.value_dtype);
}

void GPUEmbeddingLayer::accumulate(context_ptr_t& ctx, int64_t num_keys, const void* keys,
                                   int64_t value_stride, int64_t value_size, const void* values,
                                   nve_data_type_t value_type, int64_t table_id) {
  NVE_B200_CHECK(table_id < get_num_tables(), "Invalid table_id");
  modify(ctx, num_keys, keys, value_stride, value_size, values, true, value_type);
}

}  // namespace nve_b200
