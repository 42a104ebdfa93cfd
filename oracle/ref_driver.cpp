// TEST INFRASTRUCTURE — not part of the product path.
//
// Thin C-ABI driver around the UNMODIFIED reference CPU implementation
// (HostEmbeddingLayer + LinearHostTable + cpu_ops), compiled from the reference
// sources where they lie (never copied into this repository) by oracle/build.py
// into oracle/_ref/libnve_ref.so.  It exists for two jobs only:
//   1. pin the plain-C restatement in oracle/nve_oracle.c against the real reference, and
//   2. serve as the timed CPU baseline ("kind": "reference") in bench.py.
// Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load it.
//
// Reference entry points exercised here (paths relative to the reference tree):
//   src/host_embedding_layer.cpp:55-247   HostEmbeddingLayer<K>::lookup
//   include/linear_host_table.hpp:76-107  LinearHostTable<K>::find -> cpu_kernel_gather
//   src/layer_utils.cpp:330-515           pool_gathered_host -> cpu_kernel_pooling[_quant]
//   cpu_ops/cpu_pooling.hpp:581-641       cpu_kernel_pooling_dispatch<OffsetT>
//   cpu_ops/cpu_update.hpp:27-130         cpu_kernel_update / cpu_kernel_update_accumulate

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>

#include "include/host_embedding_layer.hpp"
#include "include/linear_host_table.hpp"
#include "include/nve_types.hpp"
#include "include/thread_pool.hpp"
#include "cpu_ops/cpu_pooling.hpp"

namespace {

thread_local std::string g_err;

nve::DataType_t to_dtype(int id) {
  switch (id) {
    case 1: return nve::DataType_t::Float32;
    case 3: return nve::DataType_t::Float16;
    case 7: return nve::DataType_t::QInt8RowwiseF32;
    case 8: return nve::DataType_t::QInt8RowwiseF16;
    case 9: return nve::DataType_t::QUint8RowwiseF32;
    case 10: return nve::DataType_t::QUint8RowwiseF16;
    default: return nve::DataType_t::Unknown;
  }
}

nve::PoolingType_t to_pool(int id) {
  switch (id) {
    case 1: return nve::PoolingType_t::Sum;
    case 2: return nve::PoolingType_t::Mean;
    case 3: return nve::PoolingType_t::WeightedSum;
    case 4: return nve::PoolingType_t::WeightedMean;
    default: return nve::PoolingType_t::Concatenate;
  }
}

struct RefLayer {
  std::shared_ptr<nve::LinearHostTable<int64_t>> table;
  std::shared_ptr<nve::HostEmbeddingLayer<int64_t>> layer;
  nve::context_ptr_t ctx;
};

template <typename F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown exception";
    return 1;
  }
}

}  // namespace

extern "C" {

const char* nve_ref_last_error() { return g_err.c_str(); }

// Worker count of the reference's default thread pool (max(hardware_concurrency - 2, 1),
// src/thread_pool.cpp:112-116) as seen through a freshly created context.
int64_t nve_ref_num_workers(void* handle) {
  auto* h = static_cast<RefLayer*>(handle);
  return h->ctx->get_thread_pool()->num_workers();
}

void* nve_ref_host_layer_create(void* emb_table, int64_t num_rows, int64_t row_bytes,
                                int value_dtype) {
  RefLayer* h = nullptr;
  const int rc = guarded([&] {
    nve::LinearHostTableConfig cfg;
    cfg.value_dtype = to_dtype(value_dtype);
    cfg.max_value_size = row_bytes;
    cfg.num_rows = num_rows;
    cfg.emb_table = emb_table;
    auto holder = std::make_unique<RefLayer>();
    holder->table = std::make_shared<nve::LinearHostTable<int64_t>>(cfg);
    nve::HostEmbeddingLayer<int64_t>::Config lcfg;
    lcfg.layer_name = "ref_host_layer";
    holder->layer = std::make_shared<nve::HostEmbeddingLayer<int64_t>>(lcfg, holder->table);
    holder->ctx = holder->layer->create_execution_context(0, 0, nullptr, nullptr);
    h = holder.release();
  });
  return rc == 0 ? h : nullptr;
}

void nve_ref_host_layer_destroy(void* handle) {
  auto* h = static_cast<RefLayer*>(handle);
  if (h) {
    h->ctx.reset();
    h->layer.reset();
    h->table.reset();
    delete h;
  }
}

// pooled == 0: plain lookup (pool_params == nullptr).  Offsets are int64 (the layer key type).
int nve_ref_host_layer_lookup(void* handle, int64_t num_keys, const int64_t* keys, void* output,
                              int64_t output_stride, int pooled, int pooling_type,
                              int sparse_type, const int64_t* csr_offsets,
                              int64_t num_csr_offsets, int64_t fixed_hotness,
                              const void* weights, int weight_type, int output_type,
                              float* hitrate) {
  auto* h = static_cast<RefLayer*>(handle);
  return guarded([&] {
    nve::EmbeddingLayerBase::PoolingParams pp;
    if (pooled) {
      pp.pooling_type = to_pool(pooling_type);
      pp.output_type = to_dtype(output_type);
      pp.sparse_type = sparse_type == 1 ? nve::SparseType_t::CSR : nve::SparseType_t::Fixed;
      pp.csr_offsets = csr_offsets;
      pp.num_csr_offsets = num_csr_offsets;
      pp.fixed_hotness = fixed_hotness;
      pp.weights = weights;
      pp.weight_type = to_dtype(weight_type);
    }
    h->layer->lookup(h->ctx, num_keys, keys, output, output_stride, nullptr,
                     pooled ? &pp : nullptr, hitrate);
    h->ctx->wait();
  });
}

int nve_ref_host_layer_update(void* handle, int64_t num_keys, const int64_t* keys,
                              int64_t value_stride, int64_t value_size, const void* values) {
  auto* h = static_cast<RefLayer*>(handle);
  return guarded([&] {
    h->layer->update(h->ctx, num_keys, keys, value_stride, value_size, values, 0);
    h->ctx->wait();
  });
}

int nve_ref_host_layer_accumulate(void* handle, int64_t num_keys, const int64_t* keys,
                                  int64_t value_stride, int64_t value_size, const void* values,
                                  int value_type) {
  auto* h = static_cast<RefLayer*>(handle);
  return guarded([&] {
    h->layer->accumulate(h->ctx, num_keys, keys, value_stride, value_size, values,
                         to_dtype(value_type), 0);
    h->ctx->wait();
  });
}

// Pooling of already gathered rows with int32 CSR offsets: the reference's CPU templates take the
// offset type independently of the key type (cpu_ops/cpu_pooling.hpp:581-641).
int nve_ref_pool_gathered_i32(void* handle, int value_dtype, int output_type, int weight_type,
                              int64_t num_bags, int64_t row_width, const int8_t* input,
                              int64_t input_stride, int8_t* output, int64_t output_stride,
                              int sparse_type, int64_t fixed_hotness, const int32_t* offsets,
                              int pooling_type, const void* weights) {
  auto* h = static_cast<RefLayer*>(handle);
  return guarded([&] {
    auto tp = h->ctx->get_thread_pool();
    nve::cpu_kernel_pooling_dispatch<int32_t>(
        tp, num_bags, row_width, input, input_stride, output, output_stride,
        sparse_type == 1 ? nve::SparseType_t::CSR : nve::SparseType_t::Fixed, fixed_hotness,
        offsets, to_pool(pooling_type), weights, to_dtype(weight_type), to_dtype(value_dtype),
        to_dtype(output_type), tp->num_workers());
  });
}

}  // extern "C"
