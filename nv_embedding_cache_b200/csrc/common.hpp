// Shared host-side plumbing of libnve_b200: error types that map onto nve_status_t, the
// thread-local last-error slot, CUDA call checking and small dtype helpers.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <sstream>
#include <stdexcept>
#include <string>

#include "nve_b200_ops.h"

#include <nvtx3/nvToolsExt.h>

namespace nve_b200 {

// Exceptions carry the status the C boundary reports.  The mapping follows the reference's
// NVE_C_CATCH (src/nve_c_api_internal.hpp:48-92): bad argument -> 1, CUDA failure -> 2 (5 when
// the allocation failed), not implemented -> 4, anything else -> 3.
class Error : public std::runtime_error {
 public:
  Error(nve_status_t status, const std::string& msg) : std::runtime_error(msg), status_(status) {}
  nve_status_t status() const { return status_; }

 private:
  nve_status_t status_;
};

struct InvalidArgument : Error {
  explicit InvalidArgument(const std::string& m) : Error(NVE_ERROR_INVALID_ARGUMENT, m) {}
};
struct NotImplemented : Error {
  explicit NotImplemented(const std::string& m) : Error(NVE_ERROR_NOT_IMPLEMENTED, m) {}
};
struct RuntimeFailure : Error {
  explicit RuntimeFailure(const std::string& m) : Error(NVE_ERROR_RUNTIME, m) {}
};
struct CudaFailure : Error {
  CudaFailure(cudaError_t e, const std::string& what)
      : Error(e == cudaErrorMemoryAllocation ? NVE_ERROR_OUT_OF_MEMORY : NVE_ERROR_CUDA,
              what + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")") {}
};

nve_status_t set_last_error(nve_status_t status, const std::string& message);

// Named range around an entry point for timeline profilers (the reference marks its entry points
// the same way, include/cuda_support.hpp:26-55).  Header-only NVTX: without a profiler attached a
// push or pop is a call through a null-checked pointer.
struct ScopedRange {
  explicit ScopedRange(const char* name) { nvtxRangePushA(name); }
  ~ScopedRange() { nvtxRangePop(); }
  ScopedRange(const ScopedRange&) = delete;
  ScopedRange& operator=(const ScopedRange&) = delete;
};
#define NVE_B200_RANGE() ::nve_b200::ScopedRange nve_b200_range_(__func__)

template <typename... Args>
std::string cat(Args&&... args) {
  std::ostringstream os;
  (os << ... << args);
  return os.str();
}

#define NVE_B200_CUDA(expr)                                                     \
  do {                                                                          \
    cudaError_t nve_b200_err_ = (expr);                                         \
    if (nve_b200_err_ != cudaSuccess) {                                         \
      (void)cudaGetLastError();                                                 \
      throw ::nve_b200::CudaFailure(nve_b200_err_, #expr);                      \
    }                                                                           \
  } while (0)

#define NVE_B200_ARG(cond, ...)                                                 \
  do {                                                                          \
    if (!(cond)) throw ::nve_b200::InvalidArgument(::nve_b200::cat(__VA_ARGS__)); \
  } while (0)

#define NVE_B200_CHECK(cond, ...)                                               \
  do {                                                                          \
    if (!(cond)) throw ::nve_b200::RuntimeFailure(::nve_b200::cat(__VA_ARGS__)); \
  } while (0)

// Runs `fn`, turning exceptions into a status + thread-local message.
template <typename Fn>
nve_status_t guarded(Fn&& fn) {
  try {
    fn();
    return NVE_SUCCESS;
  } catch (const Error& e) {
    return set_last_error(e.status(), e.what());
  } catch (const std::bad_alloc&) {
    return set_last_error(NVE_ERROR_OUT_OF_MEMORY, "Out of memory");
  } catch (const std::invalid_argument& e) {
    return set_last_error(NVE_ERROR_INVALID_ARGUMENT, e.what());
  } catch (const std::exception& e) {
    return set_last_error(NVE_ERROR_RUNTIME, e.what());
  } catch (...) {
    return set_last_error(NVE_ERROR_RUNTIME, "Unknown error");
  }
}

// ---- value types (ids of nve_data_type_t; semantics of reference include/nve_types.hpp:128-189)
inline bool is_quant_rowwise(nve_data_type_t t) {
  return t >= NVE_DTYPE_QINT8_ROWWISE_F32 && t <= NVE_DTYPE_QUINT8_ROWWISE_F16;
}
inline int64_t dtype_size(nve_data_type_t t) {
  switch (t) {
    case NVE_DTYPE_FLOAT32: return 4;
    case NVE_DTYPE_BFLOAT16:
    case NVE_DTYPE_FLOAT16: return 2;
    case NVE_DTYPE_FLOAT64: return 8;
    case NVE_DTYPE_UNKNOWN: return 1;
    default: return 1;
  }
}
inline nve_data_type_t quant_output_dtype(nve_data_type_t t) {
  return (t == NVE_DTYPE_QINT8_ROWWISE_F32 || t == NVE_DTYPE_QUINT8_ROWWISE_F32)
             ? NVE_DTYPE_FLOAT32
             : NVE_DTYPE_FLOAT16;
}
inline int64_t quant_meta_count(nve_data_type_t t) {
  return (t == NVE_DTYPE_QINT8_ROWWISE_F32 || t == NVE_DTYPE_QINT8_ROWWISE_F16) ? 1 : 2;
}
inline int64_t quant_meta_bytes(nve_data_type_t t) {
  return quant_meta_count(t) * dtype_size(quant_output_dtype(t));
}
inline bool is_weighted(nve_pooling_type_t p) {
  return p == NVE_POOL_WEIGHTED_SUM || p == NVE_POOL_WEIGHTED_MEAN;
}
inline int key_bytes(nve_key_type_t k) { return k == NVE_KEY_INT32 ? 4 : 8; }

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Number of SMs of the current device (cached per device).
int sm_count();

}  // namespace nve_b200
