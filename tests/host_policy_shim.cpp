// Test-only C entry points over the host-side replacement policy of the cache table
// (csrc/host/host_policy.hpp), so that the policy can be driven from Python without a GPU.
#include <cstdint>
#include <cstring>
#include <vector>

#include "host/host_policy.hpp"

using nve_b200::HostPolicy;
using nve_b200::ModifyEntry;

extern "C" {

void* hp_create(uint32_t sets, int64_t sentinel) {
  auto* p = new HostPolicy();
  p->reset(static_cast<size_t>(sets) * 8, sets, sentinel);
  return p;
}
void hp_destroy(void* h) { delete static_cast<HostPolicy*>(h); }

// Histogram order of a batch: distinct keys by falling count (ties as the sort leaves them), with
// counts and first positions.  Returns the number of distinct keys.
int64_t hp_histogram(const int64_t* keys, int64_t n, int64_t* out_keys, float* out_counts, int64_t* out_first) {
  const auto bins = HostPolicy::histogram<int64_t>(keys, n);
  for (size_t i = 0; i < bins.size(); i++) {
    out_keys[i] = bins[i].key;
    out_counts[i] = bins[i].count;
    out_first[i] = bins[i].first;
  }
  return static_cast<int64_t>(bins.size());
}

// One insert; entries come back as (line, tag, source row index).  Returns their number.
int64_t hp_insert(void* h, const int64_t* keys, int64_t n, float decay, int64_t max_entries, uint64_t* lines,
                  int64_t* tags, int64_t* rows) {
  auto* p = static_cast<HostPolicy*>(h);
  const auto bins = HostPolicy::histogram<int64_t>(keys, n);
  std::vector<ModifyEntry> list;
  p->select_inserts<int64_t>(bins, n, decay, max_entries, nullptr, 1, /*src_by_key=*/false, list);
  for (size_t i = 0; i < list.size(); i++) {
    lines[i] = list[i].line;
    tags[i] = list[i].tag;
    rows[i] = reinterpret_cast<int64_t>(list[i].src);    // base NULL, stride 1: the row index itself
  }
  return static_cast<int64_t>(list.size());
}

int64_t hp_find_resident(void* h, const int64_t* keys, int64_t n, int64_t max_entries, uint64_t* lines, int64_t* rows) {
  auto* p = static_cast<HostPolicy*>(h);
  std::vector<ModifyEntry> list;
  p->find_resident<int64_t>(keys, n, nullptr, 1, max_entries, list);
  for (size_t i = 0; i < list.size(); i++) {
    lines[i] = list[i].line;
    rows[i] = reinterpret_cast<int64_t>(list[i].src);
  }
  return static_cast<int64_t>(list.size());
}

int64_t hp_invalidate(void* h, const int64_t* keys, int64_t n, uint64_t* lines) {
  auto* p = static_cast<HostPolicy*>(h);
  std::vector<ModifyEntry> list;
  p->invalidate<int64_t>(keys, n, list);
  for (size_t i = 0; i < list.size(); i++) lines[i] = list[i].line;
  return static_cast<int64_t>(list.size());
}

void hp_state(void* h, int64_t* tags, float* counters, int64_t* set_ts) {
  auto* p = static_cast<HostPolicy*>(h);
  std::memcpy(tags, p->tags.data(), p->tags.size() * sizeof(int64_t));
  std::memcpy(counters, p->counters.data(), p->counters.size() * sizeof(float));
  std::memcpy(set_ts, p->set_ts.data(), p->set_ts.size() * sizeof(int64_t));
}

}  // extern "C"
