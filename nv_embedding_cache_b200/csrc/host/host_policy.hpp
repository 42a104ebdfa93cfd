// Host-side replacement policy of the GPU cache table (modify_on_gpu = 0).  Plain C++: no CUDA
// types, so that the policy can be compiled and tested without a device.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <type_traits>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../kernels/modify_entry.hpp"

namespace nve_b200 {

// The contract of the reference's CacheSAHostModify (include/ecache/ec_set_associative_host_modify.h
// :217-316 insert, :318-383 update / update_accumulate, :134-176 invalidate) fed by its host
// histogram (include/ecache/embed_cache.h:189-256): tags, replacement counters and per-set decay
// clocks are mirrored on the host; a modification walks the mirror on the calling thread, in batch
// order, and hands the device a list of (source row, cache line, tag) to apply.  The decisions are
// sequential by definition (a key sees the counters the keys before it left), which is what
// distinguishes this policy from the device one.
struct HostPolicy {
  std::vector<int64_t> tags;      // [sets * 8] tag (key / sets) or the sentinel
  std::vector<float> counters;    // [sets * 8]
  std::vector<int64_t> set_ts;    // [sets] insert number that last aged the set
  int64_t global_ts = 0;
  int64_t sentinel = -1;
  uint32_t sets = 0;

  void reset(size_t lines, uint32_t num_sets, int64_t sentinel_key) {
    sets = num_sets;
    sentinel = sentinel_key;
    tags.assign(lines, sentinel_key);
    counters.assign(lines, 0.f);
    set_ts.assign(num_sets, 0);
    global_ts = 0;
  }

  // Arithmetic in the key's own width, through its unsigned counterpart, as the device probe does.
  template <typename KeyT>
  struct Math {
    using U = typename std::make_unsigned<KeyT>::type;
    static uint32_t set_of(KeyT key, uint32_t sets) { return static_cast<uint32_t>(static_cast<U>(key) % sets); }
    static KeyT tag_of(KeyT key, uint32_t sets) { return static_cast<KeyT>(static_cast<U>(key) / sets); }
    static KeyT key_of(KeyT tag, uint32_t set, uint32_t sets) {
      return static_cast<KeyT>(static_cast<U>(static_cast<U>(tag) * sets + set));
    }
  };

  // Way of `set` whose stored tag spells `key`, lowest first, or -1.
  template <typename KeyT>
  int way_of(KeyT key, uint32_t set) const {
    const int64_t* ways = tags.data() + size_t(set) * 8;
    for (int j = 0; j < 8; j++) {
      if (Math<KeyT>::key_of(static_cast<KeyT>(ways[j]), set, sets) == key) return j;
    }
    return -1;
  }

  // Distinct keys of the batch in order of first appearance, sorted by falling count (std::sort on
  // the count alone, as the reference does: the order among equal counts is whatever that sort
  // leaves, and is the same here because it is the same call on the same sequence), priority =
  // count / batch size.  `first[i]` is the batch position of the key's first appearance.
  template <typename KeyT>
  struct Bin {
    KeyT key;
    float count;
    int64_t first;
  };
  template <typename KeyT>
  static std::vector<Bin<KeyT>> histogram(const KeyT* keys, int64_t n) {
    std::vector<Bin<KeyT>> bins;
    bins.reserve(size_t(n));
    std::unordered_map<KeyT, size_t> where;
    where.reserve(size_t(n));
    for (int64_t i = 0; i < n; i++) {
      auto it = where.find(keys[i]);
      if (it == where.end()) {
        where.emplace(keys[i], bins.size());
        bins.push_back({keys[i], 1.f, i});
      } else {
        bins[it->second].count += 1.f;
      }
    }
    std::sort(bins.begin(), bins.end(), [](const Bin<KeyT>& a, const Bin<KeyT>& b) { return a.count > b.count; });
    return bins;
  }

  // Replacement decisions of one insert.  A resident key has its counter raised by its priority; a
  // key that is not resident takes the way with the smallest counter unless that counter exceeds
  // the key's priority or the way was already given away in this call; at most `max_entries` lines
  // change per call.  A set's counters are aged by decay^(inserts since it was last touched) when
  // the call first touches it.
  template <typename KeyT>
  void select_inserts(const std::vector<Bin<KeyT>>& bins, int64_t batch, float decay, int64_t max_entries,
                      const uint8_t* src_base, int64_t src_stride, bool src_by_key,
                      std::vector<ModifyEntry>& out) {
    const int64_t now = ++global_ts;
    std::unordered_set<uint64_t> taken;
    out.clear();
    for (size_t b = 0; b < bins.size() && int64_t(taken.size()) < max_entries; b++) {
      const KeyT key = bins[b].key;
      const float priority = bins[b].count / static_cast<float>(batch);
      const uint32_t set = Math<KeyT>::set_of(key, sets);
      float* sc = counters.data() + size_t(set) * 8;
      if (set_ts[set] != now) {
        const float factor = static_cast<float>(
            std::pow(static_cast<double>(decay), static_cast<double>(now - set_ts[set])));
        for (int j = 0; j < 8; j++) sc[j] *= factor;
        set_ts[set] = now;
      }
      const int hit = way_of<KeyT>(key, set);
      if (hit >= 0) {
        sc[hit] += priority;
        continue;
      }
      float* victim = std::min_element(sc, sc + 8);
      if (*victim > priority) continue;
      const uint64_t line = uint64_t(set) * 8 + uint64_t(victim - sc);
      if (!taken.insert(line).second) continue;
      *victim = priority;
      const KeyT tag = Math<KeyT>::tag_of(key, sets);
      tags[line] = static_cast<int64_t>(tag);
      const int64_t row = src_by_key ? static_cast<int64_t>(key) : bins[b].first;
      out.push_back({src_base + row * src_stride, line, static_cast<int64_t>(tag)});
    }
  }

  // One entry per key that is resident (its first matching way), at most `max_entries`.
  template <typename KeyT>
  void find_resident(const KeyT* keys, int64_t n, const uint8_t* values, int64_t stride, int64_t max_entries,
                     std::vector<ModifyEntry>& out) const {
    out.clear();
    for (int64_t i = 0; i < n && int64_t(out.size()) < max_entries; i++) {
      const uint32_t set = Math<KeyT>::set_of(keys[i], sets);
      const int way = way_of<KeyT>(keys[i], set);
      if (way < 0) continue;
      const uint64_t line = uint64_t(set) * 8 + uint64_t(way);
      out.push_back({values + i * stride, line, tags[line]});
    }
  }

  // Every way that holds one of the keys is emptied.
  template <typename KeyT>
  void invalidate(const KeyT* keys, int64_t n, std::vector<ModifyEntry>& out) {
    out.clear();
    for (int64_t i = 0; i < n; i++) {
      const uint32_t set = Math<KeyT>::set_of(keys[i], sets);
      int64_t* ways = tags.data() + size_t(set) * 8;
      for (int j = 0; j < 8; j++) {
        if (Math<KeyT>::key_of(static_cast<KeyT>(ways[j]), set, sets) == keys[i]) {
          ways[j] = sentinel;
          out.push_back({nullptr, uint64_t(set) * 8 + uint64_t(j), sentinel});
        }
      }
    }
  }
};

}  // namespace nve_b200
