// Stable radix sort of 64-bit words over a bit range (see radix_sort.cu).
#pragma once

#include "../common.hpp"

namespace nve_b200 {

// What the first pass reads.  kWords: the `in` array of words.  kPacked: word i =
// ((uint32)key[i] ^ flip) << 32 | i, made on the fly from the caller's keys.  kWide (pairs sort): word i
// = key[i] ^ flip with payload i.
struct RadixSource {
  enum Form : int { kWords = 0, kPacked = 1, kWide = 2 };
  const void* keys = nullptr;
  bool key64 = true;
  uint64_t flip = 0;
  int form = kWords;
};

// Largest batch the sort takes (one thread walks a histogram row of n / 8192 entries per digit).
int64_t radix_sort_max_entries();
// Bytes of `scratch` (tile histograms) for n entries; 16-byte aligned memory.
size_t radix_sort_scratch_bytes(int64_t n);
// out = the source's words ordered by their bits [begin_bit, end_bit), ascending, equal words in
// input order.  `tmp` holds n words and is used by the passes before the last; `in` (kWords only)
// is not modified.  in, out and tmp are three different buffers.
void radix_sort_u64(const RadixSource& source, const uint64_t* in, uint64_t* out, uint64_t* tmp, int64_t n,
                    int begin_bit, int end_bit, void* scratch, cudaStream_t stream);
// The same with a 32-bit payload per word (vin -> vout, vtmp beside tmp).
void radix_sort_pairs_u64(const RadixSource& source, const uint64_t* in, uint64_t* out, uint64_t* tmp,
                          const uint32_t* vin, uint32_t* vout, uint32_t* vtmp, int64_t n, int begin_bit,
                          int end_bit, void* scratch, cudaStream_t stream);

}  // namespace nve_b200
