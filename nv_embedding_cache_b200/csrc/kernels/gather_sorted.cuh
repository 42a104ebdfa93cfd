// Sort-gather schedule of the un-pooled raw-row lookup: resolve every key first, order the work so
// that all rows read from the backing table (host link when the table sits in host memory) are
// issued before the rows served by the cache, each class in coarse address order, then copy.
//
//   resolve_words_kernel   phase 1 of lookup_rows_kernel (hit mask, miss counter, miss list) and one
//                          64-bit word per key:  [class:2][source index:idx_bits][position:pos_bits]
//                          class 0 = backing table row, 1 = cache slot, 3 = no source
//   CUB radix sort         keys only, over the class bits and the top 14 index bits of the words
//   copy_sorted_kernel     a warp walks a tile of sorted words, 32 at a time, and copies the rows
//
// Against the reference's arrangement (a 16-byte {source, destination} pair per key sorted as the
// value of an 8-byte key: 48 bytes of scratch per key and a pair sort) the schedule here sorts one
// 8-byte word per key and rebuilds both addresses from it.
//
// Same results as lookup_rows_kernel; only raw copies (no decode) take this schedule.
// Bytes per key on top of the fused kernel: 8 B written + 8 B x 2 per sort pass (two passes) + 8 B read.
#pragma once

#include "../common.hpp"
#include "lookup_rows.cuh"

namespace nve_b200 {

struct SortedGatherLayout {
  int pos_bits;   // bits of a position in the batch
  int idx_bits;   // bits of a table row index / cache slot index
};

// False when class, index and position do not fit one 64-bit word (the caller keeps the fused kernel).
bool gather_sorted_layout(const GatherKernelParams& p, SortedGatherLayout* layout);

// Scratch for n keys: two word arrays and the sort's temporary storage.
size_t gather_sorted_scratch_bytes(int64_t n);

// The two halves of the schedule, for callers that split the copy (the host-assisted pipeline form):
// resolve + sort returns the sorted words (inside `scratch`); `table_rows`, when given, is a zeroed
// device counter that receives the number of words served by the backing table, which sort first.
const uint64_t* launch_resolve_and_sort(const GatherKernelParams& p, const SortedGatherLayout& layout,
                                        void* scratch, size_t scratch_bytes, unsigned long long* table_rows,
                                        cudaStream_t stream);
// Copies the rows of `count` sorted words.  With `staged` set, word i of the range reads the row
// staged + i * staged_stride (rows a host thread gathered in sorted order) instead of its source.
void launch_copy_sorted(const GatherKernelParams& p, const SortedGatherLayout& layout, int vb, int64_t tile,
                        const uint64_t* sorted, int64_t count, const uint8_t* staged, int64_t staged_stride,
                        int sm_count, cudaStream_t stream);

// Index field of a sorted word (table row or cache slot).
inline uint64_t sorted_word_index(uint64_t word, const SortedGatherLayout& layout) {
  return (word >> layout.pos_bits) & ((uint64_t{1} << layout.idx_bits) - 1);
}

// tile: upper bound of the sorted words one warp copies (the reference's tile size); the launch
// lowers it until the grid fills the GPU.
void launch_gather_sorted(const GatherKernelParams& p, const SortedGatherLayout& layout, int vb,
                          int64_t tile, void* scratch, size_t scratch_bytes, int sm_count,
                          cudaStream_t stream);

}  // namespace nve_b200
