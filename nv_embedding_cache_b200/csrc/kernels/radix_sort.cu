// Stable least-significant-digit radix sort of 64-bit words over a bit range, eight bits per pass.
//
// Written for the de-duplication of lookup batches (around a million packed (key bits, position)
// words whose order on the key bits decides the unique keys, and whose stability keeps the positions
// of equal keys ascending).  A pass is two launches and no kernel waits on another block:
//
//   count    one block of 1024 threads per tile of 8192 words: digit histogram in shared memory
//            (per-warp bins, filled through warp votes: no atomics) -> hist[digit][tile]
//   scatter  one block per tile.  Thread d (d < 256) first walks row d of hist: the words of digit d
//            in the tiles before this one, and in all tiles; a block scan over the 256 digit totals
//            then gives where this tile's words of every digit start -- the prefix sum a separate
//            one-block kernel took 10 us for, done by every tile for itself in about a microsecond.
//            Then the tile's words in 8 rounds of 1024: a word's place is the tile's start for its
//            digit + the words of that digit earlier in the tile.  "Earlier" is kept exact, hence
//            stable: lanes with the same digit find each other with eight ballots (one per digit bit;
//            the hardware's match instruction takes a step per distinct value, about thirty for a
//            warp of random digits) and rank by lane, warps publish their digit counts, and thread d
//            turns the 32 warp counts of digit d into warp offsets and advances the running count.
//
// The first pass can read the caller's keys instead of prepared words (`RadixSource`): the packing
// of (key bits, position) then costs no pass of its own.
//
// Bytes per pass: 8 read for the count, 8 read + 8 written for the scatter per word; a million words
// stay in L2.  Bound: launch latency and the block barriers of the scatter, not memory.
#include "radix_sort.cuh"

#include <algorithm>

namespace nve_b200 {

namespace {

constexpr int kRadixBits = 8;
constexpr int kDigits = 1 << kRadixBits;          // 256
constexpr int kThreads = 1024;                    // block size of count and scatter
constexpr int kRounds = 8;
constexpr int kTile = kThreads * kRounds;         // 8192 words per tile
constexpr int kWarps = kThreads / 32;

// Lanes of the warp whose `digit` equals this lane's, among the lanes in `live`.  Whole warp calls.
__device__ __forceinline__ uint32_t lanes_with_same_digit(uint32_t digit, uint32_t live) {
  uint32_t same = live;
#pragma unroll
  for (int b = 0; b < 8; b++) {
    const bool bit = (digit >> b) & 1u;
    const uint32_t vote = __ballot_sync(0xffffffffu, bit);
    same &= bit ? vote : ~vote;
  }
  return same;
}

// Word of entry i of the first pass.
__device__ __forceinline__ uint64_t source_word(const RadixSource& src, const uint64_t* in, int64_t i) {
  if (src.form == RadixSource::kWords) return in[i];
  const int64_t key = src.key64 ? static_cast<const int64_t*>(src.keys)[i]
                                : static_cast<int64_t>(static_cast<const int32_t*>(src.keys)[i]);
  if (src.form == RadixSource::kPacked) {
    return (static_cast<uint64_t>(static_cast<uint32_t>(key) ^ static_cast<uint32_t>(src.flip)) << 32) |
           static_cast<uint32_t>(i);
  }
  return static_cast<uint64_t>(key) ^ src.flip;     // kWide: the payload is the position
}

// `mask` keeps a pass's digit inside the bit range when its width is not a multiple of eight.
__global__ void __launch_bounds__(kThreads) radix_count_kernel(const RadixSource src, const uint64_t* __restrict__ in,
                                                                int64_t n, int shift, uint32_t mask,
                                                                uint32_t row_stride, uint32_t* __restrict__ hist) {
  __shared__ uint16_t bins[kWarps][kDigits];       // a warp sees at most 32 * kRounds words of a digit
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  for (int j = t; j < kWarps * kDigits; j += kThreads) (&bins[0][0])[j] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  uint64_t words[kRounds];
#pragma unroll
  for (int r = 0; r < kRounds; r++) {
    const int64_t i = base + r * kThreads + t;
    words[r] = i < n ? source_word(src, in, i) : 0;
  }
#pragma unroll
  for (int r = 0; r < kRounds; r++) {
    const bool live = base + r * kThreads + t < n;
    const uint32_t livemask = __ballot_sync(0xffffffffu, live);
    const uint32_t digit = static_cast<uint32_t>(words[r] >> shift) & mask;
    const uint32_t same = lanes_with_same_digit(digit, livemask);
    if (live && (same & ((1u << lane) - 1u)) == 0) bins[warp][digit] += static_cast<uint16_t>(__popc(same));
    __syncwarp();
  }
  __syncthreads();
  if (t < kDigits) {
    uint32_t total = 0;
#pragma unroll 8
    for (int w = 0; w < kWarps; w++) total += bins[w][t];
    hist[static_cast<size_t>(t) * row_stride + blockIdx.x] = total;
  }
}

// PAIRS: every word carries a 32-bit payload that moves with it.
template <bool PAIRS>
__global__ void __launch_bounds__(kThreads) radix_scatter_kernel(const RadixSource src, const uint64_t* __restrict__ in,
                                                                  uint64_t* __restrict__ out,
                                                                  const uint32_t* __restrict__ vin,
                                                                  uint32_t* __restrict__ vout, int64_t n, int shift,
                                                                  uint32_t mask, uint32_t num_tiles,
                                                                  uint32_t row_stride,
                                                                  const uint32_t* __restrict__ hist) {
  __shared__ uint32_t place[kDigits];              // where the tile's next word of digit d goes
  __shared__ uint32_t warp_sum[kDigits / 32];
  __shared__ uint8_t warp_count[kWarps][kDigits];  // at most 32 per warp and round
  __shared__ uint32_t warp_place[kWarps][kDigits];
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kTile;
  // the whole tile is fetched first: the loads are in flight while the histogram rows are walked,
  // and a round is then shared-memory work only
  uint64_t words[kRounds];
  uint32_t payload[PAIRS ? kRounds : 1];
#pragma unroll
  for (int r = 0; r < kRounds; r++) {
    const int64_t i = base + r * kThreads + t;
    words[r] = i < n ? source_word(src, in, i) : 0;
    if constexpr (PAIRS) {
      payload[r] = i < n ? (src.form == RadixSource::kWide ? static_cast<uint32_t>(i) : vin[i]) : 0;
    }
  }
  for (int j = t; j < kWarps * kDigits; j += kThreads) (&warp_count[0][0])[j] = 0;
  // where this tile's words of every digit start: (all words of smaller digits) + (words of the digit
  // in earlier tiles)
  uint32_t before = 0, total = 0;
  if (t < kDigits) {
    const uint4* row4 = reinterpret_cast<const uint4*>(hist + static_cast<size_t>(t) * row_stride);
    const uint32_t tile = blockIdx.x;
    for (uint32_t q = 0; q * 4 < num_tiles; q++) {
      const uint4 v = row4[q];                      // row_stride is a multiple of 4; the padding is zero
      const uint32_t j = q * 4;
      total += v.x + v.y + v.z + v.w;
      before += (j < tile ? v.x : 0u) + (j + 1 < tile ? v.y : 0u) + (j + 2 < tile ? v.z : 0u) +
                (j + 3 < tile ? v.w : 0u);
    }
    uint32_t incl = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (lane == 31) warp_sum[warp] = incl;
    before += incl - total;                         // + smaller digits held by the same warp
  }
  __syncthreads();
  if (t < kDigits) {
    uint32_t lower = 0;
    for (int w = 0; w < warp; w++) lower += warp_sum[w];
    place[t] = before + lower;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < kRounds; r++) {
    const int64_t i = base + r * kThreads + t;
    const bool live = i < n;
    const uint64_t word = words[r];
    // lanes past the end take no part: only a tile's last rounds have any, and always at the top
    const uint32_t livemask = __ballot_sync(0xffffffffu, live);
    const uint32_t digit = static_cast<uint32_t>(word >> shift) & mask;
    const uint32_t same = lanes_with_same_digit(digit, livemask);
    const uint32_t rank = __popc(same & ((1u << lane) - 1u));
    if (live && rank == 0) warp_count[warp][digit] = static_cast<uint8_t>(__popc(same));
    __syncthreads();
    if (t < kDigits) {
      // thread d: the warps' counts of digit d -> their offsets; counts cleared for the next round
      uint32_t run = place[t];
#pragma unroll 8
      for (int w = 0; w < kWarps; w++) {
        const uint32_t c = warp_count[w][t];
        warp_place[w][t] = run;
        warp_count[w][t] = 0;
        run += c;
      }
      place[t] = run;
    }
    __syncthreads();
    if (live) {
      const uint32_t at = warp_place[warp][digit] + rank;
      out[at] = word;
      if constexpr (PAIRS) vout[at] = payload[r];
    }
  }
}

uint32_t hist_row_stride(int64_t tiles) { return static_cast<uint32_t>((tiles + 3) / 4 * 4); }

template <bool PAIRS>
void radix_sort_run(const RadixSource& source, const uint64_t* in, uint64_t* out, uint64_t* tmp,
                    const uint32_t* vin, uint32_t* vout, uint32_t* vtmp, int64_t n, int begin_bit, int end_bit,
                    void* scratch, cudaStream_t stream) {
  NVE_B200_ARG(n >= 0 && n <= radix_sort_max_entries(), "radix sort: batch size out of range");
  NVE_B200_ARG(begin_bit >= 0 && end_bit <= 64 && begin_bit < end_bit, "radix sort: bad bit range");
  if (n == 0) return;
  const int passes = (end_bit - begin_bit + kRadixBits - 1) / kRadixBits;
  const uint32_t tiles = static_cast<uint32_t>((n + kTile - 1) / kTile);
  const uint32_t stride = hist_row_stride(tiles);
  uint32_t* hist = static_cast<uint32_t*>(scratch);
  // rows are padded to a multiple of four entries; the padding must read as zero
  NVE_B200_CUDA(cudaMemsetAsync(hist, 0, static_cast<size_t>(stride) * kDigits * sizeof(uint32_t), stream));
  const uint64_t* src = in;
  const uint32_t* vsrc = vin;
  RadixSource from = source;
  for (int p = 0; p < passes; p++) {
    // the last pass writes `out`; the ones before alternate so that no pass reads what it writes
    const bool to_out = (passes - 1 - p) % 2 == 0;
    uint64_t* dst = to_out ? out : tmp;
    uint32_t* vdst = to_out ? vout : vtmp;
    const int shift = begin_bit + p * kRadixBits;
    const int width = std::min(kRadixBits, end_bit - shift);
    const uint32_t mask = (1u << width) - 1u;
    radix_count_kernel<<<tiles, kThreads, 0, stream>>>(from, src, n, shift, mask, stride, hist);
    radix_scatter_kernel<PAIRS><<<tiles, kThreads, 0, stream>>>(from, src, dst, vsrc, vdst, n, shift, mask, tiles,
                                                                stride, hist);
    src = dst;
    vsrc = vdst;
    from = RadixSource{};          // later passes read the words the pass before wrote
  }
  NVE_B200_CUDA(cudaGetLastError());
}

}  // namespace

int64_t radix_sort_max_entries() { return int64_t{1} << 24; }

size_t radix_sort_scratch_bytes(int64_t n) {
  const int64_t tiles = std::max<int64_t>(1, (n + kTile - 1) / kTile);
  return static_cast<size_t>(hist_row_stride(tiles)) * kDigits * sizeof(uint32_t) + 256;
}

void radix_sort_u64(const RadixSource& source, const uint64_t* in, uint64_t* out, uint64_t* tmp, int64_t n,
                    int begin_bit, int end_bit, void* scratch, cudaStream_t stream) {
  radix_sort_run<false>(source, in, out, tmp, nullptr, nullptr, nullptr, n, begin_bit, end_bit, scratch, stream);
}

void radix_sort_pairs_u64(const RadixSource& source, const uint64_t* in, uint64_t* out, uint64_t* tmp,
                          const uint32_t* vin, uint32_t* vout, uint32_t* vtmp, int64_t n, int begin_bit,
                          int end_bit, void* scratch, cudaStream_t stream) {
  radix_sort_run<true>(source, in, out, tmp, vin, vout, vtmp, n, begin_bit, end_bit, scratch, stream);
}

}  // namespace nve_b200
