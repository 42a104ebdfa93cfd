/*
 * TEST INFRASTRUCTURE — the parity checker, never the product path.
 *
 * Plain-C, single-threaded restatement of the reference algorithms on the embedding-lookup hot
 * path.  Every function cites the reference file:line it follows (paths relative to the reference
 * tree).  Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load this
 * library; the CUDA product never calls it.
 *
 * Parity pin: tests/test_oracle_pin.py checks these functions bit-for-bit against the
 * unmodified reference CPU build (oracle/_ref/libnve_ref.so, see oracle/build.py) and against the
 * committed golden vectors in tests/golden/.
 *
 * Arithmetic rules (built with -ffp-contract=off): fp32 accumulation in key order, one rounding
 * per multiply and per add, 1.f/denom then multiply for Mean, round-to-nearest-even to fp16.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define NVE_EXPORT __attribute__((visibility("default")))

/* dtype ids follow include/nve_c_api.h:70-89 */
enum {
  DT_UNKNOWN = 0, DT_F32 = 1, DT_BF16 = 2, DT_F16 = 3, DT_E4M3 = 4, DT_E5M2 = 5, DT_F64 = 6,
  DT_QI8_F32 = 7, DT_QI8_F16 = 8, DT_QU8_F32 = 9, DT_QU8_F16 = 10
};
/* pooling ids follow include/nve_c_api.h:96-102, sparse ids :91-94 */
enum { POOL_CONCAT = 0, POOL_SUM = 1, POOL_MEAN = 2, POOL_WSUM = 3, POOL_WMEAN = 4 };
enum { SPARSE_FIXED = 0, SPARSE_CSR = 1 };

typedef _Float16 f16;

static inline float h2f(const void* p) { f16 h; memcpy(&h, p, 2); return (float)h; }
static inline void f2h(void* p, float v) { f16 h = (f16)v; memcpy(p, &h, 2); }

static inline int is_quant(int dt) { return dt >= DT_QI8_F32 && dt <= DT_QU8_F16; }
/* include/nve_types.hpp:150-189: metadata = scale [+ offset], precision from the F32/F16 suffix */
static inline int quant_scale_bytes(int dt) { return (dt == DT_QI8_F32 || dt == DT_QU8_F32) ? 4 : 2; }
static inline int quant_has_offset(int dt) { return dt == DT_QU8_F32 || dt == DT_QU8_F16; }
static inline int elem_bytes(int dt) {
  switch (dt) { case DT_F32: return 4; case DT_F16: return 2; case DT_F64: return 8;
                case DT_BF16: return 2; default: return 1; }
}

/* include/key_utils.hpp:33-41 */
static inline int key_in_range(int64_t key, int64_t num_rows) {
  return key >= 0 && (uint64_t)key < (uint64_t)num_rows;
}

static inline int64_t load_index(const void* p, int idx_bytes, int64_t i) {
  if (idx_bytes == 4) { int32_t v; memcpy(&v, (const char*)p + 4 * i, 4); return v; }
  int64_t v; memcpy(&v, (const char*)p + 8 * i, 8); return v;
}

static inline float load_meta(const uint8_t* p, int scale_bytes) {
  if (scale_bytes == 4) { float v; memcpy(&v, p, 4); return v; }
  return h2f(p);
}

/* One stored element of a row as fp32: cpu_ops/cpu_pooling.hpp:120-131 (float/half rows) and
 * :225-246 (quantized rows: float(q)*scale + offset, metadata right after the values). */
static inline float row_elem(const uint8_t* row, int dt, int64_t e, float scale, float offset) {
  switch (dt) {
    case DT_F32: { float v; memcpy(&v, row + 4 * e, 4); return v; }
    case DT_F16: return h2f(row + 2 * e);
    case DT_QI8_F32: case DT_QI8_F16: return (float)((const int8_t*)row)[e] * scale + offset;
    default: return (float)row[e] * scale + offset;
  }
}

static inline void store_out(uint8_t* out, int dt, int64_t e, float v) {
  if (dt == DT_F32) memcpy(out + 4 * e, &v, 4); else f2h(out + 2 * e, v);
}

/* sanitize_keys_kernel, cuda_ops/sanitize_keys.cuh:31-45: a key outside [0,num_rows) becomes
 * default_row when default_row >= 0; otherwise keys are trusted. */
static inline int64_t sanitize(int64_t key, int64_t num_rows, int64_t default_row) {
  if (default_row >= 0 && !key_in_range(key, num_rows)) return default_row;
  return key;
}

/*
 * Un-pooled gather: out[i] = table[key[i]] for in-range keys, other slots untouched; returns the
 * number of rows written and ORs bit i (of word i/64) into hit_mask when given.  Keys whose bit
 * is already set are skipped.  cpu_ops/cpu_gather.hpp:28-80.
 */
NVE_EXPORT int64_t nve_oracle_gather(const void* table, int64_t num_rows, int64_t row_bytes,
                                     const void* keys, int key_bytes, int64_t n, void* out,
                                     int64_t out_stride, uint64_t* hit_mask) {
  int64_t hits = 0;
  for (int64_t i = 0; i < n; i++) {
    if (hit_mask && ((hit_mask[i / 64] >> (i % 64)) & 1)) continue;
    const int64_t key = load_index(keys, key_bytes, i);
    if (!key_in_range(key, num_rows)) continue;
    memcpy((char*)out + i * out_stride, (const char*)table + key * row_bytes, (size_t)row_bytes);
    hits++;
    if (hit_mask) hit_mask[i / 64] |= (uint64_t)1 << (i % 64);
  }
  return hits;
}

/*
 * Fused lookup + pooling over a dense table: the composition the reference host layer runs as
 * gather (cpu_ops/cpu_gather.hpp:28-80) followed by cpu_kernel_pooling / cpu_kernel_pooling_quant
 * (cpu_ops/cpu_pooling.hpp:68-150, :166-259) or cpu_kernel_concatenate[_quant] (:274-348), with
 * the dense-layer key sanitising of cuda_ops/sanitize_keys.cuh:31-45 in front.
 *
 *   row_bytes   stored bytes per row (values + quantisation metadata + padding)
 *   row_width   number of values per row
 *   offsets     CSR offsets (num_bags + 1 entries of off_bytes each) or NULL for Fixed
 * Returns 0, or 1 on an unsupported dtype combination.
 */
NVE_EXPORT int nve_oracle_lookup_pooled(const void* table, int64_t num_rows, int64_t row_bytes,
                                        int value_dtype, int64_t row_width, int64_t default_row,
                                        const void* keys, int key_bytes, int64_t num_keys,
                                        int pooling_type, int sparse_type, const void* offsets,
                                        int off_bytes, int64_t num_bags, int64_t fixed_hotness,
                                        const void* weights, int weight_dtype, void* output,
                                        int64_t output_stride, int output_dtype) {
  if (output_dtype != DT_F32 && output_dtype != DT_F16) return 1;
  if (value_dtype != DT_F32 && value_dtype != DT_F16 && !is_quant(value_dtype)) return 1;
  const int q = is_quant(value_dtype);
  const int sb = q ? quant_scale_bytes(value_dtype) : 0;
  const int has_off = q ? quant_has_offset(value_dtype) : 0;
  const uint8_t* tab = (const uint8_t*)table;

  if (pooling_type == POOL_CONCAT) {
    for (int64_t k = 0; k < num_keys; k++) {
      const int64_t key = sanitize(load_index(keys, key_bytes, k), num_rows, default_row);
      const uint8_t* row = tab + key * row_bytes;
      uint8_t* out = (uint8_t*)output + k * output_stride;
      const float scale = q ? load_meta(row + row_width, sb) : 1.f;
      const float offset = has_off ? load_meta(row + row_width + sb, sb) : 0.f;
      for (int64_t e = 0; e < row_width; e++)
        store_out(out, output_dtype, e, row_elem(row, value_dtype, e, scale, offset));
    }
    return 0;
  }

  const int weighted = pooling_type == POOL_WSUM || pooling_type == POOL_WMEAN;
  const int mean = pooling_type == POOL_MEAN || pooling_type == POOL_WMEAN;
  if (weighted && weight_dtype != DT_F32 && weight_dtype != DT_F16) return 1;
  float* acc = (float*)malloc(sizeof(float) * (size_t)(row_width > 0 ? row_width : 1));
  for (int64_t bag = 0; bag < num_bags; bag++) {
    int64_t start, end;
    if (sparse_type == SPARSE_FIXED) { start = bag * fixed_hotness; end = start + fixed_hotness; }
    else { start = load_index(offsets, off_bytes, bag); end = load_index(offsets, off_bytes, bag + 1); }
    const int64_t count = end - start;
    uint8_t* out = (uint8_t*)output + bag * output_stride;
    if (count <= 0) {
      memset(out, 0, (size_t)(row_width * elem_bytes(output_dtype)));
      continue;
    }
    for (int64_t e = 0; e < row_width; e++) acc[e] = 0.f;
    float weight_sum = 0.f;
    for (int64_t k = start; k < end; k++) {
      const int64_t key = sanitize(load_index(keys, key_bytes, k), num_rows, default_row);
      const uint8_t* row = tab + key * row_bytes;
      const float scale = q ? load_meta(row + row_width, sb) : 1.f;
      const float offset = has_off ? load_meta(row + row_width + sb, sb) : 0.f;
      float w = 1.f;
      if (weighted) {
        if (weight_dtype == DT_F32) memcpy(&w, (const char*)weights + 4 * k, 4);
        else w = h2f((const char*)weights + 2 * k);
      }
      weight_sum += w;
      for (int64_t e = 0; e < row_width; e++) {
        float v = row_elem(row, value_dtype, e, scale, offset);
        if (weighted) v *= w;
        acc[e] += v;
      }
    }
    float inv = 1.f;
    if (mean) {
      const float denom = weighted ? weight_sum : (float)count;
      inv = (denom != 0.f) ? 1.f / denom : 0.f;
    }
    for (int64_t e = 0; e < row_width; e++) store_out(out, output_dtype, e, acc[e] * inv);
  }
  free(acc);
  return 0;
}

/* table[key] = values[i] for in-range keys, in key order (a later duplicate wins).
 * cpu_ops/cpu_update.hpp:27-58; GPU twin cuda_ops/update_accumulate.cuh:27-59. */
NVE_EXPORT void nve_oracle_update(void* table, int64_t num_rows, int64_t row_bytes,
                                  const void* keys, int key_bytes, int64_t n, const void* values,
                                  int64_t value_stride) {
  for (int64_t i = 0; i < n; i++) {
    const int64_t key = load_index(keys, key_bytes, i);
    if (!key_in_range(key, num_rows)) continue;
    memcpy((char*)table + key * row_bytes, (const char*)values + i * value_stride, (size_t)row_bytes);
  }
}

/* table[key][:] += updates[i][:] for in-range keys, in key order.  fp32: cpu_ops/cpu_update.hpp:
 * 66-103.  fp16 follows the device kernel (one half-precision add per element,
 * cuda_ops/update_accumulate.cuh:61-91). */
NVE_EXPORT int nve_oracle_update_accumulate(void* table, int64_t num_rows, int64_t row_bytes,
                                            int value_dtype, const void* keys, int key_bytes,
                                            int64_t n, const void* updates, int64_t update_stride) {
  if (value_dtype != DT_F32 && value_dtype != DT_F16) return 1;
  const int64_t width = row_bytes / elem_bytes(value_dtype);
  for (int64_t i = 0; i < n; i++) {
    const int64_t key = load_index(keys, key_bytes, i);
    if (!key_in_range(key, num_rows)) continue;
    char* dst = (char*)table + key * row_bytes;
    const char* src = (const char*)updates + i * update_stride;
    for (int64_t j = 0; j < width; j++) {
      if (value_dtype == DT_F32) {
        float a, b; memcpy(&a, dst + 4 * j, 4); memcpy(&b, src + 4 * j, 4);
        a = a + b; memcpy(dst + 4 * j, &a, 4);
      } else {
        f16 a, b; memcpy(&a, dst + 2 * j, 2); memcpy(&b, src + 2 * j, 2);
        a = (f16)((double)a + (double)b); memcpy(dst + 2 * j, &a, 2);
      }
    }
  }
  return 0;
}

/* ---- Deduper ------------------------------------------------------------------------------- */
typedef struct { int64_t key; int64_t pos; } KeyPos;
static int cmp_key_pos(const void* a, const void* b) {
  const KeyPos* x = (const KeyPos*)a; const KeyPos* y = (const KeyPos*)b;
  if (x->key != y->key) return x->key < y->key ? -1 : 1;
  return x->pos < y->pos ? -1 : (x->pos > y->pos);
}

/*
 * cuda_ops/deduper.cuh:136-221: stable sort of (key, position) by the low `end_bit` bits of the
 * key (signed order when all bits take part, as the device radix sort orders signed keys), then
 * run-length encoding of the full keys in that order (so keys that differ above end_bit stay
 * separate runs; callers pass an end_bit that covers their key range).  Outputs (all int64 here): unique ascending, counts, inverse = positions
 * grouped by key with ascending position inside a group, offsets = chunk starts (+ total), loc_map
 * = group of each chunk, where a group is split into chunks of at most max_run positions when
 * max_run > 0 (:39-81).  num_runs[0] = groups, num_runs[1] = chunks.
 */
NVE_EXPORT void nve_oracle_dedup(const void* keys, int key_bytes, int64_t n, int64_t max_run,
                                 int end_bit, int64_t* unique, int64_t* counts, int64_t* inverse,
                                 int64_t* offsets, int64_t* loc_map, int64_t* num_runs) {
  num_runs[0] = num_runs[1] = 0;
  if (n <= 0) { offsets[0] = 0; return; }
  const int full = end_bit <= 0 || end_bit >= key_bytes * 8;
  KeyPos* kp = (KeyPos*)malloc(sizeof(KeyPos) * (size_t)n);
  int64_t* orig = (int64_t*)malloc(sizeof(int64_t) * (size_t)n);
  for (int64_t i = 0; i < n; i++) {
    const int64_t k = load_index(keys, key_bytes, i);
    orig[i] = k;
    kp[i].key = full ? k : (int64_t)((uint64_t)k & (((uint64_t)1 << end_bit) - 1));
    kp[i].pos = i;
  }
  qsort(kp, (size_t)n, sizeof(KeyPos), cmp_key_pos);
  int64_t groups = 0, chunks = 0;
  for (int64_t i = 0; i < n;) {
    int64_t j = i;   /* runs are runs of equal FULL keys in the (partially) sorted order */
    while (j < n && orig[kp[j].pos] == orig[kp[i].pos]) j++;
    unique[groups] = orig[kp[i].pos];
    counts[groups] = j - i;
    if (max_run > 0) {
      for (int64_t b = i; b < j; b += max_run) { offsets[chunks] = b; loc_map[chunks] = groups; chunks++; }
    } else {
      offsets[chunks++] = i;
    }
    groups++;
    i = j;
  }
  offsets[chunks] = n;
  for (int64_t i = 0; i < n; i++) inverse[i] = kp[i].pos;
  num_runs[0] = groups; num_runs[1] = chunks;
  free(orig); free(kp);
}

/*
 * Per-group gradient sum (cuda_ops/dedup_grads_kernel.cuh:56-109): every chunk is summed in fp32
 * in position order; the chunk sums of a group are added in chunk order (the device reference
 * adds them with float atomics, i.e. in no fixed order; any order is within its tolerance).
 * dst[group] = sum, fp32 rows of `width` values.
 */
NVE_EXPORT void nve_oracle_dedup_grads(const float* grads, int64_t grad_stride_elems, int64_t width,
                                       const int64_t* inverse, const int64_t* offsets,
                                       const int64_t* loc_map, int64_t num_chunks, float* dst,
                                       int64_t dst_stride_elems) {
  float* part = (float*)malloc(sizeof(float) * (size_t)width);
  for (int64_t c = 0; c < num_chunks;) {
    const int64_t g = loc_map ? loc_map[c] : c;
    int64_t ce = c;
    while (ce < num_chunks && (loc_map ? loc_map[ce] : ce) == g) ce++;
    float* out = dst + g * dst_stride_elems;
    const int single = (ce - c) == 1;
    for (int64_t e = 0; e < width; e++) out[e] = 0.f;
    for (int64_t k = c; k < ce; k++) {
      for (int64_t e = 0; e < width; e++) part[e] = 0.f;
      for (int64_t i = offsets[k]; i < offsets[k + 1]; i++) {
        const float* row = grads + inverse[i] * grad_stride_elems;
        for (int64_t e = 0; e < width; e++) part[e] = part[e] + row[e];
      }
      if (single) { for (int64_t e = 0; e < width; e++) out[e] = part[e]; }
      else { for (int64_t e = 0; e < width; e++) out[e] = out[e] + part[e]; }
    }
    c = ce;
  }
  free(part);
}
