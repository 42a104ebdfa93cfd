/*
 * TEST INFRASTRUCTURE — the parity checker, never the product path.
 *
 * Plain-C restatement of the reference's set-associative embedding cache ("ecache") with the
 * DEVICE-side modify policy: probe, hit-mask / miss-list / backed lookups, the insert replacement
 * policy (histogram -> per-set top-8 selection against lazily decayed counters), update,
 * update_accumulate, invalidate, clear.  Citations are reference file:line.
 *
 * One deliberate difference, stated in the header of the CUDA side too: the lazy decay factor is
 * decay_rate^delta computed by repeated squaring in fp32 (a fixed sequence of IEEE multiplies,
 * reproducible on any machine) instead of the reference's fast-math __powf, whose low bits are
 * not specified.  With decay_rate == 1, 0.5 or any power of two the two agree exactly.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define NVE_EXPORT __attribute__((visibility("default")))
#define WAYS 8 /* include/ecache/ec_set_associative.h:753 */

typedef struct {
  uint64_t num_sets;
  int key_bytes;         /* 4 or 8: tags are stored as the key type */
  int64_t row_bytes;
  float decay_rate;      /* include/ecache/ec_set_associative.h:120 (0.95 default) */
  int64_t sentinel;      /* empty-way tag, the table's invalid key (-1 default) */
  int64_t* tags;         /* [num_sets][8], sign-extended key-type values */
  float* counters;       /* [num_sets][8] */
  int64_t* set_ts;       /* [num_sets] */
  int64_t global_ts;
  uint8_t* data;         /* [num_sets][8][row_bytes] */
  int64_t misses;        /* miss counter of the (single) lookup context */
} Cache;

static inline uint64_t align16(uint64_t x) { return (x + 15u) & ~(uint64_t)15u; }

/* Unsigned view of a key of the cache's key width (include/ecache/ec_hash.h:36-40). */
static inline uint64_t ukey(const Cache* c, int64_t key) {
  return c->key_bytes == 4 ? (uint64_t)(uint32_t)(int32_t)key : (uint64_t)key;
}
static inline int64_t as_key(const Cache* c, uint64_t u) {
  return c->key_bytes == 4 ? (int64_t)(int32_t)(uint32_t)u : (int64_t)u;
}
/* include/ecache/ec_hash.h:36-60 */
static inline uint32_t set_of(const Cache* c, int64_t key) { return (uint32_t)(ukey(c, key) % c->num_sets); }
static inline int64_t tag_of(const Cache* c, int64_t key) { return as_key(c, ukey(c, key) / c->num_sets); }
static inline int64_t key_of(const Cache* c, int64_t tag, uint32_t set) {
  return as_key(c, ukey(c, tag) * c->num_sets + set);
}

/* Sets that fit: cache_bytes / (align16(8 tags) + align16(8 rows) + align16(8 counters)),
 * include/ecache/ec_set_associative.h:666-685 with the device-modify counter term of
 * include/ecache/ec_set_associative_device_modify.cuh:472-474. */
NVE_EXPORT uint64_t nve_oracle_cache_num_sets(uint64_t cache_bytes, int64_t row_bytes, int key_bytes) {
  const uint64_t per_set = align16((uint64_t)WAYS * key_bytes) + align16((uint64_t)WAYS * row_bytes) +
                           align16((uint64_t)WAYS * sizeof(float));
  return cache_bytes / per_set;
}

NVE_EXPORT void* nve_oracle_cache_create(uint64_t cache_bytes, int64_t row_bytes, int key_bytes,
                                         float decay_rate, int64_t sentinel) {
  Cache* c = (Cache*)calloc(1, sizeof(Cache));
  c->num_sets = nve_oracle_cache_num_sets(cache_bytes, row_bytes, key_bytes);
  if (c->num_sets == 0) { free(c); return NULL; }
  c->key_bytes = key_bytes;
  c->row_bytes = row_bytes;
  c->decay_rate = decay_rate;
  c->sentinel = sentinel;
  c->tags = (int64_t*)malloc(sizeof(int64_t) * c->num_sets * WAYS);
  c->counters = (float*)calloc(c->num_sets * WAYS, sizeof(float));
  c->set_ts = (int64_t*)calloc(c->num_sets, sizeof(int64_t));
  c->data = (uint8_t*)calloc(c->num_sets * WAYS, (size_t)row_bytes);
  for (uint64_t i = 0; i < c->num_sets * WAYS; i++) c->tags[i] = sentinel;
  return c;
}

NVE_EXPORT void nve_oracle_cache_destroy(void* h) {
  Cache* c = (Cache*)h;
  if (!c) return;
  free(c->tags); free(c->counters); free(c->set_ts); free(c->data); free(c);
}

NVE_EXPORT uint64_t nve_oracle_cache_sets(void* h) { return ((Cache*)h)->num_sets; }
NVE_EXPORT void nve_oracle_cache_get_tags(void* h, int64_t* out) {
  Cache* c = (Cache*)h;
  memcpy(out, c->tags, sizeof(int64_t) * c->num_sets * WAYS);
}
NVE_EXPORT void nve_oracle_cache_get_counters(void* h, float* out) {
  Cache* c = (Cache*)h;
  memcpy(out, c->counters, sizeof(float) * c->num_sets * WAYS);
}
NVE_EXPORT void nve_oracle_cache_get_data(void* h, uint8_t* out) {
  Cache* c = (Cache*)h;
  memcpy(out, c->data, (size_t)c->row_bytes * c->num_sets * WAYS);
}
NVE_EXPORT int64_t nve_oracle_cache_misses(void* h) { return ((Cache*)h)->misses; }
NVE_EXPORT void nve_oracle_cache_reset_misses(void* h) { ((Cache*)h)->misses = 0; }

/* First way whose reconstructed key equals `key`, else -1
 * (include/ecache/ec_set_associative.cuh:46-80: way mask then __ffs). */
static int probe(const Cache* c, int64_t key, uint32_t* set_out) {
  const uint32_t set = set_of(c, key);
  *set_out = set;
  for (int w = 0; w < WAYS; w++) {
    if (key_of(c, c->tags[(uint64_t)set * WAYS + w], set) == key) return w;
  }
  return -1;
}

static inline int64_t load_key(const void* keys, int kb, int64_t i) {
  if (kb == 4) { int32_t v; memcpy(&v, (const char*)keys + 4 * i, 4); return v; }
  int64_t v; memcpy(&v, (const char*)keys + 8 * i, 8); return v;
}

/*
 * Lookup.  For every key whose hit-mask bit is clear: a cache hit copies the cached row; a miss
 * bumps the miss counter and, when `table` is given, copies table[key] (keys outside
 * [0,table_rows) are redirected to default_row when it is >= 0, else left unresolved).
 *   - backed lookup: include/ecache/embed_cache.cuh:51-90 (query_uvm)
 *   - hit-mask lookup: include/ecache/ec_set_associative.cuh:388-466
 *   - miss list (position, key) in key order: include/ecache/ec_set_associative.cuh:263-326
 * Returns the number of unresolved keys.
 */
NVE_EXPORT int64_t nve_oracle_cache_lookup(void* h, const void* keys, int64_t n, void* out,
                                           int64_t out_stride, uint64_t* hit_mask,
                                           const void* table, int64_t table_rows,
                                           int64_t default_row, int64_t* miss_pos,
                                           int64_t* miss_keys) {
  Cache* c = (Cache*)h;
  int64_t unresolved = 0;
  for (int64_t i = 0; i < n; i++) {
    if (hit_mask && ((hit_mask[i / 64] >> (i % 64)) & 1)) continue;
    const int64_t key = load_key(keys, c->key_bytes, i);
    uint32_t set;
    const int way = probe(c, key, &set);
    const uint8_t* src = NULL;
    if (way >= 0) {
      src = c->data + ((uint64_t)set * WAYS + way) * c->row_bytes;
    } else {
      c->misses++;
      if (table) {
        int64_t k = key;
        const int in_range = k >= 0 && k < table_rows;
        if (!in_range && default_row >= 0) k = default_row;
        if (in_range || default_row >= 0) src = (const uint8_t*)table + k * c->row_bytes;
      }
    }
    if (src) {
      if (out) memcpy((char*)out + i * out_stride, src, (size_t)c->row_bytes);
      if (hit_mask) hit_mask[i / 64] |= (uint64_t)1 << (i % 64);
    } else {
      if (miss_pos) miss_pos[unresolved] = i;
      if (miss_keys) miss_keys[unresolved] = key;
      unresolved++;
    }
  }
  return unresolved;
}

/* ---- insert ------------------------------------------------------------------------------- */

typedef struct { int64_t key; int64_t idx; } KeyIdx;
static int cmp_key_idx(const void* a, const void* b) {
  const KeyIdx* x = (const KeyIdx*)a; const KeyIdx* y = (const KeyIdx*)b;
  if (x->key != y->key) return x->key < y->key ? -1 : 1;
  return x->idx < y->idx ? -1 : (x->idx > y->idx);
}
typedef struct { int64_t key; int64_t first; int32_t count; int64_t order; } Bin;
static int cmp_bin(const void* a, const void* b) {  /* count descending, stable */
  const Bin* x = (const Bin*)a; const Bin* y = (const Bin*)b;
  if (x->count != y->count) return x->count > y->count ? -1 : 1;
  return x->order < y->order ? -1 : (x->order > y->order);
}
typedef struct { uint32_t set; int64_t loc; } SetLoc;
static int cmp_set_loc(const void* a, const void* b) {
  const SetLoc* x = (const SetLoc*)a; const SetLoc* y = (const SetLoc*)b;
  if (x->set != y->set) return x->set < y->set ? -1 : 1;
  return x->loc < y->loc ? -1 : (x->loc > y->loc);
}

/* The 8-lane bitonic network of the reference (include/ecache/ec_set_associative_modify.cuh:
 * 36-70): result in descending order of `v`; equal values never swap. */
static void sort_block(float* v, uint32_t* pos) {
  for (uint32_t k = 2; k <= WAYS; k *= 2) {
    for (uint32_t j = k / 2; j > 0; j /= 2) {
      float nv[WAYS]; uint32_t np[WAYS];
      for (uint32_t i = 0; i < WAYS; i++) {
        const uint32_t pr = i ^ j;
        nv[i] = v[i]; np[i] = pos[i];
        if (v[i] != v[pr]) {
          const int in_order_pos = i > pr;
          const int in_order_val = v[i] > v[pr];
          const int ascending = (i & k) != 0;
          if (ascending ? (in_order_pos != in_order_val) : (in_order_pos == in_order_val)) {
            nv[i] = v[pr]; np[i] = pos[pr];
          }
        }
      }
      memcpy(v, nv, sizeof(nv)); memcpy(pos, np, sizeof(np));
    }
  }
}

/* Merge of two descending blocks keeping the best 8 (same file :72-103).  Note: this step has no
 * equality guard, so among equal priorities a lane may take its partner's entry while the
 * partner keeps it too — an entry can be duplicated and another dropped.  Kept as is: it decides
 * which keys become resident when more than 8 new keys of equal priority hit one set. */
static void merge_block(float* p1, uint32_t* pos1, const float* p2, const uint32_t* pos2) {
  for (uint32_t i = 0; i < WAYS; i++) {
    const float rp = p2[WAYS - 1 - i];
    const float rpos = (float)pos2[WAYS - 1 - i];   /* the reference routes it through a float */
    if (rp > p1[i]) { p1[i] = rp; pos1[i] = (uint32_t)rpos; }
  }
  for (uint32_t j = WAYS / 2; j > 0; j /= 2) {
    float nv[WAYS]; uint32_t np[WAYS];
    for (uint32_t i = 0; i < WAYS; i++) {
      const uint32_t pr = i ^ j;
      const int in_order_pos = i < pr;
      const int in_order_p = p1[i] > p1[pr];
      nv[i] = p1[i]; np[i] = pos1[i];
      if (in_order_pos != in_order_p) { nv[i] = p1[pr]; np[i] = pos1[pr]; }
    }
    memcpy(p1, nv, sizeof(nv)); memcpy(pos1, np, sizeof(np));
  }
}

static float pow_by_squaring(float base, int64_t e) {
  float r = 1.f, b = base;
  while (e > 0) {
    if (e & 1) r = r * b;
    b = b * b;
    e >>= 1;
  }
  return r;
}

/*
 * Insert a raw batch of keys (duplicates allowed) with their rows.
 *   histogram: unique keys ordered by occurrence count descending, ties by key ascending;
 *     priority = count * (1/n); source row = row of the key's first occurrence
 *     (cuda_ops/gather_keys_data_ptrs.cuh:27-57, :121-191), or table[key] when from_table != 0
 *     (src/gpu_table.cu:494-560 insert_from_uvm); at most max_modify keys are kept
 *     (src/gpu_table.cu:452).
 *   per touched set, candidates in that order (include/ecache/ec_set_associative_modify.cuh:
 *     138-310): lazily decay the 8 counters, bump counters of candidates already resident, select
 *     the best min(8, #candidates) new candidates, pair the t-th best with the t-th smallest
 *     counter (empty ways count 0) and replace where priority > counter.
 * Returns the number of replacements made.
 */
NVE_EXPORT int64_t nve_oracle_cache_insert(void* h, const void* keys, int64_t n,
                                           const void* values, int64_t value_stride,
                                           int from_table, int64_t max_modify) {
  Cache* c = (Cache*)h;
  if (n <= 0) return 0;
  KeyIdx* ki = (KeyIdx*)malloc(sizeof(KeyIdx) * (size_t)n);
  for (int64_t i = 0; i < n; i++) { ki[i].key = load_key(keys, c->key_bytes, i); ki[i].idx = i; }
  qsort(ki, (size_t)n, sizeof(KeyIdx), cmp_key_idx);
  Bin* bins = (Bin*)malloc(sizeof(Bin) * (size_t)n);
  int64_t nb = 0;
  for (int64_t i = 0; i < n;) {
    int64_t j = i;
    while (j < n && ki[j].key == ki[i].key) j++;
    bins[nb].key = ki[i].key; bins[nb].first = ki[i].idx; bins[nb].count = (int32_t)(j - i);
    bins[nb].order = nb; nb++;
    i = j;
  }
  qsort(bins, (size_t)nb, sizeof(Bin), cmp_bin);
  const float norm = 1.0f / (float)n;
  int64_t m = nb < max_modify ? nb : max_modify;

  SetLoc* sl = (SetLoc*)malloc(sizeof(SetLoc) * (size_t)m);
  float* prio = (float*)malloc(sizeof(float) * (size_t)m);
  for (int64_t i = 0; i < m; i++) {
    sl[i].set = set_of(c, bins[i].key); sl[i].loc = i;
    prio[i] = (float)bins[i].count * norm;
  }
  qsort(sl, (size_t)m, sizeof(SetLoc), cmp_set_loc);

  c->global_ts++;
  int64_t replaced = 0;
  for (int64_t g = 0; g < m;) {
    int64_t ge = g;
    while (ge < m && sl[ge].set == sl[g].set) ge++;
    const uint32_t set = sl[g].set;
    const uint32_t count = (uint32_t)(ge - g);
    int64_t* tags = c->tags + (uint64_t)set * WAYS;
    float* ctr = c->counters + (uint64_t)set * WAYS;

    const int64_t delta = c->global_ts - c->set_ts[set];
    if (delta > 0 && c->decay_rate != 1.0f) {
      const float f = pow_by_squaring(c->decay_rate, delta);
      for (int w = 0; w < WAYS; w++) ctr[w] = ctr[w] * f;
    }
    c->set_ts[set] = c->global_ts;

    float best[WAYS]; uint32_t best_pos[WAYS];
    for (uint32_t processed = 0; processed < count || processed == 0; processed += WAYS) {
      float p[WAYS]; uint32_t pos[WAYS];
      for (uint32_t t = 0; t < WAYS; t++) {
        p[t] = 0.f; pos[t] = 0;
        if (processed + t < count) {
          const int64_t loc = sl[g + processed + t].loc;
          int hit = 0;
          for (int w = 0; w < WAYS; w++) {
            if (key_of(c, tags[w], set) == bins[loc].key) { ctr[w] += prio[loc]; hit = 1; }
          }
          if (!hit) { pos[t] = (uint32_t)loc; p[t] = prio[loc]; }
        }
      }
      sort_block(p, pos);
      if (processed == 0) { memcpy(best, p, sizeof(p)); memcpy(best_pos, pos, sizeof(pos)); }
      else merge_block(best, best_pos, p, pos);
    }

    float cv[WAYS]; uint32_t cw[WAYS];
    for (uint32_t w = 0; w < WAYS; w++) { cv[w] = tags[w] == c->sentinel ? 0.f : ctr[w]; cw[w] = w; }
    sort_block(cv, cw);                       /* descending ... */
    const uint32_t num_repl = count < WAYS ? count : WAYS;
    int64_t new_tag[WAYS]; int do_write[WAYS]; uint32_t dst_way[WAYS];
    for (uint32_t t = 0; t < WAYS; t++) {     /* ... read in reverse: t-th smallest counter */
      const float counter = cv[WAYS - 1 - t];
      dst_way[t] = cw[WAYS - 1 - t];
      do_write[t] = (t < num_repl) && (best[t] > counter);
      new_tag[t] = tag_of(c, bins[best_pos[t]].key);
    }
    for (uint32_t t = 0; t < WAYS; t++) {
      if (!do_write[t]) continue;
      const int64_t loc = best_pos[t];
      const uint8_t* src = from_table
          ? (const uint8_t*)values + bins[loc].key * value_stride
          : (const uint8_t*)values + bins[loc].first * value_stride;
      memcpy(c->data + ((uint64_t)set * WAYS + dst_way[t]) * c->row_bytes, src, (size_t)c->row_bytes);
      tags[dst_way[t]] = new_tag[t];
      ctr[dst_way[t]] = best[t];
      replaced++;
    }
    g = ge;
  }
  free(prio); free(sl); free(bins); free(ki);
  return replaced;
}

/* Overwrite the cached rows of resident keys (unique keys); others ignored.
 * include/ecache/ec_set_associative_modify.cuh:515-566 + mem_update_kernel. */
NVE_EXPORT void nve_oracle_cache_update(void* h, const void* keys, int64_t n, const void* values,
                                        int64_t value_stride) {
  Cache* c = (Cache*)h;
  for (int64_t i = 0; i < n; i++) {
    const int64_t key = load_key(keys, c->key_bytes, i);
    const uint32_t set = set_of(c, key);
    for (int w = 0; w < WAYS; w++) {
      if (key_of(c, c->tags[(uint64_t)set * WAYS + w], set) == key) {
        memcpy(c->data + ((uint64_t)set * WAYS + w) * c->row_bytes,
               (const char*)values + i * value_stride, (size_t)c->row_bytes);
      }
    }
  }
}

/* cached row += update for resident keys (fp32 rows, or fp16 rows with one fp16 add each).
 * include/ecache/ec_set_associative.cuh:166-184, :328-385. */
NVE_EXPORT void nve_oracle_cache_update_accumulate(void* h, const void* keys, int64_t n,
                                                   const void* updates, int64_t update_stride,
                                                   int is_f16) {
  Cache* c = (Cache*)h;
  for (int64_t i = 0; i < n; i++) {
    const int64_t key = load_key(keys, c->key_bytes, i);
    const uint32_t set = set_of(c, key);
    for (int w = 0; w < WAYS; w++) {
      if (key_of(c, c->tags[(uint64_t)set * WAYS + w], set) != key) continue;
      uint8_t* dst = c->data + ((uint64_t)set * WAYS + w) * c->row_bytes;
      const char* src = (const char*)updates + i * update_stride;
      if (is_f16) {
        for (int64_t j = 0; j < c->row_bytes / 2; j++) {
          _Float16 a, b; memcpy(&a, dst + 2 * j, 2); memcpy(&b, src + 2 * j, 2);
          a = (_Float16)((double)a + (double)b); memcpy(dst + 2 * j, &a, 2);
        }
      } else {
        for (int64_t j = 0; j < c->row_bytes / 4; j++) {
          float a, b; memcpy(&a, dst + 4 * j, 4); memcpy(&b, src + 4 * j, 4);
          a = a + b; memcpy(dst + 4 * j, &a, 4);
        }
      }
    }
  }
}

/* Remove keys: matching ways get the sentinel tag (same file :515-566, invalidate_only). */
NVE_EXPORT void nve_oracle_cache_invalidate(void* h, const void* keys, int64_t n) {
  Cache* c = (Cache*)h;
  for (int64_t i = 0; i < n; i++) {
    const int64_t key = load_key(keys, c->key_bytes, i);
    const uint32_t set = set_of(c, key);
    for (int w = 0; w < WAYS; w++) {
      if (key_of(c, c->tags[(uint64_t)set * WAYS + w], set) == key) {
        c->tags[(uint64_t)set * WAYS + w] = c->sentinel;
      }
    }
  }
}

/* All ways empty; counters and timestamps back to zero
 * (include/ecache/ec_set_associative_device_modify.cuh clear_cache). */
NVE_EXPORT void nve_oracle_cache_clear(void* h) {
  Cache* c = (Cache*)h;
  for (uint64_t i = 0; i < c->num_sets * WAYS; i++) { c->tags[i] = c->sentinel; c->counters[i] = 0.f; }
  for (uint64_t i = 0; i < c->num_sets; i++) c->set_ts[i] = 0;
}
