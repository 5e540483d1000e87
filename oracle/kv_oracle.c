/*
 * TEST INFRASTRUCTURE - CPU oracle for the paged KV-cache bookkeeping. Not part of the product.
 *
 * Only the test suite, the smoke check and the benchmark's CPU-baseline leg may load this file.
 *
 * Plain-C restatement of the reference's host-side integer logic, bit-exact by construction:
 *   src/kv_cache/block_manager.cpp:11-144   LIFO allocator + block table rows
 *   src/kv_cache/kv_cache.cpp:79-132        KvCacheBytes, MaxBlocksForBudget, ComputeSlotMapping
 *   src/kv_cache/kv_cache_kernels.cu:17-86  append scatter / block reset / block gather addressing
 *   src/kv_cache/kv_cache_layout.cuh:32-38  element offset inside one layer
 *
 * Parity pin: tests/test_oracle_pin.py drives this file and the reference's own classes
 * (oracle/_ref/libsca_ref.so, built by oracle/build_ref.sh) through the same operation traces
 * and requires identical integers; the known-answer values of tests/kv/test_kv_cache.cpp and
 * tests/kv/test_block_manager.cpp are asserted as well.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* error codes follow the reference's AttnStatusCode numbering (status.hpp:16-28) */
enum { KV_OK = 0, KV_SHAPE_MISMATCH = 2005, KV_CAPACITY_EXCEEDED = 2007 };

typedef struct OracleBlockManager {
    int64_t num_blocks;
    int64_t max_num_seqs;
    int64_t max_blocks_per_seq;
    int32_t* free_list; /* stack: allocation pops from the back */
    int64_t free_count;
    uint8_t* in_use;
    int32_t* table; /* [max_num_seqs][max_blocks_per_seq], -1 = empty */
    uint64_t revision;
    int64_t allocation_failures;
    int64_t double_free_events;
} OracleBlockManager;

/* block_manager.cpp:11-45: the free list is filled with N-1 ... 0, so a fresh pool hands out
 * 0, 1, 2, ... */
ORACLE_API OracleBlockManager* oracle_bm_create(int64_t num_blocks, int64_t max_num_seqs,
                                                int64_t max_blocks_per_seq) {
    if (num_blocks <= 0 || max_num_seqs <= 0 || max_blocks_per_seq <= 0) return NULL;
    OracleBlockManager* bm = (OracleBlockManager*)calloc(1, sizeof(*bm));
    if (!bm) return NULL;
    bm->num_blocks = num_blocks;
    bm->max_num_seqs = max_num_seqs;
    bm->max_blocks_per_seq = max_blocks_per_seq;
    bm->free_list = (int32_t*)malloc((size_t)num_blocks * sizeof(int32_t));
    bm->in_use = (uint8_t*)calloc((size_t)num_blocks, 1);
    bm->table = (int32_t*)malloc((size_t)(max_num_seqs * max_blocks_per_seq) * sizeof(int32_t));
    if (!bm->free_list || !bm->in_use || !bm->table) {
        free(bm->free_list);
        free(bm->in_use);
        free(bm->table);
        free(bm);
        return NULL;
    }
    for (int64_t i = 0; i < num_blocks; ++i) bm->free_list[i] = (int32_t)(num_blocks - 1 - i);
    bm->free_count = num_blocks;
    for (int64_t i = 0; i < max_num_seqs * max_blocks_per_seq; ++i) bm->table[i] = -1;
    return bm;
}

ORACLE_API void oracle_bm_destroy(OracleBlockManager* bm) {
    if (!bm) return;
    free(bm->free_list);
    free(bm->in_use);
    free(bm->table);
    free(bm);
}

/* block_manager.cpp:47-68: all-or-nothing */
ORACLE_API int oracle_bm_allocate(OracleBlockManager* bm, int64_t count, int32_t* out_ids) {
    if (count <= 0) return KV_SHAPE_MISMATCH;
    if (count > bm->free_count) {
        ++bm->allocation_failures;
        return KV_CAPACITY_EXCEEDED;
    }
    for (int64_t i = 0; i < count; ++i) {
        const int32_t block = bm->free_list[--bm->free_count];
        bm->in_use[block] = 1;
        out_ids[i] = block;
    }
    return KV_OK;
}

/* block_manager.cpp:70-85: ids are pushed in argument order; bad or idle ids only count */
ORACLE_API void oracle_bm_free(OracleBlockManager* bm, const int32_t* ids, int64_t count) {
    if (!ids || count <= 0) return;
    for (int64_t i = 0; i < count; ++i) {
        const int32_t block = ids[i];
        if (block < 0 || block >= bm->num_blocks || bm->in_use[block] == 0) {
            ++bm->double_free_events;
            continue;
        }
        bm->in_use[block] = 0;
        bm->free_list[bm->free_count++] = block;
    }
}

/* block_manager.cpp:87-110 */
ORACLE_API int oracle_bm_append_to_table(OracleBlockManager* bm, int64_t seq, const int32_t* ids,
                                         int64_t count) {
    if (seq < 0 || seq >= bm->max_num_seqs) return KV_SHAPE_MISMATCH;
    if (!ids || count <= 0) return KV_SHAPE_MISMATCH;
    int32_t* row = bm->table + seq * bm->max_blocks_per_seq;
    int64_t used = 0;
    while (used < bm->max_blocks_per_seq && row[used] >= 0) ++used;
    if (used + count > bm->max_blocks_per_seq) return KV_CAPACITY_EXCEEDED;
    for (int64_t i = 0; i < count; ++i) row[used + i] = ids[i];
    ++bm->revision;
    return KV_OK;
}

/* block_manager.cpp:112-127: frees the first `count` row entries where count = number of
 * non-negative entries, then blanks the row */
ORACLE_API int oracle_bm_reset_seq(OracleBlockManager* bm, int64_t seq) {
    if (seq < 0 || seq >= bm->max_num_seqs) return KV_SHAPE_MISMATCH;
    int32_t* row = bm->table + seq * bm->max_blocks_per_seq;
    int64_t count = 0;
    for (int64_t i = 0; i < bm->max_blocks_per_seq; ++i)
        if (row[i] >= 0) ++count;
    if (count > 0) oracle_bm_free(bm, row, count);
    for (int64_t i = 0; i < bm->max_blocks_per_seq; ++i) row[i] = -1;
    ++bm->revision;
    return KV_OK;
}

ORACLE_API int64_t oracle_bm_num_free(const OracleBlockManager* bm) { return bm->free_count; }
ORACLE_API int64_t oracle_bm_allocation_failures(const OracleBlockManager* bm) {
    return bm->allocation_failures;
}
ORACLE_API int64_t oracle_bm_double_free_events(const OracleBlockManager* bm) {
    return bm->double_free_events;
}
ORACLE_API uint64_t oracle_bm_revision(const OracleBlockManager* bm) { return bm->revision; }
ORACLE_API const int32_t* oracle_bm_table(const OracleBlockManager* bm) { return bm->table; }
ORACLE_API const int32_t* oracle_bm_free_list(const OracleBlockManager* bm) { return bm->free_list; }

/* kv_cache.cpp:99-132. Returns KV_OK or the reference's error code; *bad_position receives the
 * token position that failed. */
ORACLE_API int oracle_slot_mapping(const int32_t* row, int64_t seq_start, int64_t num_tokens,
                                   int64_t block_size, int64_t max_blocks, int32_t* slots,
                                   int64_t* bad_position) {
    if (!row) return KV_SHAPE_MISMATCH;
    if (block_size <= 0 || num_tokens <= 0) return KV_SHAPE_MISMATCH;
    for (int64_t t = 0; t < num_tokens; ++t) {
        const int64_t position = seq_start + t;
        const int64_t logical = position / block_size;
        const int64_t offset = position % block_size;
        if (logical >= max_blocks) {
            if (bad_position) *bad_position = position;
            return KV_CAPACITY_EXCEEDED;
        }
        const int32_t physical = row[logical];
        if (physical < 0) {
            if (bad_position) *bad_position = position;
            return KV_SHAPE_MISMATCH;
        }
        slots[t] = (int32_t)((int64_t)physical * block_size + offset);
    }
    return KV_OK;
}

/* kv_cache.cpp:79-97 */
ORACLE_API int64_t oracle_kv_cache_bytes(int64_t num_layers, int64_t num_blocks, int64_t block_size,
                                         int64_t num_kv_heads, int64_t head_dim, int64_t elem_bytes) {
    return 2 * num_layers * (num_blocks * block_size * num_kv_heads * head_dim) * elem_bytes;
}

ORACLE_API int64_t oracle_max_blocks_for_budget(int64_t num_layers, int64_t block_size,
                                                int64_t num_kv_heads, int64_t head_dim,
                                                int64_t elem_bytes, uint64_t budget_bytes) {
    const int64_t per_block = 2 * num_layers * block_size * num_kv_heads * head_dim * elem_bytes;
    if (per_block <= 0) return 0;
    return (int64_t)(budget_bytes / (uint64_t)per_block);
}

/* kv_cache_kernels.cu:17-47: rows [num_tokens][Hkv][D*elem] -> slot (block, offset); slot < 0 or
 * block >= num_blocks is skipped. */
ORACLE_API void oracle_kv_append(uint8_t* layer_k, uint8_t* layer_v, const uint8_t* k_new,
                                 const uint8_t* v_new, const int32_t* slots, int64_t num_tokens,
                                 int64_t num_blocks, int64_t block_size, int64_t num_kv_heads,
                                 int64_t head_dim, int64_t elem_bytes) {
    const int64_t row_bytes = head_dim * elem_bytes;
    for (int64_t t = 0; t < num_tokens; ++t) {
        const int32_t slot = slots[t];
        if (slot < 0) continue;
        const int64_t block = slot / block_size;
        const int64_t offset = slot % block_size;
        if (block >= num_blocks) continue;
        for (int64_t h = 0; h < num_kv_heads; ++h) {
            const int64_t dst = (((block * block_size + offset) * num_kv_heads + h) * head_dim) * elem_bytes;
            const int64_t src = (t * num_kv_heads + h) * row_bytes;
            memcpy(layer_k + dst, k_new + src, (size_t)row_bytes);
            memcpy(layer_v + dst, v_new + src, (size_t)row_bytes);
        }
    }
}

/* kv_cache_kernels.cu:49-66 */
ORACLE_API void oracle_kv_reset(uint8_t* layer_k, uint8_t* layer_v, const int32_t* block_ids,
                                int64_t count, int64_t num_blocks, int64_t block_size,
                                int64_t num_kv_heads, int64_t head_dim, int64_t elem_bytes) {
    const int64_t per_block = block_size * num_kv_heads * head_dim * elem_bytes;
    for (int64_t i = 0; i < count; ++i) {
        const int32_t b = block_ids[i];
        if (b < 0 || b >= num_blocks) continue;
        memset(layer_k + (int64_t)b * per_block, 0, (size_t)per_block);
        memset(layer_v + (int64_t)b * per_block, 0, (size_t)per_block);
    }
}

/* kv_cache_kernels.cu:68-86: invalid ids gather zeros */
ORACLE_API void oracle_kv_gather(const uint8_t* layer, const int32_t* block_ids, int64_t count,
                                 uint8_t* out, int64_t num_blocks, int64_t block_size,
                                 int64_t num_kv_heads, int64_t head_dim, int64_t elem_bytes) {
    const int64_t per_block = block_size * num_kv_heads * head_dim * elem_bytes;
    for (int64_t i = 0; i < count; ++i) {
        const int32_t b = block_ids[i];
        if (b < 0 || b >= num_blocks) memset(out + i * per_block, 0, (size_t)per_block);
        else memcpy(out + i * per_block, layer + (int64_t)b * per_block, (size_t)per_block);
    }
}
