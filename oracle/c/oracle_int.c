/* Plain-C restatement of the integer / byte-exact pieces of the gpt_lm path. TEST
 * INFRASTRUCTURE ONLY: loaded by tests and by the oracle's self-checks, never by the product.
 *
 *   oracle_splitmix64        src/backends/metal/primitives/random/metal_random.metal:8-14
 *   oracle_dropout_mask      src/ops/dropout/metal_dropout.metal:6-19, metal_dropout.m:145-155
 *   oracle_mask_allowed      src/ops/sdpa_varlen/metal_sdpa_varlen.metal:30-55
 *   oracle_kv_append_packed  src/ops/kv_cache_append/metal_kv_cache_append.metal:65-122
 *   oracle_kv_append         src/ops/kv_cache_append/metal_kv_cache_append.metal:30-63
 *   oracle_argmax_first      examples/gpt_lm/gpt_lm_shared.c:1388-1398
 *   oracle_embedding_rows    src/ops/embedding/metal_embedding.metal:60-83
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

uint64_t oracle_splitmix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ULL;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
    return x ^ (x >> 31);
}

uint32_t oracle_dropout_threshold(float p)
{
    const double t = ceil((double)p * 16777216.0);
    if (t <= 0.0) return 0U;
    if (t >= 16777216.0) return 16777216U;
    return (uint32_t)t;
}

void oracle_dropout_mask(uint8_t *mask, uint64_t count, float p, uint64_t seed)
{
    const uint32_t threshold = oracle_dropout_threshold(p);
    for (uint64_t i = 0; i < count; ++i) {
        const uint64_t r = oracle_splitmix64(seed + i);
        mask[i] = ((uint32_t)((r >> 40) & 0xffffffULL) >= threshold) ? 1 : 0;
    }
}

int oracle_mask_allowed(int i, int j, int causal, int window, int prefix_len)
{
    if (causal) {
        if (prefix_len > 0) {
            if (i < prefix_len) {
                if (j >= prefix_len) return 0;
            } else if (j > i) {
                return 0;
            }
        } else if (j > i) {
            return 0;
        }
    }
    if (window > 0) {
        if (prefix_len > 0) {
            if (i >= prefix_len && j >= prefix_len && (i - j) >= window) return 0;
        } else if ((i - j) >= window) {
            return 0;
        }
    }
    return 1;
}

/* caches [B, Tmax, row_bytes]; new rows packed [N, row_bytes]; whole sequences that would cross
 * the capacity are dropped. */
void oracle_kv_append_packed(uint8_t *k_cache, uint8_t *v_cache, const uint8_t *k_new, const uint8_t *v_new,
                             const int32_t *cache_pos, const int32_t *cu, uint32_t batch, uint32_t tmax, uint32_t row_bytes)
{
    if (cu[0] != 0) return;
    for (uint32_t b = 0; b < batch; ++b) {
        const int32_t s0 = cu[b], s1 = cu[b + 1], pos = cache_pos[b];
        if (s0 < 0 || s1 < s0 || pos < 0 || pos + (s1 - s0) > (int32_t)tmax) continue;
        for (int32_t t = 0; t < s1 - s0; ++t) {
            const size_t dst = ((size_t)b * tmax + (size_t)(pos + t)) * row_bytes, src = (size_t)(s0 + t) * row_bytes;
            memcpy(k_cache + dst, k_new + src, row_bytes);
            memcpy(v_cache + dst, v_new + src, row_bytes);
        }
    }
}

/* new rows [B, Tnew, row_bytes] at cache_pos[b] (or the scalar when cache_pos is NULL). */
void oracle_kv_append(uint8_t *k_cache, uint8_t *v_cache, const uint8_t *k_new, const uint8_t *v_new,
                      const int32_t *cache_pos, int32_t scalar_pos, uint32_t batch, uint32_t tnew, uint32_t tmax, uint32_t row_bytes)
{
    for (uint32_t b = 0; b < batch; ++b) {
        const int32_t pos = cache_pos != NULL ? cache_pos[b] : scalar_pos;
        if (pos < 0 || pos + (int32_t)tnew > (int32_t)tmax) continue;
        for (uint32_t t = 0; t < tnew; ++t) {
            const size_t dst = ((size_t)b * tmax + (size_t)pos + t) * row_bytes, src = ((size_t)b * tnew + t) * row_bytes;
            memcpy(k_cache + dst, k_new + src, row_bytes);
            memcpy(v_cache + dst, v_new + src, row_bytes);
        }
    }
}

int32_t oracle_argmax_first(const float *logits, uint32_t n)
{
    /* index 0 when no value is finite, as the reference's `int best = 0` leaves it (gpt_lm_shared.c:1380,1397) */
    int32_t best = 0;
    int have_best = 0;
    double best_v = 0.0;
    for (uint32_t i = 0; i < n; ++i) {
        const double v = (double)logits[i];
        if (!isfinite(v)) continue;
        if (!have_best || v > best_v) {
            best = (int32_t)i;
            best_v = v;
            have_best = 1;
        }
    }
    return best;
}

/* 16-bit table rows gathered by id; invalid ids give the F16 NaN pattern 0x7e00. */
void oracle_embedding_rows(const uint16_t *table, const int32_t *ids, uint16_t *out, uint32_t n_ids, uint32_t vocab, uint32_t dim)
{
    for (uint32_t r = 0; r < n_ids; ++r) {
        const int32_t id = ids[r];
        for (uint32_t c = 0; c < dim; ++c) {
            out[(size_t)r * dim + c] = (id < 0 || (uint32_t)id >= vocab) ? 0x7e00U : table[(size_t)id * dim + c];
        }
    }
}
