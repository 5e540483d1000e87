/*
 * TEST INFRASTRUCTURE - CPU oracle for the attention hot path. Not part of the product.
 *
 * Only the test suite, the smoke check and the benchmark's CPU-baseline leg may load this file;
 * the shipped library never links or calls it.
 *
 * It restates, in plain C with double accumulation, the reference's host-side checker
 *   tests/common/test_utils.hpp:229-285   ReferenceAttention (FP64, bottom-right causal, GQA)
 *   tests/kernel/test_flash_correctness.cu:73-116   the log-sum-exp expectation
 *   tests/common/test_utils.hpp:24-38     RandomFloats (xorshift32)
 *   tests/common/test_utils.hpp:48-101    software fp16 / bf16 rounding
 * and the semantics of the reference's paged decode addressing
 *   src/backends/paged/page_table.cuh:18-36, src/backends/decode/decode_splitk.cu:102-129.
 *
 * Parity pin: oracle/build_ref.sh compiles the reference's own header next to this file
 * (oracle/_ref/libsca_ref.so) and tests/test_oracle_pin.py requires bit-identical outputs.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------ */
/* deterministic inputs: tests/common/test_utils.hpp:24-38                                     */
/* ------------------------------------------------------------------------------------------ */
ORACLE_API void oracle_random_floats(float* out, size_t count, uint32_t seed, float low, float high) {
    uint32_t state = seed == 0 ? 1u : seed;
    for (size_t i = 0; i < count; ++i) {
        state ^= state << 13;
        state ^= state >> 17;
        state ^= state << 5;
        const float unit = (float)state / (float)0xffffffffu;
        out[i] = low + unit * (high - low);
    }
}

/* ------------------------------------------------------------------------------------------ */
/* software rounding: tests/common/test_utils.hpp:48-101                                        */
/* (fp16 encode flushes results below the normal range to signed zero, exactly as the           */
/*  reference's helper does; bf16 is round-to-nearest-even on the upper 16 bits)                */
/* ------------------------------------------------------------------------------------------ */
ORACLE_API uint16_t oracle_float_to_half_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof(bits));
    const uint32_t sign = (bits >> 16) & 0x8000u;
    const int32_t exponent = (int32_t)((bits >> 23) & 0xffu) - 127 + 15;
    const uint32_t mantissa = bits & 0x7fffffu;
    if (exponent <= 0) return (uint16_t)sign;
    if (exponent >= 31) return (uint16_t)(sign | 0x7c00u);
    uint16_t half = (uint16_t)(sign | ((uint32_t)exponent << 10) | (mantissa >> 13));
    const uint32_t rest = mantissa & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u) != 0u)) half = (uint16_t)(half + 1);
    return half;
}

ORACLE_API float oracle_half_bits_to_float(uint16_t half) {
    const uint32_t sign = (uint32_t)(half & 0x8000u) << 16;
    const uint32_t exponent = (half >> 10) & 0x1fu;
    const uint32_t mantissa = half & 0x3ffu;
    uint32_t bits = sign;
    if (exponent == 0) {
        if (mantissa != 0) {
            const float v = ldexpf((float)mantissa, -24);
            return sign ? -v : v;
        }
    } else if (exponent == 31) {
        bits |= 0x7f800000u | (mantissa << 13);
    } else {
        bits |= ((exponent - 15 + 127) << 23) | (mantissa << 13);
    }
    float out;
    memcpy(&out, &bits, sizeof(out));
    return out;
}

ORACLE_API uint16_t oracle_float_to_bf16_bits(float value) {
    uint32_t bits;
    memcpy(&bits, &value, sizeof(bits));
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

ORACLE_API float oracle_bf16_bits_to_float(uint16_t b) {
    const uint32_t bits = (uint32_t)b << 16;
    float out;
    memcpy(&out, &bits, sizeof(out));
    return out;
}

/* dtype: 0 = fp32 (identity), 1 = fp16, 2 = bf16. Writes the storage bits (u16, unused for fp32)
 * and the dequantised values the oracle consumes. */
ORACLE_API void oracle_encode(const float* values, size_t count, int dtype, uint16_t* bits_out,
                              float* dequant_out) {
    for (size_t i = 0; i < count; ++i) {
        if (dtype == 1) {
            const uint16_t h = oracle_float_to_half_bits(values[i]);
            if (bits_out) bits_out[i] = h;
            if (dequant_out) dequant_out[i] = oracle_half_bits_to_float(h);
        } else if (dtype == 2) {
            const uint16_t h = oracle_float_to_bf16_bits(values[i]);
            if (bits_out) bits_out[i] = h;
            if (dequant_out) dequant_out[i] = oracle_bf16_bits_to_float(h);
        } else {
            if (dequant_out) dequant_out[i] = values[i];
        }
    }
}

/* ------------------------------------------------------------------------------------------ */
/* attention, FP64: tests/common/test_utils.hpp:229-285                                         */
/*                                                                                              */
/* q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D], out [B,Hq,Sq,D] (double), lse [B,Hq,Sq] (double, optional). */
/* scale <= 0 reproduces the reference exactly: the dot product is DIVIDED by sqrt((double)D).    */
/* scale  > 0 multiplies by (double)scale instead (used for the custom-scale cases).              */
/* The weight exp(s_j - m) / sum is hoisted out of the d loop; the reference recomputes the same  */
/* expression for every d, so the hoisted value is bit-identical.                                  */
/* Fully masked rows give out = 0 and lse = -inf.                                                  */
/* threads <= 1 runs the loop nest single-threaded as the reference does; > 1 spreads (b, h)       */
/* over OpenMP threads (each (b, h) is computed exactly as in the serial order).                   */
/* ------------------------------------------------------------------------------------------ */
ORACLE_API int oracle_attention_f64(const float* q, const float* k, const float* v, int64_t batch,
                                    int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv,
                                    int64_t head_dim, int causal, double scale, double* out,
                                    double* lse, int threads) {
    if (!q || !k || !v || !out || heads_kv <= 0 || heads_q % heads_kv != 0) return 1;
    const int64_t group = heads_q / heads_kv;
    const int64_t diagonal = causal ? (seq_kv - seq_q) : 0;
    const int64_t pairs = batch * heads_q;
    int failed = 0;
#if defined(_OPENMP)
    const int nthreads = threads > 1 ? threads : 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
#endif
    for (int64_t bh = 0; bh < pairs; ++bh) {
        const int64_t b = bh / heads_q;
        const int64_t h = bh % heads_q;
        const int64_t h_kv = h / group;
        double* scores = (double*)malloc((size_t)(seq_kv > 0 ? seq_kv : 1) * sizeof(double));
        if (!scores) {
            failed = 1;
            continue;
        }
        for (int64_t i = 0; i < seq_q; ++i) {
            const float* q_row = q + ((b * heads_q + h) * seq_q + i) * head_dim;
            double m = -INFINITY;
            for (int64_t j = 0; j < seq_kv; ++j) {
                if (causal && j > i + diagonal) {
                    scores[j] = -INFINITY;
                    continue;
                }
                const float* k_row = k + ((b * heads_kv + h_kv) * seq_kv + j) * head_dim;
                double dot = 0.0;
                for (int64_t d = 0; d < head_dim; ++d) dot += (double)q_row[d] * (double)k_row[d];
                if (scale > 0.0) dot *= scale;
                else dot /= sqrt((double)head_dim);
                scores[j] = dot;
                if (dot > m) m = dot;
            }
            double sum = 0.0;
            for (int64_t j = 0; j < seq_kv; ++j) {
                if (isinf(scores[j])) continue;
                sum += exp(scores[j] - m);
            }
            for (int64_t j = 0; j < seq_kv; ++j) {
                if (isinf(scores[j])) continue;
                scores[j] = exp(scores[j] - m) / sum; /* same expression the reference evaluates */
            }
            double* o_row = out + ((b * heads_q + h) * seq_q + i) * head_dim;
            for (int64_t d = 0; d < head_dim; ++d) {
                double acc = 0.0;
                for (int64_t j = 0; j < seq_kv; ++j) {
                    if (isinf(scores[j])) continue;
                    acc += scores[j] * (double)v[((b * heads_kv + h_kv) * seq_kv + j) * head_dim + d];
                }
                o_row[d] = acc;
            }
            if (lse) lse[(b * heads_q + h) * seq_q + i] = (sum > 0.0) ? m + log(sum) : -INFINITY;
        }
        free(scores);
    }
    return failed;
}

/* ------------------------------------------------------------------------------------------ */
/* paged decode (seq_q = 1), FP64, walking the page table the way the reference kernel does:     */
/*   token j of sequence s lives in physical block table[s*max_blocks + j/bs] at offset j%bs;     */
/*   a logical block >= max_blocks, a negative id, or an id >= num_kv_blocks contributes weight 0 */
/*   (src/backends/paged/page_table.cuh:18-36);  seq_lens == NULL scans max_blocks*bs tokens.      */
/* Pools are block-major [num_kv_blocks][bs][Hkv][D] (src/kv_cache/kv_cache_layout.cuh:32-38).     */
/* q [S,Hq,1,D], out [S,Hq,D] double.                                                              */
/* ------------------------------------------------------------------------------------------ */
ORACLE_API int oracle_paged_decode_f64(const float* q, const float* k_pool, const float* v_pool,
                                       const int32_t* page_table, const int32_t* seq_lens,
                                       int64_t num_seqs, int64_t heads_q, int64_t heads_kv,
                                       int64_t head_dim, int64_t block_size,
                                       int64_t max_blocks_per_seq, int64_t num_kv_blocks,
                                       double scale, double* out, int threads) {
    if (!q || !k_pool || !v_pool || !page_table || !out || heads_kv <= 0) return 1;
    const int64_t group = heads_q / heads_kv;
    const int64_t pairs = num_seqs * heads_q;
    int failed = 0;
#if defined(_OPENMP)
    const int nthreads = threads > 1 ? threads : 1;
#pragma omp parallel for schedule(dynamic, 1) num_threads(nthreads)
#endif
    for (int64_t sh = 0; sh < pairs; ++sh) {
        const int64_t s = sh / heads_q;
        const int64_t h = sh % heads_q;
        const int64_t h_kv = h / group;
        const int64_t len = seq_lens ? (int64_t)seq_lens[s] : max_blocks_per_seq * block_size;
        double* w = (double*)malloc((size_t)(len > 0 ? len : 1) * sizeof(double));
        int64_t* rows = (int64_t*)malloc((size_t)(len > 0 ? len : 1) * sizeof(int64_t));
        if (!w || !rows) {
            failed = 1;
            free(w);
            free(rows);
            continue;
        }
        const float* q_row = q + (s * heads_q + h) * head_dim;
        double m = -INFINITY;
        for (int64_t j = 0; j < len; ++j) {
            const int64_t logical = j / block_size;
            int64_t row = -1;
            if (logical < max_blocks_per_seq) {
                const int32_t phys = page_table[s * max_blocks_per_seq + logical];
                if (phys >= 0 && phys < num_kv_blocks) row = (int64_t)phys * block_size + j % block_size;
            }
            rows[j] = row;
            if (row < 0) {
                w[j] = -INFINITY;
                continue;
            }
            const float* k_row = k_pool + (row * heads_kv + h_kv) * head_dim;
            double dot = 0.0;
            for (int64_t d = 0; d < head_dim; ++d) dot += (double)q_row[d] * (double)k_row[d];
            if (scale > 0.0) dot *= scale;
            else dot /= sqrt((double)head_dim);
            w[j] = dot;
            if (dot > m) m = dot;
        }
        double sum = 0.0;
        for (int64_t j = 0; j < len; ++j)
            if (!isinf(w[j])) sum += exp(w[j] - m);
        for (int64_t j = 0; j < len; ++j)
            if (!isinf(w[j])) w[j] = exp(w[j] - m) / sum;
        double* o_row = out + (s * heads_q + h) * head_dim;
        for (int64_t d = 0; d < head_dim; ++d) {
            double acc = 0.0;
            for (int64_t j = 0; j < len; ++j) {
                if (isinf(w[j])) continue;
                acc += w[j] * (double)v_pool[(rows[j] * heads_kv + h_kv) * head_dim + d];
            }
            o_row[d] = acc;
        }
        free(w);
        free(rows);
    }
    return failed;
}

/* ------------------------------------------------------------------------------------------ */
/* split merge: src/backends/decode/decode_splitk.cu:143-182 restated in FP64.                   */
/* Each part p holds (m_p, l_p, O_p[D]) with O_p = sum_j exp(s_j - m_p) V_j (unnormalised).       */
/* Parts with m = -inf are skipped. Also the rule that merges the per-GPU triples of a           */
/* sequence-split decode.                                                                         */
/* ------------------------------------------------------------------------------------------ */
ORACLE_API void oracle_merge_parts_f64(const double* m, const double* l, const double* o,
                                       int64_t parts, int64_t head_dim, double* out) {
    double m_all = -INFINITY;
    for (int64_t p = 0; p < parts; ++p)
        if (m[p] > m_all) m_all = m[p];
    double l_all = 0.0;
    for (int64_t d = 0; d < head_dim; ++d) out[d] = 0.0;
    for (int64_t p = 0; p < parts; ++p) {
        if (isinf(m[p]) && m[p] < 0) continue;
        const double wgt = exp(m[p] - m_all);
        l_all += l[p] * wgt;
        for (int64_t d = 0; d < head_dim; ++d) out[d] += o[p * head_dim + d] * wgt;
    }
    const double inv = l_all > 0.0 ? 1.0 / l_all : 0.0;
    for (int64_t d = 0; d < head_dim; ++d) out[d] *= inv;
}

ORACLE_API int oracle_max_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
