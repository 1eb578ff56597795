/*
 * Test infrastructure only (checker / CPU baseline), never part of the product
 * path: only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg may load this library.
 *
 * Plain-C restatement of the reference's CPU attention and of its online-softmax
 * state merge, written from the reference's behaviour (no reference code is
 * included or linked here):
 *
 *   include/kernels_cpu.hpp:14-17    f16 <-> f32 (F16C, round-to-nearest-even)
 *   include/kernels_cpu.hpp:122-138  softmax(): max from -FLT_MAX, expf(v - max), divide by the sum
 *   include/kernels_cpu.hpp:140-167  attn(): scores = (q . K[t]) / sqrtf(head_dim), softmax,
 *                                    out[i] = sum_t p[t] * V[t][i], all in fp32, sequential order
 *   src/model/block.cpp:157-164      head loop: group = head / (n_heads / n_kv_heads)
 *   src/model/model.cpp:65-68        kv_len = pos + 1  => causal prefill row t sees rows 0..t
 *   src/attention.cu:41-65           AttentionState::merge: (m, z, o) with o already normalised
 *
 * Parity pin: the reference ships no tests or golden vectors for this path, so
 * this restatement is pinned against the reference's own header compiled into
 * oracle/_ref/libref_attn.so (tests compare the two bit for bit where both are
 * present) and against fixtures in tests/golden/ that were produced by that
 * compiled reference.
 *
 * KV layout everywhere: fp16 bit patterns, [row][kv_head][head_dim], row stride
 * given in elements (default n_kv_heads * head_dim) — include/model/block.hpp:66-67.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------- conversions */

static inline uint32_t f32_bits(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
}
static inline float bits_f32(uint32_t u) {
    float x;
    memcpy(&x, &u, 4);
    return x;
}

/* IEEE binary16 -> binary32, exact (what _cvtsh_ss does, kernels_cpu.hpp:16). */
float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: value = man * 2^-24 */
        float v = (float)man * 5.9604644775390625e-8f;
        return (sign ? -v : v);
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* binary32 -> binary16 with round-to-nearest-even (what _cvtss_sh(x, 0) does,
 * kernels_cpu.hpp:17). NaN keeps its top payload bits and is made quiet. */
uint16_t oracle_f32_to_f16(float x) {
    uint32_t u = f32_bits(x);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) { /* inf / nan */
        if (a == 0x7F800000u) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7E00u | ((a >> 13) & 0x3FFu));
    }
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 -> inf */
    if (a < 0x33000001u) return sign;                        /* <= 2^-25 -> +-0 (ties to even) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_exp;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(e + 15);
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q += 1;
    uint32_t out;
    if (half_exp == 0) {
        out = q; /* may carry into exponent 1: still correct encoding */
    } else {
        out = ((half_exp - 1) << 10) + q; /* q carries the implicit bit (0x400) */
    }
    return (uint16_t)(sign | out);
}

float oracle_bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

uint16_t oracle_f32_to_bf16(float x) {
    uint32_t u = f32_bits(x);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}

void oracle_f32_to_f16_array(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = oracle_f32_to_f16(src[i]);
}
void oracle_f16_to_f32_array(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = oracle_f16_to_f32(src[i]);
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* A launcher may export OMP_NUM_THREADS=1 to its workers (torch.distributed.run does); the timed CPU baseline asks
 * for the host's cores explicitly. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* -------------------------------------------------------------------- softmax */

/* kernels_cpu.hpp:122-138 */
void oracle_softmax(float* v, uint32_t size) {
    float max_val = -FLT_MAX;
    for (uint32_t i = 0; i < size; ++i) {
        if (v[i] > max_val) max_val = v[i];
    }
    float sum = 0.0f;
    for (uint32_t i = 0; i < size; ++i) {
        float ev = expf(v[i] - max_val);
        v[i] = ev;
        sum += ev;
    }
    for (uint32_t i = 0; i < size; ++i) v[i] /= sum;
}

/* ------------------------------------------------------------- one query head */

/* kernels_cpu.hpp:140-167. scores is scratch of >= kv_len floats. row_stride in
 * elements. kv_head selects the [head_dim] slice of every row. */
void oracle_attn_head(float* out, float* scores, const float* q, const uint16_t* k_cache, const uint16_t* v_cache,
                      uint32_t kv_head, uint32_t head_dim, size_t row_stride, uint32_t kv_len) {
    const uint16_t* k0 = k_cache + (size_t)head_dim * kv_head;
    const uint16_t* v0 = v_cache + (size_t)head_dim * kv_head;
    float denom = sqrtf((float)head_dim);
    for (uint32_t t = 0; t < kv_len; ++t) {
        const uint16_t* kt = k0 + row_stride * t;
        float score = 0.0f;
        for (uint32_t i = 0; i < head_dim; ++i) score += q[i] * oracle_f16_to_f32(kt[i]);
        scores[t] = score / denom;
    }
    oracle_softmax(scores, kv_len);
    for (uint32_t i = 0; i < head_dim; ++i) {
        float acc = 0.0f;
        for (uint32_t t = 0; t < kv_len; ++t) acc += scores[t] * oracle_f16_to_f32(v0[row_stride * t + i]);
        out[i] = acc;
    }
}

/* ------------------------------------------------------------------- decode */

/* Batched single-token decode; sequences run one after another and heads in an
 * OpenMP parallel-for, as src/model/block.cpp:157-164 does for its one sequence.
 *   q, out : fp32 [batch][n_heads][head_dim]
 *   k, v   : fp16 bits, sequence b starts at b * batch_stride elements, rows of
 *            row_stride elements
 *   kv_len : [batch]
 * Returns 0, -1 on allocation failure, -2 on bad arguments. */
int oracle_attn_decode(float* out, const float* q, const uint16_t* k, const uint16_t* v, const uint32_t* kv_len,
                       uint32_t batch, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, size_t row_stride,
                       size_t batch_stride) {
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0) return -2;
    uint32_t max_len = 1;
    for (uint32_t b = 0; b < batch; ++b)
        if (kv_len[b] > max_len) max_len = kv_len[b];
    float* scores = (float*)malloc(sizeof(float) * (size_t)n_heads * max_len);
    if (!scores) return -1;
    uint32_t g = n_heads / n_kv_heads;
    for (uint32_t b = 0; b < batch; ++b) {
        const float* qb = q + (size_t)b * n_heads * head_dim;
        float* ob = out + (size_t)b * n_heads * head_dim;
        const uint16_t* kb = k + batch_stride * b;
        const uint16_t* vb = v + batch_stride * b;
        uint32_t len = kv_len[b];
#pragma omp parallel for
        for (uint32_t h = 0; h < n_heads; ++h) {
            oracle_attn_head(ob + (size_t)h * head_dim, scores + (size_t)h * max_len, qb + (size_t)h * head_dim, kb,
                             vb, h / g, head_dim, row_stride, len);
        }
    }
    free(scores);
    return 0;
}

/* ------------------------------------------------------------------ prefill */

/* Causal prefill of one sequence: row t of head h is oracle_attn_head with
 * kv_len = t + 1 (src/model/model.cpp:68, tools/infer.cpp:271-274).
 *   q, out : fp32 [seq][n_heads][head_dim];  k, v : fp16 bits [seq][n_kv_heads][head_dim]
 * Visits rows row_begin, row_begin + row_step, ... < row_end; other rows of out
 * are left untouched. */
int oracle_attn_prefill_causal(float* out, const float* q, const uint16_t* k, const uint16_t* v, uint32_t seq,
                               uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t row_begin,
                               uint32_t row_end, uint32_t row_step) {
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0) return -2;
    if (row_step == 0) row_step = 1;
    if (row_end > seq) row_end = seq;
    int nthreads = oracle_num_threads();
    float* scores = (float*)malloc(sizeof(float) * (size_t)nthreads * (seq ? seq : 1));
    if (!scores) return -1;
    uint32_t g = n_heads / n_kv_heads;
    size_t row_stride = (size_t)n_kv_heads * head_dim;
    int64_t n_rows = row_end > row_begin ? (int64_t)(row_end - row_begin + row_step - 1) / row_step : 0;
    int64_t n_items = n_rows * n_heads;
#pragma omp parallel for schedule(dynamic, 8)
    for (int64_t item = 0; item < n_items; ++item) {
        uint32_t t = row_begin + (uint32_t)(item / n_heads) * row_step;
        uint32_t h = (uint32_t)(item % n_heads);
#ifdef _OPENMP
        int tid = omp_get_thread_num();
#else
        int tid = 0;
#endif
        size_t qo = ((size_t)t * n_heads + h) * head_dim;
        oracle_attn_head(out + qo, scores + (size_t)tid * seq, q + qo, k, v, h / g, head_dim, row_stride, t + 1);
    }
    free(scores);
    return 0;
}

/* ------------------------------------------------- online-softmax state + merge */

/* State of src/attention.cu:41-45: m = running max of the scaled scores
 * (-inf when empty), z = sum exp(score - m) (0 when empty), o = NORMALISED partial
 * output sum_t (e_t / z) V[t] (0 when empty). Computed for rows
 * [row_begin, row_end) of one head; scores is scratch of >= row_end - row_begin. */
void oracle_state_from_rows(float* m_out, float* z_out, float* o, float* scores, const float* q,
                            const uint16_t* k_cache, const uint16_t* v_cache, uint32_t kv_head, uint32_t head_dim,
                            size_t row_stride, uint32_t row_begin, uint32_t row_end) {
    uint32_t n = row_end > row_begin ? row_end - row_begin : 0;
    for (uint32_t i = 0; i < head_dim; ++i) o[i] = 0.0f;
    if (n == 0) {
        *m_out = -INFINITY;
        *z_out = 0.0f;
        return;
    }
    const uint16_t* k0 = k_cache + (size_t)head_dim * kv_head;
    const uint16_t* v0 = v_cache + (size_t)head_dim * kv_head;
    float denom = sqrtf((float)head_dim);
    float m = -INFINITY;
    for (uint32_t t = 0; t < n; ++t) {
        const uint16_t* kt = k0 + row_stride * (row_begin + t);
        float score = 0.0f;
        for (uint32_t i = 0; i < head_dim; ++i) score += q[i] * oracle_f16_to_f32(kt[i]);
        score /= denom;
        scores[t] = score;
        if (score > m) m = score;
    }
    float z = 0.0f;
    for (uint32_t t = 0; t < n; ++t) {
        scores[t] = expf(scores[t] - m);
        z += scores[t];
    }
    for (uint32_t t = 0; t < n; ++t) {
        float s = scores[t] / z;
        const uint16_t* vt = v0 + row_stride * (row_begin + t);
        for (uint32_t i = 0; i < head_dim; ++i) o[i] += s * oracle_f16_to_f32(vt[i]);
    }
    *m_out = m;
    *z_out = z;
}

/* a <- merge(a, b), src/attention.cu:47-64, with one addition the reference
 * lacks: when both sides are empty (z_c == 0) the result stays the empty state
 * instead of 0/0. */
void oracle_state_merge(float* m_a, float* z_a, float* o_a, float m_b, float z_b, const float* o_b,
                        uint32_t head_dim) {
    float m_c = fmaxf(*m_a, m_b);
    float eac = (*m_a == m_c) ? 1.0f : expf(*m_a - m_c);
    float ebc = (m_b == m_c) ? 1.0f : expf(m_b - m_c);
    float z_c = (*z_a * eac) + (z_b * ebc);
    if (!(z_c > 0.0f)) {
        for (uint32_t i = 0; i < head_dim; ++i) o_a[i] = 0.0f;
        *m_a = -INFINITY;
        *z_a = 0.0f;
        return;
    }
    float oas = (*z_a / z_c) * eac;
    float obs = (z_b / z_c) * ebc;
    for (uint32_t i = 0; i < head_dim; ++i) o_a[i] = o_a[i] * oas + o_b[i] * obs;
    *m_a = m_c;
    *z_a = z_c;
}

/* The same merge in log-sum-exp form over n partials of one head:
 * lse_i = m_i + ln z_i (-inf when empty); out = sum_i w_i o_i,
 * w_i = exp(lse_i - lse_max) / sum_j exp(lse_j - lse_max); lse_out = lse_max + ln(sum).
 * o_parts: [n][o_stride] (first head_dim entries used). All-empty input gives
 * out = 0 and lse_out = -inf. */
void oracle_lse_merge(float* out, float* lse_out, const float* o_parts, size_t o_stride, const float* lse_parts,
                      uint32_t n, uint32_t head_dim) {
    float mx = -INFINITY;
    for (uint32_t i = 0; i < n; ++i)
        if (lse_parts[i] > mx) mx = lse_parts[i];
    for (uint32_t d = 0; d < head_dim; ++d) out[d] = 0.0f;
    if (mx == -INFINITY) {
        if (lse_out) *lse_out = -INFINITY;
        return;
    }
    float sum = 0.0f;
    for (uint32_t i = 0; i < n; ++i) sum += expf(lse_parts[i] - mx);
    for (uint32_t i = 0; i < n; ++i) {
        float w = expf(lse_parts[i] - mx) / sum;
        if (w == 0.0f) continue;
        const float* oi = o_parts + o_stride * i;
        for (uint32_t d = 0; d < head_dim; ++d) out[d] += w * oi[d];
    }
    if (lse_out) *lse_out = mx + logf(sum);
}

/* Sequence-sharded decode as the multi-GPU path computes it, on the CPU: split
 * rows [0, kv_len) of one sequence into n_shards contiguous even shards (the
 * last one takes the remainder), compute the (m, z, o) state of every shard per
 * head, write them as (o, lse) partials, and also the merged result.
 *   q, out     : fp32 [n_heads][head_dim]
 *   part_o     : fp32 [n_shards][n_heads][head_dim]   (may be NULL)
 *   part_lse   : fp32 [n_shards][n_heads]             (may be NULL)
 */
int oracle_attn_decode_sharded(float* out, float* part_o, float* part_lse, const float* q, const uint16_t* k,
                               const uint16_t* v, uint32_t kv_len, uint32_t n_shards, uint32_t n_heads,
                               uint32_t n_kv_heads, uint32_t head_dim, size_t row_stride) {
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0 || n_shards == 0) return -2;
    uint32_t g = n_heads / n_kv_heads;
    uint32_t per = kv_len / n_shards;
    int fail = 0;
#pragma omp parallel for
    for (uint32_t h = 0; h < n_heads; ++h) {
        float* scores = (float*)malloc(sizeof(float) * (size_t)(kv_len ? kv_len : 1));
        float* o_tmp = (float*)malloc(sizeof(float) * (size_t)head_dim * n_shards);
        float* lse_tmp = (float*)malloc(sizeof(float) * n_shards);
        if (!scores || !o_tmp || !lse_tmp) {
            fail = 1;
        } else {
            for (uint32_t s = 0; s < n_shards; ++s) {
                uint32_t r0 = s * per;
                uint32_t r1 = (s + 1 == n_shards) ? kv_len : r0 + per;
                float m, z;
                oracle_state_from_rows(&m, &z, o_tmp + (size_t)s * head_dim, scores, q + (size_t)h * head_dim, k, v,
                                       h / g, head_dim, row_stride, r0, r1);
                lse_tmp[s] = (z > 0.0f) ? m + logf(z) : -INFINITY;
                if (part_o)
                    memcpy(part_o + ((size_t)s * n_heads + h) * head_dim, o_tmp + (size_t)s * head_dim,
                           sizeof(float) * head_dim);
                if (part_lse) part_lse[(size_t)s * n_heads + h] = lse_tmp[s];
            }
            oracle_lse_merge(out + (size_t)h * head_dim, NULL, o_tmp, head_dim, lse_tmp, n_shards, head_dim);
        }
        free(scores);
        free(o_tmp);
        free(lse_tmp);
    }
    return fail ? -1 : 0;
}

/* ------------------------------------------------ rotary embedding + cache insert */

/* include/kernels_cpu.hpp:82-100: adjacent pairs (i, i+1), freq = 1 / powf(theta, i / rotary_dim), angle = pos * freq,
 * all in fp32 with the C library's powf / cosf / sinf. Dimensions >= rotary_dim are left alone. */
void oracle_rope_f32(float* vec, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta, uint32_t rotary_dim) {
    for (uint32_t h = 0; h < n_heads; ++h) {
        float* x = vec + (size_t)h * head_dim;
        for (uint32_t i = 0; i < rotary_dim; i += 2) {
            float freq = 1.0f / powf(theta, (float)i / (float)rotary_dim);
            float deg = (float)pos * freq;
            float c = cosf(deg), s = sinf(deg);
            float v0 = x[i], v1 = x[i + 1];
            x[i] = v0 * c - v1 * s;
            x[i + 1] = v0 * s + v1 * c;
        }
    }
}

/* include/kernels_cpu.hpp:102-120: the same on fp16 storage: widen, rotate in fp32, round back (nearest even). */
void oracle_rope_f16(uint16_t* vec, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta,
                     uint32_t rotary_dim) {
    for (uint32_t h = 0; h < n_heads; ++h) {
        uint16_t* x = vec + (size_t)h * head_dim;
        for (uint32_t i = 0; i < rotary_dim; i += 2) {
            float freq = 1.0f / powf(theta, (float)i / (float)rotary_dim);
            float deg = (float)pos * freq;
            float c = cosf(deg), s = sinf(deg);
            float v0 = oracle_f16_to_f32(x[i]), v1 = oracle_f16_to_f32(x[i + 1]);
            x[i] = oracle_f32_to_f16(v0 * c - v1 * s);
            x[i + 1] = oracle_f32_to_f16(v0 * s + v1 * c);
        }
    }
}

/* src/model/block.cpp:140-155 for one token of one sequence: rotate q and k, store k and v as fp16 at row kv_pos,
 * then rotate the first kv_sink cached K rows forward by one position (attention sinks of the sliding window). */
void oracle_rope_kv_insert(float* q, float* k, const float* v, uint16_t* k_cache, uint16_t* v_cache, uint32_t n_heads,
                           uint32_t n_kv_heads, uint32_t head_dim, uint32_t rotary_dim, float theta, uint32_t pos,
                           uint32_t kv_pos, uint32_t kv_sink) {
    oracle_rope_f32(q, n_heads, head_dim, pos, theta, rotary_dim);
    oracle_rope_f32(k, n_kv_heads, head_dim, pos, theta, rotary_dim);
    size_t row = (size_t)n_kv_heads * head_dim;
    for (size_t i = 0; i < row; ++i) {
        k_cache[(size_t)kv_pos * row + i] = oracle_f32_to_f16(k[i]);
        v_cache[(size_t)kv_pos * row + i] = oracle_f32_to_f16(v[i]);
    }
    for (uint32_t s = 0; s < kv_sink; ++s) oracle_rope_f16(k_cache + (size_t)s * row, n_kv_heads, head_dim, 1, theta, rotary_dim);
}

/* ------------------------------------------------------------------ weight GEMV */

/* include/kernels_cpu.hpp:69-80 with the clamp of src/model/block.cpp:130-138: w is [d][n] fp16, n fastest. */
void oracle_matmul_clip(float* out, const float* x, const uint16_t* w, uint32_t n, uint32_t d, float clip) {
#pragma omp parallel for
    for (uint32_t j = 0; j < d; ++j) {
        float sum = 0.0f;
        for (uint32_t i = 0; i < n; ++i) sum += x[i] * oracle_f16_to_f32(w[(size_t)j * n + i]);
        if (clip > 0.0f) sum = sum > clip ? clip : (sum < -clip ? -clip : sum);
        out[j] = sum;
    }
}

/* The same GEMV over Q8_0 weights (public GGML block format: 34-byte blocks of an fp16 scale d and 32 signed bytes,
 * value = fp32(d) * q, exact in fp32). The reference has no Q8_0 path (src/model/config.cpp:11-17 rejects the type):
 * this is its fp16 matmul loop (include/kernels_cpu.hpp:69-80) applied to the dequantised value. */
void oracle_matmul_q8_0(float* out, const float* x, const uint8_t* w, uint32_t n, uint32_t d, float clip) {
    const size_t row_bytes = (size_t)(n / 32) * 34;
#pragma omp parallel for
    for (uint32_t j = 0; j < d; ++j) {
        const uint8_t* row = w + (size_t)j * row_bytes;
        float sum = 0.0f;
        for (uint32_t i = 0; i < n; ++i) {
            const uint8_t* blk = row + (size_t)(i / 32) * 34;
            const float scale = oracle_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
            sum += x[i] * (scale * (float)(int8_t)blk[2 + (i % 32)]);
        }
        if (clip > 0.0f) sum = sum > clip ? clip : (sum < -clip ? -clip : sum);
        out[j] = sum;
    }
}

/* ------------------------------------------------------------------ whole model, greedy generation */

/* Restates Block::block_cpu_ (src/model/block.cpp:105-223: RMSNorm, Q/K/V GEMVs, clamp, RoPE, cache insert, sink
 * rotation, attention, output GEMV + residual, RMSNorm, SwiGLU FFN + residual), Model::forward_cpu_
 * (src/model/model.cpp:60-98: embedding, sliding-window positions with 4 sink rows, final RMSNorm, classifier) and the
 * greedy sampler and generation loop of tools/infer.cpp:64-74,271-300 (without the end-of-sequence stop). */
typedef struct LlamaModel {
    uint32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, max_seq_len, rotary_dim;
    float norm_eps, rope_theta, qkv_clip;
    const uint16_t* embed;   /* [vocab][dim] fp16 */
    const uint16_t* wcls;    /* [vocab][dim] fp16 */
    const float* rms_final;  /* [dim] */
    const float* rms_att;    /* [layers][dim] */
    const float* rms_ffn;    /* [layers][dim] */
    const uint16_t *wq, *wk, *wv, *wo, *w1, *w2, *w3; /* stacked over layers, each [d][n] fp16 */
    uint32_t weight_type; /* 0: fp16 matrices (the engine's type); 1: every matrix incl. embed / wcls is Q8_0 blocks */
} LlamaModel;

/* include/kernels_cpu.hpp:43-67 (out may be x) */
void oracle_rmsnorm(float* out, const float* x, const float* weight, uint32_t size, float eps) {
    float rms = 0.0f;
    for (uint32_t i = 0; i < size; ++i) rms += x[i] * x[i];
    rms = sqrtf(rms / (float)size + eps);
    for (uint32_t i = 0; i < size; ++i) out[i] = x[i] / rms * weight[i];
}

/* include/kernels_cpu.hpp:198 and src/model/block.cpp:206-210 */
void oracle_swiglu(float* hb, const float* hb2, size_t count) {
    for (size_t i = 0; i < count; ++i) hb[i] = hb[i] / (1.0f + expf(-hb[i])) * hb2[i];
}

/* tools/infer.cpp:64-74 */
uint32_t oracle_argmax(const float* logits, uint32_t vocab) {
    uint32_t max_i = 0;
    float max_val = logits[0];
    for (uint32_t i = 1; i < vocab; ++i) {
        if (logits[i] > max_val) {
            max_val = logits[i];
            max_i = i;
        }
    }
    return max_i;
}

/* Row-major matrix l of a stack of [d][n] matrices, either type. */
static void model_matmul(const LlamaModel* c, float* out, const float* x, const void* w, size_t layer, uint32_t n,
                         uint32_t d, float clip) {
    if (c->weight_type == 1) {
        oracle_matmul_q8_0(out, x, (const uint8_t*)w + layer * (size_t)d * (n / 32) * 34, n, d, clip);
    } else {
        oracle_matmul_clip(out, x, (const uint16_t*)w + layer * (size_t)d * n, n, d, clip);
    }
}

static int forward_token(const LlamaModel* c, uint16_t* k_cache, uint16_t* v_cache, float* buf, uint32_t token,
                         uint32_t pos, float* logits) {
    const uint32_t q_dim = c->n_heads * c->head_dim, kv_dim = c->n_kv_heads * c->head_dim;
    float* x = buf;
    float* xb = x + c->dim;
    float* xb2 = xb + c->dim;
    float* q = xb2 + c->dim;
    float* k = q + q_dim;
    float* v = k + kv_dim;
    float* att = v + kv_dim;
    float* hb = att + q_dim;
    float* hb2 = hb + c->hidden_dim;
    float* scores = hb2 + c->hidden_dim; /* [n_heads][max_seq_len] */
    if (c->weight_type == 1) {
        const uint8_t* row = (const uint8_t*)c->embed + (size_t)token * (c->dim / 32) * 34;
        for (uint32_t i = 0; i < c->dim; ++i) {
            const uint8_t* blk = row + (size_t)(i / 32) * 34;
            x[i] = oracle_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8))) * (float)(int8_t)blk[2 + (i % 32)];
        }
    } else {
        for (uint32_t i = 0; i < c->dim; ++i) x[i] = oracle_f16_to_f32(c->embed[(size_t)token * c->dim + i]);
    }
    const uint32_t kv_sink = pos >= c->max_seq_len ? 4u : 0u;
    const uint32_t kv_pos = kv_sink + ((pos - kv_sink) % (c->max_seq_len - kv_sink));
    const uint32_t kv_len = pos >= c->max_seq_len ? c->max_seq_len : pos + 1;
    const uint32_t rotary_dim = c->rotary_dim ? c->rotary_dim : c->head_dim;
    const uint32_t group = c->n_heads / c->n_kv_heads;
    for (uint32_t l = 0; l < c->n_layers; ++l) {
        uint16_t* kc = k_cache + (size_t)l * c->max_seq_len * kv_dim;
        uint16_t* vc = v_cache + (size_t)l * c->max_seq_len * kv_dim;
        oracle_rmsnorm(xb, x, c->rms_att + (size_t)l * c->dim, c->dim, c->norm_eps);
        model_matmul(c, q, xb, c->wq, l, c->dim, q_dim, c->qkv_clip);
        model_matmul(c, k, xb, c->wk, l, c->dim, kv_dim, c->qkv_clip);
        model_matmul(c, v, xb, c->wv, l, c->dim, kv_dim, c->qkv_clip);
        oracle_rope_kv_insert(q, k, v, kc, vc, c->n_heads, c->n_kv_heads, c->head_dim, rotary_dim, c->rope_theta, pos,
                              kv_pos, kv_sink);
#pragma omp parallel for
        for (uint32_t h = 0; h < c->n_heads; ++h) {
            oracle_attn_head(att + (size_t)h * c->head_dim, scores + (size_t)h * c->max_seq_len, q + (size_t)h * c->head_dim,
                             kc, vc, h / group, c->head_dim, (size_t)kv_dim, kv_len);
        }
        model_matmul(c, xb, att, c->wo, l, q_dim, c->dim, 0.0f);
        for (uint32_t i = 0; i < c->dim; ++i) x[i] += xb[i];
        oracle_rmsnorm(xb, x, c->rms_ffn + (size_t)l * c->dim, c->dim, c->norm_eps);
        model_matmul(c, hb, xb, c->w1, l, c->dim, c->hidden_dim, 0.0f);
        model_matmul(c, hb2, xb, c->w3, l, c->dim, c->hidden_dim, 0.0f);
        oracle_swiglu(hb, hb2, c->hidden_dim);
        model_matmul(c, xb2, hb, c->w2, l, c->hidden_dim, c->dim, 0.0f);
        for (uint32_t i = 0; i < c->dim; ++i) x[i] += xb2[i] * 1.0f;
    }
    if (!logits) return 0;
    oracle_rmsnorm(x, x, c->rms_final, c->dim, c->norm_eps);
    model_matmul(c, logits, x, c->wcls, 0, c->dim, c->vocab_size, 0.0f);
    return 0;
}

int oracle_generate_greedy(const LlamaModel* m, const uint32_t* prompt, uint32_t n_prompt, uint32_t n_new,
                           uint32_t* out_tokens, float* out_logits) {
    if (!m || !prompt || n_prompt == 0 || !out_tokens) return -1;
    const size_t cache = (size_t)m->n_layers * m->max_seq_len * m->n_kv_heads * m->head_dim;
    const size_t nbuf = 3 * (size_t)m->dim + 2 * (size_t)m->n_heads * m->head_dim + 2 * (size_t)m->n_kv_heads * m->head_dim +
                        2 * (size_t)m->hidden_dim + (size_t)m->n_heads * m->max_seq_len;
    uint16_t* k_cache = (uint16_t*)calloc(cache, sizeof(uint16_t));
    uint16_t* v_cache = (uint16_t*)calloc(cache, sizeof(uint16_t));
    float* buf = (float*)malloc(nbuf * sizeof(float));
    float* logits = (float*)malloc((size_t)m->vocab_size * sizeof(float));
    int rc = -1;
    if (k_cache && v_cache && buf && logits) {
        for (uint32_t pos = 0; pos < n_prompt; ++pos)
            forward_token(m, k_cache, v_cache, buf, prompt[pos], pos, pos + 1 == n_prompt ? logits : NULL);
        for (uint32_t i = 0; i < n_new; ++i) {
            const uint32_t next = oracle_argmax(logits, m->vocab_size);
            out_tokens[i] = next;
            if (out_logits) memcpy(out_logits + (size_t)i * m->vocab_size, logits, (size_t)m->vocab_size * sizeof(float));
            if (i + 1 < n_new) forward_token(m, k_cache, v_cache, buf, next, n_prompt + i, logits);
        }
        rc = 0;
    }
    free(k_cache);
    free(v_cache);
    free(buf);
    free(logits);
    return rc;
}
