// Test infrastructure only (checker / CPU baseline), never part of the product path.
//
// C-ABI driver around the reference's own CPU attention. It includes the
// reference header include/kernels_cpu.hpp unmodified (found through -I at
// build time; no reference source is copied) and calls attn() (lines 140-167)
// the way the reference's transformer block does: an OpenMP parallel-for over
// query heads with group = head / (n_heads / n_kv_heads)
// (src/model/block.cpp:157-164). The reference has no batch dimension, so
// sequences of a batch are run one after another. Causal prefill is defined by
// the reference as "row t attends to rows 0..t" because its prefill is the
// decode step run once per prompt token with kv_len = pos + 1
// (tools/infer.cpp:271-274, src/model/model.cpp:68).
#include <kernels_cpu.hpp>

#include <cstdint>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

int ref_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* A launcher may export OMP_NUM_THREADS=1 to its workers (torch.distributed.run does); the timed CPU baseline asks
 * for the host's cores explicitly. */
void ref_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

uint16_t ref_f32_to_f16(float x) { return f32_to_f16(x); }
float ref_f16_to_f32(uint16_t x) { return f16_to_f32(x); }

void ref_f32_to_f16_array(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_f16(src[i]);
}

void ref_softmax(float* v, uint32_t size) { softmax(v, size); }

// One sequence. q: fp32 [n_heads][head_dim]; k_cache/v_cache: fp16 bit patterns
// [kv_len][n_kv_heads][head_dim]; out: fp32 [n_heads][head_dim];
// scores: fp32 scratch [n_heads][scores_stride], scores_stride >= kv_len.
void ref_attn_decode_seq(float* out, float* scores, size_t scores_stride, const float* q, const uint16_t* k_cache,
                         const uint16_t* v_cache, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                         uint32_t kv_len) {
    uint32_t heads_per_group = n_heads / n_kv_heads;
#pragma omp parallel for
    for (uint32_t head_i = 0; head_i < n_heads; ++head_i) {
        uint32_t group_i = head_i / heads_per_group;
        attn(out + static_cast<size_t>(head_i) * head_dim, scores + static_cast<size_t>(head_i) * scores_stride,
             q + static_cast<size_t>(head_i) * head_dim, k_cache, v_cache, group_i, head_dim, n_kv_heads, kv_len);
    }
}

// Batch of independent sequences, each with its own contiguous cache of
// kv_capacity rows and its own kv_len[b]. Returns 0, or -1 on allocation failure.
int ref_attn_decode_batch(float* out, const float* q, const uint16_t* k_cache, const uint16_t* v_cache,
                          const uint32_t* kv_len, uint32_t batch, uint32_t kv_capacity, uint32_t n_heads,
                          uint32_t n_kv_heads, uint32_t head_dim) {
    std::vector<float> scores;
    try {
        scores.resize(static_cast<size_t>(n_heads) * (kv_capacity ? kv_capacity : 1));
    } catch (...) {
        return -1;
    }
    size_t seq_elems = static_cast<size_t>(kv_capacity) * n_kv_heads * head_dim;
    size_t qo_elems = static_cast<size_t>(n_heads) * head_dim;
    for (uint32_t b = 0; b < batch; ++b) {
        ref_attn_decode_seq(out + b * qo_elems, scores.data(), kv_capacity ? kv_capacity : 1, q + b * qo_elems,
                            k_cache + b * seq_elems, v_cache + b * seq_elems, n_heads, n_kv_heads, head_dim,
                            kv_len[b]);
    }
    return 0;
}

// Causal prefill of one sequence, rows [row_begin, row_end) with a row step:
// q: fp32 [seq][n_heads][head_dim]; k/v: fp16 bits [seq][n_kv_heads][head_dim];
// out: fp32 [seq][n_heads][head_dim] (only the visited rows are written).
// Parallel over (row, head) pairs; each pair is exactly one attn() call with
// kv_len = row + 1.
int ref_attn_prefill_causal_seq(float* out, const float* q, const uint16_t* k, const uint16_t* v, uint32_t seq,
                                uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, uint32_t row_begin,
                                uint32_t row_end, uint32_t row_step) {
    if (row_step == 0) row_step = 1;
    if (row_end > seq) row_end = seq;
    uint32_t heads_per_group = n_heads / n_kv_heads;
    int nthreads = ref_num_threads();
    std::vector<float> scores;
    try {
        scores.resize(static_cast<size_t>(nthreads) * (seq ? seq : 1));
    } catch (...) {
        return -1;
    }
    int64_t n_rows = row_end > row_begin ? (row_end - row_begin + row_step - 1) / row_step : 0;
    int64_t n_items = n_rows * n_heads;
#pragma omp parallel for schedule(dynamic, 8)
    for (int64_t item = 0; item < n_items; ++item) {
        uint32_t t = row_begin + static_cast<uint32_t>(item / n_heads) * row_step;
        uint32_t head_i = static_cast<uint32_t>(item % n_heads);
#ifdef _OPENMP
        int tid = omp_get_thread_num();
#else
        int tid = 0;
#endif
        size_t qo = (static_cast<size_t>(t) * n_heads + head_i) * head_dim;
        attn(out + qo, scores.data() + static_cast<size_t>(tid) * seq, q + qo, k, v, head_i / heads_per_group,
             head_dim, n_kv_heads, t + 1);
    }
    return 0;
}

}  // extern "C"

// ---- rotary embedding and KV-cache insert (the step in front of attention) ----
// include/kernels_cpu.hpp:82-100 (fp32) and 102-120 (fp16 in place), called from src/model/block.cpp:140-155.
extern "C" {

void ref_rope_f32(float* vec, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta, uint32_t rotary_dim) {
    rope(vec, n_heads, head_dim, pos, theta, rotary_dim);
}

void ref_rope_f16(uint16_t* vec, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta, uint32_t rotary_dim) {
    rope(vec, n_heads, head_dim, pos, theta, rotary_dim);
}

// One token of one sequence, exactly the sequence of src/model/block.cpp:140-155: rotate q and k at `pos`, store k and v
// as fp16 at cache row kv_pos, then rotate the first kv_sink cached K rows forward by one position.
void ref_rope_kv_insert(float* q, float* k, const float* v, uint16_t* k_cache, uint16_t* v_cache, uint32_t n_heads,
                        uint32_t n_kv_heads, uint32_t head_dim, uint32_t rotary_dim, float theta, uint32_t pos,
                        uint32_t kv_pos, uint32_t kv_sink) {
    rope(q, n_heads, head_dim, pos, theta, rotary_dim);
    rope(k, n_kv_heads, head_dim, pos, theta, rotary_dim);
    const uint32_t kv_total_dim = n_kv_heads * head_dim;
    for (uint32_t i = 0; i < kv_total_dim; ++i) {
        k_cache[static_cast<size_t>(kv_pos) * kv_total_dim + i] = f32_to_f16(k[i]);
        v_cache[static_cast<size_t>(kv_pos) * kv_total_dim + i] = f32_to_f16(v[i]);
    }
    for (uint32_t s = 0; s < kv_sink; ++s) {
        rope(k_cache + static_cast<size_t>(s) * kv_total_dim, n_kv_heads, head_dim, 1, theta, rotary_dim);
    }
}

}  // extern "C"

// ---- weight GEMV (QKV / output / FFN / classifier projections) ----
// include/kernels_cpu.hpp:69-80: out[j] = sum_i x[i] * f16(w[j*n + i]), fp32 sequential sum, OpenMP over j;
// optional symmetric clamp as src/model/block.cpp:130-138.
extern "C" void ref_matmul_clip(float* out, const float* x, const uint16_t* w, uint32_t n, uint32_t d, float clip) {
    matmul(out, x, w, n, d);
    if (clip > 0.f) {
        for (uint32_t j = 0; j < d; ++j) out[j] = std::min(std::max(out[j], -clip), clip);
    }
}

// include/kernels_cpu.hpp:43-54, the engine's own rmsnorm (x / rms * weight).
extern "C" void ref_rmsnorm(float* out, const float* x, const float* weight, uint32_t size, float eps) {
    rmsnorm(out, x, weight, size, eps);
}

// ---- one token through the whole model, and greedy generation ----
// The engine's classes (Model, Block, InferenceState) need its GGUF loader and device layer; this driver instead
// calls the same primitives of include/kernels_cpu.hpp in the same order as Block::block_cpu_
// (src/model/block.cpp:105-223) and Model::forward_cpu_ (src/model/model.cpp:60-98) on plain arrays, with the
// sliding-window arithmetic of model.cpp:66-68 (KV_SINK = 4, include/model/model.hpp) and the greedy sampler of
// tools/infer.cpp:64-74. Weights are fp16 [d][n], norms fp32, stacked over the layers.
struct LlamaModel {
    uint32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, max_seq_len, rotary_dim;
    float norm_eps, rope_theta, qkv_clip;
    const uint16_t* embed;
    const uint16_t* wcls;
    const float* rms_final;
    const float* rms_att;
    const float* rms_ffn;
    const uint16_t *wq, *wk, *wv, *wo, *w1, *w2, *w3;
};

namespace {
constexpr uint32_t kKvSink = 4;

void forward_token(const LlamaModel& c, uint16_t* k_cache, uint16_t* v_cache, uint32_t token, uint32_t pos,
                   float* logits) {
    const uint32_t q_dim = c.n_heads * c.head_dim, kv_dim = c.n_kv_heads * c.head_dim;
    std::vector<float> x(c.dim), xb(c.dim), xb2(c.dim), q(q_dim), k(kv_dim), v(kv_dim), att(q_dim), hb(c.hidden_dim),
        hb2(c.hidden_dim), scores(static_cast<size_t>(c.n_heads) * c.max_seq_len);
    for (uint32_t i = 0; i < c.dim; ++i) x[i] = f16_to_f32(c.embed[static_cast<size_t>(token) * c.dim + i]);
    const uint32_t kv_sink = pos >= c.max_seq_len ? kKvSink : 0;
    const uint32_t kv_pos = kv_sink + ((pos - kv_sink) % (c.max_seq_len - kv_sink));
    const uint32_t kv_len = pos >= c.max_seq_len ? c.max_seq_len : pos + 1;
    const uint32_t rotary_dim = c.rotary_dim ? c.rotary_dim : c.head_dim;
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        uint16_t* kc = k_cache + static_cast<size_t>(l) * c.max_seq_len * kv_dim;
        uint16_t* vc = v_cache + static_cast<size_t>(l) * c.max_seq_len * kv_dim;
        rmsnorm(xb.data(), x.data(), c.rms_att + static_cast<size_t>(l) * c.dim, c.dim, c.norm_eps);
        matmul(q.data(), xb.data(), c.wq + static_cast<size_t>(l) * q_dim * c.dim, c.dim, q_dim);
        matmul(k.data(), xb.data(), c.wk + static_cast<size_t>(l) * kv_dim * c.dim, c.dim, kv_dim);
        matmul(v.data(), xb.data(), c.wv + static_cast<size_t>(l) * kv_dim * c.dim, c.dim, kv_dim);
        if (c.qkv_clip > 0.f) {
            for (auto& e : q) e = std::min(std::max(e, -c.qkv_clip), c.qkv_clip);
            for (auto& e : k) e = std::min(std::max(e, -c.qkv_clip), c.qkv_clip);
            for (auto& e : v) e = std::min(std::max(e, -c.qkv_clip), c.qkv_clip);
        }
        ref_rope_kv_insert(q.data(), k.data(), v.data(), kc, vc, c.n_heads, c.n_kv_heads, c.head_dim, rotary_dim,
                           c.rope_theta, pos, kv_pos, kv_sink);
        ref_attn_decode_seq(att.data(), scores.data(), c.max_seq_len, q.data(), kc, vc, c.n_heads, c.n_kv_heads,
                            c.head_dim, kv_len);
        matmul(xb.data(), att.data(), c.wo + static_cast<size_t>(l) * c.dim * q_dim, q_dim, c.dim);
        for (uint32_t i = 0; i < c.dim; ++i) x[i] += xb[i];
        rmsnorm(xb.data(), x.data(), c.rms_ffn + static_cast<size_t>(l) * c.dim, c.dim, c.norm_eps);
        const size_t ffn = static_cast<size_t>(l) * c.hidden_dim * c.dim;
        matmul(hb.data(), xb.data(), c.w1 + ffn, c.dim, c.hidden_dim);
        matmul(hb2.data(), xb.data(), c.w3 + ffn, c.dim, c.hidden_dim);
        for (uint32_t i = 0; i < c.hidden_dim; ++i) hb[i] = silu(hb[i]) * hb2[i];
        matmul(xb2.data(), hb.data(), c.w2 + ffn, c.hidden_dim, c.dim);
        for (uint32_t i = 0; i < c.dim; ++i) x[i] += xb2[i] * 1.F;
    }
    if (!logits) return;  // prefill mode: no classifier (model.cpp:74-76)
    rmsnorm(x.data(), c.rms_final, c.dim, c.norm_eps);
    matmul(logits, x.data(), c.wcls, c.dim, c.vocab_size);
}
}  // namespace

// Greedy generation of one sequence, token at a time (tools/infer.cpp:271-300 without the end-of-sequence stop):
// out_tokens [n_new]; out_logits optional [n_new][vocab] (the logits each token was picked from). Returns 0.
extern "C" int ref_generate_greedy(const LlamaModel* m, const uint32_t* prompt, uint32_t n_prompt, uint32_t n_new,
                                   uint32_t* out_tokens, float* out_logits) {
    if (!m || !prompt || n_prompt == 0 || !out_tokens) return -1;
    const size_t cache = static_cast<size_t>(m->n_layers) * m->max_seq_len * m->n_kv_heads * m->head_dim;
    std::vector<uint16_t> k_cache(cache), v_cache(cache);
    std::vector<float> logits(m->vocab_size);
    for (uint32_t pos = 0; pos < n_prompt; ++pos) {
        forward_token(*m, k_cache.data(), v_cache.data(), prompt[pos], pos, pos + 1 == n_prompt ? logits.data() : nullptr);
    }
    for (uint32_t i = 0; i < n_new; ++i) {
        uint32_t max_i = 0;
        float max_val = logits[0];
        for (uint32_t t = 1; t < m->vocab_size; ++t) {
            if (logits[t] > max_val) {
                max_val = logits[t];
                max_i = t;
            }
        }
        out_tokens[i] = max_i;
        if (out_logits) std::memcpy(out_logits + static_cast<size_t>(i) * m->vocab_size, logits.data(), logits.size() * sizeof(float));
        if (i + 1 < n_new) forward_token(*m, k_cache.data(), v_cache.data(), max_i, n_prompt + i, logits.data());
    }
    return 0;
}
