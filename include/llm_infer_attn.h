/*
 * C ABI of the B200 (sm_100a) attention path for the llm-infer engine.
 *
 * The engine's CUDA backend declares one attention entry point,
 *
 *     __global__ void attention(float* o, const float* q, const half* k,
 *                               const half* v, uint32_t kv_tokens);
 *                                                   (include/kernels.cuh:26)
 *
 * which no translation unit of the engine defines; its transformer block adds
 * that symbol to a CUDA graph as a kernel node (src/model/block.cu:207-233,
 * include/model/device.hpp:239-247). This library supplies that symbol (see
 * include/kernels_b200.cuh) and, for everything a five-argument kernel cannot
 * express (batches, dtypes, ragged lengths, causal prefill, KV sharded over
 * several GPUs), the host functions below.
 *
 * Conventions of every function here:
 *   - returns ATTN_OK (0) or a negative ATTN_ERR_* code; never throws;
 *   - allocates nothing, frees nothing and never synchronises the device: work
 *     is only enqueued on the stream that is passed in (a cudaStream_t, passed as
 *     void* so that this header needs no CUDA include);
 *   - the caller owns every buffer, as the engine's Tensor<T> does
 *     (include/model/tensor.hpp:29-44);
 *   - K/V caches keep the engine's layout: 16-bit elements,
 *     [row][kv_head][head_dim], one cache per sequence
 *     (include/model/block.hpp:66-67, src/model/block.cpp:71-74);
 *   - results match the engine's CPU attention, attn() in
 *     include/kernels_cpu.hpp:140-167 driven per head as in
 *     src/model/block.cpp:157-164, to 2e-3 absolute / 1e-2 relative.
 */
#ifndef LLM_INFER_ATTN_H
#define LLM_INFER_ATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    ATTN_OK = 0,
    ATTN_ERR_INVALID_ARG = -1,  /* null pointer, zero dimension, n_heads % n_kv_heads != 0 ... */
    ATTN_ERR_UNSUPPORTED = -2,  /* head_dim / group size / dtype combination with no kernel */
    ATTN_ERR_ALIGNMENT = -3,    /* pointer or stride not 16-byte aligned */
    ATTN_ERR_WORKSPACE = -4,    /* workspace missing or smaller than attn_*_workspace_bytes() */
    ATTN_ERR_CUDA = -5,         /* a CUDA runtime call failed; see attn_last_cuda_error() */
    ATTN_ERR_DEVICE = -6        /* not an sm_100 device */
};

enum {
    ATTN_DTYPE_F32 = 0,
    ATTN_DTYPE_F16 = 1,
    ATTN_DTYPE_BF16 = 2,
    /* Activations prepared for the tensor-core GEMV (attn_gemv_q8_0 with x_format = ATTN_DTYPE_SPLIT16): one 32-bit word
     * per element; elements 4r .. 4r+3 of a vector occupy words 4r .. 4r+3 as {fp16(x0) | fp16(x1) << 16,
     * fp16(x2) | fp16(x3) << 16, fp16(x0 - fp16(x0)) | ... << 16, fp16(x2 - fp16(x2)) | ... << 16}: an fp16 value and an
     * fp16 residual per element (~ 22 significant bits), |x| clamped to 65504. A producer that writes its result in
     * this form (attn_decode o_dtype, attn_gemv_q8_0 out_dtype, attn_rmsnorm_residual out_split) saves the consumer
     * the conversion that every CTA of the GEMV would otherwise repeat. */
    ATTN_DTYPE_SPLIT16 = 3
};

/* Bits of the optional device status word (AttnDecodeArgs.status etc.). A kernel
 * ORs a bit in and returns early instead of spinning for ever or trapping. */
enum {
    ATTN_STATUS_OK = 0u,
    ATTN_STATUS_WAIT_TIMEOUT = 1u, /* a bounded wait on a shared-memory barrier ran out */
    ATTN_STATUS_BAD_SHAPE = 2u,    /* device-side shape check failed */
    ATTN_STATUS_BAD_INDEX = 4u     /* checking build (-DATTN_BOUNDS_CHECK) only: an index left its buffer; the access was
                                      skipped */
};

/* Single-token (decode) attention over the KV cache. Replaces the per-head
 * attn() loop of src/model/block.cpp:157-164 for a whole batch at once. */
typedef struct AttnDecodeArgs {
    void* o;       /* out: [batch][n_heads][head_dim], o_dtype */
    const void* q; /* in : [batch][n_heads][head_dim], q_dtype (already RoPE'd), 16-byte aligned */
    const void* k; /* in : kv_dtype, sequence b at k + b*kv_batch_stride, row t at + t*kv_row_stride */
    const void* v; /* in : same geometry as k */
    float* lse;    /* optional out: [batch][n_heads] natural-log sum-exp of the scaled scores
                      (-inf for an empty sequence); NULL to skip */
    int32_t o_dtype;  /* ATTN_DTYPE_F32 | F16 | BF16 | SPLIT16 (32-bit words, n_heads*head_dim a multiple of 4) */
    int32_t q_dtype;  /* ATTN_DTYPE_F32 | F16 | BF16 */
    int32_t kv_dtype; /* ATTN_DTYPE_F16 | BF16 */
    uint32_t batch;
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t head_dim;       /* 64 or 128 */
    const uint32_t* kv_len;  /* device pointer [batch], valid rows per sequence; NULL = kv_len_uniform for all. The
                                values are read on the device and must not exceed the rows the caches hold: the
                                kernel has no capacity to clamp them to */
    uint32_t kv_len_uniform; /* used when kv_len == NULL */
    uint64_t kv_row_stride;   /* elements between rows; 0 = n_kv_heads*head_dim */
    uint64_t kv_batch_stride; /* elements between sequences; may be 0 only when batch == 1 */
    float scale;              /* 0 = 1/sqrt(head_dim), as kernels_cpu.hpp:152 */
    uint32_t max_ctas;        /* upper bound on the CTAs that share the KV rows; 0 = auto */
    void* workspace;          /* device scratch, >= attn_decode_workspace_bytes(), 16-byte aligned */
    size_t workspace_bytes;
    uint32_t* status; /* optional device word, ATTN_STATUS_* bits are ORed in; NULL to skip */
    uint32_t kv_early; /* != 0: the caller vouches that (i) kv_len[] / kv_len_uniform were in place before the previous
                          kernel of the stream was launched and (ii) the only K/V row that kernel (or any kernel still
                          running) writes is each sequence's LAST valid row, kv_len - 1 - true for the engine's step
                          outside the sliding window, where the rotary kernel appends row pos just before attention
                          (src/model/block.cu:147-161, src/model/model.cpp:65-68). The split pass then starts streaming
                          every tile that cannot hold that row before it waits for the previous kernel. 0 = wait first. */
    uint32_t kv_capacity; /* rows each sequence's caches hold (the engine's max_seq_len); 0 = not stated. When stated, a
                             length beyond it (a corrupted kv_len[] entry) is clamped to it on the device and
                             ATTN_STATUS_BAD_SHAPE is ORed into *status, instead of reading past the cache. */
} AttnDecodeArgs;

/* Scratch size for attn_decode with these dimensions on the current device. */
size_t attn_decode_workspace_bytes(uint32_t batch, uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim);

/* Enqueue: split-KV pass (per-CTA partial O and LSE) + merge pass. */
int attn_decode(const AttnDecodeArgs* args, void* stream);

/* Causal prefill attention of whole prompts. The engine has no such kernel: its prefill is the decode step
 * run once per prompt token with kv_len = pos + 1 (tools/infer.cpp:271-274, src/model/model.cpp:68), so row t
 * of the result is attn() (include/kernels_cpu.hpp:140-167) over rows 0..t. Dense layouts, 16-bit inputs:
 *   q, o : [batch][seq_len][n_heads][head_dim]      k, v : [batch][seq_len][n_kv_heads][head_dim]
 * (k, v are the engine's cache layout [row][kv_head][head_dim] per sequence). head_dim 128 or 64. */
typedef struct AttnPrefillArgs {
    void* o;          /* out, o_dtype */
    const void* q;    /* in, dtype */
    const void* k;    /* in, dtype */
    const void* v;    /* in, dtype */
    int32_t o_dtype;  /* ATTN_DTYPE_F32 or the input dtype */
    int32_t dtype;    /* ATTN_DTYPE_F16 | ATTN_DTYPE_BF16 */
    uint32_t batch;
    uint32_t seq_len;
    uint32_t n_heads;
    uint32_t n_kv_heads;
    uint32_t head_dim;
    float scale;      /* 0 = 1/sqrt(head_dim) */
    uint32_t p_mode;  /* how the probabilities P enter the tensor cores for the P.V product (ATTN_PREFILL_P_*) */
    uint32_t* status; /* optional device word for ATTN_STATUS_* bits */
} AttnPrefillArgs;

enum {
    /* P in the input type plus its rounding residual as a second MMA (~2^-17 per element): the mode that meets the
     * parity tolerance on every row, short ones included. The default. */
    ATTN_PREFILL_P_RESIDUAL = 0,
    /* P rounded once to the input type (fp16: 2^-11, bf16: 2^-9 per element): one MMA per key block, two thirds of
     * the tensor work. Within a few 1e-3 absolute, but rows with few keys miss the relative bound (their outputs pass
     * through zero, where the bound is 1e-4 of the output's RMS). */
    ATTN_PREFILL_P_INPUT_TYPE = 1
};

int attn_prefill_causal(const AttnPrefillArgs* args, void* stream);

/* The step in front of decode attention, for a batch of sequences in one launch: rotary embedding of the current
 * token's Q and K (adjacent pairs, freq_i = 1/powf(theta, i/rotary_dim), include/kernels_cpu.hpp:82-100), fp16
 * round-to-nearest-even insert of K and V into cache row kv_pos (src/model/block.cpp:144-148; on the GPU
 * src/model/block.cu:96-110,147-161), and the one-position re-rotation of the first kv_sink cached K rows
 * (src/model/block.cpp:150-155, src/model/block.cu:165-205). */
typedef struct AttnRopeInsertArgs {
    void* q_out;           /* out: rotated q [batch][n_heads][head_dim], q_out_dtype; may be the same buffer as q (fp32) */
    const float* q;        /* in : [batch][n_heads][head_dim] fp32 (InferenceState::q) */
    const float* k;        /* in : [batch][n_kv_heads][head_dim] fp32, before rotation */
    const float* v;        /* in : [batch][n_kv_heads][head_dim] fp32 */
    void* k_cache;         /* fp16, sequence b at + b*kv_batch_stride, row t at + t*kv_row_stride (elements) */
    void* v_cache;
    const float* inv_freq; /* optional device array [rotary_dim/2] = 1/powf(theta, 2i/rotary_dim) computed on the host
                              (bit-identical to the CPU path); NULL = evaluated on the device in double precision */
    const uint32_t* pos;    /* device [batch]: position of the token (rotation angle) */
    const uint32_t* kv_pos; /* device [batch]: cache row that receives the token */
    uint64_t kv_row_stride;   /* 0 = n_kv_heads*head_dim */
    uint64_t kv_batch_stride; /* may be 0 only when batch == 1 */
    uint32_t batch, n_heads, n_kv_heads, head_dim;
    uint32_t rotary_dim;   /* 0 = head_dim */
    uint32_t kv_sink;      /* number of sink rows to re-rotate (KV_SINK = 4 once the window is full, else 0) */
    float theta;
    int32_t q_out_dtype;   /* ATTN_DTYPE_F32 | F16 | BF16 */
    int32_t pos_early;     /* != 0: `pos` was in place before the previous kernel of the stream was launched; the kernel
                              then evaluates its cos/sin table while that kernel may still be running */
} AttnRopeInsertArgs;

int attn_rope_kv_insert(const AttnRopeInsertArgs* args, void* stream);

/* Weight GEMV of the projections around attention: out[b][j] = clamp(sum_i x[b][i] * W[j][i]). Replaces the engine's
 * fused_gemv_clip / fused_gemv_clip_f2h kernels (include/kernels.cuh:13-16, src/kernels.cu:117-136,229-239) and
 * matches its CPU matmul() (include/kernels_cpu.hpp:69-80) with the clamp of src/model/block.cpp:130-138. */
typedef struct AttnGemvArgs {
    void* out;          /* [batch][d] fp32 or fp16, sequence b at out + b*out_batch_stride (elements) */
    const float* x;     /* [batch][n] fp32, dense, 16-byte aligned */
    const void* w;      /* [d][n] fp16, n fastest (GGUF dims [n_in, n_out]), 32-byte aligned (attn_gemv_q8_0: blocks) */
    uint64_t out_batch_stride; /* 0 = d */
    uint32_t n;         /* f16: multiple of 512; when batch*n*4 bytes exceed shared memory the call runs as several launches
                           over column slices (fp32 out and no clamp only). q8_0: multiple of 256 (slices are internal) */
    uint32_t d;
    uint32_t batch;     /* 1 .. 8 */
    float clip;         /* > 0: clamp to [-clip, clip]; 0 = none */
    int32_t out_dtype;  /* ATTN_DTYPE_F32 | ATTN_DTYPE_F16 | (q8_0 only) ATTN_DTYPE_SPLIT16, segment widths multiples of 4 */
    int32_t accumulate; /* != 0 (fp32 out only): out += result, the residual connection of src/model/block.cpp:169-172 */
    uint32_t* status;   /* optional device word: ATTN_STATUS_WAIT_TIMEOUT is ORed in if a bounded wait ran out (Q8_0) */
    /* Optional row segments (0 / NULL = unused): rows [0, split1) go to out, [split1, split2) to out2, [split2, d) to
     * out3, each [batch][segment rows] with its own batch stride (0 = dense). One launch then serves the Q, K and V
     * projections over a stacked [q rows; k rows; v rows] matrix (src/model/block.cpp:123-125). */
    void* out2;
    void* out3;
    uint64_t out2_batch_stride, out3_batch_stride;
    uint32_t split1, split2;
    /* != 0: W holds d gate rows followed by d up rows and out[b][j] = silu(gate_j . x) * (up_j . x), the first half of
     * the SwiGLU FFN in one launch (src/model/block.cpp:198-210). d a multiple of 16, no segments. */
    int32_t swiglu;
    /* > 1 (Q8_0 only): the inner dimension is cut into k_split equal slices computed by separate sets of CTAs; out
     * then receives k_split partial results [k_split][batch][d] (fp32, batch*out_batch_stride floats apart) whose sum
     * is the product. For the FFN down projection of a batch (8 x 14336 activations do not fit in shared memory at
     * once); attn_rmsnorm_residual adds the partials into the residual stream. */
    uint32_t k_split;
    /* ATTN_DTYPE_F32 (0): x is fp32. ATTN_DTYPE_SPLIT16 (q8_0 only): x points at prepared activations, 32-bit words
     * [batch][n] dense, which the kernel copies into shared memory as they are. */
    int32_t x_format;
} AttnGemvArgs;

int attn_gemv_f16(const AttnGemvArgs* args, void* stream);

/* The same GEMV over Q8_0 weights, the public GGML block format: rows of n/32 blocks, a block = little-endian fp16
 * scale + 32 signed bytes (34 bytes), value = scale * q. `w` points at the blocks of row 0 (16-byte aligned), n is a
 * multiple of 256, |x| is clamped to 65504. The engine names the type (include/gguf.hpp:28) but neither loads nor
 * computes it (src/model/config.cpp:11-17,26-34), so there is no reference kernel this one replaces. */
int attn_gemv_q8_0(const AttnGemvArgs* args, void* stream);

/* The same product from a tiled copy of the Q8_0 weights, made once when the model is loaded: same bytes (34 per 32
 * weights), same arithmetic in the same order (results are bit-identical to attn_gemv_q8_0), but every group of
 * 16 rows x 8 blocks is one contiguous 4352-byte tile whose values already sit in the order the kernel's lanes feed
 * the tensor cores, so a pipeline stage is one plain bulk copy and a lane reads its sixteen values of a block with
 * one 16-byte shared-memory load. Layout of tile (row group rg, chunk c) at ((rg * n/256) + c) * 4352: 8 blocks of 544
 * bytes; in a block, lane L = 4 g + t (g < 8, t < 4) owns the 16 bytes at 16 L = four little-endian words
 * {row g, k-step 0}, {row g+8, k-step 0}, {row g, k-step 1}, {row g+8, k-step 1}, a word holding the row's elements
 * 32 blk + 16 s + 4 t + (0, 2, 1, 3) as bytes q + 128; then at 512 + 4 g the fp16 scales of rows g and g + 8. Rows
 * past d in the last group are zeros. With swiglu, d must be a multiple of 16 (the up rows start a row group).
 * `args->w` points at the tiled copy; everything else as attn_gemv_q8_0. */
int attn_gemv_q8_0_tiled(const AttnGemvArgs* args, void* stream);

/* Bytes of the tiled copy of a [d][n] Q8_0 matrix: ceil(d / 16) * (n / 32) * 544. */
size_t attn_q8_0_tiled_bytes(uint32_t d, uint32_t n);

/* dst (16-byte aligned, attn_q8_0_tiled_bytes(d, n) bytes) = the tiled copy of the GGML Q8_0 blocks at src
 * ([d][n/32] blocks, n a multiple of 256). One launch, to be run once per matrix at load time. */
int attn_repack_q8_0_tiled(void* dst, const void* src, uint32_t d, uint32_t n, void* stream);

/* The per-token steps between the GEMVs and attention, for a batch of sequences per launch. They restate on the device
 * the CPU steps of the engine's forward pass, which its CUDA backend does not have yet (the CUDA block ends after
 * attention, src/model/block.cu:235-239; the CUDA model has no final norm or classifier, src/model/model.cu:67-87). */

/* x[b][0..dim) = fp32(table[tokens[b]][0..dim)), fp16 table [vocab][dim] (src/model/model.cpp:101-118). A token id
 * >= vocab is not read: ATTN_STATUS_BAD_SHAPE is ORed into *status (optional) and that row of x is left as it was. */
int attn_embed_f16(float* x, const void* table, const uint32_t* tokens, uint32_t batch, uint32_t dim, uint32_t vocab,
                   uint32_t* status, void* stream);

/* The same from a Q8_0 table: rows of dim/32 GGML blocks (fp16 scale + 32 signed bytes), value = scale * q. */
int attn_embed_q8_0(float* x, const void* table, const uint32_t* tokens, uint32_t batch, uint32_t dim, uint32_t vocab,
                    uint32_t* status, void* stream);

/* out[b][i] = x[b][i] / sqrt(mean_i(x[b][i]^2) + eps) * weight[i]; out may be x (include/kernels_cpu.hpp:43-67). */
int attn_rmsnorm(float* out, const float* x, const float* weight, uint32_t batch, uint32_t dim, float eps, void* stream);

/* The same with the residual connection in front (src/model/block.cpp:219-222 followed by the next norm): first
 * x[b][i] += partials[0][b][i] + partials[1][b][i] + ... (n_partials arrays [batch][dim], partial_stride floats apart,
 * added in that order and written back to x), then out = rmsnorm(x). The partial sums are what attn_gemv_q8_0 leaves
 * with k_split > 1. out must not be x when n_partials > 0. */
int attn_rmsnorm_residual(float* out, float* x, const float* partials, uint32_t n_partials, uint64_t partial_stride,
                          const float* weight, uint32_t batch, uint32_t dim, float eps, void* stream);

/* The same, with the normalised row written as prepared activations (ATTN_DTYPE_SPLIT16 words [batch][dim], dim a
 * multiple of 4) instead of fp32. */
int attn_rmsnorm_residual_split(uint32_t* out_split, float* x, const float* partials, uint32_t n_partials,
                                uint64_t partial_stride, const float* weight, uint32_t batch, uint32_t dim, float eps,
                                void* stream);

/* hb[i] = silu(hb[i]) * hb2[i], silu(x) = x / (1 + expf(-x)), over count elements (src/model/block.cpp:206-210). */
int attn_swiglu(float* hb, const float* hb2, uint64_t count, void* stream);

/* out[b] = first index of the maximum of logits[b][0..vocab) (greedy sampling, tools/infer.cpp:64-74). */
int attn_argmax(uint32_t* out, const float* logits, uint32_t batch, uint32_t vocab, void* stream);

/* ---- Whole prompts at once -------------------------------------------------------------------------------------
 * The engine feeds a prompt one token per forward pass (tools/infer.cpp:271-274). The entry points below process
 * the tokens of all prompts together, rows = tokens packed one sequence after the other: one GEMM per projection on
 * the tensor cores instead of one GEMV per token, attn_prefill_causal() per sequence for the attention, and the
 * row-wise steps in between. Per token the results are those of the engine's forward pass (src/model/block.cpp:105-223).
 * Activations travel between these steps as a PAIR of fp16 matrices, the rounded value and the rounding residual
 * (value + residual carries about 22 bits of the fp32 number), because the tensor cores multiply 16-bit operands and a
 * single rounding (2^-11) would show in the greedy token stream. */

/* C[t][j] (+)= sum_i (a_hi[t][i] + a_lo[t][i]) * w[j][i]: t < m tokens, j < n_out, i < k. a_hi, a_lo fp16 [m][k] and
 * w fp16 [n_out][k] (the engine's weight layout, k fastest), c fp32 with row stride ldc. Replaces, for m tokens at
 * once, matmul() of include/kernels_cpu.hpp:69-80 / fused_gemv_clip of src/kernels.cu:229-239. a_lo may be NULL (one
 * MMA per k-step instead of two): a caller whose weights are not exact in fp16 (Q8_0) makes a second call with the
 * weights' residual, a_lo = NULL and accumulate = 1. k a multiple of 64, n_out a multiple of 32, pointers 16-byte
 * aligned. */
typedef struct AttnGemmArgs {
    float* c;
    const void* a_hi;
    const void* a_lo;
    const void* w;
    uint64_t ldc;        /* floats between rows of c; 0 = n_out */
    uint32_t m, n_out, k;
    int32_t accumulate;  /* != 0: c += product (the residual connections of src/model/block.cpp:169-172,219-222) */
    uint32_t* status;    /* optional device word for ATTN_STATUS_* bits */
} AttnGemmArgs;
int attn_gemm_f16(const AttnGemmArgs* args, void* stream);

/* Row-wise RMSNorm (include/kernels_cpu.hpp:43-67) of x [rows][dim] fp32, written as the fp16 pair hi, lo [rows][dim]. */
int attn_rmsnorm_f16pair(void* hi, void* lo, const float* x, const float* weight, uint32_t rows, uint32_t dim, float eps,
                         void* stream);
/* count fp32 values -> the fp16 pair (count a multiple of 4). */
int attn_split_f16pair(void* hi, void* lo, const float* x, uint64_t count, void* stream);
/* gate_up [rows][ld] fp32 holding the gate projection in columns [0, hidden) and the up projection in
 * [hidden, 2 hidden) -> silu(gate) * up (src/model/block.cpp:206-210) as the fp16 pair [rows][hidden]. ld 0 = 2 hidden. */
int attn_swiglu_f16pair(void* hi, void* lo, const float* gate_up, uint32_t rows, uint32_t hidden, uint64_t ld, void* stream);
/* Q8_0 rows (GGML blocks, see attn_gemv_q8_0) -> value = fp32(scale) * q as the fp16 pair [rows][n]. */
int attn_dequant_q8_0_f16pair(void* hi, void* lo, const void* w, uint64_t rows, uint32_t n, void* stream);

/* Rotary embedding of q and k of every prompt token and fp16 insert of k, v into the token's cache row
 * (src/model/block.cpp:140-148 per token; include/kernels_cpu.hpp:82-120): qkv [tokens][ld] fp32 holds a token's q
 * (n_heads*head_dim), k and v (n_kv_heads*head_dim each) side by side, as the stacked projection leaves them;
 * q_out receives the rotated q as fp16 [tokens][n_heads][head_dim] (what attn_prefill_causal reads). */
typedef struct AttnRopePromptArgs {
    void* q_out;
    const float* qkv;
    void* k_cache;             /* fp16, sequence s at + s*kv_batch_stride, row t at + t*kv_row_stride (elements) */
    void* v_cache;
    const float* inv_freq;     /* optional device [rotary_dim/2], see AttnRopeInsertArgs */
    const uint32_t* token_seq; /* device [tokens]: sequence of each token */
    const uint32_t* token_pos; /* device [tokens]: position = cache row of each token */
    uint64_t ld;               /* 0 = (n_heads + 2 n_kv_heads) * head_dim */
    uint64_t kv_row_stride;    /* 0 = n_kv_heads*head_dim */
    uint64_t kv_batch_stride;
    uint32_t tokens, n_heads, n_kv_heads, head_dim;
    uint32_t rotary_dim;       /* 0 = head_dim */
    float theta;
    float qkv_clip;            /* > 0: q, k, v are clamped to [-clip, clip] before the rotation (block.cpp:130-138) */
} AttnRopePromptArgs;
int attn_rope_prompt(const AttnRopePromptArgs* args, void* stream);

/* out[r][0..dim) = x[rows[r]][0..dim): the last token of every prompt continues into the final norm and classifier. */
int attn_gather_rows(float* out, const float* x, const uint32_t* rows, uint32_t n_rows, uint32_t dim, void* stream);

/* Size of the built-in scratch array used by attn_decode_static_scratch(). */
#define ATTN_STATIC_SCRATCH_BYTES (8u << 20)

/* attn_decode() for callers that may not allocate device memory (no counterpart in the
 * reference, which never got as far as needing scratch: src/attention.cu:369 stops before the
 * cross-CTA reduction). Think of a server that gave all free HBM to its KV-cache pool at start-up,
 * where a later cudaMalloc can fail and stalls the GPU while it runs, or of a host application that
 * lets nobody but its own allocator touch the device heap. args->workspace and
 * args->workspace_bytes are ignored; the partials go into a fixed ATTN_STATIC_SCRATCH_BYTES array
 * that ships inside this library and occupies that much memory on every GPU that loads it, for the
 * life of the process. Inputs and outputs are still the caller's. The function itself calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *   - Shapes that need more scratch than the array holds return ATTN_ERR_WORKSPACE.
 *   - One array per GPU is shared by every call: calls that overlap on the GPU (two streams) race
 *     on it and corrupt each other; run them on one stream or use attn_decode() with a workspace.
 *   - Nothing in the array has to be zero on entry; each call overwrites what it later reads.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress with
 *     that device current); make that first call before any stream capture begins. */
int attn_decode_static_scratch(const AttnDecodeArgs* args, void* stream);

/* Decode with the KV sequence of every sequence sharded across the GPUs of one NVLink box, exchange fused into the
 * merge pass (no counterpart in the reference, which is single-GPU: include/model/device.hpp:54,127-128). Each rank
 * calls this with its own rows in `decode` (same q on every rank). Two launches: the split pass over the local rows,
 * then one kernel whose CTAs each merge the local partials of one cell (an output row, or a 32/64-float slice of it),
 * store the cell's values and the row's LSE into every rank's exchange buffer with plain 64-bit peer stores
 * (each word = fp32 bits | step << 32, so a word is its own arrival flag: no fence, no separate flag), wait (bounded)
 * until the words of the other ranks for that cell carry the current step, and merge the world_size records.
 * decode.o / decode.lse receive the final result on every rank.
 *   peer_buffers[r]: device pointer, valid on THIS GPU, to rank r's exchange buffer (peer-mapped memory, e.g. a
 *                    symmetric allocation); peer_buffers[rank] is this rank's own buffer. Every buffer has
 *                    attn_decode_sharded_exchange_bytes() bytes, is 16-byte aligned and is zero before the first
 *                    step. Layout in 64-bit words: rec[2 (step parity)][world_size (source rank)][cells] with
 *                    cells = batch*n_heads * head_dim/c and c + 1 words per cell (c values, then the LSE),
 *                    c = attn_decode_sharded_cell_floats(); then two control words (steps completed, cells
 *                    finished in the running step).
 *   step           : 0 = the kernel counts steps itself in the exchange buffer (every rank must then make the same
 *                    sequence of calls on its buffer; the launch arguments stay constant, so the call can be
 *                    replayed from a CUDA graph). Otherwise 1, 2, 3, ...: the same value on every rank for the
 *                    same call, consecutive calls using consecutive values (records are double-buffered by the
 *                    parity of the step; a peer can be at most one step ahead, so a record is never overwritten
 *                    before it was read). Restarting the numbering needs freshly zeroed buffers.
 *   poll_limit     : polls per word before a cell gives up with ATTN_STATUS_WAIT_TIMEOUT in decode.status
 *                    (0 = a default of about a second). The context stays usable after a timeout. */
#define ATTN_MAX_PEERS 8
typedef struct AttnDecodeShardedArgs {
    AttnDecodeArgs decode;
    uint32_t world_size; /* 1 .. ATTN_MAX_PEERS */
    uint32_t rank;
    void* peer_buffers[ATTN_MAX_PEERS];
    uint32_t step;
    uint32_t poll_limit;
} AttnDecodeShardedArgs;

size_t attn_decode_sharded_exchange_bytes(uint32_t batch, uint32_t n_heads, uint32_t head_dim, uint32_t world_size);
/* Floats of head_dim per exchange cell for these dimensions (32, 64 or 128; 0 = unsupported head_dim). */
uint32_t attn_decode_sharded_cell_floats(uint32_t batch, uint32_t n_heads, uint32_t head_dim);
int attn_decode_sharded(const AttnDecodeShardedArgs* args, void* stream);

/* Merge of n partial results with the engine's online-softmax state merge
 * (src/attention.cu:41-65) in log-sum-exp form:
 *   out[r] = sum_i w_i * part_o[i][r],  w_i = exp(lse_i[r] - LSE[r]),  LSE = logsumexp_i lse_i[r]
 * for r over rows (= batch * n_heads). Used after an all-gather of per-GPU
 * partials when the KV sequence is sharded across GPUs. A row whose partials
 * are all empty (lse = -inf) yields zeros. */
typedef struct AttnMergeArgs {
    void* o;               /* out: [rows][head_dim], o_dtype */
    float* lse;            /* optional out: [rows] */
    const float* part_o;   /* partial i, row r at part_o + i*o_part_stride + r*head_dim; 16-byte aligned */
    const float* part_lse; /* partial i, row r at part_lse + i*lse_part_stride + r */
    uint64_t o_part_stride;   /* floats, multiple of 4 */
    uint64_t lse_part_stride; /* floats */
    uint32_t n_parts;
    uint32_t rows;
    uint32_t head_dim; /* 32, 64, 128 or 256 */
    int32_t o_dtype;
} AttnMergeArgs;

int attn_merge(const AttnMergeArgs* args, void* stream);

/* Human-readable text for an ATTN_ERR_* code. */
const char* attn_status_string(int code);

/* cudaError_t (as int) of the last failed CUDA call made by this library on the calling thread. */
int attn_last_cuda_error(void);

/* Number of kernels this library has launched from this process (for accounting in benchmarks). */
uint64_t attn_kernel_launch_count(void);

/* sizeof() of an argument structure as this library was compiled, so that a foreign-function binding can check its own
 * mirror of the layout: 0 AttnDecodeArgs, 1 AttnDecodeShardedArgs, 2 AttnPrefillArgs, 3 AttnRopeInsertArgs,
 * 4 AttnGemvArgs, 5 AttnMergeArgs, 6 AttnGemmArgs, 7 AttnRopePromptArgs; 0 for any other index. */
size_t attn_abi_struct_size(int which);

#ifdef __cplusplus
}
#endif
#endif /* LLM_INFER_ATTN_H */
