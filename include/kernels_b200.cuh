/*
 * Definition site of the engine's attention kernel symbol for B200 (sm_100a).
 *
 * The engine's include/kernels.cuh:26 declares
 *
 *     __global__ void attention(float* o, const float* q, const half* k,
 *                               const half* v, uint32_t kv_tokens);
 *
 * and its transformer block adds that symbol to a CUDA graph as a kernel node
 * whose grid, block and shared-memory sizes are frozen when the node is first
 * added, while the arguments are refreshed for every token
 * (src/model/block.cu:207-233, include/model/device.hpp:219-247). The kernel
 * defined by this library keeps exactly that signature:
 *
 *   o          out, fp32 [n_heads][head_dim]           (InferenceState::attn_out)
 *   q          in,  fp32 [n_heads][head_dim], rotated   (InferenceState::q)
 *   k, v       in,  fp16 caches [row][n_kv_heads][head_dim] of this layer
 *   kv_tokens  number of valid rows (kv_len of src/model/model.cpp:68)
 *
 * Everything the five arguments cannot carry (head counts, head_dim, scratch for
 * the split-KV partials) is set once per device with attention_configure(); the
 * launch geometry that the graph node must use comes from attention_launch_dims().
 * One launch does both passes: every CTA writes partial (O, LSE) results for its
 * share of the rows, and the CTAs that deliver the last partials merge them - in
 * two levels when a sequence is long (no CTA waits for another).
 */
#ifndef LLM_INFER_KERNELS_B200_CUH
#define LLM_INFER_KERNELS_B200_CUH

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <stddef.h>
#include <stdint.h>

#include <optional>

/* Replaces the undefined declaration at include/kernels.cuh:26.
 *
 * Required node parameters (attention_launch_dims() returns them; the two graph helpers below fill them in):
 *   gridDim  = (number of SMs, 1, 1)     frozen; CTAs without rows exit at once
 *   blockDim = (288, 1, 1)               eight consumer warps and one producer warp
 *   sharedMemBytes = the configured size (about 200 KB; the engine's call site leaves it at 0)
 * A launch with any other block size or with less dynamic shared memory writes nothing but
 * ATTN_STATUS_BAD_SHAPE into the status word (attention_status()) and returns. */
__global__ void attention(float* o, const float* q, const half* k, const half* v, uint32_t kv_tokens);

/* The engine's other kernel symbols, same signatures as include/kernels.cuh:9-24 (which they replace when the engine
 * is linked against this library instead of its own src/kernels.cu). Each one runs correctly under the geometry the
 * engine's call sites give it (src/model/block.cu:25-205, src/model/model.cu:28-86: 128-thread blocks, a warp per
 * GEMV output, a thread per rotary pair, one CTA for the norm) and under any other one-dimensional geometry;
 * kernels_b200_launch_dims() names the one that suits a B200. Numerics follow the engine's CPU path: two-sided clamp
 * (src/model/block.cpp:130-138), x / rms * weight (include/kernels_cpu.hpp:43-67), adjacent-pair rotation with
 * freq = 1 / powf(theta, i / rotary_dim) (include/kernels_cpu.hpp:82-120). No dynamic shared memory. */
__global__ void copy_embedding_float(float* out, const float* token_embedding_table, uint32_t token, uint32_t dim);
__global__ void copy_embedding_half(float* out, const half* token_embedding_table, uint32_t token, uint32_t dim);
__global__ void rmsnorm(float* out, const float* x, const float* weight, uint32_t size, float eps);
__global__ void fused_gemv_clip(float* out, const float* x /* 1xn */, const half* w /* nxd */, uint32_t n, uint32_t d,
                                std::optional<float> clip);
__global__ void fused_gemv_clip_f2h(half* out, const float* x /* 1xn */, const half* w /* nxd */, uint32_t n,
                                    uint32_t d, std::optional<float> clip);
__global__ void rope_f2f(float* out, const float* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta,
                         uint32_t rotary_dim);
__global__ void rope_f2h(half* out, const float* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta,
                         uint32_t rotary_dim);
__global__ void rope_h2h(half* out, const half* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos, float theta,
                         uint32_t rotary_dim);

enum {
    KERNELS_B200_COPY_EMBEDDING_FLOAT = 0,
    KERNELS_B200_COPY_EMBEDDING_HALF = 1,
    KERNELS_B200_RMSNORM = 2,
    KERNELS_B200_FUSED_GEMV_CLIP = 3,
    KERNELS_B200_FUSED_GEMV_CLIP_F2H = 4,
    KERNELS_B200_ROPE_F2F = 5,
    KERNELS_B200_ROPE_F2H = 6,
    KERNELS_B200_ROPE_H2H = 7
};

extern "C" {

/* Host-side address of one of the kernels above for cudaKernelNodeParams::func (KERNELS_B200_* index; NULL for any
 * other). Same caveat as attention_kernel_function(). */
const void* kernels_b200_function(int which);

/* Suggested gridDim.x / blockDim.x for a caller free to choose: `work` = output rows d for the GEMVs, elements
 * (n_heads * head_dim, or dim) for the rotary and embedding kernels, ignored for the norm. */
int kernels_b200_launch_dims(int which, uint32_t work, uint32_t* grid, uint32_t* block);

/* Launch one of the kernels with the given geometry, either on `stream` (graph == NULL) or as a kernel node without
 * dependencies added to `graph` (cudaGraph_t; node_out = cudaGraphNode_t*), the way the engine's
 * CudaGraph::add_or_update_kernel_node does (include/model/device.hpp:185-217). For callers that cannot name the
 * __global__ symbols or std::optional (other languages, other runtime instances). */
int kernels_b200_copy_embedding(int half_table, float* out, const void* table, uint32_t token, uint32_t dim,
                                uint32_t grid, uint32_t block, void* graph, void* node_out, void* stream);
int kernels_b200_rmsnorm(float* out, const float* x, const float* weight, uint32_t size, float eps, uint32_t grid,
                         uint32_t block, void* graph, void* node_out, void* stream);
int kernels_b200_fused_gemv_clip(int out_half, void* out, const float* x, const void* w, uint32_t n, uint32_t d,
                                 int has_clip, float clip, uint32_t grid, uint32_t block, void* graph, void* node_out,
                                 void* stream);
int kernels_b200_rope(int which, void* out, const void* x, uint32_t n_heads, uint32_t head_dim, uint32_t pos,
                      float theta, uint32_t rotary_dim, uint32_t grid, uint32_t block, void* graph, void* node_out,
                      void* stream);

/* Bytes of device scratch attention() needs for these dimensions on the current device
 * (replaces nothing in the engine: its own WIP kernel stopped before the cross-CTA
 * reduction, src/attention.cu:369). 0 = unsupported shape. */
size_t attention_workspace_bytes(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim);

/* Once per device (current device), before the node is added: records the model
 * dimensions of ModelConfig (include/model/config.hpp:30-67) and the zero-initialised
 * scratch buffer in device constant memory. The call zeroes the counters part of the
 * workspace on `stream` and returns ATTN_OK or a negative ATTN_ERR_* code of
 * llm_infer_attn.h. scale = 0 selects 1/sqrt(head_dim) (include/kernels_cpu.hpp:152). */
int attention_configure(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, float scale, void* workspace,
                        size_t workspace_bytes, void* stream);

/* gridDim.x, blockDim.x and dynamic shared-memory bytes for cudaKernelNodeParams
 * (the engine's call site leaves sharedMemBytes at 0; this kernel needs it set). */
int attention_launch_dims(uint32_t* grid, uint32_t* block, uint32_t* shared_mem_bytes);

/* Host-side address of the kernel for cudaKernelNodeParams::func. Valid for a caller that
 * shares this library's CUDA runtime instance (static linking of the objects, or both
 * sides on the shared runtime); other callers use the two graph helpers below. */
const void* attention_kernel_function(void);

/* Adds attention() as a kernel node to `graph` (what CudaGraph::add_or_update_kernel_node
 * does on first use, include/model/device.hpp:185-217). `graph`, `node_out`, `deps` are
 * cudaGraph_t, cudaGraphNode_t*, const cudaGraphNode_t*. */
int attention_graph_add_node(void* graph, void* node_out, const void* deps, size_t n_deps, float* o, const float* q,
                             const void* k, const void* v, uint32_t kv_tokens);

/* Refreshes the node's arguments in an instantiated graph (the per-token
 * cudaGraphExecKernelNodeSetParams of include/model/device.hpp:219-237). */
int attention_graph_exec_update(void* graph_exec, void* node, float* o, const float* q, const void* k, const void* v,
                                uint32_t kv_tokens);

/* Reads (and with clear != 0 resets) the kernel's status word on the current device: ATTN_STATUS_* bits of
 * llm_infer_attn.h that attention() ORs in instead of trapping or spinning for ever: BAD_SHAPE for a launch with the
 * wrong geometry, WAIT_TIMEOUT when a bounded wait ran out (the output is then left untouched; clear the word before
 * the next launch, a set WAIT_TIMEOUT bit keeps later launches from merging). Synchronises `stream`. The engine has no
 * counterpart: its kernels report nothing (include/model/device.hpp:33-43 checks runtime errors only). */
int attention_status(uint32_t* bits, int clear, void* stream);

/* Plain stream launch of the same kernel, for callers that do not use graphs. */
int attention_launch(float* o, const float* q, const void* k, const void* v, uint32_t kv_tokens, void* stream);
}

#endif /* LLM_INFER_KERNELS_B200_CUH */
