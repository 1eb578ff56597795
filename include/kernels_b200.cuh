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
 * share of the rows, and the CTA that delivers the last partial merges them
 * (no CTA waits for another).
 */
#ifndef LLM_INFER_KERNELS_B200_CUH
#define LLM_INFER_KERNELS_B200_CUH

#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <stddef.h>
#include <stdint.h>

/* Replaces the undefined declaration at include/kernels.cuh:26. */
__global__ void attention(float* o, const float* q, const half* k, const half* v, uint32_t kv_tokens);

extern "C" {

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

/* Plain stream launch of the same kernel, for callers that do not use graphs. */
int attention_launch(float* o, const float* q, const void* k, const void* v, uint32_t kv_tokens, void* stream);
}

#endif /* LLM_INFER_KERNELS_B200_CUH */
