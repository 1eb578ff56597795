"""ctypes binding of include/llm_infer_attn.h. No torch types cross this boundary:
pointers are integers (``tensor.data_ptr()``), the stream is ``cudaStream_t`` as an integer.

The library is mandatory: if it is missing or cannot be loaded this module raises;
there is no CPU or PyTorch fallback anywhere in the package.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# LLM_INFER_ATTN_LIB may name another build of the same library (the profiling build of build.py --trace)
LIB_PATH = os.environ.get("LLM_INFER_ATTN_LIB") or os.path.join(HERE, "libllm_infer_attn.so")

ATTN_OK = 0
DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
STATIC_SCRATCH_BYTES = 8 << 20
STATUS_WAIT_TIMEOUT = 1
STATUS_BAD_SHAPE = 2
PREFILL_P_RESIDUAL, PREFILL_P_INPUT_TYPE = 0, 1

# every symbol include/llm_infer_attn.h declares
EXPORTED_SYMBOLS = (
    "attn_decode_workspace_bytes",
    "attn_decode",
    "attn_decode_static_scratch",
    "attn_decode_sharded_exchange_bytes",
    "attn_decode_sharded_cell_floats",
    "attn_decode_sharded",
    "attn_merge",
    "attn_prefill_causal",
    "attn_rope_kv_insert",
    "attn_gemm_f16",
    "attn_rmsnorm_f16pair",
    "attn_split_f16pair",
    "attn_swiglu_f16pair",
    "attn_dequant_q8_0_f16pair",
    "attn_rope_prompt",
    "attn_gather_rows",
    "attn_gemv_f16",
    "attn_gemv_q8_0",
    "attn_gemv_q8_0_tiled",
    "attn_q8_0_tiled_bytes",
    "attn_repack_q8_0_tiled",
    "attn_embed_f16",
    "attn_embed_q8_0",
    "attn_rmsnorm",
    "attn_rmsnorm_residual",
    "attn_rmsnorm_residual_split",
    "attn_swiglu",
    "attn_argmax",
    "attn_status_string",
    "attn_last_cuda_error",
    "attn_kernel_launch_count",
    "attn_abi_struct_size",
)
# include/kernels_b200.cuh
SYMBOL_HELPERS = (
    "attention_workspace_bytes",
    "attention_configure",
    "attention_launch_dims",
    "attention_kernel_function",
    "attention_graph_add_node",
    "attention_graph_exec_update",
    "attention_launch",
    "attention_status",
    "kernels_b200_function",
    "kernels_b200_launch_dims",
    "kernels_b200_copy_embedding",
    "kernels_b200_rmsnorm",
    "kernels_b200_fused_gemv_clip",
    "kernels_b200_rope",
)
# mangled names of the engine's __global__ symbols this library defines (include/kernels.cuh:9-26)
ENGINE_KERNEL_SYMBOLS = (
    "_Z20copy_embedding_floatPfPKfjj",
    "_Z19copy_embedding_halfPfPK6__halfjj",
    "_Z7rmsnormPfPKfS1_jf",
    "_Z15fused_gemv_clipPfPKfPK6__halfjjSt8optionalIfE",
    "_Z19fused_gemv_clip_f2hP6__halfPKfPKS_jjSt8optionalIfE",
    "_Z8rope_f2fPfPKfjjjfj",
    "_Z8rope_f2hP6__halfPKfjjjfj",
    "_Z8rope_h2hP6__halfPKS_jjjfj",
    "_Z9attentionPfPKfPK6__halfS4_j",
)
KERNEL_IDS = {"copy_embedding_float": 0, "copy_embedding_half": 1, "rmsnorm": 2, "fused_gemv_clip": 3,
              "fused_gemv_clip_f2h": 4, "rope_f2f": 5, "rope_f2h": 6, "rope_h2h": 7}


class AttnDecodeArgs(C.Structure):
    _fields_ = [
        ("o", C.c_void_p),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("lse", C.c_void_p),
        ("o_dtype", C.c_int32),
        ("q_dtype", C.c_int32),
        ("kv_dtype", C.c_int32),
        ("batch", C.c_uint32),
        ("n_heads", C.c_uint32),
        ("n_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("kv_len", C.c_void_p),
        ("kv_len_uniform", C.c_uint32),
        ("kv_row_stride", C.c_uint64),
        ("kv_batch_stride", C.c_uint64),
        ("scale", C.c_float),
        ("max_ctas", C.c_uint32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("kv_early", C.c_uint32),
        ("kv_capacity", C.c_uint32),
    ]


MAX_PEERS = 8


class AttnDecodeShardedArgs(C.Structure):
    _fields_ = [
        ("decode", AttnDecodeArgs),
        ("world_size", C.c_uint32),
        ("rank", C.c_uint32),
        ("peer_buffers", C.c_void_p * MAX_PEERS),
        ("step", C.c_uint32),
        ("poll_limit", C.c_uint32),
    ]


class AttnPrefillArgs(C.Structure):
    _fields_ = [
        ("o", C.c_void_p),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("o_dtype", C.c_int32),
        ("dtype", C.c_int32),
        ("batch", C.c_uint32),
        ("seq_len", C.c_uint32),
        ("n_heads", C.c_uint32),
        ("n_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("scale", C.c_float),
        ("p_mode", C.c_uint32),
        ("status", C.c_void_p),
    ]


class AttnRopeInsertArgs(C.Structure):
    _fields_ = [
        ("q_out", C.c_void_p),
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("inv_freq", C.c_void_p),
        ("pos", C.c_void_p),
        ("kv_pos", C.c_void_p),
        ("kv_row_stride", C.c_uint64),
        ("kv_batch_stride", C.c_uint64),
        ("batch", C.c_uint32),
        ("n_heads", C.c_uint32),
        ("n_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("rotary_dim", C.c_uint32),
        ("kv_sink", C.c_uint32),
        ("theta", C.c_float),
        ("q_out_dtype", C.c_int32),
        ("pos_early", C.c_int32),
    ]


class AttnGemvArgs(C.Structure):
    _fields_ = [
        ("out", C.c_void_p),
        ("x", C.c_void_p),
        ("w", C.c_void_p),
        ("out_batch_stride", C.c_uint64),
        ("n", C.c_uint32),
        ("d", C.c_uint32),
        ("batch", C.c_uint32),
        ("clip", C.c_float),
        ("out_dtype", C.c_int32),
        ("accumulate", C.c_int32),
        ("status", C.c_void_p),
        ("out2", C.c_void_p),
        ("out3", C.c_void_p),
        ("out2_batch_stride", C.c_uint64),
        ("out3_batch_stride", C.c_uint64),
        ("split1", C.c_uint32),
        ("split2", C.c_uint32),
        ("swiglu", C.c_int32),
        ("k_split", C.c_uint32),
        ("x_format", C.c_int32),
    ]


class AttnMergeArgs(C.Structure):
    _fields_ = [
        ("o", C.c_void_p),
        ("lse", C.c_void_p),
        ("part_o", C.c_void_p),
        ("part_lse", C.c_void_p),
        ("o_part_stride", C.c_uint64),
        ("lse_part_stride", C.c_uint64),
        ("n_parts", C.c_uint32),
        ("rows", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("o_dtype", C.c_int32),
    ]


class AttnGemmArgs(C.Structure):
    _fields_ = [
        ("c", C.c_void_p),
        ("a_hi", C.c_void_p),
        ("a_lo", C.c_void_p),
        ("w", C.c_void_p),
        ("ldc", C.c_uint64),
        ("m", C.c_uint32),
        ("n_out", C.c_uint32),
        ("k", C.c_uint32),
        ("accumulate", C.c_int32),
        ("status", C.c_void_p),
    ]


class AttnRopePromptArgs(C.Structure):
    _fields_ = [
        ("q_out", C.c_void_p),
        ("qkv", C.c_void_p),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("inv_freq", C.c_void_p),
        ("token_seq", C.c_void_p),
        ("token_pos", C.c_void_p),
        ("ld", C.c_uint64),
        ("kv_row_stride", C.c_uint64),
        ("kv_batch_stride", C.c_uint64),
        ("tokens", C.c_uint32),
        ("n_heads", C.c_uint32),
        ("n_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32),
        ("rotary_dim", C.c_uint32),
        ("theta", C.c_float),
        ("qkv_clip", C.c_float),
    ]


class AttnError(RuntimeError):
    def __init__(self, code: int, what: str, cuda_error: int = 0):
        self.code = code
        self.cuda_error = cuda_error
        extra = f" (cudaError {cuda_error})" if cuda_error else ""
        super().__init__(f"{what}: {code}{extra}")


_lib = None


def load() -> C.CDLL:
    """Load the shared library (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python llm-infer_b200/build.py` "
            "(this package has no fallback path)")
    lib = C.CDLL(LIB_PATH)
    lib.attn_decode_workspace_bytes.restype = C.c_size_t
    lib.attn_decode_workspace_bytes.argtypes = [C.c_uint32] * 4
    lib.attn_decode.restype = C.c_int
    lib.attn_decode.argtypes = [C.POINTER(AttnDecodeArgs), C.c_void_p]
    lib.attn_decode_static_scratch.restype = C.c_int
    lib.attn_decode_static_scratch.argtypes = [C.POINTER(AttnDecodeArgs), C.c_void_p]
    lib.attn_decode_sharded_exchange_bytes.restype = C.c_size_t
    lib.attn_decode_sharded_exchange_bytes.argtypes = [C.c_uint32] * 4
    lib.attn_decode_sharded_cell_floats.restype = C.c_uint32
    lib.attn_decode_sharded_cell_floats.argtypes = [C.c_uint32] * 3
    lib.attn_decode_sharded.restype = C.c_int
    lib.attn_decode_sharded.argtypes = [C.POINTER(AttnDecodeShardedArgs), C.c_void_p]
    lib.attn_prefill_causal.restype = C.c_int
    lib.attn_prefill_causal.argtypes = [C.POINTER(AttnPrefillArgs), C.c_void_p]
    lib.attn_gemv_f16.restype = C.c_int
    lib.attn_gemv_f16.argtypes = [C.POINTER(AttnGemvArgs), C.c_void_p]
    lib.attn_gemv_q8_0.restype = C.c_int
    lib.attn_gemv_q8_0.argtypes = [C.POINTER(AttnGemvArgs), C.c_void_p]
    lib.attn_gemv_q8_0_tiled.restype = C.c_int
    lib.attn_gemv_q8_0_tiled.argtypes = [C.POINTER(AttnGemvArgs), C.c_void_p]
    lib.attn_q8_0_tiled_bytes.restype = C.c_size_t
    lib.attn_q8_0_tiled_bytes.argtypes = [C.c_uint32, C.c_uint32]
    lib.attn_repack_q8_0_tiled.restype = C.c_int
    lib.attn_repack_q8_0_tiled.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    lib.attn_embed_f16.restype = C.c_int
    lib.attn_embed_f16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p,
                                   C.c_void_p]
    lib.attn_embed_q8_0.restype = C.c_int
    lib.attn_embed_q8_0.argtypes = lib.attn_embed_f16.argtypes
    lib.attn_rmsnorm.restype = C.c_int
    lib.attn_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p]
    lib.attn_rmsnorm_residual.restype = C.c_int
    lib.attn_rmsnorm_residual.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint64, C.c_void_p, C.c_uint32,
                                          C.c_uint32, C.c_float, C.c_void_p]
    lib.attn_rmsnorm_residual_split.restype = C.c_int
    lib.attn_rmsnorm_residual_split.argtypes = lib.attn_rmsnorm_residual.argtypes
    lib.attn_swiglu.restype = C.c_int
    lib.attn_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.attn_argmax.restype = C.c_int
    lib.attn_argmax.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    lib.attn_rope_kv_insert.restype = C.c_int
    lib.attn_rope_kv_insert.argtypes = [C.POINTER(AttnRopeInsertArgs), C.c_void_p]
    lib.attn_merge.restype = C.c_int
    lib.attn_merge.argtypes = [C.POINTER(AttnMergeArgs), C.c_void_p]
    lib.attn_gemm_f16.restype = C.c_int
    lib.attn_gemm_f16.argtypes = [C.POINTER(AttnGemmArgs), C.c_void_p]
    lib.attn_rmsnorm_f16pair.restype = C.c_int
    lib.attn_rmsnorm_f16pair.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_float,
                                         C.c_void_p]
    lib.attn_split_f16pair.restype = C.c_int
    lib.attn_split_f16pair.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
    lib.attn_swiglu_f16pair.restype = C.c_int
    lib.attn_swiglu_f16pair.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint64, C.c_void_p]
    lib.attn_dequant_q8_0_f16pair.restype = C.c_int
    lib.attn_dequant_q8_0_f16pair.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint32, C.c_void_p]
    lib.attn_rope_prompt.restype = C.c_int
    lib.attn_rope_prompt.argtypes = [C.POINTER(AttnRopePromptArgs), C.c_void_p]
    lib.attn_gather_rows.restype = C.c_int
    lib.attn_gather_rows.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_void_p]
    lib.attn_status_string.restype = C.c_char_p
    lib.attn_status_string.argtypes = [C.c_int]
    lib.attn_last_cuda_error.restype = C.c_int
    lib.attn_kernel_launch_count.restype = C.c_uint64
    lib.attn_abi_struct_size.restype = C.c_size_t
    lib.attn_abi_struct_size.argtypes = [C.c_int]
    mirrors = (AttnDecodeArgs, AttnDecodeShardedArgs, AttnPrefillArgs, AttnRopeInsertArgs, AttnGemvArgs, AttnMergeArgs,
               AttnGemmArgs, AttnRopePromptArgs)
    for index, mirror in enumerate(mirrors):
        if lib.attn_abi_struct_size(index) != C.sizeof(mirror):
            raise RuntimeError(f"{mirror.__name__}: the ctypes mirror ({C.sizeof(mirror)} bytes) does not match the "
                               f"library ({lib.attn_abi_struct_size(index)} bytes)")
    # include/kernels_b200.cuh: the engine's kernel symbol and its helpers
    lib.attention_workspace_bytes.restype = C.c_size_t
    lib.attention_workspace_bytes.argtypes = [C.c_uint32] * 3
    lib.attention_configure.restype = C.c_int
    lib.attention_configure.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p, C.c_size_t,
                                        C.c_void_p]
    lib.attention_launch_dims.restype = C.c_int
    lib.attention_launch_dims.argtypes = [C.POINTER(C.c_uint32)] * 3
    lib.attention_kernel_function.restype = C.c_void_p
    lib.attention_graph_add_node.restype = C.c_int
    lib.attention_graph_add_node.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                                             C.c_void_p, C.c_void_p, C.c_uint32]
    lib.attention_graph_exec_update.restype = C.c_int
    lib.attention_graph_exec_update.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                C.c_void_p, C.c_uint32]
    lib.attention_status.restype = C.c_int
    lib.attention_status.argtypes = [C.POINTER(C.c_uint32), C.c_int, C.c_void_p]
    u32, vp, f32 = C.c_uint32, C.c_void_p, C.c_float
    lib.kernels_b200_function.restype = vp
    lib.kernels_b200_function.argtypes = [C.c_int]
    lib.kernels_b200_launch_dims.restype = C.c_int
    lib.kernels_b200_launch_dims.argtypes = [C.c_int, u32, C.POINTER(u32), C.POINTER(u32)]
    lib.kernels_b200_copy_embedding.restype = C.c_int
    lib.kernels_b200_copy_embedding.argtypes = [C.c_int, vp, vp, u32, u32, u32, u32, vp, vp, vp]
    lib.kernels_b200_rmsnorm.restype = C.c_int
    lib.kernels_b200_rmsnorm.argtypes = [vp, vp, vp, u32, f32, u32, u32, vp, vp, vp]
    lib.kernels_b200_fused_gemv_clip.restype = C.c_int
    lib.kernels_b200_fused_gemv_clip.argtypes = [C.c_int, vp, vp, vp, u32, u32, C.c_int, f32, u32, u32, vp, vp, vp]
    lib.kernels_b200_rope.restype = C.c_int
    lib.kernels_b200_rope.argtypes = [C.c_int, vp, vp, u32, u32, u32, f32, u32, u32, u32, vp, vp, vp]
    lib.attention_launch.restype = C.c_int
    lib.attention_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    if code != ATTN_OK:
        lib = load()
        msg = lib.attn_status_string(code).decode()
        raise AttnError(code, f"{what}: {msg}", lib.attn_last_cuda_error() if code == -5 else 0)
