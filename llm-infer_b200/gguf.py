"""GGUF v3 files for seed-generated models: a writer whose output the engine's loader accepts, and the matching reader.

The container is the public GGUF v3 format as the engine parses it (src/gguf.cpp:175-262, docs/gguf.md:121-324):
little-endian header ``GGUF``, version 3, tensor count, key-value count; typed key-value pairs; tensor infos (name,
dims with the fastest dimension first, GGML type, offset into the data section); padding to ``general.alignment``
(32); tensor data, each tensor padded to the alignment. The writer emits what the engine requires:
``general.architecture`` = "llama" and ``general.quantization_version`` (src/gguf.cpp:219-229), the ``llama.*`` keys
read at src/gguf.cpp:87-171 including ``llama.vocab_size`` (the loader's fallback for a missing vocab size reads a
string key as an integer and fails), and the tensor names of src/model/model.cpp:25-38 and src/model/block.cpp:18-69
with matrices stored ``[n_in, n_out]`` (n_in fastest, include/kernels_cpu.hpp:75). Matrices are F16 (the type the
engine's loader accepts) or Q8_0 blocks; norm vectors are F32. No tokenizer metadata is written: generation from
token ids does not need it.
"""
from __future__ import annotations

import struct

import numpy as np

MAGIC = 0x46554747  # the bytes "GGUF"
VERSION = 3
ALIGNMENT = 32
# metadata value types
T_UINT32, T_FLOAT32, T_STRING, T_UINT64 = 4, 6, 8, 10
# GGML tensor types (include/gguf.hpp:19-35)
GGML_F32, GGML_F16, GGML_Q8_0 = 0, 1, 8

_LAYER_NAMES = {  # model.py name -> GGUF tensor name inside blk.N.
    "rms_att": "attn_norm.weight", "rms_ffn": "ffn_norm.weight", "wq": "attn_q.weight", "wk": "attn_k.weight",
    "wv": "attn_v.weight", "wo": "attn_output.weight", "w1": "ffn_gate.weight", "w2": "ffn_down.weight",
    "w3": "ffn_up.weight",
}
_GLOBAL_NAMES = {"embed": "token_embd.weight", "rms_final": "output_norm.weight", "wcls": "output.weight"}


def _string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, value) -> bytes:
    head = _string(key) + struct.pack("<I", vtype)
    if vtype == T_UINT32:
        return head + struct.pack("<I", value)
    if vtype == T_UINT64:
        return head + struct.pack("<Q", value)
    if vtype == T_FLOAT32:
        return head + struct.pack("<f", value)
    if vtype == T_STRING:
        return head + _string(value)
    raise ValueError(vtype)


def _pad(n: int) -> int:
    return (ALIGNMENT - n % ALIGNMENT) % ALIGNMENT


def _tensor_list(cfg, weights, weight_type):
    """(gguf name, logical dims fastest-first, ggml type, numpy array of the stored bytes) for every tensor."""
    mat_type = GGML_Q8_0 if weight_type == "q8_0" else GGML_F16
    out = []

    def add(name, arr, logical_shape, is_norm):
        arr = arr.detach().cpu().numpy() if hasattr(arr, "detach") else np.asarray(arr)
        dims = tuple(reversed(logical_shape))
        out.append((name, dims, GGML_F32 if is_norm else mat_type, np.ascontiguousarray(arr)))

    from .model import NORM_NAMES, WEIGHT_SHAPES
    for key, gname in _GLOBAL_NAMES.items():
        add(gname, weights[key], WEIGHT_SHAPES[key](cfg), key in NORM_NAMES)
    for layer in range(cfg.n_layers):
        for key, gname in _LAYER_NAMES.items():
            add(f"blk.{layer}.{gname}", weights[key][layer], WEIGHT_SHAPES[key](cfg)[1:], key in NORM_NAMES)
    return out


def write_gguf(path: str, cfg, weights: dict, weight_type: str = "f16") -> None:
    """cfg: model.ModelConfig; weights: the dict of model.random_weights (torch or numpy), stacked over layers."""
    if weight_type not in ("f16", "q8_0"):
        raise ValueError("weight_type must be 'f16' or 'q8_0'")
    tensors = _tensor_list(cfg, weights, weight_type)
    kvs = [
        _kv("general.architecture", T_STRING, "llama"),
        _kv("general.quantization_version", T_UINT32, 2),
        _kv("general.alignment", T_UINT32, ALIGNMENT),
        _kv("general.name", T_STRING, "seed-generated random-init model"),
        _kv("llama.context_length", T_UINT32, cfg.max_seq_len),
        _kv("llama.embedding_length", T_UINT32, cfg.dim),
        _kv("llama.block_count", T_UINT32, cfg.n_layers),
        _kv("llama.feed_forward_length", T_UINT32, cfg.hidden_dim),
        _kv("llama.rope.dimension_count", T_UINT32, cfg.rotary_dim or cfg.head_dim),
        _kv("llama.attention.head_count", T_UINT32, cfg.n_heads),
        _kv("llama.attention.head_count_kv", T_UINT32, cfg.n_kv_heads),
        _kv("llama.attention.layer_norm_rms_epsilon", T_FLOAT32, cfg.norm_eps),
        _kv("llama.rope.freq_base", T_FLOAT32, cfg.rope_theta),
        _kv("llama.vocab_size", T_UINT32, cfg.vocab_size),
    ]
    infos, offset = [], 0
    for name, dims, gtype, arr in tensors:
        infos.append(_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) +
                     struct.pack("<IQ", gtype, offset))
        offset += arr.nbytes + _pad(arr.nbytes)
    head = struct.pack("<IIQQ", MAGIC, VERSION, len(tensors), len(kvs)) + b"".join(kvs) + b"".join(infos)
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * _pad(len(head)))
        for _, _, _, arr in tensors:
            f.write(arr.tobytes())
            f.write(b"\0" * _pad(arr.nbytes))


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        vals = struct.unpack_from("<" + fmt, self.buf, self.pos)
        self.pos += struct.calcsize("<" + fmt)
        return vals if len(vals) > 1 else vals[0]

    def string(self):
        n = self.take("Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8")
        self.pos += n
        return s


_SCALAR_FMT = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}


def _value(cur, vtype):
    if vtype in _SCALAR_FMT:
        return cur.take(_SCALAR_FMT[vtype])
    if vtype == T_STRING:
        return cur.string()
    if vtype == 9:  # array
        etype, count = cur.take("I"), cur.take("Q")
        return [_value(cur, etype) for _ in range(count)]
    raise ValueError(f"unknown metadata type {vtype}")


def read_gguf(path: str):
    """Returns (model.ModelConfig, weights dict of numpy arrays in the layout of model.random_weights, weight_type).
    The arrays are views of a memory map of the file."""
    from .model import NORM_NAMES, WEIGHT_SHAPES, ModelConfig
    buf = np.memmap(path, dtype=np.uint8, mode="r")
    cur = _Cursor(buf)
    magic, version, n_tensors, n_kv = cur.take("IIQQ")
    if magic != MAGIC or version != VERSION:
        raise ValueError("not a GGUF v3 file")
    meta = {}
    for _ in range(n_kv):
        key = cur.string()
        meta[key] = _value(cur, cur.take("I"))
    if meta.get("general.architecture") != "llama":
        raise ValueError("only the llama architecture is supported")
    infos = {}
    for _ in range(n_tensors):
        name = cur.string()
        nd = cur.take("I")
        dims = [cur.take("Q") for _ in range(nd)]
        gtype, offset = cur.take("IQ")
        infos[name] = (dims, gtype, offset)
    align = meta.get("general.alignment", 32)
    data0 = cur.pos + (align - cur.pos % align) % align
    n_heads = meta["llama.attention.head_count"]
    cfg = ModelConfig(dim=meta["llama.embedding_length"], hidden_dim=meta["llama.feed_forward_length"],
                      n_layers=meta["llama.block_count"], n_heads=n_heads,
                      n_kv_heads=meta.get("llama.attention.head_count_kv", n_heads),
                      head_dim=meta["llama.embedding_length"] // n_heads, vocab_size=meta["llama.vocab_size"],
                      max_seq_len=meta["llama.context_length"],
                      norm_eps=meta["llama.attention.layer_norm_rms_epsilon"],
                      rope_theta=meta.get("llama.rope.freq_base", 10000.0))
    rot = meta.get("llama.rope.dimension_count", cfg.head_dim)
    cfg.rotary_dim = 0 if rot == cfg.head_dim else rot
    mat_types = {infos[n][1] for n in infos if not n.endswith("norm.weight")}
    if mat_types == {GGML_F16}:
        weight_type = "f16"
    elif mat_types == {GGML_Q8_0}:
        weight_type = "q8_0"
    else:
        raise ValueError(f"unsupported tensor types {sorted(mat_types)}: matrices must be all F16 or all Q8_0")

    def fetch(name, logical_shape, is_norm):
        dims, gtype, offset = infos[name]
        if tuple(reversed(dims)) != tuple(logical_shape):
            raise ValueError(f"{name}: dims {dims} do not match the configuration")
        count = int(np.prod(logical_shape))
        if is_norm:
            if gtype != GGML_F32:
                raise ValueError(f"{name}: norm weights must be F32")
            return buf[data0 + offset:data0 + offset + count * 4].view(np.float32).reshape(logical_shape)
        if weight_type == "f16":
            return buf[data0 + offset:data0 + offset + count * 2].view(np.float16).reshape(logical_shape)
        row = logical_shape[-1] // 32 * 34
        stored = tuple(logical_shape[:-1]) + (row,)
        return buf[data0 + offset:data0 + offset + int(np.prod(stored))].reshape(stored)

    weights = {}
    for key, gname in _GLOBAL_NAMES.items():
        weights[key] = fetch(gname, WEIGHT_SHAPES[key](cfg), key in NORM_NAMES)
    for key, gname in _LAYER_NAMES.items():
        weights[key] = np.stack([fetch(f"blk.{layer}.{gname}", WEIGHT_SHAPES[key](cfg)[1:], key in NORM_NAMES)
                                 for layer in range(cfg.n_layers)])
    return cfg, weights, weight_type
