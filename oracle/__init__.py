"""ctypes access to the CPU checkers. Test infrastructure only.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product library never does, and it has no CPU fallback.

Two libraries are exposed with the same Python-level interface:

* ``Oracle("port")``      -> ``oracle/liboracle_attn.so``, the plain-C restatement
  (``attn_oracle.c``) of the reference's ``attn()``/``softmax()``
  (include/kernels_cpu.hpp:122-167) and of its state merge (src/attention.cu:41-65).
* ``Oracle("reference")`` -> ``oracle/_ref/libref_attn.so``, the reference's own
  header compiled unmodified behind a small driver (``ref_driver.cpp``).

``best()`` returns the compiled reference when it has been built, else the port.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(_HERE, "liboracle_attn.so")
REF_SO = os.path.join(_HERE, "_ref", "libref_attn.so")

_f32p = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)


class LlamaModelStruct(C.Structure):
    """Field-for-field the LlamaModel struct of attn_oracle.c / ref_driver.cpp."""
    _fields_ = [(n, C.c_uint32) for n in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "head_dim",
                                          "vocab_size", "max_seq_len", "rotary_dim")] + \
               [(n, C.c_float) for n in ("norm_eps", "rope_theta", "qkv_clip")] + \
               [(n, C.c_void_p) for n in ("embed", "wcls", "rms_final", "rms_att", "rms_ffn", "wq", "wk", "wv", "wo",
                                          "w1", "w2", "w3")] + [("weight_type", C.c_uint32)]
_u32p = C.POINTER(C.c_uint32)


def build(reference_dir: str | None = None, quiet: bool = True) -> None:
    """Compile the port (always) and the reference driver (when a checkout is given)."""
    out = subprocess.DEVNULL if quiet else None
    subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=out)
    if reference_dir and os.path.exists(os.path.join(reference_dir, "include", "kernels_cpu.hpp")):
        subprocess.check_call(["make", "-C", _HERE, "ref", f"REFERENCE_DIR={reference_dir}"], stdout=out)


def _ptr(a: np.ndarray, typ):
    return a.ctypes.data_as(typ)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u16(a) -> np.ndarray:
    a = np.asarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, "K/V must be fp16 (or their uint16 bit patterns)"
    return np.ascontiguousarray(a)


class Oracle:
    def __init__(self, kind: str = "port"):
        assert kind in ("port", "reference")
        self.kind = kind
        path = PORT_SO if kind == "port" else REF_SO
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is not built (python -c 'import oracle; oracle.build()')")
        self.lib = C.CDLL(path)
        L = self.lib
        if kind == "port":
            L.oracle_f16_to_f32.restype = C.c_float
            L.oracle_f16_to_f32.argtypes = [C.c_uint16]
            L.oracle_f32_to_f16.restype = C.c_uint16
            L.oracle_f32_to_f16.argtypes = [C.c_float]
            L.oracle_bf16_to_f32.restype = C.c_float
            L.oracle_bf16_to_f32.argtypes = [C.c_uint16]
            L.oracle_f32_to_bf16.restype = C.c_uint16
            L.oracle_f32_to_bf16.argtypes = [C.c_float]
            L.oracle_f32_to_f16_array.argtypes = [_f32p, _u16p, C.c_size_t]
            L.oracle_softmax.argtypes = [_f32p, C.c_uint32]
            L.oracle_num_threads.restype = C.c_int
            L.oracle_attn_decode.restype = C.c_int
            L.oracle_attn_decode.argtypes = [_f32p, _f32p, _u16p, _u16p, _u32p, C.c_uint32, C.c_uint32, C.c_uint32,
                                             C.c_uint32, C.c_size_t, C.c_size_t]
            L.oracle_attn_prefill_causal.restype = C.c_int
            L.oracle_attn_prefill_causal.argtypes = [_f32p, _f32p, _u16p, _u16p] + [C.c_uint32] * 7
            L.oracle_state_from_rows.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, _u16p, _u16p, C.c_uint32,
                                                 C.c_uint32, C.c_size_t, C.c_uint32, C.c_uint32]
            L.oracle_state_merge.argtypes = [_f32p, _f32p, _f32p, C.c_float, C.c_float, _f32p, C.c_uint32]
            L.oracle_lse_merge.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, _f32p, C.c_uint32, C.c_uint32]
            L.oracle_attn_decode_sharded.restype = C.c_int
            L.oracle_attn_decode_sharded.argtypes = [_f32p, _f32p, _f32p, _f32p, _u16p, _u16p, C.c_uint32,
                                                     C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_size_t]
            L.oracle_matmul_clip.argtypes = [_f32p, _f32p, _u16p, C.c_uint32, C.c_uint32, C.c_float]
            L.oracle_rope_kv_insert.argtypes = [_f32p, _f32p, _f32p, _u16p, _u16p, C.c_uint32, C.c_uint32, C.c_uint32,
                                                C.c_uint32, C.c_float, C.c_uint32, C.c_uint32, C.c_uint32]
            L.oracle_matmul_q8_0.argtypes = [_f32p, _f32p, C.POINTER(C.c_uint8), C.c_uint32, C.c_uint32, C.c_float]
            L.oracle_rmsnorm.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_float]
            L.oracle_swiglu.argtypes = [_f32p, _f32p, C.c_size_t]
            L.oracle_argmax.restype = C.c_uint32
            L.oracle_argmax.argtypes = [_f32p, C.c_uint32]
            L.oracle_generate_greedy.restype = C.c_int
            L.oracle_generate_greedy.argtypes = [C.POINTER(LlamaModelStruct), _u32p, C.c_uint32, C.c_uint32, _u32p,
                                                 _f32p]
        else:
            L.ref_generate_greedy.restype = C.c_int
            L.ref_generate_greedy.argtypes = [C.POINTER(LlamaModelStruct), _u32p, C.c_uint32, C.c_uint32, _u32p, _f32p]
            L.ref_matmul_clip.argtypes = [_f32p, _f32p, _u16p, C.c_uint32, C.c_uint32, C.c_float]
            L.ref_rope_kv_insert.argtypes = [_f32p, _f32p, _f32p, _u16p, _u16p, C.c_uint32, C.c_uint32, C.c_uint32,
                                             C.c_uint32, C.c_float, C.c_uint32, C.c_uint32, C.c_uint32]
            L.ref_f16_to_f32.restype = C.c_float
            L.ref_f16_to_f32.argtypes = [C.c_uint16]
            L.ref_f32_to_f16.restype = C.c_uint16
            L.ref_f32_to_f16.argtypes = [C.c_float]
            L.ref_f32_to_f16_array.argtypes = [_f32p, _u16p, C.c_size_t]
            L.ref_softmax.argtypes = [_f32p, C.c_uint32]
            L.ref_num_threads.restype = C.c_int
            L.ref_attn_decode_batch.restype = C.c_int
            L.ref_attn_decode_batch.argtypes = [_f32p, _f32p, _u16p, _u16p, _u32p] + [C.c_uint32] * 5
            L.ref_attn_prefill_causal_seq.restype = C.c_int
            L.ref_attn_prefill_causal_seq.argtypes = [_f32p, _f32p, _u16p, _u16p] + [C.c_uint32] * 7

    # -- scalars ---------------------------------------------------------
    def num_threads(self) -> int:
        return int(self.lib.oracle_num_threads() if self.kind == "port" else self.lib.ref_num_threads())

    def set_num_threads(self, n: int | None = None) -> int:
        """OpenMP threads for the following calls; None = every core this process may run on (a launcher such as
        torch.distributed.run exports OMP_NUM_THREADS=1 to its workers). Returns the count now in effect."""
        if n is None:
            n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        fn = self.lib.oracle_set_num_threads if self.kind == "port" else self.lib.ref_set_num_threads
        fn.argtypes = [C.c_int]
        fn.restype = None
        fn(int(n))
        return self.num_threads()

    def f32_to_f16(self, x: float) -> int:
        return int(self.lib.oracle_f32_to_f16(x) if self.kind == "port" else self.lib.ref_f32_to_f16(x))

    def f16_to_f32(self, h: int) -> float:
        return float(self.lib.oracle_f16_to_f32(h) if self.kind == "port" else self.lib.ref_f16_to_f32(h))

    def f32_to_f16_array(self, x) -> np.ndarray:
        x = _f32(x)
        out = np.empty(x.shape, dtype=np.uint16)
        fn = self.lib.oracle_f32_to_f16_array if self.kind == "port" else self.lib.ref_f32_to_f16_array
        fn(_ptr(x, _f32p), _ptr(out, _u16p), x.size)
        return out

    def softmax(self, v) -> np.ndarray:
        v = _f32(v).copy()
        fn = self.lib.oracle_softmax if self.kind == "port" else self.lib.ref_softmax
        fn(_ptr(v, _f32p), v.size)
        return v

    # -- decode ----------------------------------------------------------
    def attn_decode(self, q, k, v, kv_len=None) -> np.ndarray:
        """q [B,H,D] (any float dtype, widened to fp32); k, v fp16 [B,T,Hkv,D] -> fp32 [B,H,D]."""
        q = _f32(q)
        k, v = _u16(k), _u16(v)
        B, H, D = q.shape
        _, T, Hkv, _ = k.shape
        assert k.shape == v.shape == (B, T, Hkv, D)
        lens = np.full(B, T, dtype=np.uint32) if kv_len is None else np.ascontiguousarray(kv_len, dtype=np.uint32)
        assert lens.shape == (B,) and int(lens.max(initial=0)) <= T
        out = np.zeros((B, H, D), dtype=np.float32)
        if self.kind == "port":
            rc = self.lib.oracle_attn_decode(_ptr(out, _f32p), _ptr(q, _f32p), _ptr(k, _u16p), _ptr(v, _u16p),
                                             _ptr(lens, _u32p), B, H, Hkv, D, Hkv * D, T * Hkv * D)
        else:
            rc = self.lib.ref_attn_decode_batch(_ptr(out, _f32p), _ptr(q, _f32p), _ptr(k, _u16p), _ptr(v, _u16p),
                                                _ptr(lens, _u32p), B, T, H, Hkv, D)
        if rc != 0:
            raise RuntimeError(f"oracle attn_decode failed: {rc}")
        return out

    # -- prefill ---------------------------------------------------------
    def attn_prefill_causal(self, q, k, v, row_begin=0, row_end=None, row_step=1) -> np.ndarray:
        """q [B,S,H,D]; k, v fp16 [B,S,Hkv,D] -> fp32 [B,S,H,D]; rows not visited are NaN."""
        q = _f32(q)
        k, v = _u16(k), _u16(v)
        B, S, H, D = q.shape
        Hkv = k.shape[2]
        assert k.shape == v.shape == (B, S, Hkv, D)
        row_end = S if row_end is None else row_end
        out = np.full((B, S, H, D), np.nan, dtype=np.float32)
        fn = self.lib.oracle_attn_prefill_causal if self.kind == "port" else self.lib.ref_attn_prefill_causal_seq
        for b in range(B):
            rc = fn(_ptr(out[b], _f32p), _ptr(q[b], _f32p), _ptr(k[b], _u16p), _ptr(v[b], _u16p), S, H, Hkv, D,
                    row_begin, row_end, row_step)
            if rc != 0:
                raise RuntimeError(f"oracle attn_prefill_causal failed: {rc}")
        return out

    # -- weight GEMV --
    def matmul_clip(self, x, w, clip=0.0) -> np.ndarray:
        """x [n] fp32, w [d, n] fp16 -> out [d] fp32 (include/kernels_cpu.hpp:69-80, clamp of block.cpp:130-138)."""
        x = _f32(x)
        w = _u16(w)
        d, n = w.shape
        out = np.zeros(d, dtype=np.float32)
        fn = self.lib.oracle_matmul_clip if self.kind == "port" else self.lib.ref_matmul_clip
        fn(_ptr(out, _f32p), _ptr(x, _f32p), _ptr(w, _u16p), n, d, clip)
        return out

    # -- the small per-token steps (port only; the reference versions run inside generate_greedy) --
    def rmsnorm(self, x, weight, eps) -> np.ndarray:
        x, weight = _f32(x), _f32(weight)
        out = np.empty_like(x)
        fn = self.lib.oracle_rmsnorm if self.kind == "port" else self.lib.ref_rmsnorm
        fn.argtypes = [_f32p, _f32p, _f32p, C.c_uint32, C.c_float]
        fn(_ptr(out, _f32p), _ptr(x, _f32p), _ptr(weight, _f32p), x.size, eps)
        return out

    def swiglu(self, hb, hb2) -> np.ndarray:
        assert self.kind == "port"
        out, hb2 = _f32(hb).copy(), _f32(hb2)
        self.lib.oracle_swiglu(_ptr(out, _f32p), _ptr(hb2, _f32p), out.size)
        return out

    def argmax(self, logits) -> int:
        assert self.kind == "port"
        logits = _f32(logits)
        return int(self.lib.oracle_argmax(_ptr(logits, _f32p), logits.size))

    # -- whole model: greedy generation of one sequence, token at a time --
    def generate_greedy(self, cfg: dict, weights: dict, prompt, n_new: int, want_logits: bool = True):
        """cfg: dim, hidden_dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, max_seq_len, [rotary_dim],
        norm_eps, rope_theta, [qkv_clip]. weights: numpy arrays embed/wcls fp16 [vocab, dim], rms_final [dim],
        rms_att/rms_ffn [L, dim] fp32, wq [L, H*D, dim], wk/wv [L, Hkv*D, dim], wo [L, dim, H*D], w1/w3
        [L, hidden, dim], w2 [L, dim, hidden] fp16. Returns (tokens [n_new], logits [n_new, vocab] or None):
        src/model/model.cpp:60-98 + src/model/block.cpp:105-223 + tools/infer.cpp:64-74,271-300."""
        m = LlamaModelStruct()
        for name in ("dim", "hidden_dim", "n_layers", "n_heads", "n_kv_heads", "head_dim", "vocab_size", "max_seq_len"):
            setattr(m, name, int(cfg[name]))
        m.rotary_dim = int(cfg.get("rotary_dim", 0))
        m.norm_eps, m.rope_theta, m.qkv_clip = float(cfg["norm_eps"]), float(cfg["rope_theta"]), float(cfg.get("qkv_clip", 0.0))
        keep = []
        q8 = cfg.get("weight_type", "f16") == "q8_0"  # matrices are uint8 GGML Q8_0 blocks (port only)
        if q8 and self.kind != "port":
            raise ValueError("the reference has no Q8_0 path")
        m.weight_type = 1 if q8 else 0
        for name in ("embed", "wcls", "wq", "wk", "wv", "wo", "w1", "w2", "w3"):
            a = np.ascontiguousarray(weights[name], dtype=np.uint8) if q8 else _u16(weights[name])
            keep.append(a)
            setattr(m, name, a.ctypes.data)
        for name in ("rms_final", "rms_att", "rms_ffn"):
            a = _f32(weights[name])
            keep.append(a)
            setattr(m, name, a.ctypes.data)
        prompt = np.ascontiguousarray(prompt, dtype=np.uint32)
        tokens = np.zeros(n_new, dtype=np.uint32)
        logits = np.zeros((n_new, m.vocab_size), dtype=np.float32) if want_logits else None
        fn = self.lib.oracle_generate_greedy if self.kind == "port" else self.lib.ref_generate_greedy
        rc = fn(C.byref(m), _ptr(prompt, _u32p), prompt.size, n_new, _ptr(tokens, _u32p),
                _ptr(logits, _f32p) if want_logits else None)
        if rc != 0:
            raise RuntimeError(f"generate_greedy failed: {rc}")
        return tokens, logits

    def matmul_q8_0(self, x, w_blocks, clip=0.0) -> np.ndarray:
        """x [n] fp32, w_blocks uint8 [d, n/32*34] (GGML Q8_0) -> out [d] fp32. Port only: the reference has no Q8_0."""
        assert self.kind == "port"
        x = _f32(x)
        w = np.ascontiguousarray(w_blocks, dtype=np.uint8)
        d, n = w.shape[0], x.size
        assert w.shape[1] == n // 32 * 34
        out = np.zeros(d, dtype=np.float32)
        self.lib.oracle_matmul_q8_0(_ptr(out, _f32p), _ptr(x, _f32p), _ptr(w, C.POINTER(C.c_uint8)), n, d, clip)
        return out

    # -- rotary embedding + cache insert (the step in front of attention) --
    def rope_kv_insert(self, q, k, v, k_cache, v_cache, pos, kv_pos, kv_sink=0, theta=10000.0, rotary_dim=None):
        """One token of one sequence (src/model/block.cpp:140-155). q [H,D], k/v [Hkv,D] fp32; caches fp16
        [T,Hkv,D] are updated in place (as uint16 views). Returns rotated (q, k)."""
        q, k, v = _f32(q).copy(), _f32(k).copy(), _f32(v)
        kc, vc = k_cache.view(np.uint16), v_cache.view(np.uint16)
        assert kc.flags.c_contiguous and vc.flags.c_contiguous
        H, D = q.shape
        Hkv = k.shape[0]
        rot = D if rotary_dim is None else rotary_dim
        fn = self.lib.oracle_rope_kv_insert if self.kind == "port" else self.lib.ref_rope_kv_insert
        fn(_ptr(q, _f32p), _ptr(k, _f32p), _ptr(v, _f32p), _ptr(kc, _u16p), _ptr(vc, _u16p), H, Hkv, D, rot, theta,
           pos, kv_pos, kv_sink)
        return q, k

    # -- state / merge (port only: the reference has them only as device code) --
    def state_from_rows(self, q_head, k, v, kv_head, row_begin, row_end):
        """q_head [D]; k, v fp16 [T,Hkv,D] -> (m, z, o[D]) of rows [row_begin,row_end)."""
        assert self.kind == "port"
        q_head = _f32(q_head)
        k, v = _u16(k), _u16(v)
        T, Hkv, D = k.shape
        m = C.c_float()
        z = C.c_float()
        o = np.zeros(D, dtype=np.float32)
        scores = np.zeros(max(1, row_end - row_begin), dtype=np.float32)
        self.lib.oracle_state_from_rows(C.byref(m), C.byref(z), _ptr(o, _f32p), _ptr(scores, _f32p),
                                        _ptr(q_head, _f32p), _ptr(k, _u16p), _ptr(v, _u16p), kv_head, D, Hkv * D,
                                        row_begin, row_end)
        return float(m.value), float(z.value), o

    def state_merge(self, a, b):
        """(m, z, o) x (m, z, o) -> (m, z, o), formula of src/attention.cu:47-64."""
        assert self.kind == "port"
        m = C.c_float(a[0])
        z = C.c_float(a[1])
        o = _f32(a[2]).copy()
        ob = _f32(b[2])
        self.lib.oracle_state_merge(C.byref(m), C.byref(z), _ptr(o, _f32p), b[0], b[1], _ptr(ob, _f32p), o.size)
        return float(m.value), float(z.value), o

    def lse_merge(self, o_parts, lse_parts):
        """o_parts [n,D], lse_parts [n] -> (out[D], lse)."""
        assert self.kind == "port"
        o_parts = _f32(o_parts)
        lse_parts = _f32(lse_parts)
        n, D = o_parts.shape
        out = np.zeros(D, dtype=np.float32)
        lse = C.c_float()
        self.lib.oracle_lse_merge(_ptr(out, _f32p), C.byref(lse), _ptr(o_parts, _f32p), D, _ptr(lse_parts, _f32p), n,
                                  D)
        return out, float(lse.value)

    def attn_decode_sharded(self, q, k, v, n_shards, kv_len=None):
        """One sequence. q [H,D]; k, v fp16 [T,Hkv,D] -> (out [H,D], part_o [n,H,D], part_lse [n,H])."""
        assert self.kind == "port"
        q = _f32(q)
        k, v = _u16(k), _u16(v)
        H, D = q.shape
        T, Hkv, _ = k.shape
        kv_len = T if kv_len is None else kv_len
        out = np.zeros((H, D), dtype=np.float32)
        po = np.zeros((n_shards, H, D), dtype=np.float32)
        pl = np.zeros((n_shards, H), dtype=np.float32)
        rc = self.lib.oracle_attn_decode_sharded(_ptr(out, _f32p), _ptr(po, _f32p), _ptr(pl, _f32p), _ptr(q, _f32p),
                                                 _ptr(k, _u16p), _ptr(v, _u16p), kv_len, n_shards, H, Hkv, D, Hkv * D)
        if rc != 0:
            raise RuntimeError(f"oracle attn_decode_sharded failed: {rc}")
        return out, po, pl


def have_reference() -> bool:
    return os.path.exists(REF_SO)


def best() -> Oracle:
    """The compiled reference if present, otherwise the C restatement."""
    return Oracle("reference") if have_reference() else Oracle("port")
