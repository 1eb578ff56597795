"""Generates tests/golden/*.npz from the reference's own CPU attention.

Run where a checkout of the reference is available and its header has been
compiled into oracle/_ref/libref_attn.so (``make -C oracle ref REFERENCE_DIR=...``):

    python tests/golden/make_golden.py

Every fixture stores its inputs next to the outputs, so the tests that read
them need neither the reference nor any particular random-number stream.
Outputs come from attn() of include/kernels_cpu.hpp:140-167 driven per head as
in src/model/block.cpp:157-164 (decode) and with kv_len = t + 1 per row
(prefill; src/model/model.cpp:68).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = oracle.Oracle("reference")
    rng = np.random.Generator(np.random.PCG64(20240607))

    # ---- decode cases: (name, B, H, Hkv, D, T, kv_len or None)
    decode = [
        ("c1_tinyllama", 1, 32, 4, 64, 512, None),         # the CPU-runnable configuration, seed 0 inputs
        ("gqa4_d128_t67", 1, 16, 4, 128, 67, None),
        ("ragged_b2_d64", 2, 8, 2, 64, 33, [33, 7]),
        ("mha_d64_t17", 1, 4, 4, 64, 17, None),
        ("mqa_d128_t65", 1, 8, 1, 128, 65, [64]),
        ("len1_d128", 3, 16, 4, 128, 4, [1, 2, 4]),
    ]
    out = {}
    for name, B, H, Hkv, D, T, lens in decode:
        if name == "c1_tinyllama":
            g = np.random.Generator(np.random.PCG64(0))
        else:
            g = rng
        q = g.standard_normal((B, H, D), dtype=np.float32)
        k = g.standard_normal((B, T, Hkv, D), dtype=np.float32).astype(np.float16)
        v = g.standard_normal((B, T, Hkv, D), dtype=np.float32).astype(np.float16)
        kv_len = None if lens is None else np.asarray(lens, dtype=np.uint32)
        o = ref.attn_decode(q, k, v, kv_len)
        out[f"{name}.q"] = q
        out[f"{name}.k"] = k
        out[f"{name}.v"] = v
        out[f"{name}.kv_len"] = np.full(B, T, np.uint32) if kv_len is None else kv_len
        out[f"{name}.o"] = o
    np.savez_compressed(os.path.join(HERE, "decode_golden.npz"), **out)

    # ---- causal prefill cases: (name, B, S, H, Hkv, D)
    prefill = [
        ("s48_gqa4_d64", 1, 48, 8, 2, 64),
        ("s40_mqa_d128", 2, 40, 4, 1, 128),
    ]
    out = {}
    for name, B, S, H, Hkv, D in prefill:
        q = rng.standard_normal((B, S, H, D), dtype=np.float32).astype(np.float16)
        k = rng.standard_normal((B, S, Hkv, D), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((B, S, Hkv, D), dtype=np.float32).astype(np.float16)
        o = ref.attn_prefill_causal(q.astype(np.float32), k, v)
        out[f"{name}.q"] = q
        out[f"{name}.k"] = k
        out[f"{name}.v"] = v
        out[f"{name}.o"] = o
    np.savez_compressed(os.path.join(HERE, "prefill_golden.npz"), **out)

    # ---- scalar pins: fp16 rounding of the reference (F16C, round to nearest even) and softmax
    xs = np.concatenate([
        rng.standard_normal(2000).astype(np.float32) * s for s in (1.0, 1e-3, 1e-5, 3e-8, 1e3, 7e4)
    ] + [np.array([0.0, -0.0, 65504.0, 65519.996, 65520.0, 2.0 ** -25, np.nextafter(np.float32(2.0 ** -25), 1),
                   2.0 ** -24, 6.1e-5, np.inf, -np.inf], dtype=np.float32)])
    h = ref.f32_to_f16_array(xs)
    sm_in = (rng.standard_normal(257) * 3).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "scalar_golden.npz"), f32=xs, f16_bits=h, softmax_in=sm_in,
                        softmax_out=ref.softmax(sm_in))
    # ---- rotary embedding + cache insert of one token (src/model/block.cpp:140-155), three positions
    out = {}
    H, Hkv, D, T = 8, 2, 64, 12
    for name, pos, kv_pos, sink, theta in (("early", 5, 5, 0, 10000.0), ("window", 4097, 9, 4, 500000.0),
                                           ("late", 131071, 7, 4, 500000.0)):
        q = rng.standard_normal((H, D), dtype=np.float32)
        k = rng.standard_normal((Hkv, D), dtype=np.float32)
        v = rng.standard_normal((Hkv, D), dtype=np.float32)
        kc = rng.standard_normal((T, Hkv, D), dtype=np.float32).astype(np.float16)
        vc = rng.standard_normal((T, Hkv, D), dtype=np.float32).astype(np.float16)
        out[f"{name}.q"], out[f"{name}.k"], out[f"{name}.v"] = q, k, v
        out[f"{name}.k_cache_in"], out[f"{name}.v_cache_in"] = kc.copy(), vc.copy()
        out[f"{name}.args"] = np.array([pos, kv_pos, sink, theta], dtype=np.float64)
        q_rot, _ = ref.rope_kv_insert(q, k, v, kc, vc, pos, kv_pos, sink, theta)
        out[f"{name}.q_out"], out[f"{name}.k_cache_out"], out[f"{name}.v_cache_out"] = q_rot, kc, vc
    np.savez_compressed(os.path.join(HERE, "rope_golden.npz"), **out)
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
