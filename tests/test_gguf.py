"""Seed-generated model files: the GGUF writer against this repository's reader (round trip) and against the engine's
own GGUF parser (src/gguf.cpp compiled unmodified under oracle/_ref, when it is present)."""
import ctypes as C
import os

import numpy as np
import pytest

import oracle

REF_GGUF_SO = os.path.join(os.path.dirname(oracle.__file__), "_ref", "libref_gguf.so")


class RefGgufSummary(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("tensor_count", "context_length", "embedding_length", "block_count",
                                          "feed_forward_length", "rope_dimension_count", "attention_head_count",
                                          "attention_head_count_kv", "vocab_size")] + \
               [("rope_freq_base", C.c_float), ("layer_norm_rms_epsilon", C.c_float), ("alignment", C.c_uint32),
                ("quantization_version", C.c_uint32), ("architecture", C.c_char * 32), ("error", C.c_char * 256)]


@pytest.fixture(scope="module")
def M(pkg):
    from llm_infer_b200 import gguf, model
    return model, gguf


def _small(model, weight_type):
    cfg = model.ModelConfig(dim=256, hidden_dim=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64, vocab_size=300,
                            max_seq_len=128, norm_eps=1e-5, rope_theta=500000.0)
    return cfg, model.random_weights(cfg, 3, weight_type=weight_type)


@pytest.mark.parametrize("weight_type", ["f16", "q8_0"])
def test_round_trip(M, tmp_path, weight_type):
    model, gguf = M
    cfg, w = _small(model, weight_type)
    path = str(tmp_path / "m.gguf")
    gguf.write_gguf(path, cfg, w, weight_type)
    cfg2, w2, wt2 = gguf.read_gguf(path)
    assert wt2 == weight_type
    for k, v in cfg.as_dict().items():  # floats come back as the fp32 values the file holds
        assert getattr(cfg2, k) == (np.float32(v) if isinstance(v, float) else v), k
    for name, t in w.items():
        assert np.array_equal(np.asarray(w2[name]), t.numpy()), name
    assert os.path.getsize(path) % 32 == 0


@pytest.mark.parametrize("weight_type", ["f16", "q8_0"])
def test_engine_parser_reads_what_the_writer_wrote(M, tmp_path, weight_type):
    if not os.path.exists(REF_GGUF_SO):
        pytest.skip("compiled reference GGUF parser not present")
    model, gguf = M
    lib = C.CDLL(REF_GGUF_SO)
    cfg, w = _small(model, weight_type)
    path = str(tmp_path / "m.gguf").encode()
    gguf.write_gguf(path.decode(), cfg, w, weight_type)
    s = RefGgufSummary()
    rc = lib.ref_gguf_open(path, C.byref(s))
    assert rc == 0, s.error.decode()
    assert s.architecture == b"llama" and s.alignment == 32 and s.quantization_version == 2
    assert s.tensor_count == 3 + 9 * cfg.n_layers
    assert (s.context_length, s.embedding_length, s.block_count, s.feed_forward_length) == \
        (cfg.max_seq_len, cfg.dim, cfg.n_layers, cfg.hidden_dim)
    assert (s.attention_head_count, s.attention_head_count_kv, s.vocab_size, s.rope_dimension_count) == \
        (cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size, cfg.head_dim)
    assert s.rope_freq_base == np.float32(cfg.rope_theta) and s.layer_norm_rms_epsilon == np.float32(cfg.norm_eps)
    mat_type = 8 if weight_type == "q8_0" else 1
    lib.ref_gguf_tensor.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32),
                                    C.c_void_p, C.c_uint64]
    checks = [("token_embd.weight", [cfg.dim, cfg.vocab_size], mat_type, w["embed"]),
              ("output_norm.weight", [cfg.dim], 0, w["rms_final"]),
              ("output.weight", [cfg.dim, cfg.vocab_size], mat_type, w["wcls"]),
              ("blk.1.attn_q.weight", [cfg.dim, cfg.n_heads * cfg.head_dim], mat_type, w["wq"][1]),
              ("blk.0.attn_k.weight", [cfg.dim, cfg.n_kv_heads * cfg.head_dim], mat_type, w["wk"][0]),
              ("blk.1.attn_output.weight", [cfg.n_heads * cfg.head_dim, cfg.dim], mat_type, w["wo"][1]),
              ("blk.1.ffn_gate.weight", [cfg.dim, cfg.hidden_dim], mat_type, w["w1"][1]),
              ("blk.0.ffn_up.weight", [cfg.dim, cfg.hidden_dim], mat_type, w["w3"][0]),
              ("blk.1.ffn_down.weight", [cfg.hidden_dim, cfg.dim], mat_type, w["w2"][1]),
              ("blk.1.ffn_norm.weight", [cfg.dim], 0, w["rms_ffn"][1])]
    for name, dims, gtype, tensor in checks:
        want = tensor.numpy().tobytes()
        got_dims = (C.c_uint64 * 4)()
        got_type = C.c_uint32()
        got = (C.c_uint8 * len(want))()
        nd = lib.ref_gguf_tensor(path, name.encode(), got_dims, C.byref(got_type), got, len(want))
        assert nd == len(dims), name
        assert list(got_dims[:nd]) == dims and got_type.value == gtype, (name, list(got_dims[:nd]), got_type.value)
        assert bytes(got) == want, name


def test_engine_parser_rejects_a_file_without_required_keys(M, tmp_path):
    """The writer's required keys are required: dropping general.quantization_version makes the engine's parser throw
    (src/gguf.cpp:224-229)."""
    if not os.path.exists(REF_GGUF_SO):
        pytest.skip("compiled reference GGUF parser not present")
    model, gguf = M
    cfg, w = _small(model, "f16")
    path = str(tmp_path / "m.gguf")
    real_kv = gguf._kv
    try:
        gguf._kv = lambda key, t, v: b"" if key == "general.quantization_version" else real_kv(key, t, v)
        # the key count in the header must shrink with it: patch by writing, then fixing the count
        gguf.write_gguf(path, cfg, w, "f16")
    finally:
        gguf._kv = real_kv
    raw = bytearray(open(path, "rb").read())
    n_kv = int.from_bytes(raw[16:24], "little")
    raw[16:24] = (n_kv - 1).to_bytes(8, "little")
    open(path, "wb").write(bytes(raw))
    s = RefGgufSummary()
    rc = C.CDLL(REF_GGUF_SO).ref_gguf_open(path.encode(), C.byref(s))
    assert rc == -1 and b"quantization_version" in s.error


def test_tiled_q8_0_layout_element_by_element(pkg):
    """The tiled Q8_0 layout (what attn_repack_q8_0_tiled writes) stated one byte at a time, against the vectorised
    writer; 21 rows, so the second row group has padding rows."""
    from llm_infer_b200 import quant
    rng = np.random.default_rng(5)
    rows, n = 21, 512
    blocks = quant.quantize_q8_0(rng.standard_normal((rows, n), dtype=np.float32))
    tiled = quant.repack_q8_0_tiled(blocks)
    nb = n // 32
    assert tiled.shape == ((rows + 15) // 16, nb, 544)
    src = blocks.reshape(rows, nb, 34)
    for rg in range(tiled.shape[0]):
        for blk in range(nb):
            t544 = tiled[rg, blk]
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                for word in range(4):
                    s, half = word >> 1, word & 1
                    row = rg * 16 + g + 8 * half
                    for byte, e in enumerate((0, 2, 1, 3)):
                        want = (src[row, blk, 2 + 16 * s + 4 * t + e] ^ 0x80) if row < rows else 0x80
                        assert t544[16 * lane + 4 * word + byte] == want
            for g in range(8):
                for half in range(2):
                    row = rg * 16 + g + 8 * half
                    want = src[row, blk, :2] if row < rows else np.zeros(2, np.uint8)
                    assert (t544[512 + 4 * g + 2 * half: 512 + 4 * g + 2 * half + 2] == want).all()
