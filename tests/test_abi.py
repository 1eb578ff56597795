"""The C-ABI library: builds for sm_100a without a GPU, loads, exports every
symbol the public header declares, and rejects bad arguments before touching CUDA."""
import ctypes as C
import os
import re

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "llm_infer_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    body = text[text.index('extern "C"'):]
    return set(re.findall(r"\b(attn_[a-z0-9_]+)\s*\(", body))


def test_library_exports_every_declared_symbol(built_lib, pkg):
    declared = _declared_functions()
    assert declared, "no declarations parsed"
    assert declared == set(pkg.binding.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(built_lib, name), name


def test_graph_node_symbol_is_exported(built_lib, pkg):
    """The engine's kernel symbol (include/kernels.cuh:26) and every helper include/kernels_b200.cuh declares."""
    text = open(os.path.join(ROOT, "include", "kernels_b200.cuh")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b((?:attention|kernels_b200)_[a-z0-9_]+)\s*\(", text))
    assert declared == set(pkg.binding.SYMBOL_HELPERS)
    for name in declared:
        assert hasattr(built_lib, name), name
    # the __global__ symbols themselves, under the C++ names the engine's objects refer to (include/kernels.cuh:9-26),
    # e.g. attention(float*, float const*, __half const*, __half const*, unsigned)
    assert "_Z9attentionPfPKfPK6__halfS4_j" in pkg.binding.ENGINE_KERNEL_SYMBOLS
    for name in pkg.binding.ENGINE_KERNEL_SYMBOLS:
        assert hasattr(built_lib, name), name


def test_status_strings(built_lib):
    texts = {built_lib.attn_status_string(c).decode() for c in range(0, -7, -1)}
    assert len(texts) == 7 and "unknown status" not in texts
    assert built_lib.attn_status_string(-99).decode() == "unknown status"


def test_invalid_arguments_are_rejected_without_a_device(built_lib, pkg):
    b = pkg.binding
    assert built_lib.attn_decode(None, None) == -1
    a = b.AttnDecodeArgs()
    assert built_lib.attn_decode(C.byref(a), None) == -1  # null pointers
    a.o = a.q = a.k = a.v = 16
    a.kv_dtype = b.DTYPE_F32
    a.batch, a.n_heads, a.n_kv_heads, a.head_dim = 1, 32, 8, 128
    assert built_lib.attn_decode(C.byref(a), None) == -2  # fp32 KV cache is not a thing
    a.kv_dtype = b.DTYPE_F16
    a.n_heads = 30
    assert built_lib.attn_decode(C.byref(a), None) == -1  # heads not divisible
    a.n_heads, a.batch = 32, 2
    assert built_lib.attn_decode(C.byref(a), None) == -1  # batch > 1 needs a batch stride
    m = b.AttnMergeArgs()
    assert built_lib.attn_merge(C.byref(m), None) == -1
    m.o = m.part_o = m.part_lse = 16
    m.n_parts, m.rows, m.head_dim = 2, 4, 48
    assert built_lib.attn_merge(C.byref(m), None) == -2
    m.head_dim, m.o_part_stride = 128, 514
    assert built_lib.attn_merge(C.byref(m), None) == -3


def test_missing_library_fails_loudly(pkg, monkeypatch, tmp_path):
    b = pkg.binding
    monkeypatch.setattr(b, "_lib", None)
    monkeypatch.setattr(b, "LIB_PATH", str(tmp_path / "nope.so"))
    try:
        b.load()
    except FileNotFoundError as e:
        assert "no fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")


def test_work_split_arithmetic_matches_between_passes():
    """cta_of_tile() is the inverse of the [c*nt/a, (c+1)*nt/a) dealing used by the split pass."""
    for nt, a in ((1, 1), (2, 4), (5, 148), (148, 148), (4096, 148), (8192, 148), (1000, 7), (149, 148)):
        starts = [c * nt // a for c in range(a + 1)]
        for t in range(nt):
            c = ((t + 1) * a - 1) // nt
            assert starts[c] <= t < starts[c + 1], (nt, a, t, c)


def test_ctypes_mirrors_have_the_library_struct_sizes(built_lib, pkg):
    b = pkg.binding
    mirrors = (b.AttnDecodeArgs, b.AttnDecodeShardedArgs, b.AttnPrefillArgs, b.AttnRopeInsertArgs, b.AttnGemvArgs,
               b.AttnMergeArgs, b.AttnGemmArgs, b.AttnRopePromptArgs)
    for index, mirror in enumerate(mirrors):
        assert built_lib.attn_abi_struct_size(index) == C.sizeof(mirror), mirror.__name__
    assert built_lib.attn_abi_struct_size(99) == 0
