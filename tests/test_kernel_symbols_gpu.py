"""The engine's other kernel symbols (include/kernels.cuh:9-24) as this library defines them: each one launched with
the geometry the engine's call sites use (src/model/block.cu:25-205: 128-thread blocks, a warp per GEMV output, a
thread per rotary pair, one CTA for the norm) and, as a CUDA-graph kernel node the way the engine's CudaGraph adds
them (include/model/device.hpp:185-217), with the geometry kernels_b200_launch_dims() suggests; results against the
engine's CPU functions (include/kernels_cpu.hpp)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib, pkg):
    import torch
    assert torch.cuda.is_available()
    return built_lib, pkg.binding, torch


class _Graph:
    """A CUDA graph holding one kernel node, launched through the runtime the way the engine's CudaGraph does."""

    def __init__(self):
        self.rt = C.CDLL("libcudart.so.12")
        self.graph, self.node, self.gexec = C.c_void_p(), C.c_void_p(), C.c_void_p()
        assert self.rt.cudaGraphCreate(C.byref(self.graph), 0) == 0

    def launch(self, stream):
        self.rt.cudaGraphInstantiate.argtypes = [C.c_void_p, C.c_void_p, C.c_ulonglong]
        assert self.rt.cudaGraphInstantiate(C.byref(self.gexec), self.graph, 0) == 0
        self.rt.cudaGraphLaunch.argtypes = [C.c_void_p, C.c_void_p]
        assert self.rt.cudaGraphLaunch(self.gexec, stream) == 0

    def close(self):
        self.rt.cudaGraphExecDestroy.argtypes = [C.c_void_p]
        self.rt.cudaGraphDestroy.argtypes = [C.c_void_p]
        if self.gexec:
            self.rt.cudaGraphExecDestroy(self.gexec)
        self.rt.cudaGraphDestroy(self.graph)


def _suggested(lib, which, work):
    grid, block = C.c_uint32(), C.c_uint32()
    assert lib.kernels_b200_launch_dims(which, work, C.byref(grid), C.byref(block)) == 0
    return grid.value, block.value


def _both_ways(lib, torch, which, work, engine_geometry, call):
    """Runs `call(grid, block, graph, node_ptr, stream)` as a plain launch with the engine's geometry and as a graph
    node with the suggested one; yields a label after each so the caller can check the output."""
    stream = torch.cuda.current_stream().cuda_stream
    assert call(engine_geometry[0], engine_geometry[1], None, None, stream) == 0
    torch.cuda.synchronize()
    yield "engine geometry, plain launch"
    g = _Graph()
    grid, block = _suggested(lib, which, work)
    assert call(grid, block, g.graph, C.byref(g.node), None) == 0
    g.launch(stream)
    torch.cuda.synchronize()
    yield f"suggested geometry {grid}x{block}, graph node"
    g.close()


@pytest.mark.parametrize("d,n,clip", [(4096, 4096, 0.0), (1024, 4096, 0.5), (1000, 520, 0.0), (77, 100, 1.0)])
@pytest.mark.parametrize("out_half", [False, True])
def test_fused_gemv_clip(env, checker, d, n, clip, out_half):
    lib, b, torch = env
    rng = np.random.default_rng(d + n)
    x = rng.standard_normal(n, dtype=np.float32)
    w = (rng.standard_normal((d, n), dtype=np.float32) * 0.05).astype(np.float16)
    want = checker.matmul_clip(x, w, clip)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    out = torch.empty(d, dtype=torch.float16 if out_half else torch.float32, device="cuda")
    which = b.KERNEL_IDS["fused_gemv_clip_f2h" if out_half else "fused_gemv_clip"]

    def call(grid, block, graph, node, stream):
        out.fill_(float("nan"))
        return lib.kernels_b200_fused_gemv_clip(int(out_half), out.data_ptr(), xd.data_ptr(), wd.data_ptr(), n, d,
                                                int(clip > 0), clip, grid, block, graph, node, stream)

    engine = ((d * 32 + 127) // 128, 128)  # src/model/block.cu:46-52
    for label in _both_ways(lib, torch, which, d, engine, call):
        got = out.float().cpu().numpy()
        if out_half:
            # the engine stores V with one fp16 rounding of the fp32 sum (src/kernels.cu:133-135)
            np.testing.assert_allclose(got, want.astype(np.float16).astype(np.float32), rtol=2e-3, atol=2e-3, err_msg=label)
        else:
            np.testing.assert_allclose(got, want, rtol=1e-4, atol=2e-4, err_msg=label)
        if clip > 0:
            assert np.abs(got).max() <= clip + 1e-3 and (got <= -clip + 1e-3).any(), "clamp must be two-sided"


def test_rmsnorm(env, checker):
    lib, b, torch = env
    rng = np.random.default_rng(3)
    for size in (4096, 2048, 100):
        x = rng.standard_normal(size, dtype=np.float32) * 3
        w = rng.standard_normal(size, dtype=np.float32)
        want = checker.rmsnorm(x, w, 1e-5)
        xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
        out = torch.empty(size, device="cuda")

        def call(grid, block, graph, node, stream):
            out.fill_(float("nan"))
            return lib.kernels_b200_rmsnorm(out.data_ptr(), xd.data_ptr(), wd.data_ptr(), size, 1e-5, grid, block,
                                            graph, node, stream)

        for label in _both_ways(lib, torch, b.KERNEL_IDS["rmsnorm"], size, (1, 128), call):  # block.cu:28-34
            np.testing.assert_allclose(out.cpu().numpy(), want, rtol=2e-6, atol=1e-6, err_msg=f"{size} {label}")
        # in place, as the final norm of src/model/model.cu:67-86 runs it
        assert lib.kernels_b200_rmsnorm(xd.data_ptr(), xd.data_ptr(), wd.data_ptr(), size, 1e-5, 1, 128, None, None,
                                        torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        np.testing.assert_allclose(xd.cpu().numpy(), want, rtol=2e-6, atol=1e-6)


@pytest.mark.parametrize("half_table", [False, True])
def test_copy_embedding(env, half_table):
    lib, b, torch = env
    rng = np.random.default_rng(5)
    vocab, dim, token = 50, 4096, 37
    table = rng.standard_normal((vocab, dim), dtype=np.float32)
    if half_table:
        table = table.astype(np.float16)
    td = torch.from_numpy(table).cuda()
    out = torch.empty(dim, device="cuda")
    which = b.KERNEL_IDS["copy_embedding_half" if half_table else "copy_embedding_float"]

    def call(grid, block, graph, node, stream):
        out.fill_(float("nan"))
        return lib.kernels_b200_copy_embedding(int(half_table), out.data_ptr(), td.data_ptr(), token, dim, grid, block,
                                               graph, node, stream)

    engine = ((dim // 2 + 255) // 256, 256)  # src/model/model.cu:28-54
    for label in _both_ways(lib, torch, which, dim, engine, call):
        assert np.array_equal(out.cpu().numpy(), table[token].astype(np.float32)), label


@pytest.mark.parametrize("pos", [0, 1, 777, 100_000])
@pytest.mark.parametrize("D,rot", [(128, 128), (64, 32)])
def test_rope_symbols(env, checker, pos, D, rot):
    """rope_f2f on q (in place, as block.cu:124-138), rope_f2h on k straight into a cache row (block.cu:147-161), and
    rope_h2h moving cached rows one position forward (the sink-row rotation of block.cu:165-205), against the CPU
    rope() of include/kernels_cpu.hpp:82-120 driven as src/model/block.cpp:140-155 drives it."""
    lib, b, torch = env
    rng = np.random.default_rng(pos + D)
    H, Hkv, T, theta, sink = 8, 2, 16, 500000.0, 4
    q = rng.standard_normal((H, D), dtype=np.float32)
    k = rng.standard_normal((Hkv, D), dtype=np.float32)
    v = rng.standard_normal((Hkv, D), dtype=np.float32)
    cache0 = rng.standard_normal((T, Hkv, D), dtype=np.float32).astype(np.float16)
    kc, vc = cache0.copy(), cache0.copy()
    kv_pos = 9
    q_want, _ = checker.rope_kv_insert(q, k, v, kc, vc, pos, kv_pos, kv_sink=sink, theta=theta, rotary_dim=rot)

    stream = torch.cuda.current_stream().cuda_stream
    qd = torch.from_numpy(q).cuda()
    kd = torch.from_numpy(k).cuda()
    cache = torch.from_numpy(cache0.copy()).cuda()
    grid = lambda elems: (max(1, (elems // 2 + 127) // 128), 128)  # noqa: E731  (block.cu:118-162)
    g, bl = grid(H * D)
    assert lib.kernels_b200_rope(b.KERNEL_IDS["rope_f2f"], qd.data_ptr(), qd.data_ptr(), H, D, pos, theta, rot, g, bl,
                                 None, None, stream) == 0
    row = cache[kv_pos]
    gr = _Graph()  # K straight into the cache row, as a graph node with the suggested geometry
    sg, sb = _suggested(lib, b.KERNEL_IDS["rope_f2h"], Hkv * D)
    assert lib.kernels_b200_rope(b.KERNEL_IDS["rope_f2h"], row.data_ptr(), kd.data_ptr(), Hkv, D, pos, theta, rot, sg, sb,
                                 gr.graph, C.byref(gr.node), None) == 0
    gr.launch(stream)
    g, bl = grid(sink * Hkv * D)
    assert lib.kernels_b200_rope(b.KERNEL_IDS["rope_h2h"], cache.data_ptr(), cache.data_ptr(), sink * Hkv, D, 1, theta,
                                 rot, g, bl, None, None, stream) == 0
    torch.cuda.synchronize()
    gr.close()
    np.testing.assert_allclose(qd.cpu().numpy(), q_want, rtol=0, atol=4e-6 * max(1.0, np.abs(q_want).max()))
    got = cache.cpu().numpy()
    # fp16 rows: within one fp16 step of the CPU result, nearly all bit-equal
    diff = np.abs(got.astype(np.float32) - kc.astype(np.float32))
    step = np.maximum(np.abs(kc.astype(np.float32)), 2.0 ** -14) * 2.0 ** -10
    assert (diff <= step).all()
    assert (got.view(np.uint16) == kc.view(np.uint16)).mean() > 0.97
    untouched = [r for r in range(T) if r >= sink and r != kv_pos]
    assert np.array_equal(got[untouched], cache0[untouched])


def test_engine_geometry_with_no_sink_rows_does_nothing(env):
    """kv_sink = 0: the engine still launches the node with one thread and n_heads = 0 (block.cu:176-183)."""
    lib, b, torch = env
    buf = torch.full((64,), 3.0, device="cuda")
    assert lib.kernels_b200_rope(b.KERNEL_IDS["rope_f2f"], buf.data_ptr(), buf.data_ptr(), 0, 128, 1, 1e4, 128, 1, 1,
                                 None, None, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert bool((buf == 3.0).all())
