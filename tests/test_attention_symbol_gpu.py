"""The engine's own kernel symbol (include/kernels.cuh:26) on the GPU: plain launch and as a
CUDA-graph kernel node whose arguments are refreshed per token, the way the engine's
CudaGraph drives it (include/model/device.hpp:185-247)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib, pkg):
    import torch
    assert torch.cuda.is_available()
    return built_lib, pkg.workloads, torch


def _configure(lib, torch, H, Hkv, D):
    nbytes = lib.attention_workspace_bytes(H, Hkv, D)
    assert nbytes > 0
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.attention_configure(H, Hkv, D, 0.0, ws.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.attn_status_string(rc)
    return ws


@pytest.mark.parametrize("H,Hkv,D,T", [(32, 8, 128, 4096), (32, 4, 64, 512), (32, 8, 128, 37), (8, 1, 128, 300),
                                       (32, 8, 128, 20011), (16, 2, 64, 9001),  # the long ones: two-level merge
                                       (32, 2, 128, 777)])  # 16 query heads per kv head: the general form of the body
def test_plain_launch_matches_cpu_attn(env, checker, H, Hkv, D, T):
    from gpu_util import check_close
    lib, wl, torch = env
    ws = _configure(lib, torch, H, Hkv, D)
    q, k, v = wl.decode_inputs(wl.DecodeShape("sym", 21 + T, 1, H, Hkv, D, T, "f32", "f16"))
    qd, kd, vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
    o = torch.full((H, D), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    want_full = checker.attn_decode(q, k, v)
    for kv_tokens in sorted({T, max(1, T // 3), 1}):
        rc = lib.attention_launch(o.data_ptr(), qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), kv_tokens, stream)
        assert rc == 0
        torch.cuda.synchronize()
        want = want_full if kv_tokens == T else checker.attn_decode(q, k, v, np.array([kv_tokens], np.uint32))
        check_close(wl, o.cpu().numpy(), want[0], f"kv_tokens={kv_tokens}")
    del ws


def test_graph_node_with_per_token_argument_refresh(env, checker):
    from gpu_util import check_close
    lib, wl, torch = env
    H, Hkv, D, T = 32, 8, 128, 1024
    ws = _configure(lib, torch, H, Hkv, D)
    q, k, v = wl.decode_inputs(wl.DecodeShape("graph", 5, 1, H, Hkv, D, T, "f32", "f16"))
    qd, kd, vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
    o = torch.zeros((H, D), device="cuda")

    grid, block, smem = C.c_uint32(), C.c_uint32(), C.c_uint32()
    assert lib.attention_launch_dims(C.byref(grid), C.byref(block), C.byref(smem)) == 0
    assert block.value == 288 and grid.value >= 1 and smem.value > 48 * 1024

    rt = C.CDLL("libcudart.so.12")
    graph, node, gexec = C.c_void_p(), C.c_void_p(), C.c_void_p()
    assert rt.cudaGraphCreate(C.byref(graph), 0) == 0
    rc = lib.attention_graph_add_node(graph, C.byref(node), None, 0, o.data_ptr(), qd.data_ptr(), kd.data_ptr(),
                                      vd.data_ptr(), 100)
    assert rc == 0
    rt.cudaGraphInstantiate.argtypes = [C.c_void_p, C.c_void_p, C.c_ulonglong]
    assert rt.cudaGraphInstantiate(C.byref(gexec), graph, 0) == 0
    rt.cudaGraphLaunch.argtypes = [C.c_void_p, C.c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    for kv_tokens in (100, 101, 640, 1024):  # grid stays frozen; only the arguments change
        rc = lib.attention_graph_exec_update(gexec, node, o.data_ptr(), qd.data_ptr(), kd.data_ptr(), vd.data_ptr(),
                                             kv_tokens)
        assert rc == 0
        assert rt.cudaGraphLaunch(gexec, stream) == 0
        torch.cuda.synchronize()
        want = checker.attn_decode(q, k, v, np.array([kv_tokens], np.uint32))
        check_close(wl, o.cpu().numpy(), want[0], f"graph kv_tokens={kv_tokens}")
    rt.cudaGraphExecDestroy.argtypes = [C.c_void_p]
    rt.cudaGraphDestroy.argtypes = [C.c_void_p]
    rt.cudaGraphExecDestroy(gexec)
    rt.cudaGraphDestroy(graph)
    del ws
