"""attn_decode_static_scratch(): the decode entry point for callers that are not allowed to allocate
device memory (for instance a server whose KV-cache pool already owns all free HBM, so that any later
cudaMalloc may fail or stall the GPU). Its scratch is a fixed array inside the library; everything else
is the same two kernels, so its output must equal attn_decode()'s bit for bit. The file name sorts last
on purpose: a run that stops at the first failure has then already gone through every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _args(b, q, k, v, out, kv_len_uniform, lse=None):
    B, H, D = q.shape
    _, T, Hkv, _ = k.shape
    a = b.AttnDecodeArgs()
    a.o, a.q, a.k, a.v = out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.o_dtype, a.q_dtype, a.kv_dtype = b.DTYPE_F32, b.DTYPE_F16, b.DTYPE_F16
    a.batch, a.n_heads, a.n_kv_heads, a.head_dim = B, H, Hkv, D
    a.kv_len, a.kv_len_uniform = None, kv_len_uniform
    a.kv_row_stride, a.kv_batch_stride = Hkv * D, T * Hkv * D
    a.scale, a.max_ctas = 0.0, 0
    return a


def test_static_scratch_entry_point_matches_attn_decode_twice_in_a_row(built_lib, pkg, checker):
    import torch
    assert torch.cuda.is_available()
    b, wl = pkg.binding, pkg.workloads
    lib = built_lib
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first one's partials in the shared array
    for seed, B, T in ((31, 4, 2000), (32, 2, 517)):
        shape = wl.DecodeShape("noalloc", seed, B, 32, 8, 128, T, "f16", "f16")
        q, k, v = wl.decode_inputs(shape)
        qd, kd, vd = (torch.from_numpy(x).cuda() for x in (q, k, v))

        # existing entry point, caller-provided workspace
        ws_bytes = lib.attn_decode_workspace_bytes(B, 32, 8, 128)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        want = torch.full((B, 32, 128), float("nan"), device="cuda")
        a = _args(b, qd, kd, vd, want, T)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws_bytes
        assert lib.attn_decode(C.byref(a), stream) == 0

        # new entry point: no workspace is passed at all
        got = torch.full((B, 32, 128), float("nan"), device="cuda")
        lse = torch.full((B, 32), float("nan"), device="cuda")
        a2 = _args(b, qd, kd, vd, got, T, lse)
        assert lib.attn_decode_static_scratch(C.byref(a2), stream) == 0
        torch.cuda.synchronize()

        # same kernels, same partial slots: identical bits; and both inside the parity tolerance of the CPU attn()
        assert torch.equal(got, want)
        ref = checker.attn_decode(q.astype(np.float32), k, v)
        max_abs, max_rel = wl.error_metrics(got.cpu().numpy(), ref)
        assert max_abs <= wl.ABS_TOL and max_rel <= wl.REL_TOL, (max_abs, max_rel)
        assert torch.isfinite(lse).all()


def test_static_scratch_entry_point_refuses_shapes_beyond_its_array(built_lib, pkg):
    import torch
    b = pkg.binding
    B, T = 1024, 16  # the partials of 1024 sequences do not fit in the 8 MiB array
    assert built_lib.attn_decode_workspace_bytes(B, 32, 8, 128) > b.STATIC_SCRATCH_BYTES
    q = torch.zeros((B, 32, 128), dtype=torch.float16, device="cuda")
    kv = torch.zeros((B, T, 8, 128), dtype=torch.float16, device="cuda")
    out = torch.zeros((B, 32, 128), device="cuda")
    a = _args(b, q, kv, kv, out, T)
    rc = built_lib.attn_decode_static_scratch(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == -4 and b"workspace" in built_lib.attn_status_string(rc)
    assert built_lib.attn_decode_static_scratch(None, None) == -1
