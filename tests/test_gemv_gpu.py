"""GPU parity of the fp16-weight GEMV against the engine's CPU matmul() (include/kernels_cpu.hpp:69-80, clamp of
src/model/block.cpp:130-138). Floating point with a different summation order: |got - ref| <= 4e-6 * sum_i |x_i w_ji|
(fp32 accumulation of n <= 14336 terms), and the fp16 output form within one fp16 step of the rounded reference."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def attention(built_lib, pkg):
    from llm_infer_b200 import attention as a
    return a


@pytest.mark.parametrize("n,d,batch,clip", [(4096, 4096, 1, 0.0), (4096, 1024, 3, 0.0), (14336, 512, 1, 0.0),
                                            (4096, 777, 8, 0.5), (2048, 33, 2, 0.0), (4096, 14336, 2, 0.0)])
def test_against_cpu_matmul(attention, checker, n, d, batch, clip):
    import torch
    rng = np.random.default_rng(n + d + batch)
    x = rng.standard_normal((batch, n), dtype=np.float32)
    w = (rng.standard_normal((d, n), dtype=np.float32) * 0.03).astype(np.float16)
    got = attention.gemv_f16(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), clip=clip)
    torch.cuda.synchronize()
    got = got.cpu().numpy()
    mag = np.abs(x) @ np.abs(w.astype(np.float32)).T
    for b in range(batch):
        want = checker.matmul_clip(x[b], w, clip)
        assert (np.abs(got[b] - want) <= 4e-6 * mag[b] + 1e-7).all(), (n, d, b)


def test_fp16_result_into_a_strided_cache_row(attention, checker):
    """The f2h form: V = W_v x written as fp16 straight into each sequence's cache row (src/model/block.cu:96-110)."""
    import torch
    rng = np.random.default_rng(3)
    B, n, Hkv, D, T = 4, 4096, 8, 128, 16
    x = rng.standard_normal((B, n), dtype=np.float32)
    w = (rng.standard_normal((Hkv * D, n), dtype=np.float32) * 0.03).astype(np.float16)
    cache = torch.zeros((B, T, Hkv * D), dtype=torch.float16, device="cuda")
    row = 5
    attention.gemv_f16(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), out=cache[:, row, :])
    torch.cuda.synchronize()
    got = cache.cpu().numpy()
    for b in range(B):
        want = checker.matmul_clip(x[b], w).astype(np.float16)
        steps = np.abs(got[b, row].view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
        assert steps.max() <= 1
        assert not got[b, row - 1].any() and not got[b, row + 1].any()  # neighbours untouched


def test_streams_weights_near_hbm_rate(attention):
    """Not a parity test: the FFN-sized projection (14336 x 4096 fp16, 117 MB) must stream at a large fraction of HBM."""
    import torch
    n, d = 4096, 14336
    ws = [torch.randn(d, n, device="cuda").half() for _ in range(3)]  # 352 MB > L2, rotated
    x = torch.randn(1, n, device="cuda")
    out = torch.empty(1, d, device="cuda")
    for i in range(3):
        attention.gemv_f16(x, ws[i % 3], out=out)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(30):
        attention.gemv_f16(x, ws[i % 3], out=out)
    e.record()
    torch.cuda.synchronize()
    gbs = d * n * 2 / (s.elapsed_time(e) / 30 * 1e-3) / 1e9
    print(f"gemv 14336x4096 fp16: {gbs:.0f} GB/s")
    assert gbs > 3000
