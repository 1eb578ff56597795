"""The whole-prompt path on the GPU: the tensor-core projection GEMM (attn_gemm_f16) and the row-wise steps around it,
against the engine's CPU functions (matmul(), rmsnorm(), rope() of include/kernels_cpu.hpp and the SwiGLU of
src/model/block.cpp:206-210) applied one token at a time, the way the engine processes a prompt
(tools/infer.cpp:271-274)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def A(built_lib, pkg):
    import torch
    assert torch.cuda.is_available()
    from llm_infer_b200 import attention
    return attention


def _pair(x):
    """fp32 array -> (hi, lo) fp16 arrays the way the device writes them."""
    x = np.clip(x, -65504, 65504).astype(np.float32)
    hi = x.astype(np.float16)
    lo = (x - hi.astype(np.float32)).astype(np.float16)
    return hi, lo


@pytest.mark.parametrize("m,n_out,k", [(1, 32, 64), (127, 96, 128), (128, 256, 64), (129, 288, 192), (300, 544, 1024),
                                       (1000, 4096, 4096), (513, 6144, 256)])
def test_gemm_against_float64_and_accumulate(A, m, n_out, k):
    import torch
    rng = np.random.default_rng(m + n_out + k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = (rng.standard_normal((n_out, k), dtype=np.float32) * k ** -0.5).astype(np.float16)
    hi, lo = _pair(x)
    a64 = hi.astype(np.float64) + lo.astype(np.float64)
    want = a64 @ w.astype(np.float64).T
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    hid, lod, wd = (torch.from_numpy(t).cuda() for t in (hi, lo, w))
    out = torch.full((m, n_out), float("nan"), device="cuda")
    A.gemm_f16(hid, lod, wd, out=out, status=status)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    scale = np.abs(want).max()
    assert np.isfinite(got).all()
    # fp32 accumulation inside the tensor cores over k / 16 steps: a few 1e-6 of the largest output per 64 columns of k
    tol = 4e-6 * scale * (k / 64) ** 0.5
    assert np.abs(got - want).max() <= tol, "value + residual product"
    # accumulate on top, without the residual term, into a strided output
    wide = torch.zeros((m, n_out + 32), device="cuda")
    view = wide[:, :n_out]
    view.copy_(out)
    A.gemm_f16(hid, None, wd, out=view, accumulate=True, status=status)
    torch.cuda.synchronize()
    want2 = want + hi.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(view.cpu().numpy() - want2).max() <= 2 * tol
    assert bool((wide[:, n_out:] == 0).all()), "nothing written past the row"
    assert int(status.item()) == 0


def test_gemm_rows_equal_the_engine_matmul(A, checker):
    """Each token's row of the GEMM against the engine's own per-token matmul() on the fp32 activations."""
    import torch
    rng = np.random.default_rng(7)
    m, n_out, k = 37, 512, 1024
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = (rng.standard_normal((n_out, k), dtype=np.float32) * 0.03).astype(np.float16)
    hi, lo = A.split_pair(torch.from_numpy(x).cuda())
    out = torch.empty((m, n_out), device="cuda")
    A.gemm_f16(hi, lo, torch.from_numpy(w).cuda(), out=out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    for t in (0, 5, 36):
        want = checker.matmul_clip(x[t], w, 0.0)  # itself a sequential fp32 sum over 1024 terms (~1e-5 of its own)
        np.testing.assert_allclose(got[t], want, rtol=0, atol=3e-5 * np.abs(want).max())


def test_row_steps_against_the_cpu_functions(A, checker, port, pkg):
    import torch
    from llm_infer_b200 import quant
    rng = np.random.default_rng(9)
    rows, dim, hidden = 21, 1024, 1536
    x = rng.standard_normal((rows, dim), dtype=np.float32) * 2
    wt = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    hi, lo = A.rmsnorm_pair(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), 1e-5)
    got = hi.float().cpu().numpy().astype(np.float64) + lo.float().cpu().numpy()
    for r in (0, 20):
        want = checker.rmsnorm(x[r], wt, 1e-5)
        assert np.abs(got[r] - want).max() <= 4e-6 * np.abs(want).max()
    gu = rng.standard_normal((rows, 2 * hidden), dtype=np.float32) * 3
    hi, lo = A.swiglu_pair(torch.from_numpy(gu).cuda())
    got = hi.float().cpu().numpy().astype(np.float64) + lo.float().cpu().numpy()
    want = port.swiglu(gu[:, :hidden].copy(), gu[:, hidden:].copy())
    assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()
    wq = quant.quantize_q8_0(rng.standard_normal((48, 256), dtype=np.float32) * 0.05)
    hi, lo = A.dequant_q8_0_pair(torch.from_numpy(wq).cuda())
    got = hi.float().cpu().numpy().astype(np.float64) + lo.float().cpu().numpy()
    want = quant.dequantize_q8_0(wq)
    assert np.abs(got - want).max() <= 2.0 ** -21 * np.abs(want).max()
    idx = torch.tensor([20, 0, 7], dtype=torch.int32, device="cuda")
    out = torch.empty((3, dim), device="cuda")
    A.gather_rows(torch.from_numpy(x).cuda(), idx, out=out)
    assert np.array_equal(out.cpu().numpy(), x[[20, 0, 7]])


@pytest.mark.parametrize("D,rot,clip", [(128, 128, 0.0), (128, 64, 1.5), (64, 64, 0.0)])
def test_rope_prompt_fills_the_caches_like_the_per_token_loop(A, checker, D, rot, clip):
    """Two sequences of 5 and 3 prompt tokens packed into 8 rows: rotated q, and the K / V cache rows, against the
    engine's rope + insert (src/model/block.cpp:140-148) run token by token."""
    import torch
    rng = np.random.default_rng(D + rot)
    H, Hkv, T, theta = 4, 2, 16, 500000.0
    lens = [5, 3]
    tokens = sum(lens)
    qkv = rng.standard_normal((tokens, (H + 2 * Hkv) * D), dtype=np.float32) * 2
    seq = np.repeat(np.arange(2, dtype=np.int32), lens)
    pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
    kc = torch.zeros((2, T, Hkv, D), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    q16 = torch.empty((tokens, H, D), dtype=torch.float16, device="cuda")
    A.rope_prompt(torch.from_numpy(qkv).cuda(), q16, kc, vc, torch.from_numpy(seq).cuda(), torch.from_numpy(pos).cuda(),
                  n_heads=H, theta=theta, rotary_dim=0 if rot == D else rot, qkv_clip=clip)
    torch.cuda.synchronize()
    src = np.clip(qkv, -clip, clip) if clip > 0 else qkv
    want_k = np.zeros((2, T, Hkv, D), dtype=np.float16)
    want_v = np.zeros_like(want_k)
    for t in range(tokens):
        q = src[t, :H * D].reshape(H, D)
        k = src[t, H * D:(H + Hkv) * D].reshape(Hkv, D)
        v = src[t, (H + Hkv) * D:].reshape(Hkv, D)
        q_rot, _ = checker.rope_kv_insert(q, k, v, want_k[seq[t]], want_v[seq[t]], int(pos[t]), int(pos[t]), theta=theta,
                                          rotary_dim=rot)
        got_q = q16[t].float().cpu().numpy()
        assert np.abs(got_q - q_rot).max() <= 2.0 ** -10 * max(1.0, np.abs(q_rot).max())
    gk, gv = kc.cpu().numpy(), vc.cpu().numpy()
    assert np.array_equal(gv.view(np.uint16), want_v.view(np.uint16))
    diff = np.abs(gk.astype(np.float32) - want_k.astype(np.float32))
    assert (diff <= np.maximum(np.abs(want_k.astype(np.float32)), 2.0 ** -14) * 2.0 ** -10).all()
    assert (gk.view(np.uint16) == want_k.view(np.uint16)).mean() > 0.97
