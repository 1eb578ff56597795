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
        want32 = checker.matmul_clip(x[b], w)
        want = want32.astype(np.float16)
        # one fp16 step of the rounded reference, or (results near zero, where fp16 steps are tiny) the fp32 bound
        steps = np.abs(got[b, row].view(np.int16).astype(np.int32) - want.view(np.int16).astype(np.int32))
        near = np.abs(got[b, row].astype(np.float32) - want32) <= 4e-6 * (np.abs(x[b]) @ np.abs(w.astype(np.float32)).T) + 1e-3 * np.abs(want32)
        assert ((steps <= 1) | near).all() and (np.abs(got[b, row].astype(np.float32) - want32) <= 2e-3 * np.abs(want32) + 1e-3).all()
        assert not got[b, row - 1].any() and not got[b, row + 1].any()  # neighbours untouched


def _graph_time_us(call, n_buffers, rounds=10):
    """Device time per call with the host's launch cost taken out: the calls over all rotated buffers are captured
    in one CUDA graph and the graph is replayed."""
    import torch
    for i in range(n_buffers):
        call(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph):
            for i in range(n_buffers):
                call(i)
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(rounds):
        graph.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e3 / (rounds * n_buffers)


def test_streams_weights_near_hbm_rate(attention):
    """Not a parity test: the FFN-sized projection (14336 x 4096 fp16, 117 MB) must stream at a large fraction of HBM."""
    import torch
    n, d = 4096, 14336
    ws = [torch.randn(d, n, device="cuda").half() for _ in range(3)]  # 352 MB > L2, rotated
    x = torch.randn(1, n, device="cuda")
    out = torch.empty(1, d, device="cuda")
    us = _graph_time_us(lambda i: attention.gemv_f16(x, ws[i], out=out), 3)
    gbs = (d * n * 2 + n * 4 + d * 4) / us / 1e3
    print(f"gemv 14336x4096 fp16: {us:.1f} us, {gbs:.0f} GB/s")
    assert gbs > 3000


def test_many_sequences_long_inner_dimension_runs_as_column_slices(attention, checker):
    """batch 8 x n 14336 (the FFN down projection of a batch of 8) does not fit in shared memory at once."""
    import torch
    rng = np.random.default_rng(8)
    n, d, batch = 14336, 512, 8
    x = rng.standard_normal((batch, n), dtype=np.float32)
    w = (rng.standard_normal((d, n), dtype=np.float32) * 0.03).astype(np.float16)
    base = rng.standard_normal((batch, d), dtype=np.float32)
    out = torch.from_numpy(base.copy()).cuda()
    attention.gemv_f16(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), out=out, accumulate=True)
    got = out.cpu().numpy()
    mag = np.abs(x) @ np.abs(w.astype(np.float32)).T
    for b in range(batch):
        want = base[b] + checker.matmul_clip(x[b], w, 0.0)
        assert (np.abs(got[b] - want) <= 4e-6 * (mag[b] + np.abs(base[b])) + 1e-7).all()


# ---- Q8_0 weights ----

@pytest.mark.parametrize("n,d,batch,clip", [(4096, 4096, 1, 0.0), (4096, 1024, 3, 0.0), (14336, 512, 1, 0.0),
                                            (4096, 777, 8, 0.5), (256, 33, 2, 0.0), (2048, 14336, 2, 0.0),
                                            (14336, 100, 8, 0.0), (1280, 16, 5, 0.0)])
def test_q8_0_against_cpu_matmul(attention, port, pkg, n, d, batch, clip):
    import torch
    from llm_infer_b200 import quant
    rng = np.random.default_rng(n + d + batch)
    x = rng.standard_normal((batch, n), dtype=np.float32)
    x[0, :7] *= 300.0  # large activations: the fp16 value + residual split must still hold
    blocks = quant.quantize_q8_0(rng.standard_normal((d, n), dtype=np.float32) * 0.03)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = attention.gemv_q8_0(torch.from_numpy(x).cuda(), torch.from_numpy(blocks).cuda(), clip=clip, status=status)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = got.cpu().numpy()
    wf = quant.dequantize_q8_0(blocks)
    mag = np.abs(x) @ np.abs(wf).T
    for b in range(batch):
        want = port.matmul_q8_0(x[b], blocks, clip)
        assert (np.abs(got[b] - want) <= 4e-6 * mag[b] + 1e-7).all(), (n, d, b, np.abs(got[b] - want).max())


@pytest.mark.parametrize("batch", [1, 8])
def test_q8_0_pinned_on_the_engine_matmul_with_fp16_exact_blocks(attention, checker, batch):
    """The engine has no Q8_0 code, so the GPU kernel is pinned on its F16 matmul() (include/kernels_cpu.hpp:69-80)
    directly: blocks whose scale is a power of two dequantise to numbers that are exact in fp16 (|q| <= 127 needs 7
    bits), so the SAME weights can be handed to the engine as an fp16 matrix and to the GPU as Q8_0 blocks, and the
    two products must agree at the F16 tolerance - no restated CPU code in between."""
    import torch
    rng = np.random.default_rng(55 + batch)
    d, n = 512, 1024
    q = rng.integers(-127, 128, size=(d, n // 32, 32), dtype=np.int64).astype(np.int8)
    exp = rng.integers(-9, -4, size=(d, n // 32, 1))
    scale = (2.0 ** exp).astype(np.float16)
    blocks = np.empty((d, n // 32, 34), dtype=np.uint8)
    blocks[..., :2] = scale.view(np.uint8).reshape(d, n // 32, 2)
    blocks[..., 2:] = q.view(np.uint8)
    blocks = blocks.reshape(d, -1)
    w16 = (scale.astype(np.float32) * q.astype(np.float32)).reshape(d, n).astype(np.float16)
    assert np.array_equal(w16.astype(np.float32), (scale.astype(np.float32) * q).reshape(d, n))  # exact in fp16
    x = rng.standard_normal((batch, n), dtype=np.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = attention.gemv_q8_0(torch.from_numpy(x).cuda(), torch.from_numpy(blocks).cuda(), status=status).cpu().numpy()
    assert status.item() == 0
    mag = np.abs(x) @ np.abs(w16.astype(np.float32)).T
    for b in range(batch):
        want = checker.matmul_clip(x[b], w16, 0.0)
        assert (np.abs(got[b] - want) <= 4e-6 * mag[b] + 1e-7).all(), np.abs(got[b] - want).max()


def test_q8_0_roundtrip_and_reference_f16_path(port, checker, pkg):
    """The writer against the dequantiser (|w - dq| <= d/2 per block, plus the fp16 rounding of d itself) and the Q8_0 sum against the engine's F16 matmul
    fed the values rounded once to fp16 (2^-11 per weight: 1e-3 of the magnitude)."""
    from llm_infer_b200 import quant
    rng = np.random.default_rng(1)
    w = rng.standard_normal((64, 512), dtype=np.float32)
    blocks = quant.quantize_q8_0(w)
    assert blocks.shape == (64, 512 // 32 * 34)
    dq = quant.dequantize_q8_0(blocks)
    step = np.abs(w).reshape(64, 16, 32).max(-1, keepdims=True) / 127
    assert (np.abs(w - dq).reshape(64, 16, 32) <= step * (0.5 + 127 * 2.0 ** -11) * 1.001 + 1e-8).all()
    x = rng.standard_normal(512, dtype=np.float32)
    a = port.matmul_q8_0(x, blocks)
    b = checker.matmul_clip(x, dq.astype(np.float16), 0.0)
    assert np.abs(a - b).max() <= 1e-3 * (np.abs(x) @ np.abs(dq).T).max()


def test_q8_0_streams_weights_near_hbm_rate(attention, pkg):
    import torch
    from llm_infer_b200 import quant
    d, n = 14336, 4096
    rng = np.random.default_rng(0)
    base = torch.from_numpy(quant.quantize_q8_0(rng.standard_normal((d, n), dtype=np.float32))).cuda()
    ws = [base.clone() for _ in range(6)]  # 6 x 62 MB = 374 MB > L2, rotated
    x = torch.randn(1, n, device="cuda")
    out = torch.empty(1, d, device="cuda")
    us = _graph_time_us(lambda i: attention.gemv_q8_0(x, ws[i], out=out), 6)
    gbs = (d * n // 32 * 34 + n * 4 + d * 4) / us / 1e3
    print(f"gemv {d}x{n} q8_0: {us:.1f} us, {gbs:.0f} GB/s")
    assert gbs > 3000


def test_tiled_q8_0_copy_and_bit_identical_products(attention, pkg):
    """attn_repack_q8_0_tiled writes exactly the layout quant.repack_q8_0_tiled states, and the GEMV over the tiled copy
    returns what the GEMV over the GGML blocks returns - the same per-block arithmetic; the same bits wherever both run
    with the same split of the inner dimension over the warps, else equal up to the order of the fp32 sum over the
    warps: plain (batch 1 and 8, a row count that is not a multiple of 16), clamp, stacked Q/K/V segments, SwiGLU
    rows, split-k partials, prepared activations in and out."""
    import torch
    from llm_infer_b200 import quant
    rng = np.random.default_rng(123)

    def make(d, n):
        blocks = quant.quantize_q8_0(rng.standard_normal((d, n), dtype=np.float32) * 0.05)
        dev = torch.from_numpy(blocks).cuda()
        tiled = attention.repack_q8_0(dev)
        assert (tiled.cpu().numpy() == quant.repack_q8_0_tiled(blocks)).all()
        return dev, tiled

    def same(a, b, exact=False):
        torch.cuda.synchronize()
        if a.dtype == torch.int32:  # prepared activations: compare the numbers they stand for (value + residual)
            a, b = (t.view(torch.float16).float().view(*t.shape[:-1], -1, 2, 2, 2).sum(dim=-3) for t in (a, b))
        if exact:
            assert torch.equal(a, b)
        scale = float(b.float().abs().max())
        assert float((a.float() - b.float()).abs().max()) <= 1e-5 * scale

    for d, n, B in ((4096, 4096, 1), (4096, 4096, 8), (777, 2048, 3), (1024, 14336, 1), (48, 256, 2)):
        w, wt = make(d, n)
        x = torch.randn(B, n, device="cuda")
        same(attention.gemv_q8_0(x, w), attention.gemv_q8_0(x, wt, rows=d), exact=(n == 4096 and B == 8))
        clip = 0.5 * float(attention.gemv_q8_0(x, w).abs().max())
        same(attention.gemv_q8_0(x, w, clip=clip), attention.gemv_q8_0(x, wt, clip=clip, rows=d))
    # stacked projections, one fp16 output
    n, B = 4096, 8
    w, wt = make(4096 + 1024 + 1024, n)
    x = torch.randn(B, n, device="cuda")
    outs = []
    for m in (w, wt):
        q, k = torch.empty(B, 4096, device="cuda"), torch.empty(B, 1024, device="cuda")
        v = torch.empty(B, 1024, device="cuda")
        attention.gemv_q8_0(x, m, out=q, out2=k, out3=v)
        outs.append((q, k, v))
    for a, b in zip(*outs):
        same(a, b)
    # SwiGLU rows, prepared activations in and out
    hidden = 1040
    w, wt = make(2 * hidden, n)
    xs = attention.rmsnorm(x, torch.ones(n, device="cuda"), 1e-5, out=torch.empty(B, n, dtype=torch.int32, device="cuda"))
    same(attention.gemv_q8_0(xs, w, swiglu=True, out_dtype=torch.int32),
         attention.gemv_q8_0(xs, wt, swiglu=True, out_dtype=torch.int32))
    # split-k partials of a batch whose activations do not fit at once
    n2 = 14336
    w, wt = make(1024, n2)
    x2 = torch.randn(B, n2, device="cuda")
    same(attention.gemv_q8_0(x2, w, k_split=4), attention.gemv_q8_0(x2, wt, k_split=4))
    same(attention.gemv_q8_0(x2, w), attention.gemv_q8_0(x2, wt))


def _weights(kind, w32, port, checker):
    """(device tensor, gemv wrapper name, per-sequence CPU product, fp32 view of the stored weights)."""
    import torch
    from llm_infer_b200 import quant
    if kind == "q8_0":
        blocks = quant.quantize_q8_0(w32)
        return torch.from_numpy(blocks).cuda(), "gemv_q8_0", (lambda x, clip=0.0: port.matmul_q8_0(x, blocks, clip)), \
            quant.dequantize_q8_0(blocks)
    w16 = w32.astype(np.float16)
    return torch.from_numpy(w16).cuda(), "gemv_f16", (lambda x, clip=0.0: checker.matmul_clip(x, w16, clip)), \
        w16.astype(np.float32)


@pytest.mark.parametrize("kind", ["q8_0", "f16"])
def test_stacked_qkv_and_swiglu_epilogue(attention, port, checker, pkg, kind):
    """One launch for the Q, K and V projections (three outputs) and one for silu(W1 x) * (W3 x), batch 8."""
    import torch
    rng = np.random.default_rng(77)
    n, B = 2048, 8
    x = rng.standard_normal((B, n), dtype=np.float32)
    mats = [_weights(kind, rng.standard_normal((d, n), dtype=np.float32) * 0.03, port, checker) for d in (512, 128, 128)]
    stacked = torch.cat([m[0] for m in mats])
    gemv = getattr(attention, mats[0][1])
    q, k, v = (torch.empty(B, d, device="cuda") for d in (512, 128, 128))
    gemv(torch.from_numpy(x).cuda(), stacked, out=q, out2=k, out3=v, clip=0.8)
    for got, m in ((q, mats[0]), (k, mats[1]), (v, mats[2])):
        got = got.cpu().numpy()
        mag = np.abs(x) @ np.abs(m[3]).T
        for b in range(B):
            assert (np.abs(got[b] - m[2](x[b], 0.8)) <= 4e-6 * mag[b] + 1e-7).all()
    hidden = 1040  # 65 row groups: the up rows start at a group boundary that is not a multiple of the grid
    g1, g3 = (_weights(kind, rng.standard_normal((hidden, n), dtype=np.float32) * 0.03, port, checker) for _ in range(2))
    got = gemv(torch.from_numpy(x).cuda(), torch.cat([g1[0], g3[0]]), swiglu=True).cpu().numpy()
    assert got.shape == (B, hidden)
    for b in range(B):
        want = port.swiglu(g1[2](x[b]), g3[2](x[b]))
        assert np.abs(got[b] - want).max() <= 2e-5 * np.abs(want).max() + 1e-6


@pytest.mark.parametrize("kind", ["q8_0", "f16"])
def test_split_k_partials_and_residual_norm(attention, port, checker, pkg, kind):
    """k_split sets of CTAs each compute one slice of the inner dimension; the partial products sum to the product, and
    attn_rmsnorm_residual adds them into x before normalising."""
    import torch
    rng = np.random.default_rng(99)
    n, d, B, K = 14336, 1024, 8, 4
    x = rng.standard_normal((B, n), dtype=np.float32)
    w_dev, name, product, w_f32 = _weights(kind, rng.standard_normal((d, n), dtype=np.float32) * 0.02, port, checker)
    parts = getattr(attention, name)(torch.from_numpy(x).cuda(), w_dev, k_split=K)
    assert parts.shape == (K, B, d)
    got = parts.sum(0).cpu().numpy()
    mag = np.abs(x) @ np.abs(w_f32).T
    want = np.stack([product(x[b]) for b in range(B)])
    assert (np.abs(got - want) <= 4e-6 * mag + 1e-7).all()
    assert (parts[0].abs().sum() > 0) and (parts[K - 1].abs().sum() > 0)
    # residual + norm
    resid = rng.standard_normal((B, d), dtype=np.float32)
    wt = (1 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    xg = torch.from_numpy(resid.copy()).cuda()
    normed = attention.rmsnorm(xg, torch.from_numpy(wt).cuda(), 1e-5, out=torch.empty_like(xg), partials=parts)
    full = resid.copy()
    for s_ in range(K):
        full += parts[s_].cpu().numpy()
    assert np.array_equal(xg.cpu().numpy(), full)  # same order of additions: bit-equal
    for b in range(B):
        ref = port.rmsnorm(full[b], wt, 1e-5)
        assert np.abs(normed[b].cpu().numpy() - ref).max() <= 4e-6 * np.abs(ref).max()


def test_f16_batch_8_streams_weights_near_hbm_rate(attention):
    """The batched fp16 form on the tensor cores: 14336 x 4096, batch 8."""
    import torch
    n, d = 4096, 14336
    ws = [torch.randn(d, n, device="cuda").half() for _ in range(3)]  # 352 MB > L2, rotated
    x = torch.randn(8, n, device="cuda")
    out = torch.empty(8, d, device="cuda")
    us = _graph_time_us(lambda i: attention.gemv_f16(x, ws[i], out=out), 3)
    gbs = (d * n * 2 + 8 * (n * 4 + d * 4)) / us / 1e3
    print(f"gemv 14336x4096 fp16 batch 8: {us:.1f} us, {gbs:.0f} GB/s")
    assert gbs > 3000


def _split16_words(x):
    """numpy restatement of the prepared-activation form (ATTN_DTYPE_SPLIT16): per group of four elements the words
    {hi(x0,x1), hi(x2,x3), lo(x0,x1), lo(x2,x3)}, hi = fp16(x), lo = fp16(x - hi)."""
    x = np.clip(np.asarray(x, dtype=np.float32), -65504.0, 65504.0)
    hi = x.astype(np.float16)
    lo = (x - hi.astype(np.float32)).astype(np.float16)
    h = hi.view(np.uint16).astype(np.uint32).reshape(*x.shape[:-1], -1, 4)
    l = lo.view(np.uint16).astype(np.uint32).reshape(*x.shape[:-1], -1, 4)
    words = np.stack([h[..., 0] | (h[..., 1] << 16), h[..., 2] | (h[..., 3] << 16),
                      l[..., 0] | (l[..., 1] << 16), l[..., 2] | (l[..., 3] << 16)], axis=-1)
    return words.reshape(x.shape).astype(np.uint32)


def test_prepared_activations_from_every_producer(attention, pkg):
    """RMSNorm, the Q8_0 GEMV (SwiGLU epilogue, row segments) and decode attention can write their result as prepared
    activations (int32 tensors); the words are exactly the split of the fp32 result, and a GEMV fed with them gives
    bit for bit what it gives when it converts the fp32 activations itself."""
    import torch
    from llm_infer_b200 import quant
    rng = np.random.default_rng(123)
    B, n, hidden = 8, 2048, 1024
    x = torch.from_numpy(rng.standard_normal((B, n), dtype=np.float32) * 3).cuda()
    wt = torch.from_numpy((1 + 0.1 * rng.standard_normal(n)).astype(np.float32)).cuda()
    w13 = torch.from_numpy(quant.quantize_q8_0(rng.standard_normal((2 * hidden, n), dtype=np.float32) * 0.03)).cuda()
    w2 = torch.from_numpy(quant.quantize_q8_0(rng.standard_normal((512, hidden), dtype=np.float32) * 0.03)).cuda()
    # 1. RMSNorm
    xb32 = attention.rmsnorm(x, wt, 1e-5, out=torch.empty_like(x))
    xbw = attention.rmsnorm(x, wt, 1e-5, out=torch.empty((B, n), dtype=torch.int32, device="cuda"))
    assert np.array_equal(xbw.cpu().numpy().view(np.uint32), _split16_words(xb32.cpu().numpy()))
    # 2. GEMV reading prepared activations, writing fp32 and prepared activations (SwiGLU epilogue)
    hb32 = attention.gemv_q8_0(xb32, w13, swiglu=True)
    assert torch.equal(attention.gemv_q8_0(xbw, w13, swiglu=True), hb32)
    hbw = attention.gemv_q8_0(xbw, w13, swiglu=True, out=torch.empty((B, hidden), dtype=torch.int32, device="cuda"))
    assert np.array_equal(hbw.cpu().numpy().view(np.uint32), _split16_words(hb32.cpu().numpy()))
    assert torch.equal(attention.gemv_q8_0(hbw, w2), attention.gemv_q8_0(hb32, w2))
    # 3. row segments in prepared form
    q32, k32 = torch.empty(B, 768, device="cuda"), torch.empty(B, 256, device="cuda")
    qw, kw = (torch.empty(B, d, dtype=torch.int32, device="cuda") for d in (768, 256))
    attention.gemv_q8_0(xbw, w13[:1024], out=q32, out2=k32)
    attention.gemv_q8_0(xbw, w13[:1024], out=qw, out2=kw)
    assert np.array_equal(qw.cpu().numpy().view(np.uint32), _split16_words(q32.cpu().numpy()))
    assert np.array_equal(kw.cpu().numpy().view(np.uint32), _split16_words(k32.cpu().numpy()))
    # 4. decode attention
    H, Hkv, D, T = 8, 2, 128, 300
    q = torch.randn(B, H, D, device="cuda")
    kc, vc = torch.randn(B, T, Hkv, D, device="cuda").half(), torch.randn(B, T, Hkv, D, device="cuda").half()
    o32 = attention.attn_decode(q, kc, vc)
    ow = attention.attn_decode(q, kc, vc, out=torch.empty((B, H, D), dtype=torch.int32, device="cuda"))
    assert np.array_equal(ow.cpu().numpy().view(np.uint32).reshape(B, H * D),
                          _split16_words(o32.cpu().numpy().reshape(B, H * D)))
