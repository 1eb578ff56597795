"""Greedy end-to-end generation on the GPU against the CPU forward pass: exact token equality.

The checker runs the engine's own primitives (include/kernels_cpu.hpp) in the order of src/model/block.cpp:105-223
and src/model/model.cpp:60-98, one sequence and one token at a time, with the greedy pick of tools/infer.cpp:64-74.
The device path runs the whole ragged batch at once through the C ABI kernels. Models are random-init (seeded) and
small enough for the CPU to finish in seconds; logits are also compared (2e-3 absolute + 1e-2 relative to the row's
RMS, the attention tolerance; measured differences are ~1e-5). A pick is only required to be equal where the
checker's own top-2 margin exceeds 1e-3: below that, two correct fp32 summation orders may legitimately disagree."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def M(built_lib, pkg):
    from llm_infer_b200 import model
    return model


def _numpy_weights(w):
    return {k: v.numpy() for k, v in w.items()}


def _run_case(M, checker, cfg, prompts, n_new, seed, graph=False, weight_type="f16", prompt_mode="token"):
    import torch
    w = M.random_weights(cfg, seed, weight_type=weight_type)
    llama = M.Llama(cfg, w, batch=len(prompts), weight_type=weight_type)
    if graph:
        llama.capture()
    got_tokens, got_logits = llama.generate(prompts, n_new, want_logits=True, prompt_mode=prompt_mode)
    wn = _numpy_weights(w)
    safe_all = True
    cfg_dict = dict(cfg.as_dict(), weight_type=weight_type)
    for b, prompt in enumerate(prompts):
        want_tokens, want_logits = checker.generate_greedy(cfg_dict, wn, prompt, n_new)
        g_tok, g_log = got_tokens[b].numpy(), got_logits[b].numpy()
        for i in range(n_new):
            srt = np.sort(want_logits[i])
            margin = srt[-1] - srt[-2]
            rms = float(np.sqrt(np.mean(want_logits[i] ** 2)))
            err = np.abs(g_log[i] - want_logits[i]).max()
            assert err <= 2e-3 + 1e-2 * rms, (b, i, err, rms)
            if margin > 1e-3:
                assert g_tok[i] == want_tokens[i], (b, i, margin, g_tok[:i + 1], want_tokens[:i + 1])
            elif g_tok[i] != want_tokens[i]:
                safe_all = False
                break  # the two sequences diverged on a near-tie; later steps are not comparable
    torch.cuda.synchronize()
    return safe_all


def test_tiny_model_ragged_batch_token_equality(M, checker):
    cfg = M.ModelConfig(dim=512, hidden_dim=1024, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, vocab_size=1000,
                        max_seq_len=64, norm_eps=1e-5, rope_theta=10000.0)
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (5, 9, 3)]
    _run_case(M, checker, cfg, prompts, n_new=24, seed=1)


def test_cuda_graph_replay_gives_the_same_tokens(M, checker):
    """The step captured once per mode as a CUDA graph and replayed (one launch per step)."""
    cfg = M.ModelConfig(dim=512, hidden_dim=1024, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, vocab_size=1000,
                        max_seq_len=64, norm_eps=1e-5, rope_theta=10000.0)
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (4, 11, 7, 1, 2)]
    _run_case(M, checker, cfg, prompts, n_new=20, seed=5, graph=True)


def test_q8_0_model_token_equality(M, port):
    """Every matrix (embedding and classifier included) stored as Q8_0 blocks, graph replay, batch of 8: against the
    restated forward pass reading the same blocks (the engine itself has no Q8_0 path to compare with)."""
    cfg = M.ModelConfig(dim=512, hidden_dim=1024, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, vocab_size=1000,
                        max_seq_len=48, norm_eps=1e-5, rope_theta=500000.0)
    rng = np.random.default_rng(31)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (4, 11, 7, 1, 2, 16, 9, 5)]
    _run_case(M, port, cfg, prompts, n_new=12, seed=6, graph=True, weight_type="q8_0")


def test_q8_0_model_with_split_k_down_projection(M, port):
    """Batch 8 with an FFN wide enough (8 x 8192 activations) that the down projection runs split over the inner
    dimension and the next RMSNorm adds the partial products into the residual stream."""
    cfg = M.ModelConfig(dim=512, hidden_dim=8192, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=128, vocab_size=400,
                        max_seq_len=32, norm_eps=1e-5, rope_theta=10000.0)
    rng = np.random.default_rng(41)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (3, 8, 5, 1, 2, 6, 4, 7)]
    w = M.random_weights(cfg, 8, weight_type="q8_0")
    assert M.Llama(cfg, w, batch=8, weight_type="q8_0")._k_split == 2
    _run_case(M, port, cfg, prompts, n_new=8, seed=8, graph=True, weight_type="q8_0")
    _run_case(M, port, cfg, prompts, n_new=8, seed=8, weight_type="q8_0", prompt_mode="batched")


@pytest.mark.parametrize("weight_type", ["f16", "q8_0"])
def test_model_file_round_trip_generates_the_same_tokens(M, tmp_path, weight_type):
    """Seed-generated weights written as a GGUF file, loaded back, same greedy output as the in-memory model."""
    from llm_infer_b200 import gguf
    cfg = M.ModelConfig(dim=512, hidden_dim=1024, n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, vocab_size=600,
                        max_seq_len=40, norm_eps=1e-5, rope_theta=500000.0)
    w = M.random_weights(cfg, 9, weight_type=weight_type)
    path = str(tmp_path / "model.gguf")
    gguf.write_gguf(path, cfg, w, weight_type)
    prompts = [[5, 17, 3], [9], [100, 200, 300, 400, 500]]
    a = M.Llama(cfg, w, batch=3, weight_type=weight_type).generate(prompts, 10)
    b = M.Llama.from_gguf(path, batch=3).generate(prompts, 10)
    assert np.array_equal(a.numpy(), b.numpy()) and len(set(a.flatten().tolist())) > 3


@pytest.mark.parametrize("prompt_mode", ["token", "batched"])
def test_head_dim_128_gqa4_clip_and_partial_rotary(M, checker, prompt_mode):
    cfg = M.ModelConfig(dim=1024, hidden_dim=1536, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=128,
                        vocab_size=777, max_seq_len=96, norm_eps=1e-5, rope_theta=500000.0, rotary_dim=64,
                        qkv_clip=2.5)
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (17, 1, 40, 8)]
    _run_case(M, checker, cfg, prompts, n_new=16, seed=2, prompt_mode=prompt_mode)


def test_sliding_window_with_sink_rows(M, checker):
    """Generation runs past max_seq_len: the cache becomes a ring behind four sink rows whose K is re-rotated every
    step (src/model/model.cpp:66-68, src/model/block.cpp:150-155)."""
    cfg = M.ModelConfig(dim=512, hidden_dim=512, n_layers=2, n_heads=4, n_kv_heads=4, head_dim=128, vocab_size=500,
                        max_seq_len=16, norm_eps=1e-5, rope_theta=10000.0)
    rng = np.random.default_rng(13)
    prompts = [rng.integers(0, cfg.vocab_size, size=10).tolist() for _ in range(2)]
    _run_case(M, checker, cfg, prompts, n_new=20, seed=3)


@pytest.mark.parametrize("prompt_mode", ["token", "batched"])
def test_llama3_8b_shaped_layer(M, checker, prompt_mode):
    """One layer with the 8B model's dimensions (dim 4096, 32/8 heads of 128, FFN 14336, theta 5e5), small vocabulary;
    prompts fed token by token, and all at once through the tensor-core GEMMs and the causal prefill kernel."""
    cfg = M.ModelConfig(dim=4096, hidden_dim=14336, n_layers=1, n_heads=32, n_kv_heads=8, head_dim=128,
                        vocab_size=2048, max_seq_len=48, norm_eps=1e-5, rope_theta=500000.0)
    rng = np.random.default_rng(14)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (12, 30)]
    _run_case(M, checker, cfg, prompts, n_new=8, seed=4, prompt_mode=prompt_mode)


def test_whole_prompt_prefill_equals_the_token_loop(M, port):
    """Longer ragged prompts (several 128-row tiles, one shorter than a tile), fp16 and Q8_0 weights: the batched prompt
    phase must leave the model where the token-at-a-time loop leaves it - same greedy tokens afterwards, logits
    within the attention tolerance - and match the CPU forward pass for the Q8_0 case."""
    cfg = M.ModelConfig(dim=512, hidden_dim=1024, n_layers=3, n_heads=4, n_kv_heads=2, head_dim=128, vocab_size=900,
                        max_seq_len=420, norm_eps=1e-5, rope_theta=500000.0)
    rng = np.random.default_rng(77)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (300, 7, 129, 400)]
    for weight_type in ("f16", "q8_0"):
        w = M.random_weights(cfg, 17, weight_type=weight_type)
        a = M.Llama(cfg, w, batch=4, weight_type=weight_type)
        assert a.can_prefill(prompts, 12)
        tok_a, log_a = a.generate(prompts, 12, want_logits=True, prompt_mode="token")
        b = M.Llama(cfg, w, batch=4, weight_type=weight_type)
        tok_b, log_b = b.generate(prompts, 12, want_logits=True, prompt_mode="batched")
        la, lb = log_a.numpy(), log_b.numpy()
        rms = float(np.sqrt(np.mean(la ** 2)))
        assert np.abs(la - lb).max() <= 2e-3 + 1e-2 * rms
        srt = np.sort(la, axis=-1)
        safe = (srt[..., -1] - srt[..., -2]) > 1e-3
        ta, tb = tok_a.numpy(), tok_b.numpy()
        for s in range(4):
            upto = 12 if safe[s].all() else int(np.argmin(safe[s]))  # compare up to the first near-tie
            assert np.array_equal(ta[s, :upto], tb[s, :upto]), (weight_type, s)
    _run_case(M, port, cfg, prompts[:2], n_new=6, seed=17, weight_type="q8_0", prompt_mode="batched")


def test_full_depth_q8_0_against_its_own_weights_in_fp16(M):
    """All 32 layers at the 8B model's widths (small vocabulary): the Q8_0 model against the SAME weights expanded to
    fp16 and run through the fp16 kernels (the path that is pinned on the engine's CPU matmul). The fp16 copy rounds
    each weight once (2^-12 relative), so the two runs are compared with tolerances, teacher-forced on one token
    stream: logits within 2e-2 of the row's RMS at every step, and the first step at which the greedy picks differ is
    reported (a near-tie is the only legitimate reason)."""
    import torch
    from llm_infer_b200 import quant
    cfg = M.ModelConfig(dim=4096, hidden_dim=14336, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128,
                        vocab_size=4096, max_seq_len=96, norm_eps=1e-5, rope_theta=500000.0)
    wq = M.random_weights(cfg, 23, device="cuda", weight_type="q8_0")
    wf = {}
    for name, t in wq.items():
        if t.dtype != torch.uint8:
            wf[name] = t
            continue
        b = t.view(*t.shape[:-1], t.shape[-1] // 34, 34)
        d = b[..., :2].contiguous().view(torch.float16).float()
        q = b[..., 2:].contiguous().view(torch.int8).float()
        wf[name] = (d * q).reshape(*t.shape[:-1], -1).half()
    rng = np.random.default_rng(23)
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in (40, 64)]
    n_new = 12
    a = M.Llama(cfg, wq, batch=2, weight_type="q8_0")
    del wq
    tok_a, log_a = a.generate(prompts, n_new, want_logits=True)
    del a
    torch.cuda.empty_cache()
    b = M.Llama(cfg, wf, batch=2, weight_type="f16")
    del wf
    # teacher forcing: the fp16 model reads the Q8_0 model's picks as part of its prompt, one more per step
    first_diff = None
    for i in range(n_new):
        forced = [p + tok_a[s, :i].tolist() for s, p in enumerate(prompts)]
        tok_b, log_b = b.generate(forced, 1, want_logits=True)
        la, lb = log_a[:, i].numpy(), log_b[:, 0].numpy()
        rms = float(np.sqrt(np.mean(la ** 2)))
        assert np.abs(la - lb).max() <= 2e-2 * rms, (i, np.abs(la - lb).max(), rms)
        if first_diff is None and not np.array_equal(tok_a[:, i].numpy(), tok_b[:, 0].numpy()):
            srt = np.sort(la, axis=-1)
            first_diff = (i, float((srt[:, -1] - srt[:, -2]).min()))
    print("first step with a different greedy pick (step, smallest top-2 margin there):", first_diff)
    assert len(set(tok_a.flatten().tolist())) > 4
    if first_diff is not None:
        assert first_diff[1] < 2e-2 * rms, "the picks may only differ on a near-tie"


def test_small_steps_against_port(M, port):
    """RMSNorm, SwiGLU, embedding and argmax alone (fp32: a few ulp; argmax and embedding exact)."""
    import torch
    from llm_infer_b200 import attention as A
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 4096), dtype=np.float32) * 3
    wt = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float32)
    got = A.rmsnorm(torch.from_numpy(x).cuda(), torch.from_numpy(wt).cuda(), 1e-5).cpu().numpy()
    for b in range(3):
        want = port.rmsnorm(x[b], wt, 1e-5)
        assert np.abs(got[b] - want).max() <= 4e-6 * np.abs(want).max()
    hb, hb2 = rng.standard_normal((2, 14336), dtype=np.float32) * 4, rng.standard_normal((2, 14336), dtype=np.float32)
    got = A.swiglu_(torch.from_numpy(hb.copy()).cuda(), torch.from_numpy(hb2).cuda()).cpu().numpy()
    want = port.swiglu(hb, hb2)
    assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()
    table = rng.standard_normal((100, 512), dtype=np.float32).astype(np.float16)
    tok = np.array([7, 99, 0, 7], dtype=np.int32)
    got = A.embed_f16(torch.from_numpy(table).cuda(), torch.from_numpy(tok).cuda()).cpu().numpy()
    assert np.array_equal(got, table[tok].astype(np.float32))
    logits = rng.standard_normal((5, 128256), dtype=np.float32)
    logits[1, 777] = logits[1, 90000] = 9.0   # a tie: the first index wins
    logits[2, 0] = 10.0
    logits[3, -1] = 10.0
    got = A.argmax(torch.from_numpy(logits).cuda()).cpu().numpy()
    assert got.tolist() == [port.argmax(logits[b]) for b in range(5)] and got[1] == 777


def test_token_id_out_of_range_is_reported_not_read(M):
    import torch
    from llm_infer_b200 import attention as A
    table = torch.ones((10, 64), dtype=torch.float16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((2, 64), -1.0, device="cuda")
    A.embed_f16(table, torch.tensor([3, 10], dtype=torch.int32, device="cuda"), out=out, status=status)
    torch.cuda.synchronize()
    assert status.item() == 2 and (out[0] == 1).all() and (out[1] == -1).all()
