"""Incremental decoding with the key/value cache against the CPU oracle (GPU).

The oracle is the full-sequence forward: the logits a decode step returns for position pos must
be those of the oracle's forward over the same tokens at that position.  The decode kernels run
on the fp32 FMA pipe, so a sequence decoded from an empty cache is held to fp32-level agreement;
after a tensor-core prefill the cache holds TF32-path keys and values and the tolerance is the
forward's (2e-2 max-abs).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _model(pkg, orc, ctx, kw, B, T, round_operands):
    cfg = pkg.GPT2Config(**kw)
    ocfg = orc.GPT2Config(**kw)
    params = orc.init_params(ocfg, seed=1234)
    model = pkg.GPT2(ctx, cfg, B, T)
    model.set_options(round_operands=round_operands)  # 0: the weights stay the oracle's, bit for bit
    model.load_params(params)
    model.enable_kv_cache()
    return cfg, ocfg, params, model


@pytest.mark.parametrize("kw,B,T,use_graph", [(dict(num_layers=2), 3, 64, 0), (dict(num_layers=2), 3, 64, 1),
                                              (dict(num_layers=2, num_heads=25, channels=1600), 2, 64, 1),
                                              (dict(num_layers=1), 11, 64, 0)])
def test_decode_from_empty_cache_matches_oracle(pkg, orc, ctx, kw, B, T, use_graph):
    """Every position decoded one token at a time (pos = 0 .. T-1): fp32-level agreement.  With
    use_graph the steps after the first are replays of one captured graph (the position is data)."""
    import torch
    cfg, ocfg, params, model = _model(pkg, orc, ctx, kw, B, T, 0)
    model.set_options(round_operands=0, use_graph=use_graph)
    tokens = orc.fill_tokens((B, T), seed=99, vocab=cfg.vocab_size)
    want = orc.gpt2_forward(params, ocfg, tokens, precise=True)  # [B,T,Vp]
    d_tok = torch.from_numpy(tokens).cuda()
    worst = 0.0
    for pos in range(T):
        col = d_tok[:, pos].contiguous()
        torch.cuda.synchronize()
        logits = model.decode_step(col, B, pos)
        ctx.sync_check()
        got = logits.cpu().numpy()
        worst = max(worst, float(np.abs(got - want[:, pos, :]).max()))
        assert np.array_equal(got[:, :cfg.vocab_size].argmax(-1), want[:, pos, :cfg.vocab_size].argmax(-1)), pos
    assert worst < 2e-4 * max(1.0, float(np.abs(want).max())), worst
    model.close()


def test_prefill_then_decode_matches_oracle(pkg, orc, ctx):
    """Tensor-core prefill of 64 positions, then 16 decode steps through the host-buffer call."""
    B, T0, T = 4, 64, 128
    cfg, ocfg, params, model = _model(pkg, orc, ctx, dict(num_layers=3), B, T, 1)
    import torch
    tokens = orc.fill_tokens((B, T), seed=5, vocab=cfg.vocab_size)
    want = orc.gpt2_forward(params, ocfg, tokens, precise=False)
    d_tok = torch.from_numpy(np.ascontiguousarray(tokens[:, :T0])).cuda()
    torch.cuda.synchronize()
    pre = model.prefill(d_tok, B, T0)
    ctx.sync_check()
    assert np.abs(pre.cpu().numpy() - want[:, :T0, :]).max() < 2e-2
    logits = np.empty((B, cfg.padded_vocab_size), np.float32)
    amax = np.empty((B,), np.int32)
    for pos in range(T0, T0 + 16):
        model.decode_step_host(np.ascontiguousarray(tokens[:, pos]), B, pos, logits_host=logits, argmax_host=amax)
        assert np.abs(logits - want[:, pos, :]).max() < 2e-2, pos
        assert np.array_equal(amax, logits[:, :cfg.vocab_size].argmax(-1))
    model.close()


def test_decode_preconditions(pkg, orc, ctx):
    import torch
    cfg = pkg.GPT2Config(num_layers=1)
    model = pkg.GPT2(ctx, cfg, 2, 64)
    tok = torch.zeros(2, dtype=torch.int32, device="cuda")
    lib = pkg.lib()
    assert lib.b200_gpt2_decode_step(model._h, tok.data_ptr(), 2, 0) == pkg.B200_ERR_STATE  # no cache yet
    model.enable_kv_cache()
    assert lib.b200_gpt2_decode_step(model._h, tok.data_ptr(), 2, 64) == pkg.B200_ERR_SHAPE  # pos beyond max_T
    assert lib.b200_gpt2_decode_step(model._h, tok.data_ptr(), 3, 0) == pkg.B200_ERR_SHAPE   # B beyond max_B
    assert lib.b200_gpt2_prefill(model._h, tok.data_ptr(), 2, 32) == pkg.B200_ERR_SHAPE      # T % 64
    model.close()


@pytest.mark.parametrize("T0,use_graph", [(5, 0), (64, 1)])
def test_generate_greedy_follows_the_oracle(pkg, orc, ctx, T0, use_graph):
    """Greedy continuation: every generated token must be the arg-max of the oracle's logits for
    the sequence so far.  T0 = 5 feeds the prompt token by token (fp32 path throughout); T0 = 64
    goes through the tensor-core prefill.  A near-tie in the oracle's own logits is allowed to fall
    either way: then the check continues with the token the engine chose."""
    B, n_new = 3, 6
    cfg, ocfg, params, model = _model(pkg, orc, ctx, dict(num_layers=2), B, 128, 0)
    model.set_options(round_operands=0, use_graph=use_graph)
    prompt = orc.fill_tokens((B, T0), seed=21, vocab=cfg.vocab_size)
    out = np.empty((B, n_new), np.int32)
    model.generate_greedy(np.ascontiguousarray(prompt), B, T0, n_new, out)
    seq = prompt.copy()
    V = cfg.vocab_size
    for i in range(n_new):
        T = seq.shape[1]
        Tpad = (T + 63) // 64 * 64  # the oracle's forward is causal: padding behind the sequence changes nothing
        padded = np.zeros((B, Tpad), np.int32)
        padded[:, :T] = seq
        logits = orc.gpt2_forward(params, ocfg, padded, precise=True)[:, T - 1, :V]
        for b in range(B):
            top2 = np.sort(logits[b])[-2:]
            if out[b, i] != logits[b].argmax():
                assert top2[1] - top2[0] < 2e-3 and logits[b, out[b, i]] >= top2[0] - 1e-6, (b, i)
        seq = np.concatenate([seq, out[:, i:i + 1]], axis=1)
    model.close()


# ------------------------------------------------------------------ sampling
def _mix32(x):
    x = x.astype(np.uint64)
    x ^= x >> np.uint64(16); x = (x * np.uint64(0x7feb352d)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(15); x = (x * np.uint64(0x846ca68b)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    return x


def _gumbel(seed, stream, cols):
    """numpy restatement of the device's counter-based Gumbel noise (float64 logs)."""
    a = _mix32(np.uint64(seed) ^ ((stream.astype(np.uint64) * np.uint64(0x9E3779B1)) & np.uint64(0xFFFFFFFF)))
    h = _mix32(a[:, None] ^ ((cols.astype(np.uint64)[None, :] * np.uint64(0x85EBCA77)) & np.uint64(0xFFFFFFFF)))
    u = ((h >> np.uint64(8)).astype(np.float64) + 0.5) / 16777216.0
    return -np.log(-np.log(u))


def test_sample_rows_draws_from_the_softmax(ctx, dev):
    """Gumbel-max sampling: the draws equal the arg-max of logit/T + noise computed in numpy with
    the same counter-based noise, their frequencies follow softmax(logits/T), a call is
    reproducible, and temperature 0 is the arg-max."""
    import torch
    M, V, temp, seed = 20000, 8, 0.7, 1234
    row = np.array([0.3, -1.0, 1.2, 0.0, 2.0, -0.5, 0.9, 1.5], np.float32)
    logits = dev.to(np.tile(row, (M, 1)))
    out = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ctx.sample_rows(out, logits, M, V, V, temp, seed, 77)
    ctx.sync_check()
    got = out.cpu().numpy()
    score = row.astype(np.float64)[None, :] / temp + _gumbel(seed, np.arange(77, 77 + M), np.arange(V))
    assert (got == score.argmax(1)).mean() > 0.9995  # float32 logs on the device: a rare near-tie may flip
    p = np.exp(row.astype(np.float64) / temp); p /= p.sum()
    freq = np.bincount(got, minlength=V) / M
    assert (np.abs(freq - p) < 5 * np.sqrt(p * (1 - p) / M)).all(), (freq, p)
    out2 = torch.empty_like(out)
    ctx.sample_rows(out2, logits, M, V, V, temp, seed, 77)
    ctx.sync_check()
    assert torch.equal(out, out2)
    ctx.sample_rows(out2, logits, M, V, V, temp, seed + 1, 77)
    ctx.sync_check()
    assert not torch.equal(out, out2)
    ctx.sample_rows(out2, logits, M, V, V, 0.0, seed, 77)
    ctx.sync_check()
    assert (out2.cpu().numpy() == int(row.argmax())).all()


@pytest.mark.parametrize("T0", [5, 64])
def test_generate_with_temperature_is_reproducible_and_follows_its_logits(pkg, orc, ctx, T0):
    """Sampled generation: same seed, same continuation; and every drawn token is the arg-max of
    the oracle's logits for the sequence so far, divided by the temperature, plus the noise of its
    (position, sequence) stream - up to near-ties."""
    B, n_new, temp, seed = 3, 5, 0.8, 99
    cfg, ocfg, params, model = _model(pkg, orc, ctx, dict(num_layers=2), B, 128, 0)
    model.set_options(round_operands=0)
    prompt = np.ascontiguousarray(orc.fill_tokens((B, T0), seed=31, vocab=cfg.vocab_size))
    out, again, greedy = (np.empty((B, n_new), np.int32) for _ in range(3))
    model.generate(prompt, B, T0, n_new, out, temperature=temp, seed=seed)
    model.generate(prompt, B, T0, n_new, again, temperature=temp, seed=seed)
    model.generate(prompt, B, T0, n_new, greedy, temperature=0.0)
    assert np.array_equal(out, again)
    assert not np.array_equal(out, greedy)
    V = cfg.vocab_size
    assert out.min() >= 0 and out.max() < V
    seq = prompt.copy()
    for i in range(n_new):
        T = seq.shape[1]
        padded = np.zeros((B, (T + 63) // 64 * 64), np.int32)
        padded[:, :T] = seq
        logits = orc.gpt2_forward(params, ocfg, padded, precise=True)[:, T - 1, :V].astype(np.float64)
        for b in range(B):
            score = logits[b] / temp + _gumbel(seed, np.array([T * 16 + b]), np.arange(V))[0]
            assert score[out[b, i]] >= score.max() - 5e-3, (b, i)
        seq = np.concatenate([seq, out[:, i:i + 1]], axis=1)
    model.close()


@pytest.mark.parametrize("V,k", [(50257, 40), (50257, 1), (1000, 999), (4096, 64)])
def test_top_k_sampling_draws_only_among_the_k_largest(ctx, dev, orc, V, k):
    """Top-k: every draw is the arg-max of logit/T + noise over the k largest logits of its row
    (found on the device by a radix select over order-preserving keys), for rows with distinct
    random logits, negative ones included; and a row with ties at the threshold keeps all tied
    columns."""
    import torch
    M, temp, seed = 64, 1.3, 7
    ld = (V + 3) // 4 * 4
    logits = np.zeros((M, ld), np.float32)
    logits[:, :V] = orc.fill_normal((M, V), 401, std=3.0)
    logits[:, V:] = 1e9  # padding columns must never be drawn
    logits[0, :V] = np.round(logits[0, :V])  # many exact ties
    out = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    d_logits = dev.to(logits)
    ctx.sample_rows(out, d_logits, M, V, ld, temp, seed, 5, top_k=k)
    ctx.sync_check()
    got = out.cpu().numpy()
    noise = _gumbel(seed, np.arange(5, 5 + M), np.arange(V))
    for r in range(M):
        x = logits[r, :V].astype(np.float64)
        kth = np.sort(x)[-k]
        keep = x >= kth  # ties with the k-th largest stay in
        score = np.where(keep, x / temp + noise[r], -np.inf)
        assert keep[got[r]], (r, got[r])
        assert score[got[r]] >= score.max() - 1e-4, (r, got[r], int(score.argmax()))
    if k == 1:
        assert np.array_equal(got[1:], logits[1:, :V].argmax(1))


def test_generate_with_top_k_stays_inside_the_oracle_top_k(pkg, orc, ctx):
    B, T0, n_new, k = 2, 7, 4, 5
    cfg, ocfg, params, model = _model(pkg, orc, ctx, dict(num_layers=2), B, 128, 0)
    model.set_options(round_operands=0)
    prompt = np.ascontiguousarray(orc.fill_tokens((B, T0), seed=41, vocab=cfg.vocab_size))
    out = np.empty((B, n_new), np.int32)
    model.generate(prompt, B, T0, n_new, out, temperature=5.0, seed=3, top_k=k)
    V = cfg.vocab_size
    seq = prompt.copy()
    for i in range(n_new):
        T = seq.shape[1]
        padded = np.zeros((B, 64), np.int32)
        padded[:, :T] = seq
        logits = orc.gpt2_forward(params, ocfg, padded, precise=True)[:, T - 1, :V]
        for b in range(B):
            kth = np.sort(logits[b])[-k]
            assert logits[b, out[b, i]] >= kth - 1e-4, (b, i)  # up to the fp32 noise of the two forwards
        seq = np.concatenate([seq, out[:, i:i + 1]], axis=1)
    model.close()


@pytest.mark.parametrize("V,k,p", [(50257, 0, 0.9), (50257, 50, 0.5), (2000, 0, 0.3), (4096, 0, 0.999)])
def test_top_p_sampling_keeps_the_smallest_set_that_reaches_p(ctx, dev, orc, V, k, p):
    """Nucleus sampling (after an optional top-k): every draw lies inside the nucleus computed by
    numpy with a slightly larger p and is the arg-max of the perturbed score over the nucleus
    computed with a slightly smaller p - the device sums probabilities in fp32 and in arrival
    order, so a column exactly on the boundary may fall either way."""
    import torch
    M, temp, seed = 48, 0.9, 11
    ld = (V + 3) // 4 * 4
    logits = np.zeros((M, ld), np.float32)
    logits[:, :V] = orc.fill_normal((M, V), 501, std=2.5)
    out = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    ctx.sample_rows(out, dev.to(logits), M, V, ld, temp, seed, 9, top_k=k, top_p=p)
    ctx.sync_check()
    got = out.cpu().numpy()
    noise = _gumbel(seed, np.arange(9, 9 + M), np.arange(V))

    def nucleus(x, pp):
        keep = np.ones(V, bool) if k == 0 else x >= np.sort(x)[-k]
        w = np.where(keep, np.exp((x - x[keep].max()) / temp), 0.0)
        order = np.argsort(-x, kind="stable")
        cum = np.cumsum(w[order])
        last = int(np.searchsorted(cum, pp * w.sum(), side="left"))  # first prefix whose mass reaches pp
        return keep & (x >= x[order[min(last, V - 1)]])

    sizes = []
    for r in range(M):
        x = logits[r, :V].astype(np.float64)
        outer, inner = nucleus(x, min(p + 1e-4, 1.0)), nucleus(x, p - 1e-4)
        sizes.append(int(inner.sum()))
        assert outer[got[r]], (r, got[r])
        score = np.where(inner, x / temp + noise[r], -np.inf)
        assert x[got[r]] / temp + noise[r, got[r]] >= score.max() - 1e-4, (r, got[r])
    assert min(sizes) >= 1 and (p > 0.99 or max(sizes) < V)
