"""End-to-end parity of the gpt2_forward driver against the CPU oracle (GPU).

Tolerances are the ones stated for the default path: logits within 2e-2 max-abs of the
fp32 forward and at least 99.9 % top-1 token agreement; the encoder output is bit-exact.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _make(pkg, orc, ctx, cfg_kwargs, B, T):
    cfg = pkg.GPT2Config(**cfg_kwargs)
    ocfg = orc.GPT2Config(**cfg_kwargs)
    params = orc.init_params(ocfg, seed=1234)
    model = pkg.GPT2(ctx, cfg, B, T)
    model.load_params(params)
    return cfg, ocfg, params, model


def test_param_offsets_match_oracle(pkg, orc):
    for kw in (dict(), dict(num_layers=48, num_heads=25, channels=1600)):
        assert pkg.param_offsets(pkg.GPT2Config(**kw)) == orc.param_offsets(orc.GPT2Config(**kw))


def test_gpt2_124m_b4_t64_matches_oracle(pkg, orc, ctx):
    """The CPU-runnable configuration: GPT-2 124M, B=4, T=64, seeded random-init weights."""
    B, T = 4, 64
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(), B, T)
    tokens = orc.fill_tokens((B, T), seed=4321, vocab=cfg.vocab_size)
    want = orc.gpt2_forward(params, ocfg, tokens, precise=False)
    logits = np.empty((B, T, cfg.padded_vocab_size), np.float32)
    last = np.empty((B, cfg.padded_vocab_size), np.float32)
    amax = np.empty((B, T), np.int32)
    model.forward_host(tokens, B, T, logits_host=logits, last_logits_host=last, argmax_host=amax)
    # encoder output is kept in no buffer after the forward (the residual stream is updated in
    # place), so it is checked on its own through the same entry point the driver uses
    assert np.abs(logits - want).max() < 2e-3
    agree = (logits[..., :cfg.vocab_size].argmax(-1) == want[..., :cfg.vocab_size].argmax(-1)).mean()
    assert agree >= 0.996, agree  # 256 positions: at most one near-tie flip; the 99.9 % bar is held on 8192 positions below
    assert np.array_equal(last, logits[:, -1, :])
    assert np.array_equal(amax, logits[..., :cfg.vocab_size].argmax(-1))
    model.close()


def _compare(got, want, V):
    err = np.abs(got - want)
    a_got, a_want = got[:, :V].argmax(-1), want[:, :V].argmax(-1)
    miss = np.nonzero(a_got != a_want)[0]
    srt = np.sort(want[:, :V], axis=-1)
    gaps = (srt[:, -1] - srt[:, -2])[miss]  # the oracle's own top-1/top-2 margin where they differ
    return float(err.max()), float(np.sqrt((err ** 2).mean())), 1.0 - len(miss) / len(a_want), gaps


@pytest.mark.parametrize("mode", ["bf16x3", "tf32", "bf16x3_att_tf32", "tf32x3"])
def test_gpt2_124m_full_length_sequences(pkg, orc, ctx, mode):
    """The benchmark configuration (B=8, T=1024) against the oracle on ALL eight sequences
    (sequences are independent, so the oracle runs them one at a time).

    Stated tolerances: logits within 2e-2 max-abs of the fp32 forward and >= 99.9 % top-1
    agreement.  With seeded random-init weights the logits are nearly tied (the oracle's own
    top-1/top-2 margin is below 5.4e-4 at 0.1 % and below 1.3e-3 at 1 % of the positions), so the
    agreement is a direct reading of the logit error:
      bf16x3       the default: GEMM operands carried as two bf16 terms (16 significant bits), attention
                   on fp16 planes of q, k, v: logit error about 5e-5 rms; held to 99.9 % over the 8192
                   positions, to 99.7 % on every sequence (1024 positions: three flips) and to "every miss
                   is a tie within the error" (the oracle's own margin there is below 2.5e-4)
      tf32x3       3xTF32 GEMMs and attention: fp32-level logits (about 1e-5 rms), 99.9 % per
                   sequence and 1e-4 of the largest logit
      bf16x3_att_tf32  bf16x3 GEMMs with the single-pass TF32 attention kernel: about 1.1e-4 rms (what
                   is left comes from the attention's P.V product); holds 99.9 % over the 8192 positions
      tf32         one TF32 pass per GEMM, round-to-nearest operands: 4.6e-4 rms, which flips 0.2-0.3 %
                   of the arg-maxes; held to max-abs, to >= 99 % and to "only near-ties are missed"."""
    import torch
    assert pkg.DEFAULT_MODE_NAME == "bf16x3"
    B, T = 8, 1024
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(), B, T)
    if mode != pkg.DEFAULT_MODE_NAME:  # the default is what a fresh model runs
        model.set_options(**pkg.MODES[mode])
    tokens = orc.fill_tokens((B, T), seed=4321, vocab=cfg.vocab_size)
    d_tok = torch.from_numpy(tokens).cuda()
    torch.cuda.synchronize()
    logits = model.forward(d_tok, B, T)
    ctx.sync_check()
    assert torch.isfinite(logits).all()
    got_all = logits.cpu().numpy()
    model.close()
    misses = 0
    for b in range(B):
        want = orc.gpt2_forward(params, ocfg, tokens[b:b + 1], precise=False)[0]
        mx, rms, agree, gaps = _compare(got_all[b], want, cfg.vocab_size)
        misses += len(gaps)
        print(f"{mode} seq {b}: max-abs {mx:.3e}, rms {rms:.3e}, top-1 agreement {agree:.5f}, "
              f"largest oracle margin among the misses {gaps.max() if len(gaps) else 0:.2e}")
        assert mx < 2e-2
        if mode == "tf32":
            assert agree >= 0.99, agree
            assert rms < 7e-4
            assert len(gaps) == 0 or gaps.max() < 4e-3, "a top-1 miss that is not a near-tie"
        elif mode == "bf16x3_att_tf32":
            assert agree >= 0.997, agree
            assert rms < 2e-4
            assert len(gaps) == 0 or gaps.max() < 1e-3, "a top-1 miss that is not a near-tie"
        elif mode == "bf16x3":
            assert agree >= 0.997, agree
            assert rms < 1e-4
            assert mx < 2e-3
            assert len(gaps) == 0 or gaps.max() < 2.5e-4, "a top-1 miss that is not a near-tie"
        else:
            assert agree >= 0.999, agree
            assert rms < 5e-5
            assert mx < 1e-4 * np.abs(want).max()  # "within 1e-4 relative error"
    total = 1.0 - misses / (B * T)
    print(f"{mode}: top-1 agreement over all {B * T} positions {total:.5f} ({misses} misses)")
    if mode != "tf32":
        assert total >= 0.999, total


def test_batch_rows_are_independent_and_deterministic(pkg, orc, ctx):
    """A sequence's logits do not depend on what else is in the batch nor on its position in
    it (bitwise): this is what makes batch sharding across GPUs exact."""
    import torch
    B, T = 4, 128
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(num_layers=2), B, T)
    tokens = orc.fill_tokens((B, T), seed=99, vocab=cfg.vocab_size)
    d_tok = torch.from_numpy(tokens).cuda()
    torch.cuda.synchronize()
    # the forward runs on the context's stream: synchronise before torch touches the logits
    out = model.forward(d_tok, B, T)
    ctx.sync_check()
    full = out.clone()
    out = model.forward(d_tok, B, T)
    ctx.sync_check()
    again = out.clone()
    torch.cuda.synchronize()
    assert torch.equal(full, again)
    for start, stop in (pkg.shard_batch(B, 2, r) for r in range(2)):
        part = model.forward(d_tok[start:stop].contiguous(), stop - start, T)
        ctx.sync_check()
        assert torch.equal(part, full[start:stop])
    model.close()


def test_graph_replay_matches_eager(pkg, orc, ctx):
    import torch
    B, T = 2, 128
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(num_layers=2), B, T)
    tokens = orc.fill_tokens((B, T), seed=7, vocab=cfg.vocab_size)
    d_tok = torch.from_numpy(tokens).cuda()
    torch.cuda.synchronize()
    out = model.forward(d_tok, B, T)
    ctx.sync_check()
    eager = out.clone()
    torch.cuda.synchronize()
    model.set_options(use_graph=1)
    n0 = ctx.launches
    for _ in range(3):
        g = model.forward(d_tok, B, T)
        ctx.sync_check()
        assert torch.equal(g, eager), f"max diff {(g - eager).abs().max().item()} nan {torch.isnan(g).sum().item()}"
    assert ctx.launches - n0 >= 3 * (2 + 7 * cfg.num_layers + 1)
    model.close()


@pytest.mark.parametrize("use_graph", [0, 1])
def test_fused_argmax_matches_the_logits(pkg, orc, ctx, use_graph):
    """The host-buffer call takes the per-position arg-max out of the lm-head GEMM's epilogue
    instead of a second pass over the logits: it must equal the arg-max of the logits the same
    call returns, bit for bit (ties to the lowest index, padded vocabulary columns excluded).
    B*T = 2048 rows puts the lm-head on the CTA-pair kernel, as in the benchmark configuration;
    the second call repeats the first (keys are reset per call; with use_graph it is a replay)."""
    B, T = 2, 1024
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(num_layers=1), B, T)
    model.set_options(use_graph=use_graph)
    for seed in (11, 12, 11):
        tokens = orc.fill_tokens((B, T), seed=seed, vocab=cfg.vocab_size)
        logits = np.empty((B, T, cfg.padded_vocab_size), np.float32)
        amax = np.empty((B, T), np.int32)
        model.forward_host(tokens, B, T, logits_host=logits, argmax_host=amax)
        assert np.array_equal(amax, logits[..., :cfg.vocab_size].argmax(-1))
    # a column of the padding that would win if it were not excluded
    params2 = params.copy()
    off = pkg.param_offsets(cfg)
    wte = params2[off[0]:off[0] + cfg.padded_vocab_size * cfg.channels].reshape(cfg.padded_vocab_size, cfg.channels)
    wte[cfg.vocab_size:] = 50.0 * np.sign(wte[0])  # large positive logit wherever it correlates
    model.load_params(params2)
    tokens = orc.fill_tokens((B, T), seed=13, vocab=cfg.vocab_size)
    logits = np.empty((B, T, cfg.padded_vocab_size), np.float32)
    amax = np.empty((B, T), np.int32)
    model.forward_host(tokens, B, T, logits_host=logits, argmax_host=amax)
    assert (logits.argmax(-1) >= cfg.vocab_size).any(), "the padding never wins: the case tests nothing"
    assert np.array_equal(amax, logits[..., :cfg.vocab_size].argmax(-1))
    model.close()


def test_xl_shapes_small_batch(pkg, orc, ctx):
    """GPT-2 XL dimensions (C=1600, 25 heads) on a 4-layer stack, B=1 T=128, against the oracle."""
    B, T = 1, 128
    kw = dict(num_layers=4, num_heads=25, channels=1600)
    cfg, ocfg, params, model = _make(pkg, orc, ctx, kw, B, T)
    tokens = orc.fill_tokens((B, T), seed=5, vocab=cfg.vocab_size)
    want = orc.gpt2_forward(params, ocfg, tokens, precise=False)
    logits = np.empty((B, T, cfg.padded_vocab_size), np.float32)
    model.forward_host(tokens, B, T, logits_host=logits)
    assert np.abs(logits - want).max() < 2e-2
    agree = (logits[..., :cfg.vocab_size].argmax(-1) == want[..., :cfg.vocab_size].argmax(-1)).mean()
    assert agree >= 0.99, agree
    model.close()


def test_out_of_range_token_is_reported(pkg, orc, ctx):
    B, T = 1, 64
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(num_layers=1), B, T)
    tokens = np.zeros((B, T), np.int32)
    tokens[0, 3] = cfg.padded_vocab_size + 5
    with pytest.raises(pkg.B200Error):
        model.forward_host(tokens, B, T)
    # the context stays usable
    tokens[0, 3] = 1
    model.forward_host(tokens, B, T)
    model.close()


def test_forward_rejects_sizes_beyond_the_allocation(pkg, orc, ctx):
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(num_layers=1), 1, 64)
    tokens = np.zeros((2, 64), np.int32)
    with pytest.raises(pkg.B200Error, match="maximum"):
        model.forward_host(tokens, 2, 64)
    with pytest.raises(pkg.B200Error):
        model.forward_host(tokens, 1, 100)  # T % 64
    model.close()


@pytest.mark.parametrize("lmhead_bf16", [True, False])
def test_bf16_operand_mode_stays_close_to_the_fp32_forward(pkg, orc, ctx, lmhead_bf16):
    """The optional bf16 mode (GEMM operands rounded to bf16, fp32 accumulation, everything between
    the GEMMs in fp32; attention stays on the TF32 path).  bf16 keeps 8 significant bits against
    TF32's 11, so its bar is four times the TF32 one: logits within 8e-2 max-abs (measured: a
    quarter of that) and top-1 misses only on near-ties of the oracle's own logits."""
    import torch
    B, T = 2, 256
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(), B, T)
    model.set_options(round_operands=1, gemm_mode=pkg.B200_BF16,
                      lmhead_mode=pkg.B200_BF16 if lmhead_bf16 else pkg.B200_TF32)
    tokens = orc.fill_tokens((B, T), seed=4321, vocab=cfg.vocab_size)
    want = orc.gpt2_forward(params, ocfg, tokens, precise=False)
    d_tok = torch.from_numpy(tokens).cuda()
    torch.cuda.synchronize()
    logits = model.forward(d_tok, B, T)
    ctx.sync_check()
    assert torch.isfinite(logits).all()
    got = logits.cpu().numpy()
    mx, rms, agree, gaps = _compare(got.reshape(B * T, -1), want.reshape(B * T, -1), cfg.vocab_size)
    print(f"bf16 (lm-head bf16: {lmhead_bf16}): max-abs {mx:.3e}, rms {rms:.3e}, top-1 agreement {agree:.5f}, "
          f"largest oracle margin among the misses {gaps.max() if len(gaps) else 0:.2e}")
    assert mx < 8e-2
    assert rms < 6e-3
    assert agree >= 0.95, agree
    assert len(gaps) == 0 or gaps.max() < 2e-2, "a top-1 miss that is not a near-tie"
    # the arg-max fused into the bf16 lm-head agrees with the logits it wrote
    if lmhead_bf16:
        amax = np.empty((B, T), np.int32)
        lg = np.empty((B, T, cfg.padded_vocab_size), np.float32)
        model.forward_host(tokens, B, T, logits_host=lg, argmax_host=amax)
        assert np.array_equal(amax, lg[..., :cfg.vocab_size].argmax(-1))
    model.close()


def test_load_params_file_reads_raw_parameters_behind_a_header(pkg, orc, ctx, tmp_path):
    """The raw parameter-file loader: skip the caller's header, copy the fp32 parameters in
    param_offsets order; a file of the wrong size or a missing file is refused."""
    kw = dict(num_layers=2)
    cfg, ocfg, params, model = _make(pkg, orc, ctx, kw, 1, 64)
    good = tmp_path / "params.bin"
    with open(good, "wb") as f:
        f.write(b"\x5a" * 1024)
        f.write(params.tobytes())
    fresh = pkg.GPT2(ctx, cfg, 1, 64)
    fresh.load_params_file(str(good), 1024)
    assert np.array_equal(fresh.params_tensor().cpu().numpy(), params)
    tokens = orc.fill_tokens((1, 64), seed=5, vocab=cfg.vocab_size)
    a = np.empty((1, 64, cfg.padded_vocab_size), np.float32)
    b = np.empty_like(a)
    model.forward_host(tokens, 1, 64, logits_host=a)
    fresh.forward_host(tokens, 1, 64, logits_host=b)
    assert np.array_equal(a, b)
    with pytest.raises(pkg.B200Error):
        fresh.load_params_file(str(good), 1020)          # size does not match
    with pytest.raises(pkg.B200Error):
        fresh.load_params_file(str(tmp_path / "absent.bin"), 0)
    fresh.close()
    model.close()


@pytest.mark.parametrize("use_graph,bf16", [(0, False), (1, False), (0, True)])
def test_enqueue_wait_pair_matches_the_synchronous_host_call(pkg, orc, ctx, use_graph, bf16):
    """Two batches in flight through forward_host_enqueue / _wait return exactly what the
    synchronous forward_host returns for each of them; a bad token id is reported by the wait of
    the batch that holds it."""
    import torch
    B, T = 2, 128
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(num_layers=2), B, T)
    mode = pkg.B200_BF16 if bf16 else pkg.B200_TF32
    model.set_options(round_operands=1, gemm_mode=mode, lmhead_mode=mode, use_graph=use_graph)  # graph replay: results go through copies
    V, Vp = cfg.vocab_size, cfg.padded_vocab_size
    toks = [torch.from_numpy(orc.fill_tokens((B, T), seed=s, vocab=V)).pin_memory() for s in (11, 12, 13)]
    want = []
    for t in toks:
        last, amax = np.empty((B, Vp), np.float32), np.empty((B, T), np.int32)
        model.forward_host(t.numpy(), B, T, last_logits_host=last, argmax_host=amax)
        want.append((last, amax))
    # without logits_host the lm-head skips the stores of all but the last-position rows: ids and
    # last logits must still be those of the full logits
    full = np.empty((B, T, Vp), np.float32)
    model.forward_host(toks[0].numpy(), B, T, logits_host=full)
    assert np.array_equal(want[0][0], full[:, -1, :])
    assert np.array_equal(want[0][1], full[..., :V].argmax(-1))
    bufs = [(torch.empty((B, Vp)).pin_memory(), torch.empty((B, T), dtype=torch.int32).pin_memory()) for _ in range(2)]
    got = []
    model.forward_host_enqueue(toks[0].numpy(), B, T, 0, last_logits_host=bufs[0][0].numpy(), argmax_host=bufs[0][1].numpy())
    for i in (1, 2):
        model.forward_host_enqueue(toks[i].numpy(), B, T, i & 1, last_logits_host=bufs[i & 1][0].numpy(), argmax_host=bufs[i & 1][1].numpy())
        model.forward_host_wait((i - 1) & 1)
        got.append((bufs[(i - 1) & 1][0].numpy().copy(), bufs[(i - 1) & 1][1].numpy().copy()))
    model.forward_host_wait(0)
    got.append((bufs[0][0].numpy().copy(), bufs[0][1].numpy().copy()))
    for (wl, wa), (gl, ga) in zip(want, got):
        assert np.array_equal(wl, gl) and np.array_equal(wa, ga)
    bad = toks[0].clone().pin_memory()
    bad[1, 5] = V + 1000
    model.forward_host_enqueue(bad.numpy(), B, T, 1, last_logits_host=bufs[1][0].numpy())
    with pytest.raises(pkg.B200Error):
        model.forward_host_wait(1)
    model.forward_host_enqueue(toks[0].numpy(), B, T, 0, last_logits_host=bufs[0][0].numpy())
    model.forward_host_wait(0)  # the context is usable again
    assert np.array_equal(bufs[0][0].numpy(), want[0][0])
    model.close()


@pytest.mark.parametrize("mode,temperature", [("bf16x3", 0.8), ("tf32", 1.3), ("bf16x3", 0.0)])
def test_sampling_and_lse_fused_into_the_lmhead(pkg, orc, ctx, mode, temperature):
    """b200_gpt2_forward_sample draws every position's token and forms log-sum-exp in the lm-head
    GEMM's epilogue.  The draw must be exactly the one b200_sample_rows makes from the stored logits of
    the plain forward (same noise function, same logits bits), and lse must be the log-sum-exp of those
    logits over the real vocabulary; without stored logits the results must not change."""
    import torch
    B, T = 2, 1024   # 2048 rows: CTA-pair kernel, as in the benchmark configuration
    cfg, ocfg, params, model = _make(pkg, orc, ctx, dict(num_layers=1), B, T)
    model.set_options(**pkg.MODES[mode])
    V, Vp = cfg.vocab_size, cfg.padded_vocab_size
    tokens = orc.fill_tokens((B, T), seed=21, vocab=V)
    d_tok = torch.from_numpy(tokens).cuda()
    torch.cuda.synchronize()
    logits = model.forward(d_tok, B, T)
    ctx.sync_check()
    logits = logits.clone()
    want_ids = torch.empty((B * T,), dtype=torch.int32, device="cuda")
    ctx.sample_rows(want_ids, logits.view(B * T, Vp), B * T, V, Vp, temperature, 1234, 0)
    ctx.sync_check()
    want_lse = torch.logsumexp(logits.view(B * T, Vp)[:, :V].double(), dim=-1).float()
    for store in (True, False):
        ids = torch.full((B, T), -1, dtype=torch.int32, device="cuda")
        lse = torch.full((B, T), float("nan"), device="cuda")
        torch.cuda.synchronize()
        model.forward_sample(d_tok, B, T, ids, temperature=temperature, seed=1234, lse_out=lse, store_logits=store)
        ctx.sync_check()
        assert torch.equal(ids.view(-1), want_ids), f"{(ids.view(-1) != want_ids).sum().item()} draws differ"
        assert (lse.view(-1) - want_lse).abs().max().item() < 1e-4
        if store:
            got = model.forward(d_tok, B, T)  # same bits as before: the extra epilogue work does not touch the logits
            ctx.sync_check()
            assert torch.equal(got, logits)
    if temperature > 0:
        # the draws follow the softmax: their mean log-probability is close to its expectation (minus the entropy)
        lp = torch.log_softmax(logits.view(B * T, Vp)[:, :V].double() / temperature, dim=-1)
        mean_lp = lp.gather(1, want_ids.long().view(-1, 1)).mean().item()
        ent = -(lp.exp() * lp).sum(-1).mean().item()
        assert abs(mean_lp + ent) < 0.2, (mean_lp, ent)
    model.close()
