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
