"""CPU self-checks of the oracle: against numpy fp64, hand-computable cases, and a blockwise
(flash-style) restatement of the softmax."""
import numpy as np
import pytest


def test_generators_are_deterministic_and_counter_based(orc):
    a = orc.fill_normal((1001,), seed=5, stream=2)
    b = orc.fill_normal((2000,), seed=5, stream=2)
    assert np.array_equal(a, b[:1001])  # element i depends only on (seed, stream, i)
    assert not np.array_equal(a, orc.fill_normal((1001,), seed=5, stream=3))
    big = orc.fill_normal((200000,), seed=9, mean=1.0, std=0.02)
    assert abs(big.mean() - 1.0) < 3e-4 and abs(big.std() - 0.02) < 2e-4
    t = orc.fill_tokens((4, 64), seed=4321)
    assert t.min() >= 0 and t.max() < 50257 and np.array_equal(t, orc.fill_tokens((4, 64), seed=4321))


def test_tiny_hand_case(orc):
    # C=4, T=2: everything checkable by hand
    x = np.array([[[1, 2, 3, 4], [0, 0, 0, 8]]], np.float32)
    w = np.array([[1, 0, 0, 0], [1, 1, 1, 1]], np.float32)
    out = orc.matmul_forward(x, w, np.array([10, -1], np.float32))
    assert np.array_equal(out, np.array([[[11, 9], [10, 7]]], np.float32))
    y, mean, rstd = orc.layernorm_forward(x, np.ones(4, np.float32), np.zeros(4, np.float32), precise=True)
    assert np.allclose(mean, [[2.5, 2.0]])
    assert np.allclose(rstd, [[1 / np.sqrt(1.25 + 1e-5), 1 / np.sqrt(12 + 1e-5)]], rtol=1e-6)
    assert np.allclose(y[0, 0], (np.array([1, 2, 3, 4]) - 2.5) / np.sqrt(1.25 + 1e-5), rtol=1e-6)
    enc = orc.encoder_forward(np.array([[1, 0]], np.int32), np.array([[1, 1, 1, 1], [2, 2, 2, 2]], np.float32),
                              np.array([[10, 20, 30, 40], [1, 2, 3, 4]], np.float32))
    assert np.array_equal(enc, np.array([[[12, 22, 32, 42], [2, 3, 4, 5]]], np.float32))


@pytest.mark.parametrize("precise", [False, True])
def test_matmul_epilogues_against_numpy(orc, precise):
    x = orc.fill_normal((2, 33, 100), 1)
    w = orc.fill_normal((52, 100), 2, std=0.1)
    b = orc.fill_normal((52,), 3)
    r = orc.fill_normal((2, 33, 52), 4)
    z = x.astype(np.float64) @ w.astype(np.float64).T + b
    gelu = 0.5 * z * (1 + np.tanh(np.sqrt(2 / np.pi) * (z + 0.044715 * z ** 3)))
    assert np.abs(orc.matmul_forward(x, w, b, precise=precise) - z).max() < 1e-5
    assert np.abs(orc.matmul_forward(x, w, b, act=1, precise=precise) - gelu).max() < 1e-5
    assert np.abs(orc.matmul_forward(x, w, b, act=1, residual=r, precise=precise) - (gelu + r)).max() < 1e-5
    assert np.abs(orc.matmul_forward(x, w, None, precise=precise) - (z - b)).max() < 1e-5


def test_layernorm_single_pass_vs_two_pass(orc):
    x = orc.fill_normal((2, 16, 1600), 5, mean=0.5, std=2.0)
    w = orc.fill_normal((1600,), 6, mean=1.0, std=0.1)
    b = orc.fill_normal((1600,), 7)
    y32, m32, r32 = orc.layernorm_forward(x, w, b, precise=False)
    y64, m64, r64 = orc.layernorm_forward(x, w, b, precise=True)
    assert np.abs(y32 - y64).max() < 2e-5 and np.abs(m32 - m64).max() < 1e-6 and np.abs(r32 / r64 - 1).max() < 1e-5


def _attention_blockwise(qkv, NH, block=64):
    """Online-softmax over key blocks, the way the GPU kernel proceeds."""
    B, T, C3 = qkv.shape
    C = C3 // 3
    HS = C // NH
    out = np.zeros((B, T, C))
    q, k, v = (qkv[..., i * C:(i + 1) * C].reshape(B, T, NH, HS).transpose(0, 2, 1, 3).astype(np.float64) for i in range(3))
    for b in range(B):
        for h in range(NH):
            m = np.full(T, -np.inf)
            l = np.zeros(T)
            acc = np.zeros((T, HS))
            for j0 in range(0, T, block):
                s = q[b, h] @ k[b, h, j0:j0 + block].T / np.sqrt(HS)
                cols = np.arange(j0, min(j0 + block, T))
                s = np.where(cols[None, :] <= np.arange(T)[:, None], s, -np.inf)
                mn = np.maximum(m, s.max(-1))
                live = np.isfinite(mn)
                alpha = np.where(live, np.exp(np.where(live, m - mn, 0.0)), 1.0)
                p = np.where(live[:, None], np.exp(s - np.where(live, mn, 0.0)[:, None]), 0.0)
                l = l * alpha + p.sum(-1)
                acc = acc * alpha[:, None] + p @ v[b, h, j0:j0 + block]
                m = mn
            out[b, :, h * HS:(h + 1) * HS] = acc / l[:, None]
    return out


@pytest.mark.parametrize("precise", [False, True])
def test_attention_direct_vs_blockwise_online_softmax(orc, precise):
    qkv = orc.fill_normal((2, 192, 3 * 128), 8)
    out, lse = orc.attention_forward(qkv, 2, precise=precise)
    assert np.abs(out - _attention_blockwise(qkv, 2)).max() < 2e-6
    # first position attends only to itself
    assert np.allclose(out[:, 0], qkv[:, 0, 256:384], atol=1e-6)
    assert np.isfinite(lse).all()


def test_attention_is_causal(orc):
    qkv = orc.fill_normal((1, 64, 3 * 64), 9)
    base, _ = orc.attention_forward(qkv, 1)
    qkv2 = qkv.copy()
    qkv2[0, 40:] += 5.0  # changing later positions must not change earlier outputs
    out2, _ = orc.attention_forward(qkv2, 1)
    assert np.array_equal(base[0, :40], out2[0, :40])


def test_forward_fp32_vs_fp64_accumulation_small_model(orc):
    cfg = orc.GPT2Config(max_seq_len=64, vocab_size=300, padded_vocab_size=320, num_layers=2, num_heads=2, channels=128)
    params = orc.init_params(cfg, 1)
    tok = orc.fill_tokens((2, 64), 2, vocab=300)
    a = orc.gpt2_forward(params, cfg, tok, precise=False)
    b = orc.gpt2_forward(params, cfg, tok, precise=True)
    assert a.shape == (2, 64, 320) and np.abs(a - b).max() < 2e-5
    views = orc.param_views(params, cfg)
    assert np.all(views["ln1w"] == 1) and np.all(views["qkvb"] == 0) and abs(views["wte"].std() - 0.02) < 1e-3
    # sequences are independent
    assert np.array_equal(orc.gpt2_forward(params, cfg, tok[1:], precise=False)[0], a[1])
