"""b200_gpt2_forward_static: the forward for callers that may not allocate device memory.

Some users of this library run where cudaMalloc is off limits - the application owns the whole
GPU through its own pool, the host process forbids driver allocations after start-up, or a serving
loop cannot take the device-wide synchronisation an allocation implies.  The entry point keeps the
activations in an array built into the library; this test checks, through the C ABI, that it gives
exactly the logits of the allocating entry point (b200_gpt2_forward with round_operands = 0 and
single-pass TF32 GEMMs: same
kernels, same order, so the comparison is bitwise), twice in a row with different inputs - the
second call finds the first call's leftovers in the shared scratch array.  The file sorts last so
that a run stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = dict(max_seq_len=128, vocab_size=1000, padded_vocab_size=1024, num_layers=2, num_heads=2, channels=128)


def test_static_forward_matches_allocating_forward_twice(pkg, orc, ctx):
    import torch
    cfg = pkg.GPT2Config(**CFG)
    params = orc.init_params(orc.GPT2Config(**CFG), seed=77)
    d_params = torch.from_numpy(params).cuda()
    model = pkg.GPT2(ctx, cfg, 2, 128)
    model.load_params(params)
    model.set_options(round_operands=0, gemm_mode=pkg.B200_TF32, lmhead_mode=pkg.B200_TF32)
    for seed, (B, T) in ((1, (2, 128)), (2, (1, 64))):
        tokens = orc.fill_tokens((B, T), seed=seed, vocab=cfg.vocab_size)
        d_tok = torch.from_numpy(tokens).cuda()
        want = model.forward(d_tok, B, T)
        ctx.sync_check()
        want = want.clone()
        got = torch.full((B, T, cfg.padded_vocab_size), float("nan"), device="cuda")
        torch.cuda.synchronize()
        st = pkg.gpt2_forward_static(ctx, cfg, d_params, d_tok, B, T, got)
        assert st == 0, pkg.lib().b200_status_string(st)
        ctx.sync_check()
        assert torch.isfinite(got).all()
        assert torch.equal(got, want), f"max diff {(got - want).abs().max().item()}"
        # and against the CPU oracle, within the tolerance of the other forward tests
        ref = orc.gpt2_forward(params, orc.GPT2Config(**CFG), tokens)
        assert np.abs(got.cpu().numpy() - ref).max() < 2e-2
    model.close()


def test_static_forward_rejects_sizes_beyond_its_scratch(pkg, ctx):
    import torch
    cfg = pkg.GPT2_124M
    B, T = 8, 64  # 8*64*768 = 393216 > 196608
    assert B * T * cfg.channels > pkg.STATIC_MAX_TOKEN_CHANNELS
    dummy = torch.zeros(16, device="cuda")
    tok = torch.zeros((B, T), dtype=torch.int32, device="cuda")
    st = pkg.gpt2_forward_static(ctx, cfg, dummy, tok, B, T, dummy)
    assert st == 8  # B200_ERR_LIMIT, before anything is launched or read
    assert b"exceeds the built-in scratch" in pkg.lib().b200_ctx_last_error(ctx._h)
    assert pkg.gpt2_forward_static(ctx, cfg, dummy, tok, 1, 100, dummy) == 2  # T % 64
    ctx.sync_check()


def test_static_forward_at_its_documented_maximum(pkg, orc, ctx):
    """GPT-2 124M with B=4, T=64 is exactly B*T*C = 196608, the largest problem the built-in scratch
    array holds; bitwise against the allocating forward, as above."""
    import torch
    cfg = pkg.GPT2_124M
    B, T = 4, 64
    assert B * T * cfg.channels == pkg.STATIC_MAX_TOKEN_CHANNELS
    params = orc.init_params(orc.GPT2_124M, seed=1234)
    d_params = torch.from_numpy(params).cuda()
    model = pkg.GPT2(ctx, cfg, B, T)
    model.load_params(params)
    model.set_options(round_operands=0, gemm_mode=pkg.B200_TF32, lmhead_mode=pkg.B200_TF32)
    tokens = orc.fill_tokens((B, T), seed=4321, vocab=cfg.vocab_size)
    d_tok = torch.from_numpy(tokens).cuda()
    want = model.forward(d_tok, B, T)
    ctx.sync_check()
    want = want.clone()
    got = torch.full((B, T, cfg.padded_vocab_size), float("nan"), device="cuda")
    torch.cuda.synchronize()
    assert pkg.gpt2_forward_static(ctx, cfg, d_params, d_tok, B, T, got) == 0
    ctx.sync_check()
    assert torch.equal(got, want)
    model.close()


_FRESH_PROCESS = r"""
import sys, numpy as np, torch
sys.path.insert(0, {root!r})
import __graft_entry__ as ge
from oracle import oracle as orc
pkg = ge.load_package()
torch.cuda.set_device(0)
stream = torch.cuda.Stream()
ctx = pkg.Context(0, stream)
kw = dict(max_seq_len=128, vocab_size=1000, padded_vocab_size=1024, num_layers=2, num_heads=2, channels=128)
cfg = pkg.GPT2Config(**kw)
params = orc.init_params(orc.GPT2Config(**kw), seed=77)
B, T = 2, 128
tokens = orc.fill_tokens((B, T), seed=1, vocab=cfg.vocab_size)
d_params = torch.from_numpy(params).cuda()
d_tok = torch.from_numpy(tokens).cuda()
got = torch.empty((B, T, cfg.padded_vocab_size), device="cuda")
assert pkg.gpt2_static_prepare(ctx) == 0          # the last moment at which allocation is allowed
torch.cuda.synchronize()
free_before = torch.cuda.mem_get_info()[0]
for _ in range(2):
    assert pkg.gpt2_forward_static(ctx, cfg, d_params, d_tok, B, T, got) == 0
    ctx.sync_check()
free_after = torch.cuda.mem_get_info()[0]
ref = orc.gpt2_forward(params, orc.GPT2Config(**kw), tokens)
assert np.abs(got.cpu().numpy() - ref).max() < 2e-2
print("FREE", free_before, free_after)
"""


def test_no_device_memory_is_taken_after_the_prepare_step():
    """In a fresh process (no kernel of the library has run yet): after b200_gpt2_static_prepare the
    static forward must not reduce the device's free memory - not through cudaMalloc and not
    through the CUDA runtime loading kernel code at a first launch."""
    import os
    import subprocess
    import sys
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", _FRESH_PROCESS.format(root=root)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    line = [l for l in out.stdout.splitlines() if l.startswith("FREE")][-1].split()
    before, after = int(line[1]), int(line[2])
    assert after >= before, f"free device memory went from {before} to {after} bytes across b200_gpt2_forward_static"
