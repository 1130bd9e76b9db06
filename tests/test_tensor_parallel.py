"""Tensor-parallel (Megatron-style) split of the forward: the sharding plan on CPU (numpy, and as
two gloo ranks around the oracle's operators), and the CUDA driver on two GPUs when present."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = dict(max_seq_len=64, vocab_size=300, padded_vocab_size=320, num_layers=2, num_heads=5, channels=320)


def test_head_split_is_a_partition(pkg):
    for nh, n in ((25, 2), (25, 4), (25, 8), (12, 4), (5, 2)):
        spans = [pkg.tp_heads(nh, n, r) for r in range(n)]
        assert spans[0][0] == 0 and sum(c for _, c in spans) == nh
        assert all(a[0] + a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert [pkg.tp_heads(25, 8, r)[1] for r in range(8)] == [4, 3, 3, 3, 3, 3, 3, 3]


@pytest.mark.parametrize("tp_size", [2, 4])
def test_shard_params_against_numpy_slices(pkg, orc, tp_size):
    cfg, ocfg = pkg.GPT2Config(**SMALL), orc.GPT2Config(**SMALL)
    full = orc.fill_normal((orc.param_offsets(ocfg)[16],), 5)
    fv = orc.param_views(full, ocfg)
    C, L = cfg.channels, cfg.num_layers
    for r in range(tp_size):
        local = pkg.shard_params(cfg, tp_size, r, full)
        off = pkg.param_offsets_tp(cfg, tp_size, r)
        h0, nh = pkg.tp_heads(cfg.num_heads, tp_size, r)
        A, a0, F, f0 = nh * 64, h0 * 64, 4 * C // tp_size, r * (4 * C // tp_size)
        get = lambda i, shape: local[off[i]:off[i + 1]].reshape(shape)
        qkvw = fv["qkvw"].reshape(L, 3, C, C)[:, :, a0:a0 + A, :].reshape(L, 3 * A, C)
        assert np.array_equal(get(4, (L, 3 * A, C)), qkvw)
        assert np.array_equal(get(5, (L, 3 * A)), fv["qkvb"].reshape(L, 3, C)[:, :, a0:a0 + A].reshape(L, 3 * A))
        assert np.array_equal(get(6, (L, C, A)), fv["attprojw"][:, :, a0:a0 + A])
        assert np.array_equal(get(10, (L, F, C)), fv["fcw"][:, f0:f0 + F, :])
        assert np.array_equal(get(11, (L, F)), fv["fcb"][:, f0:f0 + F])
        assert np.array_equal(get(12, (L, C, F)), fv["fcprojw"][:, :, f0:f0 + F])
        for i, name in ((7, "attprojb"), (13, "fcprojb")):
            assert np.array_equal(get(i, (L, C)), fv[name] if r == 0 else np.zeros((L, C), np.float32))
        for i, name in ((0, "wte"), (1, "wpe"), (2, "ln1w"), (9, "ln2b"), (14, "lnfw")):
            assert np.array_equal(local[off[i]:off[i + 1]], fv[name].ravel())


_CPU_RANK = r"""
import sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
import __graft_entry__ as ge
from oracle import oracle as orc
pkg = ge.load_package()
dist.init_process_group("gloo")
r, n = dist.get_rank(), dist.get_world_size()
kw = {small!r}
cfg, ocfg = pkg.GPT2Config(**kw), orc.GPT2Config(**kw)
full = orc.init_params(ocfg, 11)
full[orc.param_offsets(ocfg)[7]:orc.param_offsets(ocfg)[8]] = 0.01   # non-zero projection biases
tokens = orc.fill_tokens((2, 64), 12, vocab=cfg.vocab_size)
local = pkg.shard_params(cfg, n, r, full)
off = pkg.param_offsets_tp(cfg, n, r)
C, L = cfg.channels, cfg.num_layers
h0, nh = pkg.tp_heads(cfg.num_heads, n, r)
A, F = nh * 64, 4 * C // n
P = lambda i, shape: local[off[i]:off[i + 1]].reshape(shape)
def allreduce(x):
    t = torch.from_numpy(x); dist.all_reduce(t); return t.numpy()
x = orc.encoder_forward(tokens, P(0, (cfg.padded_vocab_size, C)), P(1, (cfg.max_seq_len, C)))
ln, _, _ = orc.layernorm_forward(x, P(2, (L, C))[0], P(3, (L, C))[0])
for l in range(L):
    qkv = orc.matmul_forward(ln, P(4, (L, 3 * A, C))[l], P(5, (L, 3 * A))[l])
    att, _ = orc.attention_forward(qkv, nh)
    br = allreduce(orc.matmul_forward(att, P(6, (L, C, A))[l], P(7, (L, C))[l]))      # one all-reduce per block
    x, ln, _, _ = orc.fused_residual_layernorm_forward(x, br, P(8, (L, C))[l], P(9, (L, C))[l])
    fch = orc.matmul_forward(ln, P(10, (L, F, C))[l], P(11, (L, F))[l], act=1)
    br = allreduce(orc.matmul_forward(fch, P(12, (L, C, F))[l], P(13, (L, C))[l]))
    nw, nb = (P(2, (L, C))[l + 1], P(3, (L, C))[l + 1]) if l + 1 < L else (P(14, (C,)), P(15, (C,)))
    x, ln, _, _ = orc.fused_residual_layernorm_forward(x, br, nw, nb)
Vl = cfg.padded_vocab_size // n
mine = orc.matmul_forward(ln, P(0, (cfg.padded_vocab_size, C))[r * Vl:(r + 1) * Vl], None)   # logits stay sharded
parts = [None] * n
dist.all_gather_object(parts, mine)
if r == 0:
    want = orc.gpt2_forward(full, ocfg, tokens)
    got = np.concatenate(parts, axis=-1)
    err = np.abs(got - want).max()
    assert err < 2e-5, err
    print("TP_PLAN_OK", err)

# The same forward with the sequence-parallel hand-over in place of the all-reduce (the plan of
# b200_gpt2_tp_sp_*): rank s owns the rows [s, s+1) * M / n; every rank hands the owner its partial sum
# for the owner's rows, the owner adds the n parts in rank order to its rows of the residual stream,
# normalises them, and every rank gathers the normalised rows of all owners.
M = tokens.size
rows = M // n
def handover(x_own, partial, w, b):
    mine = [np.ascontiguousarray(partial.reshape(M, C)[s * rows:(s + 1) * rows]) for s in range(n)]
    got = [None] * n
    for s in range(n):  # (gloo has no all-to-all for numpy objects: one gather per owner)
        box = [None] * n if s == r else None
        dist.gather_object(mine[s], box, dst=s)
        if s == r:
            got = box
    total = got[0].copy()
    for s in range(1, n):
        total += got[s]
    x_new, ln_own, _, _ = orc.fused_residual_layernorm_forward(x_own[None], total[None], w, b)
    every = [None] * n
    dist.all_gather_object(every, ln_own[0])
    return x_new[0], np.concatenate(every, axis=0).reshape(tokens.shape + (C,))
x = orc.encoder_forward(tokens, P(0, (cfg.padded_vocab_size, C)), P(1, (cfg.max_seq_len, C)))
ln, _, _ = orc.layernorm_forward(x, P(2, (L, C))[0], P(3, (L, C))[0])
x_own = x.reshape(M, C)[r * rows:(r + 1) * rows].copy()
for l in range(L):
    qkv = orc.matmul_forward(ln, P(4, (L, 3 * A, C))[l], P(5, (L, 3 * A))[l])
    att, _ = orc.attention_forward(qkv, nh)
    x_own, ln = handover(x_own, orc.matmul_forward(att, P(6, (L, C, A))[l], P(7, (L, C))[l]), P(8, (L, C))[l], P(9, (L, C))[l])
    fch = orc.matmul_forward(ln, P(10, (L, F, C))[l], P(11, (L, F))[l], act=1)
    nw, nb = (P(2, (L, C))[l + 1], P(3, (L, C))[l + 1]) if l + 1 < L else (P(14, (C,)), P(15, (C,)))
    x_own, ln = handover(x_own, orc.matmul_forward(fch, P(12, (L, C, F))[l], P(13, (L, C))[l]), nw, nb)
mine = orc.matmul_forward(ln, P(0, (cfg.padded_vocab_size, C))[r * Vl:(r + 1) * Vl], None)
parts = [None] * n
dist.all_gather_object(parts, mine)
if r == 0:
    got = np.concatenate(parts, axis=-1)
    err = np.abs(got - want).max()
    assert err < 2e-5, err
    print("TP_SP_PLAN_OK", err)
dist.barrier(); dist.destroy_process_group()
"""


def test_tp_plan_two_gloo_ranks(tmp_path):
    """The sharding plan with the oracle's operators and a gloo all-reduce on CPU: one all-reduce
    after attn-proj and one after fc-proj per block reproduces the unsharded forward."""
    script = tmp_path / "tp_rank.py"
    script.write_text(_CPU_RANK.format(root=ROOT, small=SMALL))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29544", str(script)],
                         capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2"), cwd=ROOT)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "TP_PLAN_OK" in out.stdout
    assert "TP_SP_PLAN_OK" in out.stdout


_GPU_RANK = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
import __graft_entry__ as ge
from oracle import oracle as orc
pkg = ge.load_package()
r = int(os.environ["LOCAL_RANK"]); torch.cuda.set_device(r)
dist.init_process_group("nccl", device_id=torch.device("cuda", r))
n = dist.get_world_size()
kw = dict(max_seq_len=128, vocab_size=1000, padded_vocab_size=1024, num_layers=3, num_heads=5, channels=320)
cfg, ocfg = pkg.GPT2Config(**kw), orc.GPT2Config(**kw)
full = orc.init_params(ocfg, 21)
tokens = orc.fill_tokens((4, 128), 22, vocab=cfg.vocab_size)
stream = torch.cuda.Stream(); ctx = pkg.Context(r, stream)
model = pkg.GPT2(ctx, cfg, 4, 128, tp_size=n, tp_rank=r)
model.load_params(pkg.shard_params(cfg, n, r, full))
model.set_allreduce_torch(stream)
d_tok = torch.from_numpy(tokens).cuda(); torch.cuda.synchronize()
for _ in range(2):
    logits = model.forward(d_tok, 4, 128); ctx.sync_check()
parts = [torch.empty_like(logits) for _ in range(n)]
dist.all_gather(parts, logits.contiguous())
if r == 0:
    got = torch.cat(parts, dim=-1).cpu().numpy()
    want = orc.gpt2_forward(full, ocfg, tokens)
    err = np.abs(got - want).max()
    assert err < 2e-2, err
    print("TP_GPU_OK", err, model.read_profile() if False else "")
# the same forward with the partial sums handed over through peer memory instead of all-reduces:
# local + peer is the all-reduce's sum, bit for bit, on both ranks
nccl_logits = logits.clone()
model.connect_tp_peer()
for _ in range(3):
    logits = model.forward(d_tok, 4, 128); ctx.sync_check()
    assert torch.equal(logits, nccl_logits), float((logits - nccl_logits).abs().max())
# another shape (the hand-over's tensor maps follow the row count)
l2 = model.forward(d_tok[:1, :64].contiguous(), 1, 64); ctx.sync_check()
assert torch.equal(l2[0], nccl_logits[0, :64]) or float((l2[0] - nccl_logits[0, :64]).abs().max()) < 2e-3
# off (the all-reduce callback again) and on again: same bits every way
model.enable_tp_peer(False)
logits = model.forward(d_tok, 4, 128); ctx.sync_check()
assert torch.equal(logits, nccl_logits)
model.enable_tp_peer(True)
logits = model.forward(d_tok, 4, 128); ctx.sync_check()
assert torch.equal(logits, nccl_logits)
# the sequence-parallel hand-over (each rank normalises its own half of the rows): for two ranks again
# the all-reduce's bits.  The all-reduce callback is taken away first, so a silent fall-back would fail.
model.connect_tp_sequence_parallel()
import ctypes
pkg.lib().b200_gpt2_set_allreduce(model._h, pkg.ALLREDUCE_FN(), None)
for _ in range(3):
    logits = model.forward(d_tok, 4, 128); ctx.sync_check()
    assert torch.equal(logits, nccl_logits), float((logits - nccl_logits).abs().max())
model.set_allreduce_torch(stream)
dist.barrier()
if r == 0:
    print("TP_SP_OK")
dist.barrier()
if r == 0:
    print("TP_PEER_OK")
# the default arithmetic of the unsharded model (split-bf16 GEMMs, fp16 attention) on the sharded one
model.set_options(**pkg.MODES["bf16x3"])
lx = model.forward(d_tok, 4, 128); ctx.sync_check()
parts = [torch.empty_like(lx) for _ in range(n)]
dist.all_gather(parts, lx.contiguous())
if r == 0:
    got = torch.cat(parts, dim=-1).cpu().numpy()
    want = orc.gpt2_forward(full, ocfg, tokens)
    err = np.abs(got - want).max()
    assert err < 2e-3, err
    assert np.sqrt(np.mean((got - want) ** 2)) < 1e-4
    print("TP_X3_OK", err)
dist.barrier(); dist.destroy_process_group()
"""


@pytest.mark.gpu
def test_tp_forward_two_gpus(tmp_path):
    """Two CUDA ranks, one NCCL all-reduce per block (NVLS off: a plain ring is all this needs); then the
    same forward with the partial sums handed over through peer memory (b200_gpt2_tp_peer_*): identical bits."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "tp_gpu_rank.py"
    script.write_text(_GPU_RANK.format(root=ROOT))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="4")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29545", str(script)],
                         capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "TP_GPU_OK" in out.stdout
    assert "TP_PEER_OK" in out.stdout
    assert "TP_SP_OK" in out.stdout
    assert "TP_X3_OK" in out.stdout
