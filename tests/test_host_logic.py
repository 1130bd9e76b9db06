"""Host-side logic that needs no GPU: parameter layout, batch sharding (also as two gloo ranks)."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_param_layout_matches_oracle(pkg, orc):
    for kw in (dict(), dict(num_layers=48, num_heads=25, channels=1600),
               dict(max_seq_len=64, vocab_size=300, padded_vocab_size=320, num_layers=2, num_heads=2, channels=128)):
        assert pkg.param_offsets(pkg.GPT2Config(**kw)) == orc.param_offsets(orc.GPT2Config(**kw))
    assert pkg.GPT2_124M.num_params() == 124475904
    assert pkg.GPT2_XL.num_params() == 1557686400
    assert pkg.PARAM_NAMES == orc.PARAM_NAMES


def test_flops_per_token(pkg):
    # 2.179 TFLOP for 8192 tokens at T=1024 (GEMMs 2*M*K*N, causal-exact attention)
    assert abs(pkg.GPT2_124M.flops_per_token(1024) * 8192 / 1e12 - 2.179) < 0.005


@pytest.mark.parametrize("B,world", [(64, 8), (64, 4), (8, 3), (5, 8), (0, 2), (7, 1)])
def test_shard_batch_partitions_contiguously(pkg, B, world):
    spans = [pkg.shard_batch(B, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == B
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        pkg.shard_batch(B, world, world)


_RANK_SCRIPT = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
import __graft_entry__ as ge
from oracle import oracle as orc
pkg = ge.load_package()
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
cfg = orc.GPT2Config(max_seq_len=64, vocab_size=300, padded_vocab_size=320, num_layers=1, num_heads=2, channels=128)
params = orc.init_params(cfg, 3)                 # every rank holds the full replica
tokens = orc.fill_tokens((5, 64), 4, vocab=300)  # global batch of 5 over 2 ranks: 3 + 2
lo, hi = pkg.shard_batch(5, world, rank)
mine = orc.gpt2_forward(params, cfg, tokens[lo:hi])        # stands in for the GPU forward
# the forward itself needs no collective; gathering is only done here to check the shards
parts = [None] * world
dist.all_gather_object(parts, (lo, hi, mine))
if rank == 0:
    full = orc.gpt2_forward(params, cfg, tokens)
    got = np.concatenate([p[2] for p in sorted(parts, key=lambda p: p[0])])
    assert np.array_equal(got, full), "sharded forward differs from the whole-batch forward"
    print("SHARD_OK", [(p[0], p[1]) for p in parts])
dist.barrier()
dist.destroy_process_group()
"""


def test_batch_sharded_forward_two_gloo_ranks(tmp_path):
    """world_size 2 on CPU: each rank runs its contiguous shard with no data-path collective and
    the concatenation equals the whole-batch result bit for bit."""
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT.format(root=ROOT))
    env = dict(os.environ, OMP_NUM_THREADS="2")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "SHARD_OK [(0, 3), (3, 5)]" in out.stdout


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the CPU port on a bounded sample and prints
    one JSON line with the benchmark's metric, unit and config plus the cpu_baseline / e2e objects."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "gpt2_forward_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["steps"] == 1
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0
    assert "workload" in line["config"]


def test_clock_sampler_without_a_gpu_returns_an_empty_record():
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    s = bench.ClockSampler(0)
    s.start()
    rec = s.stop()
    assert set(("sm_mhz", "sm_max_mhz", "reasons", "samples")) <= set(rec)


def test_shard_params_torch_equals_the_host_cut(pkg):
    """The device-side cut of a tensor-parallel rank's parameters (used by bench.py's multi-GPU checks)
    is the same selection as b200_gpt2_shard_params_host, for an uneven head split."""
    import numpy as np
    import torch
    cfg = pkg.GPT2Config(max_seq_len=64, vocab_size=100, padded_vocab_size=128, num_layers=2, num_heads=5, channels=320)
    n = pkg.param_offsets(cfg)[16]
    full = np.arange(n, dtype=np.float32) * 0.001
    for tp in (2, 4):
        for r in range(tp):
            want = pkg.shard_params(cfg, tp, r, full)
            got = pkg.shard_params_torch(cfg, tp, r, torch.from_numpy(full)).numpy()
            assert np.array_equal(got, want)
