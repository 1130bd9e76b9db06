#!/usr/bin/env python
"""Benchmark of the GPT-2 forward hot path.

  python bench.py --gpus N --steps K --warmup W            this repository's CUDA path
  python bench.py --impl reference --gpus N --steps K ...   the CPU forward on the host cores

A step is one full-sequence forward of GPT-2 124M on B=8 x T=1024 synthetic token ids per GPU
(seeded random-init weights: there is no checkpoint to load).  With N > 1 it is launched with
one process per GPU (torch.distributed.run); the batch is sharded, sequences are independent,
so there is no collective on the data path and the scaling is weak (8 sequences per GPU).
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# Measured DRAM traffic of the GEMM kernels of the 124M forward, launch-weighted average over the 49
# launches of a step (ncu dram__bytes_read.sum + dram__bytes_write.sum), by arithmetic mode; the
# capture and the per-shape figures are in the named profile.
GEMM_DRAM_TRAFFIC = {
    "bf16x3": {"dram_bytes_per_launch": 122.0e6, "algorithmic_bytes_per_launch": 155.2e6,
               "source": "profiles/gemm_pair_bf16x3_dram_traffic_by_shape.md (lone launches per shape, launch-weighted)"},
}

METRIC = "gpt2_forward_tokens_per_s"
UNIT = "tokens/s"
B_PER_GPU, T = 8, 1024
WORKLOAD = "GPT-2 124M full-sequence forward, B=8 T=1024 per GPU, fp32 storage, tensor-core GEMMs (configs[1]; arithmetic: see config.arithmetic)"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"],
                "bf16_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """SM clock and clock-event reasons sampled (read-only) while the timed region runs: a
    background thread polling NVML every few milliseconds; `nvidia-smi -lms` as a fall-back when
    the NVML bindings are missing."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index: int, uuid: str | None = None, period_s: float = 0.004):
        self.gpu_index, self.uuid, self.period_s = gpu_index, uuid, period_s
        self.proc = None
        self.path = None
        self.thread = None
        self.stop_flag = None
        self.clocks, self.maxes, self.reasons = [], [], set()

    def _nvml_loop(self, nv, handle):
        try:
            max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
        except Exception:
            max_mhz = None
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self.stop_flag.is_set():
            try:
                self.clocks.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                if max_mhz:
                    self.maxes.append(max_mhz)
                if reasons_fn:
                    mask = int(reasons_fn(handle))
                    for bit, name in self.REASON_BITS.items():
                        if mask & bit:
                            self.reasons.add(name)
            except Exception:
                pass
            self.stop_flag.wait(self.period_s)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            handle = None
            if self.uuid:
                try:
                    handle = nv.nvmlDeviceGetHandleByUUID(self.uuid if self.uuid.startswith("GPU-") else "GPU-" + self.uuid)
                except Exception:
                    handle = None
            if handle is None:
                handle = nv.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self.stop_flag = threading.Event()
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            if self.clocks:
                out.update(sm_mhz=statistics.median(self.clocks), sm_max_mhz=max(self.maxes) if self.maxes else None,
                           reasons=sorted(self.reasons), samples=len(self.clocks), source="nvml")
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 9:
                        continue
                    try:
                        clocks.append(float(parts[1]))
                        maxes.append(float(parts[2]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         parts[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if clocks:
            out.update(sm_mhz=statistics.median(clocks), sm_max_mhz=max(maxes), reasons=sorted(reasons),
                       samples=len(clocks), source="nvidia-smi")
        return out


def _random_init_(model, pkg, torch, seed: int):
    """Random-init weights of the architecture, written in place on the device: matrices
    N(0, 0.02), layernorm weight 1 / bias 0, linear biases 0.  (With tensor parallelism the
    replicated tensors - wte, wpe, layernorms - come out identical on every rank: same seed,
    same sizes, drawn first.)"""
    cfg = model.cfg
    offs = pkg.param_offsets_tp(cfg, model.tp_size, model.tp_rank)
    p = model.params_tensor()
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    for i, name in enumerate(pkg.PARAM_NAMES):
        view = p[offs[i]:offs[i + 1]]
        if name in ("ln1w", "ln2w", "lnfw"):
            view.fill_(1.0)
        elif name in ("wte", "wpe", "qkvw", "attprojw", "fcw", "fcprojw"):
            view.normal_(0.0, 0.02, generator=g)
        else:
            view.zero_()


def _headline_mode(pkg):
    """The arithmetic the headline is measured in: the library's default options."""
    return pkg.DEFAULT_MODE_NAME, dict(pkg.MODES[pkg.DEFAULT_MODE_NAME])


def _config(world: int, tp: bool = False, xl: bool = False) -> dict:
    """The `config` object of the JSON line; the same for this repository's arm and the reference arm."""
    workload = WORKLOAD if not xl else ("GPT-2 XL 1.5B full-sequence forward, B=8 T=1024 per " +
                                        ("tensor-parallel group" if tp else "GPU") + ", fp32 storage (configs[4] shapes)")
    par = (f"tensor-parallel x{world}: heads / MLP / vocabulary split, one NCCL all-reduce per attention and MLP block" if tp
           else f"batch-sharded x{world}, no collective")
    return {"workload": workload, "global_batch": (1 if tp else world) * B_PER_GPU, "seq_len": T, "parallelism": par,
            "l2": "no flush: each step streams the weights (0.5 GB for 124M) and writes 1.65 GB of logits, far beyond the 126 MB L2"}


def _oracle_all_threads():
    """Loads the CPU oracle and gives it every core this process may run on (torch.distributed.run
    exports OMP_NUM_THREADS=1 to its workers)."""
    from oracle import oracle as orc
    orc.build()
    cores = orc.use_all_host_threads()
    return orc, cores


def run_reference(args):
    """The reference project has no CPU implementation and cannot run without a GPU, so the
    reference arm times this repository's CPU restatement of its forward (oracle/, a port)
    with all host threads, each step one sequence of the benchmark workload (or a shorter
    prefix when K+W steps of a full sequence would not finish in a few minutes)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np
    orc, cores = _oracle_all_threads()
    cfg = orc.GPT2_124M
    params = orc.init_params(cfg, seed=1234)
    # calibrate on a short prefix, then size the per-step sample so the run stays bounded
    tok64 = orc.fill_tokens((1, 64), seed=4321, vocab=cfg.vocab_size)
    t0 = time.perf_counter()
    orc.gpt2_forward(params, cfg, tok64)
    tps_small = 64 / (time.perf_counter() - t0)
    budget_s = 150.0
    n_steps = args.steps + args.warmup
    sample_T = 1024
    while sample_T > 64 and n_steps * sample_T / (0.8 * tps_small) > budget_s:
        sample_T //= 2
    tokens = orc.fill_tokens((1, sample_T), seed=4321, vocab=cfg.vocab_size)
    for _ in range(args.warmup):
        orc.gpt2_forward(params, cfg, tokens)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.gpt2_forward(params, cfg, tokens)
    dt = time.perf_counter() - t0
    value = args.steps * sample_T / dt
    sample = (f"1 sequence of {sample_T} tokens per step (of the B=8 x T=1024 workload), fp32 accumulate, C/OpenMP, "
              f"{cores} threads" + ("" if cores > 1 else " (ONE thread only: no more cores are available to this process)"))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": _config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def _measure_matmul_peaks(torch, seconds: float = 2.0):
    """cuBLAS through torch.matmul, 8192^3: TF32 (fp32 tensors, TF32 allowed) and bf16, each as the
    best of 10 launches (burst) and back to back for `seconds` (sustained).  Harness only: the
    denominators of the roofline fractions, never on the product path."""
    out = {}
    n = 8192
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        for name, dt in (("tf32", torch.float32), ("bf16", torch.bfloat16)):
            a = torch.randn(n, n, device="cuda", dtype=dt)
            b = torch.randn(n, n, device="cuda", dtype=dt)
            c = torch.empty(n, n, device="cuda", dtype=dt)
            for _ in range(3):
                torch.matmul(a, b, out=c)
            torch.cuda.synchronize()
            best = 1e9
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch.matmul(a, b, out=c)
                e1.record()
                e1.synchronize()
                best = min(best, e0.elapsed_time(e1))
            flop = 2.0 * n ** 3
            out[name + "_burst_tflops"] = flop / (best * 1e-3) / 1e12
            reps = max(10, int(seconds / (best * 1e-3)))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                torch.matmul(a, b, out=c)
            e1.record()
            e1.synchronize()
            out[name + "_sustained_tflops"] = flop * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12
            del a, b, c
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    out["how"] = f"torch.matmul {n}^3, best of 10 (burst) and back to back for {seconds:.0f} s (sustained), measured in this run"
    return out


def _time_reference_gpu_kernels(torch, np):
    """The reference project's own CUDA kernels (built from its headers into oracle/_ref/ where a
    checkout was present) timed on this GPU at the sweep shapes that satisfy their asserts: the
    GPU-vs-GPU baseline per operator.  Returns None when the library is not there."""
    import ctypes as C
    path = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")
    if not os.path.exists(path):
        return None
    ref = C.CDLL(path)
    p = lambda t: C.c_void_p(t.data_ptr())
    Bb, Tt, M = 8, 1024, 8192
    g = torch.Generator(device="cuda").manual_seed(7)
    res = {"source": "oracle/_ref/libref_kernels.so (the reference's headers compiled for sm_100a)", "kernels": {}}

    def timed(fn, reps=5):
        for _ in range(2):
            rc = fn()
            if rc != 0:
                raise RuntimeError(f"reference kernel returned {rc}")
        ts = []
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    for name, K, N, gelu in (("gemm_qkv", 768, 2304, 0), ("gemm_attproj", 768, 768, 0), ("gemm_fc", 768, 3072, 1),
                             ("gemm_fcproj", 3072, 768, 0), ("gemm_lmhead", 768, 50304, 0)):
        x = torch.empty(M, K, device="cuda").normal_(0, 1, generator=g)
        w = torch.empty(N, K, device="cuda").normal_(0, 0.02, generator=g)
        b = torch.zeros(N, device="cuda")
        o = torch.empty(M, N, device="cuda")
        torch.cuda.synchronize()
        ms = timed(lambda: ref.ref_matmul_forward_tf32_gelu(p(o), p(x), p(w), p(b), Bb, Tt, K, N, gelu))
        res["kernels"][name] = {"kernel": "matmul_forward_async_cg_tf32_gelu (kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh)",
                                "ms": round(ms, 4), "tflops": round(2.0 * M * K * N / (ms * 1e-3) / 1e12, 1)}
        del x, w, b, o
    NH, Cc = 12, 768
    qkv = torch.empty(Bb, Tt, 3 * Cc, device="cuda").normal_(0, 1, generator=g)
    o = torch.empty(Bb, Tt, Cc, device="cuda")
    torch.cuda.synchronize()
    ms = timed(lambda: ref.ref_flash_attention_permute_forward(p(o), p(qkv), Bb, Tt, Cc, NH))
    res["kernels"]["attention"] = {"kernel": "flash_attention_permute_forward (kernels/attention/3_flash_attention_permute.cuh)",
                                   "ms": round(ms, 4),
                                   "tflops_causal": round(4.0 * 64 * Tt * (Tt + 1) / 2 * NH * Bb / (ms * 1e-3) / 1e12, 1)}
    x = torch.empty(Bb, Tt, Cc, device="cuda").normal_(0, 1, generator=g)
    w, b = torch.ones(Cc, device="cuda"), torch.zeros(Cc, device="cuda")
    mean, rstd = torch.empty(M, device="cuda"), torch.empty(M, device="cuda")
    torch.cuda.synchronize()
    ms = timed(lambda: ref.ref_layernorm_forward_block_vectorized(p(o), p(mean), p(rstd), p(x), p(w), p(b), Bb, Tt, Cc))
    res["kernels"]["layernorm"] = {"kernel": "layernorm_forward_block_vectorized (kernels/layernorm/2_layernorm_block_vectorized.cuh)",
                                   "ms": round(ms, 4), "gbs": round((2.0 * M * Cc + 2 * M + 2 * Cc) * 4 / (ms * 1e-3) / 1e9, 1)}
    # a forward made of these kernels (the reference leaves the driver to llm.c): twelve blocks of QKV, attention,
    # projection, two layernorms, fc and fc-proj, then the final layernorm and the lm-head; its two residual adds
    # per block and the encoder are left out, so this is a lower bound on the chain's time
    k = {n: v["ms"] for n, v in res["kernels"].items()}
    chain = 12 * (k["gemm_qkv"] + k["attention"] + k["gemm_attproj"] + 2 * k["layernorm"] + k["gemm_fc"] + k["gemm_fcproj"]) \
        + k["layernorm"] + k["gemm_lmhead"]
    res["forward_as_a_chain_of_these_kernels"] = {"ms_per_step": round(chain, 3), "tokens_per_s": round(M / (chain * 1e-3), 1),
                                                  "note": "sum of the kernel times above for the 124M forward at B=8, T=1024 (residual adds and encoder not counted)"}
    return res


def _seq_hashes(torch, logits):
    """Two 63-bit checksums per sequence over the bit patterns of logits [B,T,V] (order-dependent)."""
    Bn = logits.shape[0]
    bits = logits.contiguous().view(torch.int32).view(Bn, -1).to(torch.int64)
    idx = torch.arange(bits.shape[1], device=bits.device, dtype=torch.int64) % 65521 + 1
    return torch.stack([bits.sum(1), (bits * idx).sum(1)], dim=1)


def _time_steps(torch, model, ctx, stream, tok, Bn, Tn, steps, warmup, barrier, max_over_ranks):
    for _ in range(warmup):
        model.forward(tok, Bn, Tn)
    ctx.sync_check()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        model.forward(tok, Bn, Tn)
    e1.record(stream)
    barrier()
    ctx.sync_check()
    return max_over_ranks(e0.elapsed_time(e1)) / steps


def run_ours(args):
    import numpy as np
    import torch
    import __graft_entry__ as ge

    pkg = ge.load_package()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    stream = torch.cuda.Stream()
    ctx = pkg.Context(local_rank, stream)
    xl = args.model == "xl"
    cfg = pkg.GPT2_XL if xl else pkg.GPT2_124M
    tp = bool(args.tp) and world > 1   # one tensor-parallel group over all ranks, one global batch
    B = B_PER_GPU
    mode_name, mode_opts = _headline_mode(pkg)
    if tp:
        mode_name, mode_opts = "tf32", dict(pkg.MODES["tf32"])  # the tensor-parallel driver runs the TF32 kernels
    model = pkg.GPT2(ctx, cfg, B, T, tp_size=world if tp else 1, tp_rank=rank if tp else 0)
    model.set_options(**mode_opts)
    if tp:
        model.set_allreduce_torch()
    with torch.cuda.stream(stream):
        _random_init_(model, pkg, torch, seed=1234 + 0)  # same weights on every rank
        tok_dev = torch.randint(0, cfg.vocab_size, (B, T), dtype=torch.int32, device="cuda",
                                generator=torch.Generator(device="cuda").manual_seed(4321 + (0 if tp else rank)))
    stream.synchronize()
    tok_host = torch.empty((B, T), dtype=torch.int32).pin_memory()
    tok_host.copy_(tok_dev.cpu())
    last_host = torch.empty((B, model.logits_width), dtype=torch.float32).pin_memory()
    amax_host = None if tp else torch.empty((B, T), dtype=torch.int32).pin_memory()
    amax_np = None if tp else amax_host.numpy()
    replicas = 1 if tp else world   # independent batches processed per step

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------------------------------------------------------- device-resident arm
    for _ in range(max(args.warmup, 3)):
        model.forward(tok_dev, B, T)
    ctx.sync_check()
    sampler = ClockSampler(local_rank, uuid=str(getattr(torch.cuda.get_device_properties(local_rank), "uuid", "") or "") or None)
    barrier()
    if rank == 0:
        sampler.start()
    ctx.reset_launches()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        model.forward(tok_dev, B, T)
    ev1.record(stream)
    barrier()
    ctx.sync_check()
    launches = ctx.launches
    elapsed_ms = max_over_ranks(ev0.elapsed_time(ev1))
    clocks = sampler.stop() if rank == 0 else None
    # logits of the headline mode for the parity figures (rank 0's first sequences)
    n_par = 0 if (tp or xl) else (8 if world == 1 else 2)
    head_logits = model.forward(tok_dev, B, T)[:n_par].clone() if n_par else None
    ctx.sync_check()

    # ---------------------------------------------------------------- end-to-end arm
    # Every step brings its tokens in from pinned host memory, runs the forward and puts the
    # last-position logits and the arg-max ids back into pinned host memory (the library moves them
    # with its own kernels over PCIe instead of queueing copies).  First the call split
    # into enqueue / wait with two steps in flight (each slot has its own host buffers), so the host's
    # share of a step hides behind the GPU's - the headline `e2e`; then the synchronous call, one
    # step at a time.
    tok_h = [tok_host.numpy(), tok_host.clone().pin_memory().numpy()]
    last_h = [last_host.numpy(), torch.empty_like(last_host).pin_memory().numpy()]
    amax_h = [amax_np, None if tp else torch.empty_like(amax_host).pin_memory().numpy()]

    def pipelined(n):
        model.forward_host_enqueue(tok_h[0], B, T, 0, last_logits_host=last_h[0], argmax_host=amax_h[0])
        for i in range(1, n):
            model.forward_host_enqueue(tok_h[i & 1], B, T, i & 1, last_logits_host=last_h[i & 1], argmax_host=amax_h[i & 1])
            model.forward_host_wait((i - 1) & 1)
        model.forward_host_wait((n - 1) & 1)

    pipelined(3)
    barrier()
    t0 = time.perf_counter()
    pipelined(args.steps)
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    for _ in range(3):
        model.forward_host(tok_host.numpy(), B, T, last_logits_host=last_host.numpy(), argmax_host=amax_np)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        model.forward_host(tok_host.numpy(), B, T, last_logits_host=last_host.numpy(), argmax_host=amax_np)
    e2e_sync_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    # the same call returning ALL logits [B,T,Vp] to pinned host memory: the deliverable the benchmark
    # configuration names, bound by the PCIe copy of 1.65 GB per step
    e2e_full = None
    if not tp and not xl:
        try:
            full_host = torch.empty((B, T, model.logits_width), dtype=torch.float32).pin_memory()
            n_full = max(2, min(args.steps, 8))
            for _ in range(2):
                model.forward_host(tok_host.numpy(), B, T, logits_host=full_host.numpy())
            barrier()
            t0 = time.perf_counter()
            for _ in range(n_full):
                model.forward_host(tok_host.numpy(), B, T, logits_host=full_host.numpy())
            full_s = max_over_ranks(time.perf_counter() - t0)
            e2e_full = {"value": replicas * B * T * n_full / full_s, "unit": UNIT, "ms_per_step": 1e3 * full_s / n_full,
                        "steps": n_full, "h2d_bytes_per_step": B * T * 4, "d2h_bytes_per_step": B * T * model.logits_width * 4,
                        "result": "all logits [B,T,Vp] in pinned host memory", "call": "b200_gpt2_forward_host, one step at a time"}
            del full_host
        except Exception as e:
            e2e_full = {"error": str(e)}
        barrier()

    # the same K steps again with one CUDA-event pair around every kernel launch (on the launching
    # stream): per-operator durations for the roofline figures; not part of `value`
    model.set_profile(True)
    for _ in range(args.steps):
        model.forward(tok_dev, B, T)
    prof = model.read_profile()
    model.set_profile(False)

    # ------------------------------------------------ the same workload in the other arithmetic modes
    other = {}
    other_logits = {}
    if not tp:
        for name in ("tf32", "bf16x3", "bf16x3_att_tf32", "bf16x3_lm_tf32", "bf16"):
            if name == mode_name or (xl and name in ("bf16x3_att_tf32", "bf16x3_lm_tf32")):
                continue
            try:
                model.set_options(**pkg.MODES[name])
                n_o = max(2, args.steps // 2)
                ms = _time_steps(torch, model, ctx, stream, tok_dev, B, T, n_o, 3, barrier, max_over_ranks)
                other[name] = {"value": replicas * B * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "note": pkg.MODE_NOTES[name]}
                if n_par:
                    other_logits[name] = model.forward(tok_dev, B, T)[:n_par].clone()
                    ctx.sync_check()
            except Exception as e:
                other[name] = {"error": str(e)}
        model.set_options(**mode_opts)

    # ---------------------------------------------- incremental decoding (key/value cache)
    # One new token per sequence against a cache filled by a prefill of T/2 positions; each step
    # reads every weight and the used part of the cache once (HBM-bound).  Extra measurement on
    # rank 0; not part of `value`.
    decode = None
    if rank == 0 and not tp and not xl and B <= 16:
        try:
            model.enable_kv_cache()
            model.set_options(**dict(mode_opts, use_graph=1))
            T0 = T // 2
            model.prefill(tok_dev[:, :T0].contiguous(), B, T0)
            col = tok_dev[:, 0].contiguous()
            for i in range(3):
                model.decode_step(col, B, T0)
            ctx.sync_check()
            n_dec = 64
            ev4, ev5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev4.record(stream)
            for i in range(n_dec):
                model.decode_step(col, B, T0 + i)
            ev5.record(stream)
            ctx.sync_check()
            dec_us = ev4.elapsed_time(ev5) * 1e3 / n_dec
            Cc_, L_ = cfg.channels, cfg.num_layers
            w_bytes = 4.0 * (L_ * 12 * Cc_ * Cc_ + cfg.padded_vocab_size * Cc_)
            kv_bytes = 4.0 * L_ * B * (T0 + n_dec / 2 + 1) * 2 * Cc_
            decode = {"value": B / (dec_us * 1e-6), "unit": "tokens/s", "us_per_step": dec_us, "batch": B,
                      "positions": [T0, T0 + n_dec - 1],
                      "algorithmic_bytes_per_step": w_bytes + kv_bytes,
                      "achieved_gbs": (w_bytes + kv_bytes) / (dec_us * 1e-6) / 1e9,
                      "frac_of_hbm_peak": (w_bytes + kv_bytes) / (dec_us * 1e-6) / 1e9 / _peaks()["hbm_gbs"],
                      "note": "b200_gpt2_decode_step replayed as a CUDA graph; bytes = all weight matrices once + keys and values of the cached positions"}
            model.set_options(**mode_opts)
        except Exception as e:  # an extra measurement must not take the benchmark line down
            decode = {"error": str(e)}

    # ---------------------------------------------- parity of the timed arithmetic against the CPU oracle
    # and the CPU baseline (rank 0): the oracle's fp32 forward on the first sequences of rank 0's batch
    # with the model's own weights; the first one is timed.
    parity, cpu_tps, cores, cpu_T = None, None, None, (256 if xl else 1024)
    if rank == 0:
        orc, cores = _oracle_all_threads()
        ocfg = orc.GPT2Config(**cfg.__dict__)
        host_params = model.params_tensor().cpu().numpy() if not tp else None
        tok_np = tok_host.numpy()
        if host_params is None:  # tensor parallel: weights are sharded on the device; time the oracle on its own weights
            host_params = orc.init_params(ocfg, seed=1234)
        wants = []
        for b in range(max(1, n_par)):
            t0 = time.perf_counter()
            w = orc.gpt2_forward(host_params, ocfg, tok_np[b:b + 1, :cpu_T], precise=False)[0]
            if b == 0:
                cpu_tps = cpu_T / (time.perf_counter() - t0)
            wants.append(w)
        if n_par:
            V = cfg.vocab_size

            def compare(lg):
                got = lg.cpu().numpy()
                miss, mx, sq = 0, 0.0, 0.0
                for b in range(n_par):
                    err = np.abs(got[b] - wants[b])
                    mx = max(mx, float(err.max()))
                    sq += float((err.astype(np.float64) ** 2).mean())
                    miss += int((got[b][:, :V].argmax(-1) != wants[b][:, :V].argmax(-1)).sum())
                return {"top1": 1.0 - miss / (n_par * T), "top1_misses": miss, "positions": n_par * T,
                        "max_abs": mx, "rms": (sq / n_par) ** 0.5}

            parity = {"mode": mode_name, **compare(head_logits),
                      "against": f"oracle fp32 forward (CPU) on the first {n_par} sequences of rank 0's batch, same weights",
                      "bars": "max-abs <= 2e-2, top-1 agreement >= 0.999",
                      "other_modes": {k: compare(v) for k, v in other_logits.items()}}
        del host_params
    head_logits = None
    other_logits = None

    # ---------------------------------------------- measured matmul peaks and the reference's own kernels
    peaks_now, ref_gpu = None, None
    if rank == 0:
        try:
            peaks_now = _measure_matmul_peaks(torch)
        except Exception as e:
            peaks_now = {"error": str(e)}
        if world == 1 and not xl:
            try:
                ref_gpu = _time_reference_gpu_kernels(torch, np)
            except Exception as e:
                ref_gpu = {"error": str(e)}
    barrier()

    # ---------------------------------------------- GPT-2 XL (configs[4]) and the multi-GPU checks
    extras = {}
    if not xl and not tp and not args.no_xl:
        model.close()
        model = None
        torch.cuda.empty_cache()
        try:
            extras = _xl_and_multi_gpu(pkg, torch, dist, ctx, stream, world, rank, barrier, max_over_ranks, mode_name)
        except Exception as e:
            extras = {"xl_config4": {"error": str(e)}}

    if rank != 0:
        if model is not None:
            model.close()
        ctx.close()
        if dist is not None:
            dist.destroy_process_group()
        return 0

    tokens_total = replicas * B * T * args.steps
    value = tokens_total / (elapsed_ms * 1e-3)
    peaks = _peaks()
    # dominant kernel: the tcgen05 GEMM (five shapes, 4L+1 launches per step); rank-local widths
    M = B * T
    Cc, L = cfg.channels, cfg.num_layers
    n_tp = world if tp else 1
    Ac, Fc, Vl = pkg.tp_heads(cfg.num_heads, n_tp, 0)[1] * 64, 4 * Cc // n_tp, (cfg.padded_vocab_size // n_tp if tp else cfg.padded_vocab_size)
    if tp and (cfg.padded_vocab_size % n_tp or (cfg.padded_vocab_size // n_tp) % 4):
        Vl = cfg.padded_vocab_size
    gemm_flops = {"gemm_qkv": 2.0 * M * Cc * 3 * Ac, "gemm_attproj": 2.0 * M * Ac * Cc, "gemm_fc": 2.0 * M * Cc * Fc,
                  "gemm_fcproj": 2.0 * M * Fc * Cc, "gemm_lmhead": 2.0 * M * Cc * Vl}
    tot_flops = sum(gemm_flops[k] * prof[k][1] for k in gemm_flops)
    tot_ms = sum(prof[k][0] for k in gemm_flops)
    n_gemm = sum(prof[k][1] for k in gemm_flops)
    achieved = tot_flops / (tot_ms * 1e-3) / 1e12 if tot_ms > 0 else 0.0
    # Denominator: the tensor-pipe rate this arithmetic can reach per algorithmic flop.  TF32: the
    # cuBLAS TF32 GEMM measured in this run (burst: best launch; sustained: seconds back to back).
    # bf16x3: three bf16 products per algorithmic product, so a third of the measured bf16 GEMM rate.
    have_now = isinstance(peaks_now, dict) and "tf32_burst_tflops" in peaks_now
    if mode_name.startswith("bf16x3"):
        pk_burst = (peaks_now["bf16_burst_tflops"] if have_now else peaks["bf16_burst"]) / 3.0
        pk_sust = (peaks_now["bf16_sustained_tflops"] if have_now else peaks["bf16_sustained"]) / 3.0
        pk_src = ("bf16 cuBLAS GEMM " + ("measured in this run" if have_now else f"from MEASURED_PEAKS.json ({peaks['source']})") +
                  " / 3: the kernel issues three bf16 products (hi.hi + hi.lo + lo.hi) per algorithmic product")
    elif mode_name == "bf16":
        pk_burst = peaks_now["bf16_burst_tflops"] if have_now else peaks["bf16_burst"]
        pk_sust = peaks_now["bf16_sustained_tflops"] if have_now else peaks["bf16_sustained"]
        pk_src = "bf16 cuBLAS GEMM " + ("measured in this run" if have_now else f"from MEASURED_PEAKS.json ({peaks['source']})")
    else:
        pk_burst = peaks_now["tf32_burst_tflops"] if have_now else peaks["bf16_burst"] / 2.0
        pk_sust = peaks_now["tf32_sustained_tflops"] if have_now else peaks["bf16_sustained"] / 2.0
        pk_src = ("TF32 cuBLAS GEMM measured in this run" if have_now else
                  f"{peaks['source']} bf16 / 2 (TF32 issues at half the bf16 rate; no TF32 measurement was possible)")
    per_op = {}
    hbm_bytes = {"layernorm": (2.0 * M * Cc + 2 * Cc) * 4, "fused_residual_layernorm": (4.0 * M * Cc + 2 * Cc) * 4,
                 "encoder": (2.0 * M * Cc + T * Cc) * 4 + M * 4}
    att_flops = 4.0 * 64 * T * (T + 1) / 2 * (Ac // 64) * B
    prof_total = sum(v[0] for v in prof.values())
    for name, (ms, n) in prof.items():
        if n == 0:
            continue
        avg = ms / n
        entry = {"launches_per_step": n / args.steps, "avg_ms": round(avg, 5), "share": round(ms / prof_total, 4)}
        if name in gemm_flops:
            entry["tflops"] = round(gemm_flops[name] / (avg * 1e-3) / 1e12, 1)
            entry["frac_burst"] = round(entry["tflops"] / pk_burst, 3)
        elif name == "attention":
            entry["tflops_causal"] = round(att_flops / (avg * 1e-3) / 1e12, 1)
        elif name in hbm_bytes:
            entry["gbs"] = round(hbm_bytes[name] / (avg * 1e-3) / 1e9, 1)
            entry["frac_hbm"] = round(entry["gbs"] / peaks["hbm_gbs"], 3)
        if isinstance(ref_gpu, dict) and name in ref_gpu.get("kernels", {}):
            entry["vs_reference_kernel"] = round(ref_gpu["kernels"][name]["ms"] / avg, 2)
        per_op[name] = entry
    traffic = None if (xl or tp) else GEMM_DRAM_TRAFFIC.get(mode_name)
    cfg_obj = _config(world, tp, xl)
    cfg_obj["flop_per_token"] = cfg.flops_per_token(T)
    cfg_obj["arithmetic"] = pkg.MODE_NOTES[mode_name]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": mode_name, "data": "synthetic",
        "config": cfg_obj,
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel and gemm_tf32_kernel (all five GEMM shapes of the forward)",
                     "achieved": achieved, "peak": pk_burst, "unit": "TFLOP/s", "frac": achieved / pk_burst,
                     "frac_burst": achieved / pk_burst, "frac_sustained": achieved / pk_sust, "peak_sustained": pk_sust,
                     "matches_timed_region": "burst: the timed region lasts a fraction of a second (see clocks.sm_mhz)",
                     "peak_source": pk_src, "peaks_measured_in_run": peaks_now,
                     "launches_per_step": n_gemm / args.steps,
                     "event_timing": "one event pair per launch serialises the launches: per-operator times add up to slightly more than ms_per_step",
                     "traffic": None if traffic is None else traffic["dram_bytes_per_launch"],
                     "algorithmic_bytes": None if traffic is None else traffic["algorithmic_bytes_per_launch"],
                     "traffic_source": None if traffic is None else traffic["source"],
                     "per_operator": per_op},
        "parity": parity,
        "cpu_baseline": {"value": cpu_tps, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"1 sequence of {cpu_T} tokens (B=1), fp32-accumulate C/OpenMP forward, {cores} host threads, one run"},
        "e2e": {"value": replicas * B * T * args.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": B * T * 4,
                "d2h_bytes_per_step": B * model_logits_width(pkg, cfg, n_tp if tp else 1) * 4 + (0 if tp else B * T * 4),
                "ms_per_step": 1e3 * e2e_s / args.steps,
                "result": "last-position logits [B,Vp]" + ("" if tp else " and per-position arg-max token ids [B,T]"),
                "call": "b200_gpt2_forward_host_enqueue / _wait, two steps in flight, double-buffered pinned host buffers",
                "synchronous_call": {"value": replicas * B * T * args.steps / e2e_sync_s, "ms_per_step": 1e3 * e2e_sync_s / args.steps,
                                     "call": "b200_gpt2_forward_host, one step at a time"}},
        "e2e_full_logits": e2e_full,
        "gpu_launches": launches,
        "clocks": clocks,
        "other_modes": other,
        "decode": decode,
        "ref_gpu_kernels": ref_gpu,
    }
    if isinstance(ref_gpu, dict) and "forward_as_a_chain_of_these_kernels" in ref_gpu:
        # the GPU-vs-GPU figure for the whole step: this library's device-resident value over the reference kernels' chain
        line["vs_reference_gpu_kernels_chain"] = round(value / ref_gpu["forward_as_a_chain_of_these_kernels"]["tokens_per_s"], 2)
    line.update(extras)
    print(json.dumps(line), flush=True)
    if model is not None:
        model.close()
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def model_logits_width(pkg, cfg, n_tp):
    Vp = cfg.padded_vocab_size
    return Vp // n_tp if (Vp % n_tp == 0 and (Vp // n_tp) % 4 == 0) else Vp


def _xl_and_multi_gpu(pkg, torch, dist, ctx, stream, world, rank, barrier, max_over_ranks, mode_name):
    """GPT-2 XL at global batch 64 split over the ranks (strong scaling of configs[4]); with more
    than one rank also the tensor-parallel XL forward (B=8) with its all-reduce share, and the
    sharding checks: batch shards bitwise equal to the unsharded run, tensor-parallel logits
    against the unsharded ones."""
    out = {}
    cfg = pkg.GPT2_XL
    GB = 64
    Bl = GB // world
    g = torch.Generator(device="cuda").manual_seed(4321)
    tok_all = torch.randint(0, cfg.vocab_size, (GB, T), dtype=torch.int32, device="cuda", generator=g)  # same on every rank
    xlm = pkg.GPT2(ctx, cfg, max(Bl, 8), T)
    xlm.set_options(**pkg.MODES[mode_name])
    with torch.cuda.stream(stream):
        _random_init_(xlm, pkg, torch, seed=99)
    stream.synchronize()
    lo = rank * Bl
    tok_mine = tok_all[lo:lo + Bl].contiguous()
    steps = 2 if world == 1 else 3
    ms = _time_steps(torch, xlm, ctx, stream, tok_mine, Bl, T, steps, 1, barrier, max_over_ranks)
    out["xl_config4"] = {"value": GB * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "global_batch": GB, "batch_per_gpu": Bl,
                         "n_gpus": world, "steps": steps, "scaling": "strong", "dtype": mode_name,
                         "workload": "GPT-2 XL 1.5B (48 layers, 25 heads, C=1600) full-sequence forward, global batch 64 x T=1024 "
                                     "sharded over the GPUs, no collective (configs[4])"}
    if world == 1:
        xlm.close()
        return out

    # ---- batch sharding is exact: sequences [0,8) computed by every rank as one batch, and each rank's
    # own slice of them computed alone, give the same bits everywhere
    with torch.no_grad():
        ref8 = xlm.forward(tok_all[:8].contiguous(), 8, T)
        ctx.sync_check()
        ref8 = ref8.clone()  # the model's logits buffer is written again below
        h_full = _seq_hashes(torch, ref8)
        s0, s1 = pkg.shard_batch(8, world, rank)
        h_shard = torch.zeros((8, 2), dtype=torch.int64, device="cuda")
        diff = torch.zeros(1, device="cuda")
        if s1 > s0:
            part = xlm.forward(tok_all[s0:s1].contiguous(), s1 - s0, T)
            ctx.sync_check()
            h_shard[s0:s1] = _seq_hashes(torch, part)
            diff = (part - ref8[s0:s1]).abs().max().reshape(1)
        gather_full = [torch.empty_like(h_full) for _ in range(world)]
        dist.all_gather(gather_full, h_full)
        dist.all_reduce(h_shard)  # every sequence is filled in by exactly one rank
        dist.all_reduce(diff, op=dist.ReduceOp.MAX)
        same_full = all(torch.equal(gather_full[0], x) for x in gather_full)
        same_shard = torch.equal(h_shard, gather_full[0])
        out["shard_check"] = {"same_batch_on_every_rank": "bitwise" if same_full else "MISMATCH",
                              "batch_sharded": "bitwise" if same_shard else "not bitwise",
                              "batch_sharded_max_abs_vs_full_batch": float(diff.item()),
                              "how": "GPT-2 XL, 8 sequences: per-sequence checksums of the logits' bit patterns, the full batch on "
                                     "every rank and each rank's own shard alone, compared across the ranks.  The accumulate-GEMMs "
                                     "choose their number of K slices from the number of rows, and the order of an fp32 sum "
                                     "follows it: a shard whose GEMMs run with the full batch's configuration (8 / N >= 4 "
                                     "sequences) gives the same bits, a smaller one differs by rounding (the figure above)"}

    # ---- tensor parallel over all ranks (B = 8): weights cut out of the unsharded model's on the device
    tpm = pkg.GPT2(ctx, cfg, 8, T, tp_size=world, tp_rank=rank)
    tpm.set_allreduce_torch()
    with torch.cuda.stream(stream):
        tpm.params_tensor().copy_(pkg.shard_params_torch(cfg, world, rank, xlm.params_tensor()))
    stream.synchronize()
    tok8 = tok_all[:8].contiguous()
    tp_logits = tpm.forward(tok8, 8, T)
    ctx.sync_check()
    Vl = tpm.logits_width
    full_slice = ref8[..., rank * Vl:(rank + 1) * Vl] if Vl != cfg.padded_vocab_size else ref8
    diff = (tp_logits - full_slice).abs().max().reshape(1).to(torch.float64)
    dist.all_reduce(diff, op=dist.ReduceOp.MAX)
    out["shard_check"]["tensor_parallel_max_abs_vs_unsharded"] = float(diff.item())
    ms_tp = _time_steps(torch, tpm, ctx, stream, tok8, 8, T, 3, 1, barrier, max_over_ranks)
    tpm.set_profile(True)
    for _ in range(2):
        tpm.forward(tok8, 8, T)
    prof = tpm.read_profile()
    tpm.set_profile(False)
    tot = sum(v[0] for v in prof.values())
    ser_ms, ar_ms = tot / 2, prof["allreduce"][0] / 2
    out["tp_xl"] = {"value": 8 * T / (ms_tp * 1e-3), "unit": UNIT, "ms_per_step": ms_tp, "batch": 8, "tp_size": world,
                    "ms_per_step_serialised": ser_ms, "allreduce_ms_per_step": ar_ms,
                    "allreduce_share_serialised": ar_ms / ser_ms if ser_ms else None,
                    "exposed_allreduce_ms": max(0.0, ms_tp - (ser_ms - ar_ms)),
                    "exposed_allreduce_share": max(0.0, ms_tp - (ser_ms - ar_ms)) / ms_tp if ms_tp else None,
                    "allreduce_launches_per_step": prof["allreduce"][1] / 2,
                    "dtype": pkg.DEFAULT_MODE_NAME,
                    "note": "GPT-2 XL, one tensor-parallel group over all ranks (heads / MLP / vocabulary split), one NCCL all-reduce "
                            "per attention and MLP block on the compute stream (row-chunked overlap on a communication stream is an "
                            "option that measured slower); the serialised figures come from a pass with one event pair per launch; "
                            "exposed = ms_per_step - (serialised - all-reduce)"}
    # single-pass TF32 arithmetic on the same sharded model (what this measurement ran in before the
    # split-bf16 arithmetic was wired for sharded weights)
    tpm.set_options(**pkg.MODES["tf32"])
    for _ in range(2):
        tpm.forward(tok8, 8, T)
    ctx.sync_check()
    ms_tf32 = _time_steps(torch, tpm, ctx, stream, tok8, 8, T, 3, 1, barrier, max_over_ranks)
    out["tp_xl"]["tf32"] = {"value": 8 * T / (ms_tf32 * 1e-3), "unit": UNIT, "ms_per_step": ms_tf32}
    tpm.set_options(**pkg.MODES[pkg.DEFAULT_MODE_NAME])
    tpm.forward(tok8, 8, T)
    ctx.sync_check()
    if world == 2:
        # the same model with the partial sums handed over through peer memory instead of all-reduces
        try:
            tpm.connect_tp_peer()
            peer_logits = tpm.forward(tok8, 8, T)
            ctx.sync_check()
            same = bool(torch.equal(peer_logits, tp_logits))
            ms_peer = _time_steps(torch, tpm, ctx, stream, tok8, 8, T, 3, 1, barrier, max_over_ranks)
            tpm.set_profile(True)
            for _ in range(2):
                tpm.forward(tok8, 8, T)
            prof = tpm.read_profile()
            tpm.set_profile(False)
            tot = sum(v[0] for v in prof.values())
            ser_ms, ar_ms = tot / 2, prof["allreduce"][0] / 2
            tpm.set_options(**pkg.MODES["tf32"])
            for _ in range(2):
                tpm.forward(tok8, 8, T)
            ctx.sync_check()
            ms_peer_tf32 = _time_steps(torch, tpm, ctx, stream, tok8, 8, T, 3, 1, barrier, max_over_ranks)
            tpm.set_options(**pkg.MODES[pkg.DEFAULT_MODE_NAME])
            out["tp_xl"]["peer_handover"] = {
                "value": 8 * T / (ms_peer * 1e-3), "unit": UNIT, "ms_per_step": ms_peer, "logits_equal_to_allreduce_run": "bitwise" if same else "MISMATCH",
                "tf32_ms_per_step": ms_peer_tf32,
                "ms_per_step_serialised": ser_ms, "handover_ms_per_step": ar_ms,
                "exposed_handover_ms": max(0.0, ms_peer - (ser_ms - ar_ms)),
                "exposed_handover_share": max(0.0, ms_peer - (ser_ms - ar_ms)) / ms_peer if ms_peer else None,
                "note": "b200_gpt2_tp_peer_*: each projection GEMM also stores its tiles into the other GPU's memory (TMA stores over "
                        "NVLink, under the GEMM); a flag word and a bounded wait replace the all-reduce; the fused residual + layernorm "
                        "adds the two partial sums; hand-over = the signal and wait kernels"}
        except Exception as e:  # noqa: BLE001
            out["tp_xl"]["peer_handover"] = {"error": str(e)}
    # the sequence-parallel hand-over (any group size): tiles to the owner of their rows, layernorm on the own rows
    try:
        tpm.set_options(**pkg.MODES[pkg.DEFAULT_MODE_NAME])
        tpm.connect_tp_sequence_parallel()
        sp_logits = tpm.forward(tok8, 8, T)
        ctx.sync_check()
        sp_diff = (sp_logits - tp_logits).abs().max().reshape(1).to(torch.float64)
        dist.all_reduce(sp_diff, op=dist.ReduceOp.MAX)
        ms_sp = _time_steps(torch, tpm, ctx, stream, tok8, 8, T, 3, 1, barrier, max_over_ranks)
        tpm.set_profile(True)
        for _ in range(2):
            tpm.forward(tok8, 8, T)
        prof = tpm.read_profile()
        tpm.set_profile(False)
        tot = sum(v[0] for v in prof.values())
        ser_ms, ar_ms = tot / 2, prof["allreduce"][0] / 2
        tpm.set_options(**pkg.MODES["tf32"])
        for _ in range(2):
            tpm.forward(tok8, 8, T)
        ctx.sync_check()
        ms_sp_tf32 = _time_steps(torch, tpm, ctx, stream, tok8, 8, T, 3, 1, barrier, max_over_ranks)
        out["tp_xl"]["sequence_parallel_handover"] = {
            "value": 8 * T / (ms_sp * 1e-3), "unit": UNIT, "ms_per_step": ms_sp, "tf32_ms_per_step": ms_sp_tf32,
            "max_abs_vs_allreduce_run": float(sp_diff.item()),
            "ms_per_step_serialised": ser_ms, "handover_ms_per_step": ar_ms,
            "exposed_handover_ms": max(0.0, ms_sp - (ser_ms - ar_ms)),
            "exposed_handover_share": max(0.0, ms_sp - (ser_ms - ar_ms)) / ms_sp if ms_sp else None,
            "note": "b200_gpt2_tp_sp_*: every projection tile is stored only to the rank that owns its rows (TMA stores over NVLink "
                    "under the GEMM), that rank's layernorm adds the partial sums of its rows and writes the result into every rank's "
                    "layernorm output; hand-over = the signal and wait kernels around it"}
    except Exception as e:  # noqa: BLE001
        out["tp_xl"]["sequence_parallel_handover"] = {"error": str(e)}
    tpm.close()
    xlm.close()
    return out


def run_kernel_sweep(args):
    """Per-kernel timings at the sweep sizes (8192 rows): one JSON line per case on stdout.
    --op picks one family; --case N picks one case of it (for a profiler capture of one kernel).
    Inputs are larger than L2 only for the big cases; --flush-l2 writes a 256 MB buffer between
    launches so that every launch starts with a cold L2."""
    import torch
    import __graft_entry__ as ge

    pkg = ge.load_package()
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    ctx = pkg.Context(0, stream)
    peaks = _peaks()
    M, Bb, Tt = 8192, 8, 1024
    g = torch.Generator(device="cuda").manual_seed(1)

    def randn(*shape, std=1.0):
        t = torch.empty(shape, device="cuda").normal_(0.0, std, generator=g)
        torch.cuda.synchronize()  # made on torch's stream; the library reads it on the context's
        return t

    cases = []
    if args.op in ("matmul", "all"):
        for (K, N, act, res, bias) in ((768, 2304, 0, False, True), (768, 768, 0, False, True), (768, 3072, 1, False, True),
                                       (3072, 768, 0, True, True), (768, 50304, 0, False, False),
                                       (1600, 4800, 0, False, True), (1600, 6400, 1, False, True), (6400, 1600, 0, True, True)):
            for mode in ((0, 1) if args.modes == "both" else (0,)):
                cases.append(("matmul", dict(K=K, N=N, act=act, res=res, bias=bias, mode=mode)))
    if args.op in ("matmul_bf16", "all"):
        for (K, N, act, bias, out_h) in ((768, 2304, 0, True, False), (768, 768, 0, True, False), (768, 3072, 1, True, True),
                                         (3072, 768, 0, True, False), (768, 50304, 0, False, False),
                                         (1600, 4800, 0, True, False), (1600, 6400, 1, True, True), (6400, 1600, 0, True, False)):
            cases.append(("matmul_bf16", dict(K=K, N=N, act=act, bias=bias, out_h=out_h)))
    if args.op in ("matmul_bf16x3", "all"):
        # K, N, act, bias, output: fp32 / split planes / accumulate onto the output
        for (K, N, act, bias, outk) in ((768, 2304, 0, True, "split"), (768, 768, 0, True, "accumulate"), (768, 3072, 1, True, "split"),
                                        (3072, 768, 0, True, "accumulate"), (768, 50304, 0, False, "fp32"),
                                        (1600, 4800, 0, True, "split"), (1600, 6400, 1, True, "split"), (6400, 1600, 0, True, "accumulate")):
            cases.append(("matmul_bf16x3", dict(K=K, N=N, act=act, bias=bias, outk=outk)))
    if args.op in ("matmul_fp8", "all"):
        for (K, N, act, bias, acc) in ((768, 2304, 0, True, False), (768, 768, 0, True, True), (768, 3072, 1, True, False),
                                       (3072, 768, 0, True, True), (768, 50304, 0, False, False),
                                       (1600, 4800, 0, True, False), (1600, 6400, 1, True, False), (6400, 1600, 0, True, True)):
            cases.append(("matmul_fp8", dict(K=K, N=N, act=act, bias=bias, acc=acc)))
    if args.op in ("attention", "all"):
        cases += [("attention", dict(NH=12)), ("attention", dict(NH=25))]
    if args.op in ("attention_fp16", "all"):
        cases += [("attention_fp16", dict(NH=12)), ("attention_fp16", dict(NH=25))]
    if args.op in ("layernorm", "all"):
        cases += [("layernorm", dict(C=768)), ("layernorm", dict(C=1600))]
    if args.op in ("fused_residual_layernorm", "all"):
        cases += [("fused_residual_layernorm", dict(C=768)), ("fused_residual_layernorm", dict(C=1600))]
    if args.op in ("rowwise", "all"):
        cases += [("residual", dict(C=768)), ("gelu", dict(C=3072)), ("encoder", dict(C=768))]
    if args.case is not None:
        cases = [cases[args.case]]
    flush = torch.empty(64 * 1024 * 1024, device="cuda") if args.flush_l2 else None
    nsets = max(1, args.stream)  # rotating buffer sets of the memory-bound kernels
    for op, c in cases:
        if op == "matmul":
            K, N = c["K"], c["N"]
            x, w = randn(Bb, Tt, K), randn(N, K, std=0.02)
            bias = randn(N, std=0.01) if c["bias"] else None
            res = randn(Bb, Tt, N) if c["res"] else None
            out = torch.empty(Bb, Tt, N, device="cuda")
            fn = lambda: ctx.matmul_forward(out, x, w, bias, Bb, Tt, K, N, act=c["act"], residual=res, mode=c["mode"])
            work, unit, peak = 2.0 * M * K * N / 1e12, "TFLOP/s", peaks["bf16_burst"] / 2
            name = f"matmul {K}->{N}" + ("+gelu" if c["act"] else "") + ("+residual" if c["res"] else "") + (" 3xTF32" if c["mode"] else "")
        elif op == "matmul_bf16":
            K, N = c["K"], c["N"]
            x, w = randn(Bb, Tt, K).to(torch.bfloat16), randn(N, K, std=0.02).to(torch.bfloat16)
            bias = randn(N, std=0.01) if c["bias"] else None
            out = None if c["out_h"] else torch.empty(Bb, Tt, N, device="cuda")
            outh = torch.empty(Bb, Tt, N, device="cuda", dtype=torch.bfloat16) if c["out_h"] else None
            fn = lambda: ctx.matmul_forward_bf16(out, outh, x, w, bias, Bb, Tt, K, N, act=c["act"])
            work, unit, peak = 2.0 * M * K * N / 1e12, "TFLOP/s", peaks["bf16_burst"]
            name = f"matmul bf16 {K}->{N}" + ("+gelu" if c["act"] else "") + (" bf16 out" if c["out_h"] else "")
        elif op == "matmul_bf16x3":
            K, N = c["K"], c["N"]
            xs = torch.empty(2, Bb, Tt, K, device="cuda", dtype=torch.bfloat16)
            ctx.split_bf16(xs[0], xs[1], randn(Bb, Tt, K), M * K)
            wh = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
            wl = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
            ctx.split_bf16(wh, wl, randn(N, K, std=0.02), N * K)
            bias = randn(N, std=0.01) if c["bias"] else None
            out = None if c["outk"] == "split" else torch.zeros(Bb, Tt, N, device="cuda")
            outs = torch.empty(2, Bb, Tt, N, device="cuda", dtype=torch.bfloat16) if c["outk"] == "split" else None
            fn = lambda: ctx.matmul_forward_bf16x3(out, outs, xs, wh, wl, bias, Bb, Tt, K, N, act=c["act"],
                                                   accumulate=c["outk"] == "accumulate")
            work, unit, peak = 2.0 * M * K * N / 1e12, "TFLOP/s", peaks["bf16_burst"] / 3
            name = f"matmul bf16x3 {K}->{N}" + ("+gelu" if c["act"] else "") + {"split": " split out", "accumulate": " accumulate", "fp32": ""}[c["outk"]]
        elif op == "matmul_fp8":
            K, N = c["K"], c["N"]
            xq = torch.empty(Bb, Tt, K, device="cuda", dtype=torch.uint8)
            wq = torch.empty(N, K, device="cuda", dtype=torch.uint8)
            ctx.quantize_e4m3(xq, randn(Bb, Tt, K), M * K, 1.0)
            ctx.quantize_e4m3(wq, randn(N, K, std=0.02), N * K, 1024.0)
            bias = randn(N, std=0.01) if c["bias"] else None
            out = torch.zeros(Bb, Tt, N, device="cuda")
            fn = lambda: ctx.matmul_forward_fp8(out, xq, wq, bias, Bb, Tt, K, N, act=c["act"], alpha=1.0 / 1024.0, accumulate=c["acc"])
            work, unit, peak = 2.0 * M * K * N / 1e12, "TFLOP/s", peaks["bf16_burst"] * 2
            name = f"matmul fp8 (e4m3) {K}->{N}" + ("+gelu" if c["act"] else "") + (" accumulate" if c["acc"] else "")
        elif op == "attention_fp16":
            NH = c["NH"]
            Cc = NH * 64
            planes = torch.empty(2, Bb, Tt, 3 * Cc, device="cuda", dtype=torch.float16)
            ctx.split_fp16(planes[0], planes[1], randn(Bb, Tt, 3 * Cc), M * 3 * Cc)
            out = torch.empty(Bb, Tt, Cc, device="cuda")
            lse = torch.empty(Bb, NH, Tt, device="cuda")
            fn = lambda: ctx.attention_forward_fp16(out, lse, planes, Bb, Tt, Cc, NH)
            work, unit, peak = 4.0 * 64 * Tt * (Tt + 1) / 2 * NH * Bb / 1e12, "TFLOP/s", peaks["bf16_burst"]
            name = f"attention fp16 B=8 T=1024 NH={NH} (causal-exact flop)"
        elif op == "attention":
            NH = c["NH"]
            Cc = NH * 64
            qkv, out = randn(Bb, Tt, 3 * Cc), torch.empty(Bb, Tt, Cc, device="cuda")
            lse = torch.empty(Bb, NH, Tt, device="cuda")
            fn = lambda: ctx.attention_forward(out, None, lse, qkv, Bb, Tt, Cc, NH)
            work, unit, peak = 4.0 * 64 * Tt * (Tt + 1) / 2 * NH * Bb / 1e12, "TFLOP/s", peaks["bf16_burst"] / 2
            name = f"attention B=8 T=1024 NH={NH} (causal-exact flop)"
        elif op in ("layernorm", "fused_residual_layernorm"):
            Cc = c["C"]
            S = [dict(x=randn(Bb, Tt, Cc), x2=randn(Bb, Tt, Cc), out=torch.empty(Bb, Tt, Cc, device="cuda"),
                      res=torch.empty(Bb, Tt, Cc, device="cuda")) for _ in range(nsets)]
            w, b = randn(Cc), randn(Cc)
            mean, rstd = torch.empty(Bb, Tt, device="cuda"), torch.empty(Bb, Tt, device="cuda")
            if op == "layernorm":
                fn = lambda k=0: ctx.layernorm_forward(S[k]["out"], mean, rstd, S[k]["x"], w, b, Bb, Tt, Cc)
                work = (2.0 * M * Cc + 2 * M + 2 * Cc) * 4 / 1e9
            else:
                fn = lambda k=0: ctx.fused_residual_layernorm_forward(S[k]["res"], S[k]["out"], mean, rstd, S[k]["x"],
                                                                      S[k]["x2"], w, b, Bb, Tt, Cc)
                work = (4.0 * M * Cc + 2 * M + 2 * Cc) * 4 / 1e9
            unit, peak, name = "GB/s", peaks["hbm_gbs"], f"{op} [8192,{Cc}]"
        else:
            Cc = c["C"]
            S = [dict(x=randn(Bb, Tt, Cc), x2=randn(Bb, Tt, Cc), out=torch.empty(Bb, Tt, Cc, device="cuda"))
                 for _ in range(nsets)]
            if op == "residual":
                fn = lambda k=0: ctx.residual_forward(S[k]["out"], S[k]["x"], S[k]["x2"], M * Cc)
                work = 3.0 * M * Cc * 4 / 1e9
            elif op == "gelu":
                fn = lambda k=0: ctx.gelu_forward(S[k]["out"], S[k]["x"], M * Cc)
                work = 2.0 * M * Cc * 4 / 1e9
            else:
                tok = torch.randint(0, 50257, (Bb, Tt), dtype=torch.int32, device="cuda", generator=g)
                wte, wpe = randn(50304, Cc, std=0.02), randn(Tt, Cc, std=0.02)
                fn = lambda k=0: ctx.encoder_forward(S[k]["out"], tok, wte, wpe, Bb, Tt, Cc)
                work = ((2.0 * M * Cc + Tt * Cc) * 4 + M * 4) / 1e9
            unit, peak, name = "GB/s", peaks["hbm_gbs"], f"{op} [8192,{Cc}]"
        streaming = args.stream > 1 and op not in ("matmul", "matmul_bf16", "matmul_bf16x3", "matmul_fp8", "attention", "attention_fp16")
        torch.cuda.synchronize()
        for _ in range(args.warmup):
            fn()
        ctx.sync_check()
        times = []
        for _ in range(args.steps):
            if flush is not None:
                with torch.cuda.stream(stream):
                    flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            if streaming:
                for k in range(2 * nsets):
                    fn(k % nsets)
            else:
                fn()
            e1.record(stream)
            e1.synchronize()
            times.append(e0.elapsed_time(e1) / (2 * nsets if streaming else 1))
        ctx.sync_check()
        med, best = statistics.median(times), min(times)
        scale = 1e3  # work is in T(FLOP) or G(B); time in ms
        print(json.dumps({"kernel": name, "median_ms": round(med, 5), "min_ms": round(best, 5), "cold_l2": bool(args.flush_l2),
                          "back_to_back_sets": nsets if streaming else 1,
                          "achieved": round(work / (med / scale), 1), "unit": unit, "peak": peak,
                          "frac": round(work / (med / scale) / peak, 4), "peak_source": peaks["source"]}), flush=True)
    ctx.close()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="124m", choices=["124m", "xl"],
                    help="124m = the benchmark configuration; xl = GPT-2 XL shapes, B=8 T=1024 per GPU (extra measurement)")
    ap.add_argument("--no-xl", action="store_true", help="skip the GPT-2 XL / multi-GPU extras behind the main measurement")
    ap.add_argument("--tp", action="store_true",
                    help="with --gpus N > 1: one tensor-parallel group over all ranks instead of batch sharding")
    ap.add_argument("--op", default=None,
                    choices=["all", "matmul", "matmul_bf16", "matmul_bf16x3", "matmul_fp8", "attention", "attention_fp16", "layernorm",
                             "fused_residual_layernorm", "rowwise"],
                    help="per-kernel sweep at 8192 rows instead of the forward benchmark")
    ap.add_argument("--case", type=int, default=None, help="with --op: run only this case of the family")
    ap.add_argument("--modes", default="tf32", choices=["tf32", "both"], help="with --op matmul: also time 3xTF32")
    ap.add_argument("--flush-l2", action="store_true", help="with --op: cold L2 before every launch")
    ap.add_argument("--stream", type=int, default=1,
                    help="with --op, memory-bound kernels: time 2N back-to-back launches over N rotating buffer sets "
                         "(N x 100-200 MB, beyond L2): steady-state HBM rate without per-launch latency")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.op:
        return run_kernel_sweep(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
