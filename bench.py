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

METRIC = "gpt2_forward_tokens_per_s"
UNIT = "tokens/s"
B_PER_GPU, T = 8, 1024
WORKLOAD = "GPT-2 124M full-sequence forward, B=8 T=1024 per GPU, fp32 storage, TF32 tensor-core GEMMs (configs[1])"


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


def cpu_forward_tokens_per_s(sample_T: int, repeats: int = 1, threads: int | None = None, xl: bool = False):
    """Times the CPU oracle's fp32 forward of GPT-2 (124M, or XL) on one sequence of sample_T tokens."""
    import numpy as np
    from oracle import oracle as orc
    if threads:
        os.environ["OMP_NUM_THREADS"] = str(threads)
    cfg = orc.GPT2_XL if xl else orc.GPT2_124M
    offs = orc.param_offsets(cfg)
    rng = np.random.default_rng(1234)
    params = np.zeros(offs[16], dtype=np.float32)
    for i, name in enumerate(orc.PARAM_NAMES):
        if name in ("ln1w", "ln2w", "lnfw"):
            params[offs[i]:offs[i + 1]] = 1.0
        elif name in ("wte", "wpe", "qkvw", "attprojw", "fcw", "fcprojw"):
            params[offs[i]:offs[i + 1]] = rng.standard_normal(offs[i + 1] - offs[i], dtype=np.float32) * 0.02
    tokens = orc.fill_tokens((1, sample_T), seed=4321, vocab=cfg.vocab_size)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.gpt2_forward(params, cfg, tokens)
        times.append(time.perf_counter() - t0)
    return sample_T / min(times), orc.num_threads(), params, cfg


def run_reference(args):
    """The reference project has no CPU implementation and cannot run without a GPU, so the
    reference arm times this repository's CPU restatement of its forward (oracle/, a port)
    with all host threads, each step one sequence of the benchmark workload (or a shorter
    prefix when K+W steps of a full sequence would not finish in a few minutes)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np
    from oracle import oracle as orc
    orc.build()
    # calibrate on a short prefix, then size the per-step sample so the run stays bounded
    tps_small, cores, params, cfg = cpu_forward_tokens_per_s(64)
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
    sample = f"1 sequence of {sample_T} tokens per step (of the B=8 x T=1024 workload), fp32 accumulate, OpenMP"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "tokens_per_step": sample_T},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


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
    model = pkg.GPT2(ctx, cfg, B, T, tp_size=world if tp else 1, tp_rank=rank if tp else 0)
    if tp:
        model.set_allreduce_torch(stream)
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

    # the same K steps again with one CUDA-event pair around every kernel launch (on the launching
    # stream): per-operator durations for the roofline figures; not part of `value`
    model.set_profile(True)
    for _ in range(args.steps):
        model.forward(tok_dev, B, T)
    prof = model.read_profile()
    model.set_profile(False)

    # ------------------------------------------------ the same workload in the 3xTF32 mode
    # (split-operand GEMMs and attention: the mode that holds the 99.9 % top-1 / 1e-4 bars)
    x3_ms = None
    if not xl:
        model.set_options(round_operands=0, gemm_mode=pkg.B200_TF32X3, lmhead_mode=pkg.B200_TF32X3)
        for _ in range(2):
            model.forward(tok_dev, B, T)
        barrier()
        ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_x3 = max(1, args.steps // 2)
        ev2.record(stream)
        for _ in range(n_x3):
            model.forward(tok_dev, B, T)
        ev3.record(stream)
        barrier()
        ctx.sync_check()
        x3_ms = max_over_ranks(ev2.elapsed_time(ev3)) / n_x3
        model.set_options(round_operands=1, gemm_mode=pkg.B200_TF32, lmhead_mode=pkg.B200_TF32)

    # ------------------------------------------------ the same workload with bf16 GEMM operands
    # (optional reduced-precision mode; never the headline, which stays TF32)
    bf16_ms = None
    if not args.tp:
        model.set_options(round_operands=1, gemm_mode=pkg.B200_BF16, lmhead_mode=pkg.B200_BF16)
        for _ in range(3):
            model.forward(tok_dev, B, T)
        barrier()
        ev4, ev5 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev4.record(stream)
        for _ in range(args.steps):
            model.forward(tok_dev, B, T)
        ev5.record(stream)
        barrier()
        ctx.sync_check()
        bf16_ms = max_over_ranks(ev4.elapsed_time(ev5)) / args.steps
        model.set_options(round_operands=1, gemm_mode=pkg.B200_TF32, lmhead_mode=pkg.B200_TF32)

    # ---------------------------------------------- incremental decoding (key/value cache)
    # One new token per sequence against a cache filled by a prefill of T/2 positions; each step
    # reads every weight and the used part of the cache once (HBM-bound).  Extra measurement on
    # rank 0; not part of `value`.
    decode = None
    if rank == 0 and not tp and not xl and B <= 16:
        try:
            model.enable_kv_cache()
            model.set_options(round_operands=1, gemm_mode=pkg.B200_TF32, lmhead_mode=pkg.B200_TF32, use_graph=1)
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
        except Exception as e:  # an extra measurement must not take the benchmark line down
            decode = {"error": str(e)}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return 0

    tokens_total = replicas * B * T * args.steps
    value = tokens_total / (elapsed_ms * 1e-3)
    peaks = _peaks()
    # dominant kernel: the tcgen05 TF32 GEMM (five shapes, 4L+1 launches per step); rank-local widths
    M = B * T
    Cc, L = cfg.channels, cfg.num_layers
    n_tp = world if tp else 1
    Ac, Fc, Vl = pkg.tp_heads(cfg.num_heads, n_tp, 0)[1] * 64, 4 * Cc // n_tp, model.logits_width
    gemm_flops = {"gemm_qkv": 2.0 * M * Cc * 3 * Ac, "gemm_attproj": 2.0 * M * Ac * Cc, "gemm_fc": 2.0 * M * Cc * Fc,
                  "gemm_fcproj": 2.0 * M * Fc * Cc, "gemm_lmhead": 2.0 * M * Cc * Vl}
    tot_flops = sum(gemm_flops[k] * prof[k][1] for k in gemm_flops)
    tot_ms = sum(prof[k][0] for k in gemm_flops)
    n_gemm = sum(prof[k][1] for k in gemm_flops)
    tf32_peak = peaks["bf16_sustained"] / 2.0
    achieved = tot_flops / (tot_ms * 1e-3) / 1e12 if tot_ms > 0 else 0.0
    per_op = {}
    hbm_bytes = {"layernorm": (2.0 * M * Cc + 2 * Cc) * 4, "fused_residual_layernorm": (4.0 * M * Cc + 2 * Cc) * 4,
                 "encoder": (2.0 * M * Cc + T * Cc) * 4 + M * 4}
    att_flops = 4.0 * 64 * T * (T + 1) / 2 * (Ac // 64) * B
    for name, (ms, n) in prof.items():
        if n == 0:
            continue
        avg = ms / n
        entry = {"launches_per_step": n / args.steps, "avg_ms": round(avg, 5), "share": round(ms / sum(v[0] for v in prof.values()), 4)}
        if name in gemm_flops:
            entry["tflops"] = round(gemm_flops[name] / (avg * 1e-3) / 1e12, 1)
        elif name == "attention":
            entry["tflops_causal"] = round(att_flops / (avg * 1e-3) / 1e12, 1)
        elif name in hbm_bytes:
            entry["gbs"] = round(hbm_bytes[name] / (avg * 1e-3) / 1e9, 1)
        per_op[name] = entry

    cpu_T = 256 if xl else 1024
    cpu_tps, cores, _, _ = cpu_forward_tokens_per_s(cpu_T, repeats=1, xl=xl)
    d2h = B * model.logits_width * 4 + (0 if tp else B * T * 4)
    workload = WORKLOAD if not xl else "GPT-2 XL 1.5B full-sequence forward, B=8 T=1024 per " + ("tensor-parallel group" if tp else "GPU") + ", fp32 storage, TF32 tensor-core GEMMs (configs[4] shapes)"
    par = (f"tensor-parallel x{world}: heads / MLP / vocabulary split, one NCCL all-reduce per attention and MLP block" if tp
           else f"batch-sharded x{world}, no collective")
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
        "config": {"workload": workload, "global_batch": replicas * B, "seq_len": T, "parallelism": par,
                   "l2": "no flush: each step streams the weights (0.5 GB for 124M) and writes 1.65 GB of logits, far beyond the 126 MB L2",
                   "flop_per_token": cfg.flops_per_token(T)},
        "roofline": {"bound": "tensor", "kernel": "gemm_tf32_pair_kernel and gemm_tf32_kernel (all five GEMM shapes of the forward)",
                     "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak,
                     "peak_source": f"{peaks['source']} bf16 sustained {peaks['bf16_sustained']} TFLOP/s / 2 (TF32 runs at half the bf16 rate; no TF32 peak is measured)",
                     "launches_per_step": n_gemm / args.steps,
                     # ncu dram__bytes_read.sum + dram__bytes_write.sum, average per GEMM launch of the 124M
                     # forward (profiles/gemm_tf32_dram_traffic_by_shape.md); not captured for other models
                     "traffic": None if (xl or tp) else 116.2e6, "algorithmic_bytes": None if (xl or tp) else 142.9e6,
                     "per_operator": per_op},
        "cpu_baseline": {"value": cpu_tps, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"1 sequence of {cpu_T} tokens (B=1), fp32-accumulate C/OpenMP forward, all host threads, one run"},
        "e2e": {"value": replicas * B * T * args.steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": B * T * 4,
                "d2h_bytes_per_step": d2h, "ms_per_step": 1e3 * e2e_s / args.steps,
                "result": "last-position logits [B,Vp]" + ("" if tp else " and per-position arg-max token ids [B,T]"),
                "call": "b200_gpt2_forward_host_enqueue / _wait, two steps in flight, double-buffered pinned host buffers",
                "synchronous_call": {"value": replicas * B * T * args.steps / e2e_sync_s, "ms_per_step": 1e3 * e2e_sync_s / args.steps,
                                     "call": "b200_gpt2_forward_host, one step at a time"}},
        "gpu_launches": launches,
        "clocks": clocks,
        "tf32x3": None if x3_ms is None else {
            "value": replicas * B * T / (x3_ms * 1e-3), "unit": UNIT, "ms_per_step": x3_ms,
            "note": "same workload with gemm_mode = lmhead_mode = B200_TF32X3 (split-operand GEMMs and attention)"},
        "bf16_operands": None if bf16_ms is None else {
            "value": replicas * B * T / (bf16_ms * 1e-3), "unit": UNIT, "ms_per_step": bf16_ms,
            "note": "same workload with gemm_mode = lmhead_mode = B200_BF16 (bf16 GEMM operands, fp32 accumulation; "
                    "reduced precision, not comparable with the headline)"},
        "decode": decode,
    }
    print(json.dumps(line), flush=True)
    model.close()
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


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
        return torch.empty(shape, device="cuda").normal_(0.0, std, generator=g)

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
    if args.op in ("attention", "all"):
        cases += [("attention", dict(NH=12)), ("attention", dict(NH=25))]
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
        streaming = args.stream > 1 and op not in ("matmul", "matmul_bf16", "attention")
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
    ap.add_argument("--tp", action="store_true",
                    help="with --gpus N > 1: one tensor-parallel group over all ranks instead of batch sharding")
    ap.add_argument("--op", default=None,
                    choices=["all", "matmul", "matmul_bf16", "attention", "layernorm", "fused_residual_layernorm", "rowwise"],
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
