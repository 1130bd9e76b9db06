"""Records the golden fixtures (reference_kernels.npz) from the REFERENCE project's own CUDA
kernels.

Run on a machine with a GPU, after `make -C oracle ref` has built oracle/_ref/libref_kernels.so
from a checkout of GJ0407790/CUDA-GPT2-Inference:

    python tests/golden/make_golden.py [output.npz]

Inputs are drawn with the oracle's seeded generator (oracle_fill_normal), stored alongside the
reference outputs, and the CPU tests (tests/test_oracle_golden.py) check the oracle against them.
A second file beside it, reference_kernels_sizes.npz, holds the cases at the real models' widths
(see SIZES below): outputs and seeds only.
Only kernels that compile and are correct by reading are used (see oracle/ref_harness.cu).
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_kernels.npz")
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so"))
    keep = []  # every device buffer stays alive until the end (the caching allocator reuses freed blocks)

    def dev(a):
        t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
        keep.append(t)
        return t

    p = lambda t: C.c_void_p(t.data_ptr())
    fx = {}

    def check(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} returned {rc}")

    # matmul, fp32 FMA: kernels/matmul/1_matmul_tiling.cuh (ragged shapes, bias and no bias)
    for tag, (B, T, Cc, OC, has_bias) in {"mm_a": (2, 24, 40, 56, True), "mm_b": (1, 33, 768, 100, False)}.items():
        x = orc.fill_normal((B, T, Cc), 1001)
        w = orc.fill_normal((OC, Cc), 1002, std=0.02)
        b = orc.fill_normal((OC,), 1003, std=0.01) if has_bias else None
        out = torch.empty((B, T, OC), device="cuda")
        check(ref.ref_matmul_forward_tiling(p(out), p(dev(x)), p(dev(w)), p(dev(b)) if has_bias else None, B, T, Cc, OC), tag)
        fx[f"{tag}_x"], fx[f"{tag}_w"], fx[f"{tag}_out"] = x, w, out.cpu().numpy()
        if has_bias:
            fx[f"{tag}_bias"] = b

    # matmul, TF32 wmma + bias (+GELU): kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh
    for tag, gelu in {"mmtf32": 0, "mmtf32_gelu": 1}.items():
        B, T, Cc, OC = 1, 128, 64, 128
        x = orc.fill_normal((B, T, Cc), 1011)
        w = orc.fill_normal((OC, Cc), 1012, std=0.05)
        b = orc.fill_normal((OC,), 1013, std=0.1)
        out = torch.empty((B, T, OC), device="cuda")
        check(ref.ref_matmul_forward_tf32_gelu(p(out), p(dev(x)), p(dev(w)), p(dev(b)), B, T, Cc, OC, gelu), tag)
        fx[f"{tag}_x"], fx[f"{tag}_w"], fx[f"{tag}_bias"], fx[f"{tag}_out"] = x, w, b, out.cpu().numpy()

    # layernorm: kernels/layernorm/1_layernorm_block.cuh and 2_layernorm_block_vectorized.cuh
    for tag, fn in {"ln_block": ref.ref_layernorm_forward_block, "ln_vec": ref.ref_layernorm_forward_block_vectorized}.items():
        B, T, Cc = 2, 8, 768
        x = orc.fill_normal((B, T, Cc), 1021, mean=0.3, std=1.5)
        w = orc.fill_normal((Cc,), 1022, mean=1.0, std=0.2)
        b = orc.fill_normal((Cc,), 1023, std=0.2)
        out, mean, rstd = torch.empty((B, T, Cc), device="cuda"), torch.empty((B, T), device="cuda"), torch.empty((B, T), device="cuda")
        check(fn(p(out), p(mean), p(rstd), p(dev(x)), p(dev(w)), p(dev(b)), B, T, Cc), tag)
        fx[f"{tag}_x"], fx[f"{tag}_w"], fx[f"{tag}_b"] = x, w, b
        fx[f"{tag}_out"], fx[f"{tag}_mean"], fx[f"{tag}_rstd"] = out.cpu().numpy(), mean.cpu().numpy(), rstd.cpu().numpy()

    # residual: kernels/residual/1_residual_naive.cuh
    a, b2 = orc.fill_normal((1000,), 1031), orc.fill_normal((1000,), 1032)
    out = torch.empty(1000, device="cuda")
    check(ref.ref_residual_forward_naive(p(out), p(dev(a)), p(dev(b2)), 1000), "residual")
    fx["res_a"], fx["res_b"], fx["res_out"] = a, b2, out.cpu().numpy()

    # causal flash attention on the packed buffer: kernels/attention/3_flash_attention_permute.cuh
    B, T, NH = 1, 128, 2
    Cc = NH * 64
    qkv = orc.fill_normal((B, T, 3 * Cc), 1041)
    out = torch.empty((B, T, Cc), device="cuda")
    check(ref.ref_flash_attention_permute_forward(p(out), p(dev(qkv)), B, T, Cc, NH), "attention")
    fx["att_qkv"], fx["att_out"], fx["att_nh"] = qkv, out.cpu().numpy(), np.int32(NH)

    np.savez_compressed(out_path, **fx)
    print("wrote", out_path, {k: v.shape for k, v in fx.items() if k.endswith("_out")})
    record_sizes(ref, dev, p, check, os.path.join(os.path.dirname(out_path), "reference_kernels_sizes.npz"))


# Second fixture: the same reference kernels at the widths and depths of the real models (K = 768, 1600,
# 3072; C = 1600; T = 1024; several heads and sequences).  Only the outputs are stored; the inputs are
# regenerated from the seeds in `meta` (the generator is counter-based and pinned by its own test), and a
# float64 sum of every input is stored so that a drifted generator is told apart from a drifted oracle.
SIZES = {
    "mm_k3072": dict(kind="mm", B=1, T=64, C=3072, OC=64, seed=2001),
    "mmtf32_k768_gelu": dict(kind="mmtf32", B=2, T=128, C=768, OC=256, gelu=1, seed=2011),
    "mmtf32_k3072": dict(kind="mmtf32", B=1, T=128, C=3072, OC=128, gelu=0, seed=2021),
    "mmtf32_k1600_gelu": dict(kind="mmtf32", B=1, T=128, C=1600, OC=128, gelu=1, seed=2031),
    "ln_block_1600": dict(kind="ln_block", B=1, T=16, C=1600, seed=2041),
    "ln_vec_1600": dict(kind="ln_vec", B=1, T=16, C=1600, seed=2051),
    "att_b2_t256_nh3": dict(kind="att", B=2, T=256, NH=3, seed=2061),
    "att_t1024_nh1": dict(kind="att", B=1, T=1024, NH=1, seed=2071),
}


def sizes_inputs(c):
    """The inputs of one case of SIZES, from its seed (also used by tests/test_oracle_golden.py)."""
    k, s = c["kind"], c["seed"]
    if k in ("mm", "mmtf32"):
        return dict(x=orc.fill_normal((c["B"], c["T"], c["C"]), s), w=orc.fill_normal((c["OC"], c["C"]), s + 1, std=0.02),
                    bias=orc.fill_normal((c["OC"],), s + 2, std=0.05))
    if k in ("ln_block", "ln_vec"):
        return dict(x=orc.fill_normal((c["B"], c["T"], c["C"]), s, mean=-0.2, std=2.0),
                    w=orc.fill_normal((c["C"],), s + 1, mean=1.0, std=0.2), b=orc.fill_normal((c["C"],), s + 2, std=0.2))
    return dict(qkv=orc.fill_normal((c["B"], c["T"], 3 * 64 * c["NH"]), s))


def record_sizes(ref, dev, p, check, out_path):
    import json
    fx = {"meta": np.array(json.dumps(SIZES))}
    for tag, c in SIZES.items():
        a = sizes_inputs(c)
        for name, v in a.items():
            fx[f"{tag}_sum_{name}"] = np.float64(v.astype(np.float64).sum())
        k = c["kind"]
        if k in ("mm", "mmtf32"):
            out = torch.empty((c["B"], c["T"], c["OC"]), device="cuda")
            if k == "mm":
                check(ref.ref_matmul_forward_tiling(p(out), p(dev(a["x"])), p(dev(a["w"])), p(dev(a["bias"])), c["B"], c["T"], c["C"], c["OC"]), tag)
            else:
                check(ref.ref_matmul_forward_tf32_gelu(p(out), p(dev(a["x"])), p(dev(a["w"])), p(dev(a["bias"])), c["B"], c["T"], c["C"], c["OC"], c["gelu"]), tag)
        elif k in ("ln_block", "ln_vec"):
            fn = ref.ref_layernorm_forward_block if k == "ln_block" else ref.ref_layernorm_forward_block_vectorized
            out = torch.empty((c["B"], c["T"], c["C"]), device="cuda")
            mean, rstd = torch.empty((c["B"], c["T"]), device="cuda"), torch.empty((c["B"], c["T"]), device="cuda")
            check(fn(p(out), p(mean), p(rstd), p(dev(a["x"])), p(dev(a["w"])), p(dev(a["b"])), c["B"], c["T"], c["C"]), tag)
            fx[f"{tag}_mean"], fx[f"{tag}_rstd"] = mean.cpu().numpy(), rstd.cpu().numpy()
        else:
            Cc = 64 * c["NH"]
            out = torch.empty((c["B"], c["T"], Cc), device="cuda")
            check(ref.ref_flash_attention_permute_forward(p(out), p(dev(a["qkv"])), c["B"], c["T"], Cc, c["NH"]), tag)
        fx[f"{tag}_out"] = out.cpu().numpy()
    np.savez_compressed(out_path, **fx)
    print("wrote", out_path, {k: v.shape for k, v in fx.items() if k.endswith("_out")})


if __name__ == "__main__":
    main()
