"""Pins the CPU oracle against outputs of the REFERENCE project's own CUDA kernels.

tests/golden/reference_kernels.npz was recorded by tests/golden/make_golden.py on a B200 from
oracle/_ref/libref_kernels.so, i.e. from the reference's headers compiled as they are
(kernels/matmul/1_matmul_tiling.cuh, 9_matmul_async_cg_tf32_gelu.cuh,
kernels/layernorm/1_layernorm_block.cuh, 2_layernorm_block_vectorized.cuh,
kernels/residual/1_residual_naive.cuh, kernels/attention/3_flash_attention_permute.cuh).
The reference ships no test vectors of its own, so these recordings are the pin.

tests/golden/reference_kernels_sizes.npz (same script, same library) adds the cases at the real
models' widths: K = 768, 1600 and 3072 for the GEMMs, C = 1600 for the layernorms, T = 1024 and
several heads and sequences for the attention.  It stores outputs and seeds; the inputs are drawn
again here.  A second recording on another B200 reproduced every array of both files bit for bit
except the layernorm outputs (the reference kernels sum with shared-memory atomics, whose order
varies: differences up to 1e-6).
"""
import json
import os
import sys

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz")
GOLD_SIZES = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels_sizes.npz")


@pytest.fixture(scope="module")
def g():
    return np.load(GOLD)


def trunc_tf32(a):
    """What the tensor cores do with fp32 operand bits: drop the low 13 mantissa bits."""
    return (np.ascontiguousarray(a).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


@pytest.mark.parametrize("tag", ["mm_a", "mm_b"])
@pytest.mark.parametrize("precise", [False, True])
def test_matmul_matches_reference_fp32_kernel(g, orc, tag, precise):
    bias = g[tag + "_bias"] if tag + "_bias" in g else None
    y = orc.matmul_forward(g[tag + "_x"], g[tag + "_w"], bias, precise=precise)
    # fp32 FMA kernel vs a different summation order: a few ulp of the K-term sums
    assert np.abs(y - g[tag + "_out"]).max() < 5e-6


@pytest.mark.parametrize("tag,act", [("mmtf32", 0), ("mmtf32_gelu", 1)])
def test_matmul_gelu_matches_reference_tf32_kernel(g, orc, tag, act):
    x, w, b, want = g[tag + "_x"], g[tag + "_w"], g[tag + "_bias"], g[tag + "_out"]
    # the reference feeds raw fp32 bits to wmma tf32 (kernels/matmul/ptx.cuh:51-84): the hardware
    # truncates them.  With the same truncation applied to the oracle's inputs the two agree to
    # fp32 rounding, which pins matmul + bias + tanh-GELU; without it they differ by TF32 error.
    y_t = orc.matmul_forward(trunc_tf32(x), trunc_tf32(w), b, act=act, precise=True)
    assert np.abs(y_t - want).max() < 5e-6
    y = orc.matmul_forward(x, w, b, act=act, precise=True)
    assert np.abs(y - want).max() < 3e-3


@pytest.mark.parametrize("tag", ["ln_block", "ln_vec"])
@pytest.mark.parametrize("precise", [False, True])
def test_layernorm_matches_reference_kernels(g, orc, tag, precise):
    y, mean, rstd = orc.layernorm_forward(g[tag + "_x"], g[tag + "_w"], g[tag + "_b"], precise=precise)
    assert np.abs(y - g[tag + "_out"]).max() < 5e-6
    assert np.abs(mean - g[tag + "_mean"]).max() < 1e-6
    assert np.abs(rstd / g[tag + "_rstd"] - 1).max() < 2e-6


def test_residual_matches_reference_kernel_bitwise(g, orc):
    assert np.array_equal(orc.residual_forward(g["res_a"], g["res_b"]), g["res_out"])


def test_fused_residual_layernorm_is_residual_then_layernorm(g, orc):
    # the reference's fused kernel reads the wrong rows (float4 pointer stride,
    # fused_residual_layernorm.cuh:19,48-50), so the fused oracle is pinned through its two
    # pinned halves instead
    x = g["ln_block_x"]
    x2 = orc.fill_normal(x.shape, 77)
    res, out, mean, rstd = orc.fused_residual_layernorm_forward(x, x2, g["ln_block_w"], g["ln_block_b"])
    assert np.array_equal(res, orc.residual_forward(x, x2))
    y, m, r = orc.layernorm_forward(res, g["ln_block_w"], g["ln_block_b"])
    assert np.array_equal(out, y) and np.array_equal(mean, m) and np.array_equal(rstd, r)


def test_attention_matches_reference_flash_kernel(g, orc):
    qkv, want, nh = g["att_qkv"], g["att_out"], int(g["att_nh"])
    y, _ = orc.attention_forward(qkv, nh, precise=True)
    # TF32 operands (truncated q, k, v and p) and __expf in the reference kernel
    assert np.abs(y - want).max() < 4e-3
    y_t, _ = orc.attention_forward(trunc_tf32(qkv), nh, precise=True)
    assert np.abs(y_t - want).max() < 1e-3  # what is left is the truncation of P


# ---------------------------------------------------------------- the cases at the real models' widths
@pytest.fixture(scope="module")
def gs():
    return np.load(GOLD_SIZES)


def _case(gs, orc, tag):
    """Inputs of a case, drawn from its recorded seed exactly as the recording script drew them."""
    sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
    try:
        import make_golden
    finally:
        sys.path.pop(0)
    c = json.loads(str(gs["meta"]))[tag]
    inp = make_golden.sizes_inputs(c)
    for name, v in inp.items():  # the generator still produces what was fed to the reference kernels
        assert float(gs[f"{tag}_sum_{name}"]) == v.astype(np.float64).sum()
    return c, inp, gs[tag + "_out"]


@pytest.mark.parametrize("precise", [False, True])
def test_matmul_k3072_matches_reference_fp32_kernel(gs, orc, precise):
    c, a, want = _case(gs, orc, "mm_k3072")
    y = orc.matmul_forward(a["x"], a["w"], a["bias"], precise=precise)
    assert np.abs(y - want).max() < 2e-5  # 3072-term fp32 sums in another order, outputs up to 4.3


@pytest.mark.parametrize("tag", ["mmtf32_k768_gelu", "mmtf32_k3072", "mmtf32_k1600_gelu"])
def test_matmul_real_widths_match_reference_tf32_kernel(gs, orc, tag):
    c, a, want = _case(gs, orc, tag)
    y_t = orc.matmul_forward(trunc_tf32(a["x"]), trunc_tf32(a["w"]), a["bias"], act=c["gelu"], precise=True)
    # same truncated operands: what is left is the tensor core's fp32 accumulation, whose error grows
    # with the number of terms (measured 4.5e-6, 8.3e-6 and 1.6e-5 of the largest output at K = 768, 1600, 3072)
    assert np.abs(y_t - want).max() < 1e-8 * c["C"] * np.abs(want).max()
    y = orc.matmul_forward(a["x"], a["w"], a["bias"], act=c["gelu"], precise=True)
    assert 2e-4 < np.abs(y - want).max() < 6e-3  # TF32 operand error, and visibly so


@pytest.mark.parametrize("tag", ["ln_block_1600", "ln_vec_1600"])
@pytest.mark.parametrize("precise", [False, True])
def test_layernorm_1600_matches_reference_kernels(gs, orc, tag, precise):
    c, a, want = _case(gs, orc, tag)
    y, mean, rstd = orc.layernorm_forward(a["x"], a["w"], a["b"], precise=precise)
    assert np.abs(y - want).max() < 8e-6
    assert np.abs(mean - gs[tag + "_mean"]).max() < 1e-6
    assert np.abs(rstd / gs[tag + "_rstd"] - 1).max() < 2e-6


@pytest.mark.parametrize("tag", ["att_b2_t256_nh3", "att_t1024_nh1"])
def test_attention_more_heads_and_long_rows_match_reference_flash_kernel(gs, orc, tag):
    c, a, want = _case(gs, orc, tag)
    y, _ = orc.attention_forward(a["qkv"], c["NH"], precise=True)
    assert np.abs(y - want).max() < 4e-3
    y_t, _ = orc.attention_forward(trunc_tf32(a["qkv"]), c["NH"], precise=True)
    assert np.abs(y_t - want).max() < 1e-3
