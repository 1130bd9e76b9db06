"""Pins the CPU oracle against outputs of the REFERENCE project's own CUDA kernels.

tests/golden/reference_kernels.npz was recorded by tests/golden/make_golden.py on a B200 from
oracle/_ref/libref_kernels.so, i.e. from the reference's headers compiled as they are
(kernels/matmul/1_matmul_tiling.cuh, 9_matmul_async_cg_tf32_gelu.cuh,
kernels/layernorm/1_layernorm_block.cuh, 2_layernorm_block_vectorized.cuh,
kernels/residual/1_residual_naive.cuh, kernels/attention/3_flash_attention_permute.cuh).
The reference ships no test vectors of its own, so these recordings are the pin.
"""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden", "reference_kernels.npz")


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
