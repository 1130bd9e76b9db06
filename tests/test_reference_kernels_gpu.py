"""The library's operators against the REFERENCE project's own CUDA kernels, on the same GPU, on the
same inputs, at the sizes of the GPT-2 124M forward (B=8, T=1024).

oracle/_ref/libref_kernels.so holds the reference's kernels compiled from its headers as they are
(oracle/ref_harness.cu lists them with file:line); it is built where a checkout of the reference is
present and travels with the tree.  Where it is missing these tests skip: the oracle tests pin the
same math on the CPU.  The reference kernels run on the default stream and synchronise; the library
runs on the context's stream.

Bars, with the reason for each:
  residual     bit for bit (one fp32 add)
  layernorm    1e-6 of the largest output (measured 2-3e-6 on outputs up to 7; the reference sums in
               shared-memory atomics, in varying order)
  matmul       both feed raw fp32 bits to the tensor cores, which drop the low 13 mantissa bits
               (reference: kernels/matmul/ptx.cuh:51-84), so what differs is the order and rounding of
               the fp32 accumulation: within 1e-8 * K of the largest output (measured 8e-6 at K = 768,
               5e-5 at K = 3072, on outputs of 3-6), against 2-4e-3 of TF32 operand error to the exact product
  attention    both truncate q, k, v and the probabilities to TF32; the exponentials differ
               (__expf there, ex2 on a pre-scaled argument here): 1.5e-3 (measured 6.4e-4, 2.8e-4 relative rms)
"""
import ctypes as C
import os

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B, T = 8, 1024
M = B * T


@pytest.fixture(scope="module")
def ref():
    path = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")
    if not os.path.exists(path):
        pytest.skip("the reference's kernels are not built here (oracle/_ref)")
    return C.CDLL(path)


def _p(t):
    return C.c_void_p(t.data_ptr())


def _randn(shape, seed, std=1.0, mean=0.0):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    t = torch.empty(shape, device="cuda").normal_(mean, std, generator=g)
    torch.cuda.synchronize()  # made on torch's stream; both libraries read it on others
    return t


@pytest.mark.parametrize("K,N,gelu", [(768, 2304, 0), (768, 768, 0), (768, 3072, 1), (3072, 768, 0),
                                       (768, 50304, 0), (1600, 6400, 1)])  # + the lm-head width and the XL GELU GEMM
def test_matmul_equals_reference_tf32_kernel_at_8192_rows(ctx, ref, K, N, gelu):
    """kernels/matmul/9_matmul_async_cg_tf32_gelu.cuh:237-275 against b200_matmul_forward (single TF32 pass,
    raw operands) on the four per-layer GEMM shapes, the lm-head's and one of GPT-2 XL's."""
    import torch
    x, w, bias = _randn((B, T, K), 1), _randn((N, K), 2, std=0.02), _randn((N,), 3, std=0.05)
    want = torch.empty((B, T, N), device="cuda")
    assert ref.ref_matmul_forward_tf32_gelu(_p(want), _p(x), _p(w), _p(bias), B, T, K, N, gelu) == 0
    got = torch.full((B, T, N), float("nan"), device="cuda")
    torch.cuda.synchronize()
    ctx.matmul_forward(got, x, w, bias, B, T, K, N, act=gelu)
    ctx.sync_check()
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    scale = want.abs().max().item()
    assert err <= 1e-8 * K * scale, (err, scale)
    # and the two are far closer to each other than either is to the exact product: same truncated operands
    exact = torch.nn.functional.linear(x[0, :256].double(), w.double(), bias.double())
    if gelu:
        exact = torch.nn.functional.gelu(exact, approximate="tanh")
    tf32_err = (want[0, :256].double() - exact).abs().max().item()
    assert err < 0.05 * tf32_err, (err, tf32_err)


def test_attention_equals_reference_flash_kernel_b8_t1024(ctx, ref):
    """kernels/attention/3_flash_attention_permute.cuh:346-355 against b200_attention_forward (TF32 kernel),
    B=8, T=1024, NH=12 on the packed QKV buffer."""
    import torch
    NH, Cc = 12, 768
    qkv = _randn((B, T, 3 * Cc), 11)
    want = torch.empty((B, T, Cc), device="cuda")
    assert ref.ref_flash_attention_permute_forward(_p(want), _p(qkv), B, T, Cc, NH) == 0
    got = torch.full((B, T, Cc), float("nan"), device="cuda")
    lse = torch.empty((B, NH, T), device="cuda")
    torch.cuda.synchronize()
    ctx.attention_forward(got, None, lse, qkv, B, T, Cc, NH)
    ctx.sync_check()
    assert torch.isfinite(got).all()
    assert (got - want).abs().max().item() < 1.5e-3
    assert ((got - want).double().pow(2).mean().sqrt() / want.double().pow(2).mean().sqrt()).item() < 5e-4


@pytest.mark.parametrize("Cc", [768, 1600])
@pytest.mark.parametrize("which", ["block", "vectorized"])
def test_layernorm_equals_reference_kernels_at_8192_rows(ctx, ref, Cc, which):
    """kernels/layernorm/1_layernorm_block.cuh:63 and 2_layernorm_block_vectorized.cuh:74."""
    import torch
    x = _randn((B, T, Cc), 21, std=1.5, mean=0.3)
    w, b = _randn((Cc,), 22, std=0.2, mean=1.0), _randn((Cc,), 23, std=0.2)
    want, mean_w, rstd_w = torch.empty((B, T, Cc), device="cuda"), torch.empty(M, device="cuda"), torch.empty(M, device="cuda")
    fn = ref.ref_layernorm_forward_block if which == "block" else ref.ref_layernorm_forward_block_vectorized
    assert fn(_p(want), _p(mean_w), _p(rstd_w), _p(x), _p(w), _p(b), B, T, Cc) == 0
    got, mean_g, rstd_g = torch.full((B, T, Cc), float("nan"), device="cuda"), torch.empty((B, T), device="cuda"), torch.empty((B, T), device="cuda")
    torch.cuda.synchronize()
    ctx.layernorm_forward(got, mean_g, rstd_g, x, w, b, B, T, Cc)
    ctx.sync_check()
    assert (got - want).abs().max().item() < 1e-6 * max(1.0, want.abs().max().item())
    assert (mean_g.reshape(-1) - mean_w).abs().max().item() < 1e-6
    assert (rstd_g.reshape(-1) / rstd_w - 1).abs().max().item() < 3e-6


def test_residual_equals_reference_kernel_bitwise(ctx, ref):
    """kernels/residual/1_residual_naive.cuh:15 at the residual stream's size."""
    import torch
    n = M * 768
    a, b2 = _randn((n,), 31), _randn((n,), 32)
    want = torch.empty(n, device="cuda")
    assert ref.ref_residual_forward_naive(_p(want), _p(a), _p(b2), n) == 0
    got = torch.full((n,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    ctx.residual_forward(got, a, b2, n)
    ctx.sync_check()
    assert torch.equal(got, want)
