"""Parity of every C-ABI operator against the CPU oracle on the same seeded inputs (GPU).

Tolerances (frozen from the measured gap between a correct TF32 kernel and the fp64-accumulate
oracle, see the per-test comments):
  encoder, residual          bit-exact
  layernorm / fused          1e-5 absolute on N(0,1) rows
  gelu                       2e-6 absolute
  GEMM, TF32                 relative RMS error <= 1e-3, max-abs <= 6e-3 * sqrt(K/768) on N(0,1) x N(0,0.02)
  attention, TF32            5e-3 absolute on N(0,1) Q/K/V (the tensor core truncates fp32 operands to
                             TF32: |v| * 2^-10 with |v| up to ~4.5); lse 4e-3
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rel_rms(a, b):
    return float(np.sqrt(np.mean((a.astype(np.float64) - b) ** 2)) / (np.sqrt(np.mean(b.astype(np.float64) ** 2)) + 1e-30))


# ------------------------------------------------------------------ memory-bound kernels
@pytest.mark.parametrize("B,T,C", [(4, 64, 768), (2, 64, 1600), (1, 64, 128), (3, 64, 1024), (1, 192, 4096)])
def test_layernorm_matches_oracle(ctx, dev, orc, B, T, C):
    x = orc.fill_normal((B, T, C), 11)
    w = orc.fill_normal((C,), 12, mean=1.0, std=0.1)
    b = orc.fill_normal((C,), 13, std=0.1)
    want, wmean, wrstd = orc.layernorm_forward(x, w, b, precise=True)
    out, mean, rstd = dev.empty((B, T, C)), dev.empty((B, T)), dev.empty((B, T))
    ctx.layernorm_forward(out, mean, rstd, dev.to(x), dev.to(w), dev.to(b), B, T, C)
    assert np.abs(dev.back(out) - want).max() < 1e-5
    assert np.abs(dev.back(mean) - wmean).max() < 1e-6
    assert np.abs(dev.back(rstd) / wrstd - 1).max() < 1e-5


def test_layernorm_null_stats_and_shifted_rows(ctx, dev, orc):
    # mean/rstd may be NULL; rows with a large common offset stress the variance formula
    B, T, C = 2, 64, 768
    x = orc.fill_normal((B, T, C), 21) + 100.0
    w = np.ones(C, np.float32)
    b = np.zeros(C, np.float32)
    want, _, _ = orc.layernorm_forward(x, w, b, precise=True)
    out = dev.empty((B, T, C))
    ctx.layernorm_forward(out, None, None, dev.to(x), dev.to(w), dev.to(b), B, T, C)
    assert np.abs(dev.back(out) - want).max() < 2e-4  # fp32 input resolution at |x|~100 is 7.6e-6 * rstd~1


@pytest.mark.parametrize("B,T,C", [(4, 64, 768), (2, 64, 1600)])
def test_fused_residual_layernorm_matches_oracle(ctx, dev, orc, B, T, C):
    x1 = orc.fill_normal((B, T, C), 31)
    x2 = orc.fill_normal((B, T, C), 32)
    w = orc.fill_normal((C,), 33, mean=1.0, std=0.1)
    b = orc.fill_normal((C,), 34, std=0.1)
    wres, wout, wmean, wrstd = orc.fused_residual_layernorm_forward(x1, x2, w, b, precise=True)
    res, out, mean, rstd = dev.empty((B, T, C)), dev.empty((B, T, C)), dev.empty((B, T)), dev.empty((B, T))
    ctx.fused_residual_layernorm_forward(res, out, mean, rstd, dev.to(x1), dev.to(x2), dev.to(w), dev.to(b), B, T, C)
    assert np.array_equal(dev.back(res), wres)  # one fp32 add
    assert np.abs(dev.back(out) - wout).max() < 1e-5
    assert np.abs(dev.back(mean) - wmean).max() < 1e-6


def test_fused_residual_layernorm_in_place(ctx, dev, orc):
    # res_out aliasing inp1 is how the driver keeps the residual stream
    B, T, C = 2, 64, 768
    x1 = orc.fill_normal((B, T, C), 41)
    x2 = orc.fill_normal((B, T, C), 42)
    w = np.ones(C, np.float32)
    b = np.zeros(C, np.float32)
    wres, wout, _, _ = orc.fused_residual_layernorm_forward(x1, x2, w, b, precise=True)
    d1, out = dev.to(x1), dev.empty((B, T, C))
    ctx.fused_residual_layernorm_forward(d1, out, None, None, d1, dev.to(x2), dev.to(w), dev.to(b), B, T, C)
    assert np.array_equal(dev.back(d1), wres)
    assert np.abs(dev.back(out) - wout).max() < 1e-5


@pytest.mark.parametrize("N", [1, 3, 4, 1000, 768 * 256 + 3])
def test_residual_bit_exact(ctx, dev, orc, N):
    a = orc.fill_normal((N,), 51)
    b = orc.fill_normal((N,), 52)
    npad = (N + 3) // 4 * 4
    da, db, out = dev.to(np.resize(a, npad)), dev.to(np.resize(b, npad)), dev.empty((npad,))
    ctx.residual_forward(out, da, db, N)
    assert np.array_equal(dev.back(out)[:N], orc.residual_forward(a, b))


@pytest.mark.parametrize("N", [5, 4096, 3072 * 256])
def test_gelu_matches_oracle(ctx, dev, orc, N):
    x = orc.fill_normal((N,), 61, std=3.0)
    x[:5] = [0.0, -20.0, 20.0, -1e-8, 100.0][: min(5, N)]
    npad = (N + 3) // 4 * 4
    out = dev.empty((npad,))
    ctx.gelu_forward(out, dev.to(np.resize(x, npad)), N)
    want = orc.gelu_forward(x, precise=True)
    assert np.abs(dev.back(out)[:N] - want).max() < 2e-6 * max(1.0, float(np.abs(want).max()) / 10)


@pytest.mark.parametrize("B,T,C,V", [(4, 64, 768, 50304), (2, 128, 1600, 1024), (1, 64, 128, 7)])
def test_encoder_bit_exact(ctx, dev, orc, B, T, C, V):
    import torch
    wte = orc.fill_normal((V, C), 71, std=0.02)
    wpe = orc.fill_normal((T, C), 72, std=0.02)
    tok = orc.fill_tokens((B, T), 73, vocab=V)
    tok[0, 0], tok[-1, -1] = 0, V - 1  # both ends of the table
    out = dev.empty((B, T, C))
    ctx.encoder_forward(out, dev.to(tok), dev.to(wte), dev.to(wpe), B, T, C)
    assert np.array_equal(dev.back(out), orc.encoder_forward(tok, wte, wpe))
    assert out.dtype == torch.float32


# ------------------------------------------------------------------------------- GEMM
GEMM_SHAPES = [
    # B, T, C(K), OC(N), bias, act, residual
    (1, 128, 64, 64, True, 0, False),        # one tile, two K blocks
    (2, 64, 768, 2304, True, 0, False),      # QKV, c0-sized M
    (4, 64, 768, 768, True, 0, False),       # attn-proj
    (4, 64, 768, 3072, True, 1, False),      # fc + GELU
    (4, 64, 3072, 768, True, 0, True),       # fc-proj + residual
    (2, 64, 768, 50304, False, 0, False),    # lm-head, no bias, ragged last N tile
    (1, 192, 1600, 4800, True, 0, False),    # XL QKV, M not a multiple of 128
    (1, 64, 1600, 6400, True, 1, False),     # XL fc, M < 128
    (1, 64, 100, 36, True, 0, False),        # K not a multiple of 32, tiny N
    (8, 128, 768, 768, True, 0, False),      # several M tiles
    (2, 1024, 128, 4608, True, 1, False),    # wide output: CTA-pair kernel (M = 2048, 18 N tiles of 256)
    (17, 128, 96, 4672, True, 0, True),      # CTA-pair kernel, odd number of 128-row tiles, ragged N tile
]


@pytest.mark.parametrize("B,T,C,OC,has_bias,act,has_res", GEMM_SHAPES)
def test_matmul_tf32_matches_oracle(ctx, dev, orc, B, T, C, OC, has_bias, act, has_res):
    x = orc.fill_normal((B, T, C), 81)
    w = orc.fill_normal((OC, C), 82, std=0.02)
    bias = orc.fill_normal((OC,), 83, std=0.01) if has_bias else None
    res = orc.fill_normal((B, T, OC), 84) if has_res else None
    want = orc.matmul_forward(x, w, bias, act=act, residual=res, precise=True)
    out = dev.full((B, T, OC), float("nan"))
    ctx.matmul_forward(out, dev.to(x), dev.to(w), None if bias is None else dev.to(bias), B, T, C, OC,
                       act=act, residual=None if res is None else dev.to(res))
    got = dev.back(out)
    assert np.isfinite(got).all(), "unwritten or non-finite outputs"
    ref_scale = want - (res if has_res else 0)  # error is relative to the GEMM part
    rr = float(np.sqrt(np.mean((got.astype(np.float64) - want) ** 2)) / np.sqrt(np.mean(ref_scale.astype(np.float64) ** 2)))
    assert rr < 1e-3, f"relative RMS error {rr}"
    assert np.abs(got - want).max() < 6e-3 * max(1.0, (C / 768) ** 0.5)


def test_matmul_linearity_full_size(ctx, dev, orc):
    # size-independent property at the benchmark's row count (M = 8192): f(x1 + x2) = f(x1) + f(x2)
    # up to TF32 rounding, and an oracle spot check on the last rows
    import torch
    B, T, C, OC = 8, 1024, 768, 2304
    x1, x2 = orc.fill_normal((B, T, C), 91), orc.fill_normal((B, T, C), 92)
    w = orc.fill_normal((OC, C), 93, std=0.02)
    dw = dev.to(w)
    outs = []
    for x in (x1, x2, x1 + x2):
        o = dev.empty((B, T, OC))
        ctx.matmul_forward(o, dev.to(x), dw, None, B, T, C, OC)
        ctx.sync_check()
        outs.append(o)
    lin = (outs[0] + outs[1] - outs[2]).abs().max().item()
    assert lin < 8e-3
    want = orc.matmul_forward(x1[-1:, -256:], w, None, precise=True)
    assert np.abs(outs[0][-1:, -256:].cpu().numpy() - want).max() < 6e-3
    assert torch.isfinite(outs[2]).all()


# -------------------------------------------------------------------------- attention
@pytest.mark.parametrize("B,T,NH", [(1, 64, 1), (2, 128, 2), (1, 256, 12), (2, 192, 3), (1, 1024, 2), (1, 384, 25)])
def test_attention_matches_oracle(ctx, dev, orc, B, T, NH):
    C = NH * 64
    qkv = orc.fill_normal((B, T, 3 * C), 101)
    want, wlse = orc.attention_forward(qkv, NH, precise=True)
    out, lse = dev.full((B, T, C), float("nan")), dev.full((B, NH, T), float("nan"))
    d_in = dev.to(qkv)
    ctx.attention_forward(out, None, lse, d_in, B, T, C, NH)
    got = dev.back(out)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() < 5e-3
    assert np.abs(dev.back(lse) - wlse).max() < 4e-3
    assert np.array_equal(d_in.cpu().numpy(), qkv), "inp must not be modified"


def test_attention_without_stats_and_large_scores(ctx, dev, orc):
    # att == NULL; scores far below zero except the diagonal exercise the running-max path
    B, T, NH = 1, 256, 2
    C = NH * 64
    qkv = orc.fill_normal((B, T, 3 * C), 111, std=4.0)
    want, _ = orc.attention_forward(qkv, NH, precise=True)
    out = dev.empty((B, T, C))
    ctx.attention_forward(out, None, None, dev.to(qkv), B, T, C, NH)
    # |s| reaches ~100 here, so TF32 operand rounding moves the softmax weights by a few percent
    assert np.abs(dev.back(out) - want).max() < 0.5
    assert _rel_rms(dev.back(out), want) < 3e-2


# ------------------------------------------------------------------------ error paths
def test_precondition_failures_return_status(ctx, dev, pkg):
    x = dev.empty((1, 64, 768))
    w = dev.empty((768, 768))
    assert ctx.raw("matmul_forward", x, x, w, None, 1, 64, 768, 766, 0, None, 0) == 2      # OC % 4
    assert ctx.raw("matmul_forward", None, x, w, None, 1, 64, 768, 768, 0, None, 0) == 1   # NULL out
    assert ctx.raw("attention_forward", x, None, None, x, 1, 64, 768, 8) == 2              # head size 96
    assert ctx.raw("attention_forward", x, None, None, x, 1, 63, 768, 12) == 2             # T % 64
    assert ctx.raw("layernorm_forward", x, None, None, x, w, w, 1, 64, 770) == 2           # C % 4
    import torch
    mis = torch.empty(64 * 768 + 1, device="cuda")[1:]
    assert ctx.raw("layernorm_forward", x, None, None, mis, w, w, 1, 64, 768) == 3         # misaligned
    ctx.sync_check()


def test_void_shims_run_on_default_stream(ctx, dev, orc, pkg):
    import torch
    B, T, C = 2, 64, 768
    a, b = orc.fill_normal((B * T * C,), 121), orc.fill_normal((B * T * C,), 122)
    da, db, out = dev.to(a), dev.to(b), dev.empty((B * T * C,))
    lib = pkg.lib()
    lib.residual_forward(out.data_ptr(), da.data_ptr(), db.data_ptr(), B * T * C)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), a + b)
    x = orc.fill_normal((B, T, C), 123)
    w = orc.fill_normal((C, C), 124, std=0.02)
    bias = orc.fill_normal((C,), 125, std=0.01)
    o2 = dev.empty((B, T, C))
    dx, dw, dbias = dev.to(x), dev.to(w), dev.to(bias)  # keep the buffers alive across the call
    lib.matmul_forward(o2.data_ptr(), dx.data_ptr(), dw.data_ptr(), dbias.data_ptr(), B, T, C, C)
    torch.cuda.synchronize()
    assert np.abs(o2.cpu().numpy() - orc.matmul_forward(x, w, bias, precise=True)).max() < 6e-3


# --------------------------------------------------------------------- 3xTF32 mode
@pytest.mark.parametrize("B,T,C,OC,has_bias,act,has_res", [
    (2, 64, 768, 2304, True, 0, False),
    (4, 64, 768, 3072, True, 1, False),
    (4, 64, 3072, 768, True, 0, True),
    (1, 192, 1600, 4800, True, 0, False),
    (1, 64, 100, 36, True, 0, False),
    (2, 64, 768, 50304, False, 0, False),
])
def test_matmul_tf32x3_within_1e4_relative(ctx, dev, orc, pkg, B, T, C, OC, has_bias, act, has_res):
    """The three-term split mode: within 1e-4 of the result's magnitude.  What is left at large K
    is the tensor core's own fp32 accumulation (over a thousand chained partial sums), not the
    operand precision."""
    x = orc.fill_normal((B, T, C), 131)
    w = orc.fill_normal((OC, C), 132, std=0.02)
    bias = orc.fill_normal((OC,), 133, std=0.01) if has_bias else None
    res = orc.fill_normal((B, T, OC), 134) if has_res else None
    want = orc.matmul_forward(x, w, bias, act=act, residual=res, precise=True)
    out = dev.full((B, T, OC), float("nan"))
    ctx.matmul_forward(out, dev.to(x), dev.to(w), None if bias is None else dev.to(bias), B, T, C, OC,
                       act=act, residual=None if res is None else dev.to(res), mode=pkg.B200_TF32X3)
    got = dev.back(out)
    assert np.isfinite(got).all()
    scale = float(np.abs(want - (res if has_res else 0)).max())
    assert np.abs(got - want).max() <= 1e-4 * scale, (np.abs(got - want).max(), scale)


@pytest.mark.parametrize("B,T,NH", [(1, 64, 1), (2, 128, 2), (1, 256, 12), (2, 192, 3), (1, 1024, 2)])
def test_attention_x3_matches_oracle(ctx, dev, orc, B, T, NH):
    """Split-operand attention of the 3xTF32 mode: fp32-level agreement with the oracle."""
    C = NH * 64
    qkv = orc.fill_normal((B, T, 3 * C), 141)
    want, wlse = orc.attention_forward(qkv, NH, precise=True)
    out, lse = dev.full((B, T, C), float("nan")), dev.full((B, NH, T), float("nan"))
    scratch = dev.empty((B, T, 3 * C))
    d_in = dev.to(qkv)
    ctx.attention_forward_x3(out, scratch, lse, d_in, B, T, C, NH)
    got = dev.back(out)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() < 2e-5, np.abs(got - want).max()
    assert np.abs(dev.back(lse) - wlse).max() < 2e-5
    assert np.array_equal(d_in.cpu().numpy(), qkv), "inp must not be modified"
    assert ctx.raw("attention_forward_x3", out, None, None, d_in, B, T, C, NH) == 1  # scratch is required


def test_device_wait_that_runs_out_is_reported_and_context_survives(ctx, dev, orc, pkg):
    """Failure detection without harming the GPU: a wait on a barrier that nothing signals gives
    up after its limit, the kernel returns, the host reads B200_ERR_TIMEOUT once, and the same
    context keeps working."""
    import time
    lib = pkg.lib()
    t0 = time.time()
    assert lib.b200_ctx_wait_timeout_probe(ctx._h, 100) == 0
    assert ctx.sync_status() == 6  # B200_ERR_TIMEOUT
    assert 0.05 < time.time() - t0 < 5.0
    assert b"101" in lib.b200_ctx_last_error(ctx._h)
    assert ctx.sync_status() == 0  # reported once, then clear
    a, b = orc.fill_normal((1024,), 1), orc.fill_normal((1024,), 2)
    out = dev.empty((1024,))
    ctx.residual_forward(out, dev.to(a), dev.to(b), 1024)
    assert np.array_equal(dev.back(out), a + b)
    assert lib.b200_ctx_wait_timeout_probe(ctx._h, 0) == 2  # limit out of range
    # the wait on a hand-over word that a peer GPU would write (tensor parallelism over peer memory)
    t0 = time.time()
    assert lib.b200_ctx_peer_wait_probe(ctx._h, 100) == 0
    assert ctx.sync_status() == 6
    assert 0.05 < time.time() - t0 < 5.0
    assert b"105" in lib.b200_ctx_last_error(ctx._h)
    assert ctx.sync_status() == 0


# ------------------------------------------------------------------ bf16 operand GEMM
def _bf16_round(a):
    """fp32 -> nearest bf16 (ties to even), returned as fp32 values and as the 16-bit patterns."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32)
    return (r << 16).view(np.float32).reshape(a.shape), r.astype(np.uint16).reshape(a.shape)


def test_convert_bf16_is_round_to_nearest_even(ctx, dev, orc):
    import torch
    x = orc.fill_normal((4, 1000), 301)
    x[0, :8] = [1.00390625, 1.01171875, -1.00390625, 0.0, 3.0e38, -1e-30, 1.0, 65280.0]  # ties, large, tiny
    out = torch.empty((4, 1000), dtype=torch.int16, device="cuda")
    ctx.convert_bf16(out, dev.to(x), x.size)
    ctx.sync_check()
    _, bits = _bf16_round(x)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), bits)


@pytest.mark.parametrize("B,T,C,OC,has_bias,act,out_h", [
    (1, 128, 64, 64, False, 0, False),
    (2, 192, 768, 2304, True, 0, False),     # qkv shape, ragged M
    (4, 512, 768, 3072, True, 1, True),      # fc + GELU, bf16 out, CTA pairs
    (1, 1000, 3072, 768, True, 0, False),    # fc-proj, M not a multiple of 128
    (1, 320, 776, 200, True, 1, True),       # K tail (776 = 12 * 64 + 8), narrow ragged N, bf16 out
    (2, 1024, 768, 50304, False, 0, False),  # lm-head width, CTA pairs
])
def test_matmul_bf16_matches_oracle_on_rounded_operands(ctx, dev, orc, B, T, C, OC, has_bias, act, out_h):
    """bf16 x bf16 products are exact in fp32, so against the oracle fed the same bf16-rounded
    operands only the accumulation order is left: 2e-5 of the result's magnitude.  A bf16 output
    may differ from the rounded oracle value by one bf16 step where the fp32 value sits on a
    rounding boundary."""
    import torch
    x, xb = _bf16_round(orc.fill_normal((B, T, C), 311))
    w, wb = _bf16_round(orc.fill_normal((OC, C), 312, std=0.02))
    bias = orc.fill_normal((OC,), 313, std=0.01) if has_bias else None
    rows = slice(None) if B * T * OC < 40_000_000 else slice(-300, None)  # oracle on the last rows of the big case
    want = orc.matmul_forward(x.reshape(B * T, C)[rows][None], w, bias, act=act, precise=True)[0]
    d = "cuda"
    d_x = torch.from_numpy(xb.view(np.int16)).to(d)
    d_w = torch.from_numpy(wb.view(np.int16)).to(d)
    out = None if out_h else dev.full((B, T, OC), float("nan"))
    outh = torch.full((B, T, OC), -1, dtype=torch.int16, device=d) if out_h else None
    ctx.matmul_forward_bf16(out, outh, d_x, d_w, None if bias is None else dev.to(bias), B, T, C, OC, act=act)
    ctx.sync_check()
    scale = float(np.abs(want).max())
    if out_h:
        got = (outh.cpu().numpy().view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(B * T, OC)[rows]
        assert np.isfinite(got).all()
        assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -8 + 2e-5 * scale).all()
    else:
        got = dev.back(out).reshape(B * T, OC)[rows]
        assert np.isfinite(dev.back(out)).all(), "unwritten or non-finite outputs"
        assert np.abs(got - want).max() <= 2e-5 * scale, (np.abs(got - want).max(), scale)


# ------------------------------------------------------------------ fp8 (e4m3) operand GEMM
def _e4m3_round(a):
    """fp32 -> nearest e4m3 (1-4-3 bits, bias 7, no infinities; ties to even; values beyond the largest
    finite one, 448, saturate), returned as fp32 values and as the byte patterns."""
    a = np.ascontiguousarray(a, np.float32)
    mag = np.abs(a).astype(np.float64)
    e = np.floor(np.log2(np.maximum(mag, 2.0 ** -20)))
    e = np.maximum(e, -6.0)                       # below 2^-6 the step stays 2^-9 (subnormals)
    step = 2.0 ** (e - 3)
    q = np.minimum(np.round(mag / step) * step, 448.0)   # np.round: half to even
    e2 = np.floor(np.log2(np.maximum(q, 2.0 ** -20)))
    normal = q >= 2.0 ** -6
    expf = np.where(normal, e2 + 7, 0).astype(np.uint8)
    mant = np.where(normal, (q / 2.0 ** np.where(normal, e2, 0) - 1.0) * 8.0, q * 2.0 ** 9).astype(np.uint8)
    bits = (np.signbit(a).astype(np.uint8) << 7) | (expf << 3) | mant
    return np.copysign(q, a).astype(np.float32), bits


def test_quantize_e4m3_is_round_to_nearest_even_and_saturates(ctx, dev, orc):
    import torch
    x = orc.fill_normal((4, 1000), 401) * np.repeat(np.float32([1.0, 30.0, 0.01, 200.0]), 1000).reshape(4, 1000)
    x[0, :16] = [0.0, -0.0, 448.0, 460.0, 500.0, 1e6, -1e6, 2.0 ** -9, 2.0 ** -10, 3 * 2.0 ** -10, 0.0019, 17.0, 19.0, -17.0, 1.0625, 1.1875]
    out = torch.empty((4, 1000), dtype=torch.uint8, device="cuda")
    ctx.quantize_e4m3(out, dev.to(x), x.size, 1.0)
    ctx.sync_check()
    vals, bits = _e4m3_round(x)
    got = out.cpu().numpy()
    assert np.array_equal(got, bits), np.flatnonzero(got.ravel() != bits.ravel())[:10]
    # the byte patterns mean what the helper says they mean (torch's own e4m3 type as a second opinion)
    assert np.array_equal(out.cpu().view(torch.float8_e4m3fn).to(torch.float32).numpy(), vals)
    # a scale is applied before rounding
    ctx.quantize_e4m3(out, dev.to(x), x.size, 64.0)
    ctx.sync_check()
    assert np.array_equal(out.cpu().numpy(), _e4m3_round(x * np.float32(64.0))[1])


@pytest.mark.parametrize("B,T,C,OC,has_bias,act,accumulate", [
    (1, 128, 64, 64, False, 0, False),
    (2, 192, 768, 2304, True, 0, False),      # qkv shape, ragged M
    (4, 512, 768, 3072, True, 1, False),      # fc + GELU
    (1, 1000, 3072, 768, True, 0, False),     # fc-proj, M not a multiple of 128
    (1, 320, 784, 200, True, 1, False),       # K tail (784 = 6 * 128 + 16), narrow ragged N
    (8, 1024, 3072, 768, True, 0, True),      # 8192 rows added onto the output (K slices)
    (8, 1024, 768, 3072, True, 1, False),     # 8192 rows, GELU: left-over tiles in quarter width
])
def test_matmul_fp8_matches_oracle_on_quantised_operands(ctx, dev, orc, B, T, C, OC, has_bias, act, accumulate):
    """Products of e4m3 values are exact in fp32, so against the oracle fed the same quantised
    operands (with the power-of-two scales taken out again) only the accumulation order is left:
    2e-5 of the result's magnitude."""
    import torch
    sx, sw = 2.0, 1024.0
    x, w = orc.fill_normal((B, T, C), 411), orc.fill_normal((OC, C), 412, std=0.02)
    xv, xb = _e4m3_round(x * np.float32(sx))
    wv, wb = _e4m3_round(w * np.float32(sw))
    bias = orc.fill_normal((OC,), 413, std=0.01) if has_bias else None
    rows = slice(None) if B * T * OC < 20_000_000 else slice(-300, None)
    want = orc.matmul_forward((xv / np.float32(sx)).reshape(B * T, C)[rows][None], wv / np.float32(sw), bias, act=act, precise=True)[0]
    res = orc.fill_normal((B, T, OC), 414) if accumulate else None
    out = dev.to(res) if accumulate else dev.full((B, T, OC), float("nan"))
    if accumulate:
        want = want + res.reshape(B * T, OC)[rows]
    ctx.matmul_forward_fp8(out, torch.from_numpy(xb).cuda(), torch.from_numpy(wb).cuda(), None if bias is None else dev.to(bias),
                           B, T, C, OC, act=act, alpha=1.0 / (sx * sw), accumulate=accumulate)
    ctx.sync_check()
    got = dev.back(out).reshape(B * T, OC)[rows]
    assert np.isfinite(dev.back(out)).all(), "unwritten or non-finite outputs"
    scale = float(np.abs(want).max())
    assert np.abs(got - want).max() <= 2e-5 * scale, (np.abs(got - want).max(), scale)


# ------------------------------------------------------------------ split bf16 (bf16x3) GEMM
def _bits_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _split_bf16(a):
    """x -> (hi, lo) bit patterns with hi = bf16(x), lo = bf16(x - hi), as the library defines them."""
    hi_f, hi_b = _bf16_round(a)
    _, lo_b = _bf16_round((np.ascontiguousarray(a, np.float32) - hi_f).astype(np.float32))
    return hi_b, lo_b


def test_split_bf16_matches_its_definition(ctx, dev, orc):
    import torch
    x = orc.fill_normal((3, 1000), 401)
    x[0, :6] = [1.00390625, -1.01171875, 0.0, 3.0e38, -1e-30, 1.0]
    hi = torch.empty((3, 1000), dtype=torch.int16, device="cuda")
    lo = torch.empty((3, 1000), dtype=torch.int16, device="cuda")
    ctx.split_bf16(hi, lo, dev.to(x), x.size)
    ctx.sync_check()
    hb, lb = _split_bf16(x)
    assert np.array_equal(hi.cpu().numpy().view(np.uint16), hb)
    assert np.array_equal(lo.cpu().numpy().view(np.uint16), lb)
    # the two terms carry 16 significant bits of x
    back = _bits_to_f32(hb) + _bits_to_f32(lb)
    ok = np.abs(x) < 1e30
    assert (np.abs(back - x)[ok] <= np.abs(x)[ok] * 2.0 ** -16).all()


@pytest.mark.parametrize("B,T,C,OC,has_bias,act,mode", [
    (1, 128, 64, 64, False, 0, "plain"),
    (2, 192, 768, 2304, True, 0, "plain"),      # ragged M (384 rows), QKV shape
    (4, 64, 768, 768, True, 0, "accumulate"),   # attention projection onto a residual
    (4, 512, 768, 3072, True, 1, "split"),      # fc + GELU, split output feeding the next product
    (1, 1024, 3072, 768, True, 0, "accumulate"),
    (1, 320, 776, 200, True, 1, "split"),       # K tail, narrow ragged N
    (1, 64, 1600, 4800, True, 0, "plain"),      # XL width, M < 128
    (2, 1024, 768, 50304, False, 0, "plain"),   # lm-head width
    (8, 1024, 768, 3072, True, 1, "split"),     # the forward's GELU GEMM: 384 tiles on 74 pairs, left-over tiles in quarter width
    (5, 1000, 768, 3072, True, 0, "plain"),     # 240 tiles: quarter-width left-over tiles again, ragged last row block, fp32 stores
])
def test_matmul_bf16x3_close_to_fp32(ctx, dev, orc, B, T, C, OC, has_bias, act, mode):
    """Split-operand product (hi.hi + hi.lo + lo.hi on the bf16 pipe) against the fp64-accumulate
    oracle on the unsplit fp32 operands: within 1e-4 of the result's magnitude (what is dropped is
    below 2^-16 per operand; at large K the tensor core's own fp32 accumulation is what is left)."""
    import torch
    x = orc.fill_normal((B, T, C), 411)
    w = orc.fill_normal((OC, C), 412, std=0.02)
    bias = orc.fill_normal((OC,), 413, std=0.01) if has_bias else None
    base = orc.fill_normal((B, T, OC), 414) if mode == "accumulate" else None
    rows = slice(None) if B * T * OC < 20_000_000 else slice(-300, None)  # the oracle on the last rows of the big cases
    want = orc.matmul_forward(x.reshape(B * T, C)[rows][None], w, bias, act=act, precise=True)[0]
    d_x = torch.empty((2, B, T, C), dtype=torch.int16, device="cuda")
    ctx.split_bf16(d_x[0], d_x[1], dev.to(x), x.size)
    d_wh = torch.empty((OC, C), dtype=torch.int16, device="cuda")
    d_wl = torch.empty((OC, C), dtype=torch.int16, device="cuda")
    ctx.split_bf16(d_wh, d_wl, dev.to(w), w.size)
    d_bias = None if bias is None else dev.to(bias)
    scale = float(np.abs(want).max())
    if mode == "split":
        outs = torch.full((2, B, T, OC), -1, dtype=torch.int16, device="cuda")
        ctx.matmul_forward_bf16x3(None, outs, d_x, d_wh, d_wl, d_bias, B, T, C, OC, act=act)
        ctx.sync_check()
        bits = outs.cpu().numpy().view(np.uint16)
        got = (_bits_to_f32(bits[0]) + _bits_to_f32(bits[1])).reshape(B * T, OC)[rows]
        assert np.isfinite(got).all()
        # the split output itself keeps 16 bits of each value
        assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -15 + 1e-4 * scale).all()
        # the second plane is small against the first: it only holds what the rounding dropped
        lo_f, hi_f = _bits_to_f32(bits[1]), _bits_to_f32(bits[0])
        assert (np.abs(lo_f) <= np.abs(hi_f) * 2.0 ** -8 + 1e-30).all()
    else:
        out = dev.full((B, T, OC), float("nan")) if base is None else dev.to(base)
        ctx.matmul_forward_bf16x3(out, None, d_x, d_wh, d_wl, d_bias, B, T, C, OC, act=act, accumulate=base is not None)
        got_all = dev.back(out)
        assert np.isfinite(got_all).all(), "unwritten or non-finite outputs"
        got = got_all.reshape(B * T, OC)[rows]
        if base is not None:
            got = got - base.reshape(B * T, OC)[rows]  # one fp32 add: exact up to its rounding
            assert np.abs(got - want).max() <= 1e-4 * scale + 4e-7 * float(np.abs(base).max() + scale)
        else:
            assert np.abs(got - want).max() <= 1e-4 * scale, (np.abs(got - want).max(), scale)
        assert _rel_rms(got, want) < (5e-5 if base is None else 2e-4)


def test_attention_fp16_moves_its_reference_maximum(ctx, dev, orc):
    """The kernel keeps O in tensor memory and only rescales it when a block of keys raises a row's
    maximum by more than 2^8.  On N(0,1) inputs that happens on the first block of a tile only; here
    the keys grow from block to block (x1, x4, x16, x64 per 128 positions, then back down), so that
    the running maximum jumps far beyond the threshold in some blocks, by less in others and falls
    in the rest.  q and k are given as exact fp16 values: what is compared is the softmax and P.V
    machinery, not the 11-bit scores."""
    import torch
    B, T, NH = 2, 768, 2
    C = NH * 64
    qkv = orc.fill_normal((B, T, 3 * C), 171)
    gain = np.float32([1, 4, 16, 64, 8, 2])[np.arange(T) // 128]
    qkv[:, :, C:2 * C] *= gain[None, :, None]
    qkv[:, :, :2 * C] = qkv[:, :, :2 * C].astype(np.float16).astype(np.float32)
    want, wlse = orc.attention_forward(qkv, NH, precise=True)
    planes = torch.empty((2, B, T, 3 * C), dtype=torch.int16, device="cuda")
    ctx.split_fp16(planes[0], planes[1], dev.to(qkv), qkv.size)
    out, lse = dev.full((B, T, C), float("nan")), dev.full((B, NH, T), float("nan"))
    ctx.attention_forward_fp16(out, lse, planes, B, T, C, NH)
    ctx.sync_check()
    got = dev.back(out)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() < 2.5e-3, np.abs(got - want).max()
    assert np.abs(dev.back(lse) - wlse).max() < 2e-3 + 1e-5 * np.abs(wlse).max()


@pytest.mark.parametrize("B,T,NH", [(1, 64, 1), (2, 128, 2), (1, 256, 12), (2, 192, 3), (1, 1024, 2), (1, 384, 25)])
def test_attention_fp16_matches_oracle(ctx, dev, orc, B, T, NH):
    """The attention of the default mode: q, k, v as two fp16 planes, q.k from the hi planes (11 bits,
    rounded to nearest), p.v with both terms of v and p rounded to fp16.  On N(0,1) inputs the scores
    reach |s| ~ 4 and carry 2^-12 relative error, i.e. the output is good to about 1e-3 absolute at
    worst and far better on average: half the TF32 kernel's bound and a tenth of its rms."""
    import torch
    C = NH * 64
    qkv = orc.fill_normal((B, T, 3 * C), 151)
    want, wlse = orc.attention_forward(qkv, NH, precise=True)
    planes = torch.empty((2, B, T, 3 * C), dtype=torch.int16, device="cuda")
    ctx.split_fp16(planes[0], planes[1], dev.to(qkv), qkv.size)
    # the split itself: hi is the nearest fp16, hi + lo carries 21 bits or more
    hi = planes[0].cpu().numpy().view(np.float16).astype(np.float32)
    lo = planes[1].cpu().numpy().view(np.float16).astype(np.float32)
    assert np.array_equal(hi, qkv.astype(np.float16).astype(np.float32))
    assert np.abs(hi + lo - qkv).max() <= 2.0 ** -20 * np.abs(qkv).max()
    out, lse = dev.full((B, T, C), float("nan")), dev.full((B, NH, T), float("nan"))
    ctx.attention_forward_fp16(out, lse, planes, B, T, C, NH)
    got = dev.back(out)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() < 2.5e-3, np.abs(got - want).max()
    assert np.sqrt(np.mean((got - want) ** 2)) < 2e-4
    assert np.abs(dev.back(lse) - wlse).max() < 2e-3
