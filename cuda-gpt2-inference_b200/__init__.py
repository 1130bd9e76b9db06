"""B200-native GPT-2 forward engine: Python host side over the C ABI of libb200gpt2.so.

The directory name carries a hyphen, so load it with
``importlib.util.spec_from_file_location("cuda_gpt2_inference_b200", ".../__init__.py")``
(see ``__graft_entry__.load_package``).

The functions mirror the reference project's host wrappers one for one - same names, same
argument order, device buffers owned by the caller, nothing allocated by the callee
(GJ0407790/CUDA-GPT2-Inference: kernels/matmul/1_matmul_tiling.cuh:57,
kernels/attention/3_flash_attention_permute.cuh:346, kernels/layernorm/1_layernorm_block.cuh:63,
kernels/fused_residual_layernorm/fused_residual_layernorm.cuh:88, kernels/residual/1_residual_naive.cuh:15).
Buffers are torch CUDA tensors (fp32 / int32, contiguous); torch is used only for device
memory and streams.  There is no CPU fallback: every call goes through the CUDA library and
raises if it is missing or if the call returns a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200gpt2.so")

B200_OK = 0
(B200_ERR_NULL, B200_ERR_SHAPE, B200_ERR_ALIGN, B200_ERR_CUDA, B200_ERR_DEVICE, B200_ERR_TIMEOUT,
 B200_ERR_STATE, B200_ERR_LIMIT) = range(1, 9)
B200_TF32, B200_TF32X3, B200_BF16, B200_BF16X3 = 0, 1, 2, 3
ACT_NONE, ACT_GELU = 0, 1

EXPORTS = (
    "b200_ctx_create", "b200_ctx_destroy", "b200_ctx_set_stream", "b200_ctx_sync_check",
    "b200_ctx_launch_count", "b200_ctx_reset_launch_count", "b200_status_string",
    "b200_ctx_last_error", "b200_ctx_wait_timeout_probe", "b200_ctx_peer_wait_probe",
    "b200_matmul_forward", "b200_matmul_forward_bf16", "b200_convert_bf16", "b200_matmul_forward_bf16x3", "b200_split_bf16",
    "b200_matmul_forward_fp8", "b200_quantize_e4m3", "b200_gpt2_tp_peer_export", "b200_gpt2_tp_peer_connect", "b200_gpt2_tp_peer_enable",
    "b200_gpt2_tp_sp_export", "b200_gpt2_tp_sp_connect", "b200_gpt2_tp_sp_enable",
    "b200_gpt2_set_attention_mode", "b200_attention_forward", "b200_attention_forward_x3", "b200_attention_forward_fp16", "b200_split_fp16", "b200_layernorm_forward",
    "b200_fused_residual_layernorm_forward", "b200_residual_forward", "b200_gelu_forward",
    "b200_encoder_forward",
    "matmul_forward", "matmul_forward_gelu", "attention_forward", "layernorm_forward",
    "fused_residual_layernorm_forward", "fused_residual_layernorm", "residual_forward",
    "gelu_forward", "encoder_forward",
    "b200_gpt2_param_offsets", "b200_gpt2_create", "b200_gpt2_destroy", "b200_gpt2_params",
    "b200_gpt2_load_params_host", "b200_gpt2_load_params_file", "b200_gpt2_set_options", "b200_gpt2_forward", "b200_gpt2_forward_sample",
    "b200_gpt2_logits", "b200_gpt2_forward_host", "b200_gpt2_forward_host_enqueue", "b200_gpt2_forward_host_wait", "b200_gpt2_activation",
    "b200_gpt2_set_profile", "b200_gpt2_read_profile",
    "b200_gpt2_forward_static", "b200_gpt2_static_prepare",
    "b200_gpt2_enable_kv_cache", "b200_gpt2_prefill", "b200_gpt2_decode_step", "b200_gpt2_decode_step_host", "b200_gpt2_generate_greedy", "b200_gpt2_generate", "b200_sample_rows",
    "b200_gpt2_create_tp", "b200_gpt2_set_allreduce", "b200_gpt2_set_tp_overlap", "b200_gpt2_param_offsets_tp", "b200_gpt2_shard_params_host",
)

# Arithmetic modes of the forward as keyword arguments of GPT2.set_options
MODES = {
    "tf32": dict(round_operands=1, gemm_mode=B200_TF32, lmhead_mode=B200_TF32, attention_mode=-1),
    "bf16x3": dict(round_operands=1, gemm_mode=B200_BF16X3, lmhead_mode=B200_BF16X3, attention_mode=-1),
    "bf16x3_att_tf32": dict(round_operands=1, gemm_mode=B200_BF16X3, lmhead_mode=B200_BF16X3, attention_mode=B200_TF32),
    "bf16x3_lm_tf32": dict(round_operands=1, gemm_mode=B200_BF16X3, lmhead_mode=B200_TF32, attention_mode=-1),
    "tf32x3": dict(round_operands=0, gemm_mode=B200_TF32X3, lmhead_mode=B200_TF32X3, attention_mode=-1),
    "bf16": dict(round_operands=1, gemm_mode=B200_BF16, lmhead_mode=B200_BF16, attention_mode=-1),
}
MODE_NOTES = {
    "tf32": "fp32 storage, single-pass TF32 tensor-core GEMMs (tcgen05 kind::tf32) on round-to-nearest operands, TF32 attention",
    "bf16x3": "fp32 storage, GEMM operands split into two bf16 terms (16 significant bits), three kind::f16 products per K step, "
              "fp32 accumulation; attention on fp16 planes of q, k, v (q.k one product, p.v two)",
    "bf16x3_att_tf32": "bf16x3 GEMMs with the single-pass TF32 attention kernel",
    "bf16x3_lm_tf32": "bf16x3 GEMMs and fp16 attention in the blocks, the lm-head as one TF32 pass on round-to-nearest operands",
    "tf32x3": "3xTF32 GEMMs and attention (three kind::tf32 products per K step)",
    "bf16": "bf16 GEMM operands (reduced precision; not comparable with the fp32-level modes)",
}
DEFAULT_MODE_NAME = "bf16x3"  # what b200_gpt2_create and b200_gpt2_create_tp set

STATIC_MAX_TOKEN_CHANNELS = 196608  # B*T*C limit of b200_gpt2_forward_static

PROF_NAMES = ("encoder", "layernorm", "gemm_qkv", "attention", "gemm_attproj", "fused_residual_layernorm",
              "gemm_fc", "gemm_fcproj", "gemm_lmhead", "allreduce")

ALLREDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p)

_lib = None


class B200Error(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Loads libb200gpt2.so; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}`")
        l = C.CDLL(LIB_PATH)
        vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
        l.b200_ctx_create.argtypes = [C.POINTER(vp), i, vp]
        l.b200_ctx_destroy.argtypes = [vp]
        l.b200_ctx_set_stream.argtypes = [vp, vp]
        l.b200_ctx_sync_check.argtypes = [vp]
        l.b200_ctx_wait_timeout_probe.argtypes = [vp, i]
        l.b200_ctx_peer_wait_probe.argtypes = [vp, i]
        l.b200_ctx_launch_count.argtypes = [vp]
        l.b200_ctx_launch_count.restype = C.c_uint64
        l.b200_ctx_reset_launch_count.argtypes = [vp]
        l.b200_ctx_reset_launch_count.restype = None
        l.b200_status_string.argtypes = [i]
        l.b200_status_string.restype = C.c_char_p
        l.b200_ctx_last_error.argtypes = [vp]
        l.b200_ctx_last_error.restype = C.c_char_p
        l.b200_matmul_forward.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, vp, i]
        l.b200_matmul_forward_bf16.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i]
        l.b200_convert_bf16.argtypes = [vp, vp, vp, sz]
        l.b200_matmul_forward_bf16x3.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i]
        l.b200_split_bf16.argtypes = [vp, vp, vp, vp, sz]
        l.b200_matmul_forward_fp8.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, C.c_float, i]
        l.b200_quantize_e4m3.argtypes = [vp, vp, vp, sz, C.c_float]
        l.b200_gpt2_tp_peer_export.argtypes = [vp, vp]
        l.b200_gpt2_tp_peer_connect.argtypes = [vp, vp]
        l.b200_gpt2_tp_peer_enable.argtypes = [vp, i]
        l.b200_gpt2_tp_sp_export.argtypes = [vp, vp]
        l.b200_gpt2_tp_sp_connect.argtypes = [vp, vp]
        l.b200_gpt2_tp_sp_enable.argtypes = [vp, i]
        l.b200_gpt2_set_attention_mode.argtypes = [vp, i]
        l.b200_attention_forward.argtypes = [vp, vp, vp, vp, vp, i, i, i, i]
        l.b200_attention_forward_x3.argtypes = [vp, vp, vp, vp, vp, i, i, i, i]
        l.b200_attention_forward_fp16.argtypes = [vp, vp, vp, vp, i, i, i, i]
        l.b200_split_fp16.argtypes = [vp, vp, vp, vp, sz]
        l.b200_layernorm_forward.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i]
        l.b200_fused_residual_layernorm_forward.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i]
        l.b200_residual_forward.argtypes = [vp, vp, vp, vp, sz]
        l.b200_gelu_forward.argtypes = [vp, vp, vp, sz]
        l.b200_encoder_forward.argtypes = [vp, vp, vp, vp, vp, i, i, i]
        for name, at in (("matmul_forward", [vp, vp, vp, vp, i, i, i, i]),
                         ("matmul_forward_gelu", [vp, vp, vp, vp, i, i, i, i, i]),
                         ("attention_forward", [vp, vp, vp, vp, i, i, i, i]),
                         ("layernorm_forward", [vp, vp, vp, vp, vp, vp, i, i, i]),
                         ("fused_residual_layernorm_forward", [vp] * 8 + [i, i, i]),
                         ("fused_residual_layernorm", [vp] * 8 + [i, i, i]),
                         ("residual_forward", [vp, vp, vp, i]),
                         ("gelu_forward", [vp, vp, i]),
                         ("encoder_forward", [vp, vp, vp, vp, i, i, i])):
            f = getattr(l, name)
            f.argtypes = at
            f.restype = None
        l.b200_gpt2_param_offsets.argtypes = [vp, C.POINTER(sz)]
        l.b200_gpt2_param_offsets.restype = sz
        l.b200_gpt2_create.argtypes = [C.POINTER(vp), vp, vp, i, i]
        l.b200_gpt2_destroy.argtypes = [vp]
        l.b200_gpt2_params.argtypes = [vp]
        l.b200_gpt2_params.restype = vp
        l.b200_gpt2_load_params_host.argtypes = [vp, vp, sz]
        l.b200_gpt2_load_params_file.argtypes = [vp, C.c_char_p, sz]
        l.b200_gpt2_set_options.argtypes = [vp, i, i, i, i]
        l.b200_gpt2_forward.argtypes = [vp, vp, i, i]
        l.b200_gpt2_forward_sample.argtypes = [vp, vp, i, i, C.c_float, C.c_uint, vp, vp, i]
        l.b200_gpt2_logits.argtypes = [vp]
        l.b200_gpt2_logits.restype = vp
        l.b200_gpt2_forward_host.argtypes = [vp, vp, i, i, vp, vp, vp]
        l.b200_gpt2_forward_host_enqueue.argtypes = [vp, vp, i, i, vp, vp, vp, i]
        l.b200_gpt2_forward_host_wait.argtypes = [vp, i]
        l.b200_gpt2_activation.argtypes = [vp, C.c_char_p]
        l.b200_gpt2_activation.restype = vp
        l.b200_gpt2_set_profile.argtypes = [vp, i]
        l.b200_gpt2_read_profile.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(C.c_long)]
        l.b200_gpt2_forward_static.argtypes = [vp, vp, vp, vp, i, i, vp]
        l.b200_gpt2_static_prepare.argtypes = [vp]
        l.b200_gpt2_enable_kv_cache.argtypes = [vp]
        l.b200_gpt2_prefill.argtypes = [vp, vp, i, i]
        l.b200_gpt2_decode_step.argtypes = [vp, vp, i, i]
        l.b200_gpt2_decode_step_host.argtypes = [vp, vp, i, i, vp, vp]
        l.b200_gpt2_generate_greedy.argtypes = [vp, vp, i, i, i, vp]
        l.b200_gpt2_generate.argtypes = [vp, vp, i, i, i, C.c_float, i, C.c_float, C.c_uint, vp]
        l.b200_sample_rows.argtypes = [vp, vp, vp, i, i, i, C.c_float, i, C.c_float, C.c_uint, C.c_uint]
        l.b200_gpt2_create_tp.argtypes = [C.POINTER(vp), vp, vp, i, i, i, i]
        l.b200_gpt2_set_allreduce.argtypes = [vp, ALLREDUCE_FN, vp]
        l.b200_gpt2_set_tp_overlap.argtypes = [vp, i, i]
        l.b200_gpt2_param_offsets_tp.argtypes = [vp, i, i, C.POINTER(sz)]
        l.b200_gpt2_param_offsets_tp.restype = sz
        l.b200_gpt2_shard_params_host.argtypes = [vp, i, i, vp, vp]
        _lib = l
    return _lib


def _ptr(t):
    """Device (or host) address of a tensor / numpy array / None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        if not t.is_contiguous():
            raise B200Error("tensor must be contiguous")
        return C.c_void_p(t.data_ptr())
    return C.c_void_p(t.ctypes.data)


class Context:
    """One context per GPU / host thread: owns the stream binding and the device status word."""

    def __init__(self, device: int = 0, stream=None):
        self._h = C.c_void_p()
        self.device = device
        handle = None
        if stream is not None:
            handle = C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))
        st = lib().b200_ctx_create(C.byref(self._h), device, handle)
        if st != B200_OK:
            raise B200Error(f"b200_ctx_create: {lib().b200_status_string(st).decode()}")

    def check(self, st: int, what: str):
        if st != B200_OK:
            msg = lib().b200_status_string(st).decode()
            extra = lib().b200_ctx_last_error(self._h).decode()
            raise B200Error(f"{what}: {msg}" + (f" ({extra})" if extra else ""))

    def status(self, st: int) -> int:
        return st

    def set_stream(self, stream):
        handle = None if stream is None else C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))
        self.check(lib().b200_ctx_set_stream(self._h, handle), "set_stream")

    def sync_check(self):
        self.check(lib().b200_ctx_sync_check(self._h), "sync_check")

    def sync_status(self) -> int:
        return lib().b200_ctx_sync_check(self._h)

    @property
    def launches(self) -> int:
        return int(lib().b200_ctx_launch_count(self._h))

    def reset_launches(self):
        lib().b200_ctx_reset_launch_count(self._h)

    def close(self):
        if self._h:
            lib().b200_ctx_destroy(self._h)
            self._h = C.c_void_p()

    # ---- operators: reference argument order, status-checked ---------------------------
    def matmul_forward(self, out, inp, weight, bias, B, T, Cc, OC, act=ACT_NONE, residual=None, mode=B200_TF32):
        self.check(lib().b200_matmul_forward(self._h, _ptr(out), _ptr(inp), _ptr(weight), _ptr(bias), B, T, Cc, OC,
                                             act, _ptr(residual), mode), "matmul_forward")

    def matmul_forward_bf16(self, out, out_bf16, inp, weight, bias, B, T, Cc, OC, act=ACT_NONE):
        """inp / weight (and out_bf16, if given) hold bf16 elements; out is fp32."""
        self.check(lib().b200_matmul_forward_bf16(self._h, _ptr(out), _ptr(out_bf16), _ptr(inp), _ptr(weight), _ptr(bias),
                                                  B, T, Cc, OC, act), "matmul_forward_bf16")

    def convert_bf16(self, out, inp, n):
        self.check(lib().b200_convert_bf16(self._h, _ptr(out), _ptr(inp), n), "convert_bf16")

    def split_bf16(self, hi, lo, inp, n):
        """hi = bf16(inp), lo = bf16(inp - hi)."""
        self.check(lib().b200_split_bf16(self._h, _ptr(hi), _ptr(lo), _ptr(inp), n), "split_bf16")

    def matmul_forward_bf16x3(self, out, out_split, inp_split, weight_hi, weight_lo, bias, B, T, Cc, OC, act=ACT_NONE,
                              accumulate=False):
        """inp_split: bf16 [2,B,T,C] (hi plane, lo plane); weight_hi / weight_lo bf16 [OC,C]; out fp32 or
        out_split bf16 [2,B,T,OC]."""
        self.check(lib().b200_matmul_forward_bf16x3(self._h, _ptr(out), _ptr(out_split), _ptr(inp_split), _ptr(weight_hi),
                                                    _ptr(weight_lo), _ptr(bias), B, T, Cc, OC, act, int(accumulate)),
                   "matmul_forward_bf16x3")

    def quantize_e4m3(self, out, inp, n, scale=1.0):
        """out (uint8) = e4m3(inp * scale), round to nearest even, saturating at 448."""
        self.check(lib().b200_quantize_e4m3(self._h, _ptr(out), _ptr(inp), n, float(scale)), "quantize_e4m3")

    def matmul_forward_fp8(self, out, inp_q, weight_q, bias, B, T, Cc, OC, act=ACT_NONE, alpha=1.0, accumulate=False):
        """inp_q [B,T,C] and weight_q [OC,C] hold e4m3 bytes; out (fp32) = act(alpha * inp_q . weight_q^T + bias)."""
        self.check(lib().b200_matmul_forward_fp8(self._h, _ptr(out), _ptr(inp_q), _ptr(weight_q), _ptr(bias), B, T, Cc, OC, act,
                                                 float(alpha), int(accumulate)), "matmul_forward_fp8")

    def sample_rows(self, out, logits, M, V, ld, temperature, seed, stream0, top_k=0, top_p=0.0):
        self.check(lib().b200_sample_rows(self._h, _ptr(out), _ptr(logits), M, V, ld, float(temperature), int(top_k), float(top_p),
                                          int(seed) & 0xFFFFFFFF, int(stream0) & 0xFFFFFFFF), "sample_rows")

    def attention_forward(self, out, qkvr, att, inp, B, T, Cc, NH):
        self.check(lib().b200_attention_forward(self._h, _ptr(out), _ptr(qkvr), _ptr(att), _ptr(inp), B, T, Cc, NH),
                   "attention_forward")

    def attention_forward_x3(self, out, qkvr, att, inp, B, T, Cc, NH):
        """3xTF32 attention; qkvr ([B,T,3C] scratch) is required."""
        self.check(lib().b200_attention_forward_x3(self._h, _ptr(out), _ptr(qkvr), _ptr(att), _ptr(inp), B, T, Cc, NH),
                   "attention_forward_x3")

    def attention_forward_fp16(self, out, att, inp_split, B, T, Cc, NH):
        """fp16 attention; inp_split: fp16 [2,B,T,3C] (hi plane, lo plane)."""
        self.check(lib().b200_attention_forward_fp16(self._h, _ptr(out), _ptr(att), _ptr(inp_split), B, T, Cc, NH),
                   "attention_forward_fp16")

    def split_fp16(self, hi, lo, inp, n):
        """hi = fp16(inp), lo = fp16(inp - hi)."""
        self.check(lib().b200_split_fp16(self._h, _ptr(hi), _ptr(lo), _ptr(inp), n), "split_fp16")

    def layernorm_forward(self, out, mean, rstd, inp, weight, bias, B, T, Cc):
        self.check(lib().b200_layernorm_forward(self._h, _ptr(out), _ptr(mean), _ptr(rstd), _ptr(inp), _ptr(weight),
                                                _ptr(bias), B, T, Cc), "layernorm_forward")

    def fused_residual_layernorm_forward(self, res_out, layernorm_out, mean, rstd, inp1, inp2, weight, bias, B, T, Cc):
        self.check(lib().b200_fused_residual_layernorm_forward(self._h, _ptr(res_out), _ptr(layernorm_out), _ptr(mean),
                                                               _ptr(rstd), _ptr(inp1), _ptr(inp2), _ptr(weight),
                                                               _ptr(bias), B, T, Cc), "fused_residual_layernorm_forward")

    def residual_forward(self, out, inp1, inp2, N):
        self.check(lib().b200_residual_forward(self._h, _ptr(out), _ptr(inp1), _ptr(inp2), N), "residual_forward")

    def gelu_forward(self, out, inp, N):
        self.check(lib().b200_gelu_forward(self._h, _ptr(out), _ptr(inp), N), "gelu_forward")

    def encoder_forward(self, out, inp, wte, wpe, B, T, Cc):
        self.check(lib().b200_encoder_forward(self._h, _ptr(out), _ptr(inp), _ptr(wte), _ptr(wpe), B, T, Cc),
                   "encoder_forward")

    def raw(self, name: str, *args) -> int:
        """Calls b200_<name>(ctx, ...) and returns the status without raising (for error-path tests)."""
        return getattr(lib(), "b200_" + name)(self._h, *[_ptr(a) if (a is None or hasattr(a, "data_ptr")) else a for a in args])


class GPT2ConfigC(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("max_seq_len", "vocab_size", "padded_vocab_size",
                                       "num_layers", "num_heads", "channels")]


@dataclass(frozen=True)
class GPT2Config:
    max_seq_len: int = 1024
    vocab_size: int = 50257
    padded_vocab_size: int = 50304
    num_layers: int = 12
    num_heads: int = 12
    channels: int = 768

    def c(self) -> GPT2ConfigC:
        return GPT2ConfigC(self.max_seq_len, self.vocab_size, self.padded_vocab_size,
                           self.num_layers, self.num_heads, self.channels)

    def num_params(self) -> int:
        return param_offsets(self)[16]

    def flops_per_token(self, T: int) -> float:
        """Forward FLOP per token at sequence length T: GEMMs 2*K*N each, causal-exact attention."""
        Cc, L, Vp = self.channels, self.num_layers, self.padded_vocab_size
        gemm = 2.0 * (Cc * 3 * Cc + Cc * Cc + Cc * 4 * Cc + 4 * Cc * Cc) * L + 2.0 * Cc * Vp
        att = 4.0 * 64 * (T + 1) / 2 * self.num_heads * L
        return gemm + att


GPT2_124M = GPT2Config()
GPT2_XL = GPT2Config(num_layers=48, num_heads=25, channels=1600)

PARAM_NAMES = ("wte", "wpe", "ln1w", "ln1b", "qkvw", "qkvb", "attprojw", "attprojb",
               "ln2w", "ln2b", "fcw", "fcb", "fcprojw", "fcprojb", "lnfw", "lnfb")


def param_offsets(cfg: GPT2Config) -> list[int]:
    """Offsets (in floats) of the 16 parameter tensors; pure host arithmetic, same as the C side."""
    Cc, L, Vp, mT = cfg.channels, cfg.num_layers, cfg.padded_vocab_size, cfg.max_seq_len
    sizes = [Vp * Cc, mT * Cc, L * Cc, L * Cc, L * 3 * Cc * Cc, L * 3 * Cc, L * Cc * Cc, L * Cc,
             L * Cc, L * Cc, L * 4 * Cc * Cc, L * 4 * Cc, L * Cc * 4 * Cc, L * Cc, Cc, Cc]
    offs = [0]
    for s in sizes:
        offs.append(offs[-1] + s)
    return offs


def shard_batch(B: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous batch shard [start, stop) of rank `rank`: sequences are independent, so the
    forward needs no collective.  Earlier ranks take the remainder."""
    if world_size <= 0 or not (0 <= rank < world_size) or B < 0:
        raise ValueError("bad shard arguments")
    base, rem = divmod(B, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def tp_heads(num_heads: int, tp_size: int, tp_rank: int) -> tuple[int, int]:
    """(first head, number of heads) of a tensor-parallel rank: NH // n each, the first NH % n
    ranks one more."""
    base, rem = divmod(num_heads, tp_size)
    return tp_rank * base + min(tp_rank, rem), base + (1 if tp_rank < rem else 0)


def param_offsets_tp(cfg: GPT2Config, tp_size: int, tp_rank: int) -> list[int]:
    """Offsets of the 16 tensors in a tensor-parallel rank's local parameter array."""
    offs = (C.c_size_t * 17)()
    cc = cfg.c()
    if lib().b200_gpt2_param_offsets_tp(C.byref(cc), tp_size, tp_rank, offs) == 0:
        raise ValueError("model cannot be split this way")
    return [int(o) for o in offs]


def shard_params(cfg: GPT2Config, tp_size: int, tp_rank: int, full_params):
    """Cuts a tensor-parallel rank's parameters out of a full host parameter array (numpy)."""
    import numpy as np
    local = np.empty(param_offsets_tp(cfg, tp_size, tp_rank)[16], dtype=np.float32)
    cc = cfg.c()
    st = lib().b200_gpt2_shard_params_host(C.byref(cc), tp_size, tp_rank, _ptr(full_params), _ptr(local))
    if st != B200_OK:
        raise B200Error(f"shard_params: {lib().b200_status_string(st).decode()}")
    return local


def shard_params_torch(cfg: GPT2Config, tp_size: int, tp_rank: int, full):
    """The same cut as shard_params on a flat CUDA tensor of the full parameters (no host round trip)."""
    import torch
    fo, lo = param_offsets(cfg), param_offsets_tp(cfg, tp_size, tp_rank)
    Cc, L = cfg.channels, cfg.num_layers
    h0, nh = tp_heads(cfg.num_heads, tp_size, tp_rank)
    A, a0 = nh * 64, h0 * 64
    F = 4 * Cc // tp_size
    f0 = tp_rank * F
    local = torch.empty(lo[16], dtype=torch.float32, device=full.device)
    fv = lambda i, *shape: full[fo[i]:fo[i + 1]].view(*shape)
    lv = lambda i, *shape: local[lo[i]:lo[i + 1]].view(*shape)
    for t in (0, 1, 2, 3, 8, 9, 14, 15):  # wte, wpe and the layernorm tensors are replicated
        local[lo[t]:lo[t + 1]] = full[fo[t]:fo[t + 1]]
    lv(4, L, 3, A, Cc).copy_(fv(4, L, 3, Cc, Cc)[:, :, a0:a0 + A, :])   # q, k, v rows of the local heads
    lv(5, L, 3, A).copy_(fv(5, L, 3, Cc)[:, :, a0:a0 + A])
    lv(6, L, Cc, A).copy_(fv(6, L, Cc, Cc)[:, :, a0:a0 + A])            # input columns of the two projections
    lv(12, L, Cc, F).copy_(fv(12, L, Cc, 4 * Cc)[:, :, f0:f0 + F])
    lv(10, L, F, Cc).copy_(fv(10, L, 4 * Cc, Cc)[:, f0:f0 + F, :])
    lv(11, L, F).copy_(fv(11, L, 4 * Cc)[:, f0:f0 + F])
    for t in (7, 13):  # the projection biases are added once: by rank 0
        if tp_rank == 0:
            lv(t, L, Cc).copy_(fv(t, L, Cc))
        else:
            lv(t, L, Cc).zero_()
    return local


class GPT2:
    """gpt2_forward driver (C++ inside the library).  Allocates parameters and one reusable set
    of activations for up to max_B x max_T tokens.  With tp_size > 1 this is one rank of a
    tensor-parallel group: load shard_params(...) and set an all-reduce (set_allreduce_torch)."""

    def __init__(self, ctx: Context, cfg: GPT2Config, max_B: int, max_T: int, tp_size: int = 1, tp_rank: int = 0):
        self.ctx, self.cfg, self.max_B, self.max_T = ctx, cfg, max_B, max_T
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self._h = C.c_void_p()
        self._allreduce_cb = None
        cc = cfg.c()
        ctx.check(lib().b200_gpt2_create_tp(C.byref(self._h), ctx._h, C.byref(cc), max_B, max_T, tp_size, tp_rank),
                  "gpt2_create")

    @property
    def logits_width(self) -> int:
        Vp = self.cfg.padded_vocab_size
        return Vp // self.tp_size if (Vp % self.tp_size == 0 and (Vp // self.tp_size) % 4 == 0) else Vp

    def num_local_params(self) -> int:
        return param_offsets_tp(self.cfg, self.tp_size, self.tp_rank)[16]

    def set_allreduce_torch(self, torch_stream=None, group=None):
        """Uses torch.distributed (NCCL) for the one all-reduce per attention / MLP block.  The
        library names the stream every all-reduce has to be ordered on (its compute stream or its
        communication stream); torch_stream is accepted for compatibility and ignored."""
        import torch
        import torch.distributed as dist
        dev = self.ctx.device
        streams = {}

        def _cb(user, buf, count, stream):
            try:
                key = int(stream or 0)
                if key not in streams:
                    streams[key] = torch.cuda.ExternalStream(key, device=dev) if key else torch.cuda.default_stream(dev)
                t = _view_device(int(buf), (int(count),), torch.float32, dev)
                with torch.cuda.stream(streams[key]):
                    dist.all_reduce(t, group=group)
                return 0
            except Exception:  # the C side turns this into B200_ERR_CUDA
                return 1

        self._allreduce_cb = ALLREDUCE_FN(_cb)  # keep the trampoline alive
        self.ctx.check(lib().b200_gpt2_set_allreduce(self._h, self._allreduce_cb, None), "set_allreduce")

    def set_tp_overlap(self, chunks: int = 1, reserve_sms: int = 0):
        """Row chunks of a tensor-parallel projection and the SMs its later chunks leave to the all-reduce kernels."""
        self.ctx.check(lib().b200_gpt2_set_tp_overlap(self._h, int(chunks), int(reserve_sms)), "set_tp_overlap")

    def connect_tp_peer(self, group=None):
        """Two-way tensor parallelism over peer memory instead of all-reduces: exchanges the CUDA IPC
        handles of the receive buffers with the other rank of the (two-rank) group through
        torch.distributed and switches the hand-over on.  Collective: both ranks call it, and either
        both end up connected or both raise."""
        import torch
        import torch.distributed as dist
        if dist.get_world_size(group) != 2:
            raise B200Error("connect_tp_peer needs a group of two ranks")
        dev = f"cuda:{self.ctx.device}"

        def both(ok: bool) -> bool:  # the step succeeded on both ranks
            t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            return bool(t.item())

        mine = (C.c_ubyte * 192)()
        st = lib().b200_gpt2_tp_peer_export(self._h, mine)
        if not both(st == 0):
            raise B200Error(f"tp_peer_export failed on a rank (here: {st}, {lib().b200_ctx_last_error(self.ctx._h).decode()})")
        t = torch.tensor(list(bytes(mine)), dtype=torch.uint8, device=dev)
        parts = [torch.empty_like(t) for _ in range(2)]
        dist.all_gather(parts, t, group=group)
        other = parts[1 - dist.get_rank(group)].cpu().numpy().tobytes()
        theirs = (C.c_ubyte * 192).from_buffer_copy(other)
        st = lib().b200_gpt2_tp_peer_connect(self._h, theirs)
        if not both(st == 0):  # (also the barrier: both sides are mapped before either starts a forward)
            if st == 0:
                lib().b200_gpt2_tp_peer_enable(self._h, 0)
            raise B200Error(f"tp_peer_connect failed on a rank (here: {st}, {lib().b200_ctx_last_error(self.ctx._h).decode()})")

    def connect_tp_sequence_parallel(self, group=None):
        """The sequence-parallel hand-over for groups of 2 to 8 ranks (b200_gpt2_tp_sp_*): exchanges the
        CUDA IPC handles of all ranks through torch.distributed and switches it on.  Collective; either
        every rank ends up connected or every rank raises."""
        import torch
        import torch.distributed as dist
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world != self.tp_size:
            raise B200Error("the group is not the model's tensor-parallel group")
        dev = f"cuda:{self.ctx.device}"

        def everyone(ok: bool) -> bool:
            t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            return bool(t.item())

        mine = (C.c_ubyte * 192)()
        st = lib().b200_gpt2_tp_sp_export(self._h, mine)
        if not everyone(st == 0):
            raise B200Error(f"tp_sp_export failed on a rank (here: {st}, {lib().b200_ctx_last_error(self.ctx._h).decode()})")
        t = torch.tensor(list(bytes(mine)), dtype=torch.uint8, device=dev)
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t, group=group)
        blob = b"".join(p.cpu().numpy().tobytes() for p in parts)
        every = (C.c_ubyte * (192 * world)).from_buffer_copy(blob)
        st = lib().b200_gpt2_tp_sp_connect(self._h, every)
        if not everyone(st == 0):
            if st == 0:
                lib().b200_gpt2_tp_sp_enable(self._h, 0)
            raise B200Error(f"tp_sp_connect failed on a rank (here: {st}, {lib().b200_ctx_last_error(self.ctx._h).decode()})")

    def enable_tp_sequence_parallel(self, on: bool = True):
        self.ctx.check(lib().b200_gpt2_tp_sp_enable(self._h, int(on)), "tp_sp_enable")

    def enable_tp_peer(self, on: bool = True):
        self.ctx.check(lib().b200_gpt2_tp_peer_enable(self._h, int(on)), "tp_peer_enable")

    def params_ptr(self) -> int:
        return int(lib().b200_gpt2_params(self._h))

    def params_tensor(self):
        """The flat fp32 parameter array as a torch view over the library's device memory."""
        import torch
        n = self.num_local_params()
        return _view_device(self.params_ptr(), (n,), torch.float32, self.ctx.device)

    def load_params(self, host_params):
        self.ctx.check(lib().b200_gpt2_load_params_host(self._h, _ptr(host_params), host_params.size), "load_params")

    def load_params_file(self, path: str, header_bytes: int = 0):
        """Raw fp32 parameters in param_offsets order behind a header of header_bytes."""
        self.ctx.check(lib().b200_gpt2_load_params_file(self._h, os.fsencode(path), header_bytes), "load_params_file")

    def set_options(self, round_operands=1, gemm_mode=None, lmhead_mode=None, use_graph=0, attention_mode=-1):
        """gemm_mode / lmhead_mode default to the library's default arithmetic (DEFAULT_MODE_NAME)."""
        d = MODES[DEFAULT_MODE_NAME]
        gemm_mode = d["gemm_mode"] if gemm_mode is None else gemm_mode
        lmhead_mode = d["lmhead_mode"] if lmhead_mode is None else lmhead_mode
        self.ctx.check(lib().b200_gpt2_set_attention_mode(self._h, int(attention_mode)), "set_attention_mode")
        self.ctx.check(lib().b200_gpt2_set_options(self._h, int(round_operands), gemm_mode, lmhead_mode, int(use_graph)),
                       "set_options")

    def set_attention_mode(self, mode: int = -1):
        """-1: follow gemm_mode; B200_TF32: single-pass kernel; B200_TF32X3: split-operand kernel."""
        self.ctx.check(lib().b200_gpt2_set_attention_mode(self._h, int(mode)), "set_attention_mode")

    def forward(self, tokens, B: int, T: int):
        """tokens: CUDA int32 [B,T].  Asynchronous; returns a view of the logits [B,T,Vp]."""
        import torch
        self.ctx.check(lib().b200_gpt2_forward(self._h, _ptr(tokens), B, T), "gpt2_forward")
        return _view_device(int(lib().b200_gpt2_logits(self._h)), (B, T, self.logits_width),
                            torch.float32, self.ctx.device)

    def forward_sample(self, tokens, B: int, T: int, ids_out, temperature: float = 1.0, seed: int = 0, lse_out=None,
                       store_logits: bool = False):
        """The forward with one token per position drawn in the lm-head's epilogue (ids_out: CUDA int32
        [B,T]) and, if lse_out (CUDA fp32 [B,T]) is given, the log-sum-exp of every row of logits."""
        self.ctx.check(lib().b200_gpt2_forward_sample(self._h, _ptr(tokens), B, T, float(temperature), int(seed) & 0xFFFFFFFF,
                                                      _ptr(ids_out), _ptr(lse_out), int(store_logits)), "gpt2_forward_sample")

    def forward_host(self, tokens_host, B: int, T: int, logits_host=None, last_logits_host=None, argmax_host=None):
        """Host-buffer call: H2D of tokens, forward, D2H of what is asked for; synchronous."""
        self.ctx.check(lib().b200_gpt2_forward_host(self._h, _ptr(tokens_host), B, T, _ptr(logits_host),
                                                    _ptr(last_logits_host), _ptr(argmax_host)), "gpt2_forward_host")

    def forward_host_enqueue(self, tokens_host, B: int, T: int, slot: int, logits_host=None, last_logits_host=None,
                             argmax_host=None):
        """forward_host without the wait: queues copy in, forward, copies back for slot 0 or 1."""
        self.ctx.check(lib().b200_gpt2_forward_host_enqueue(self._h, _ptr(tokens_host), B, T, _ptr(logits_host),
                                                            _ptr(last_logits_host), _ptr(argmax_host), slot),
                       "gpt2_forward_host_enqueue")

    def forward_host_wait(self, slot: int):
        """Blocks until the results of that slot are in the host buffers."""
        self.ctx.check(lib().b200_gpt2_forward_host_wait(self._h, slot), "gpt2_forward_host_wait")

    # ---- incremental decoding with a key/value cache
    def enable_kv_cache(self):
        """Allocates keys and values of every layer for max_B sequences of max_T positions."""
        self.ctx.check(lib().b200_gpt2_enable_kv_cache(self._h), "enable_kv_cache")

    def prefill(self, tokens, B: int, T: int):
        """forward() that also stores the keys and values of positions [0,T); logits [B,T,Vp]."""
        import torch
        self.ctx.check(lib().b200_gpt2_prefill(self._h, _ptr(tokens), B, T), "gpt2_prefill")
        return _view_device(int(lib().b200_gpt2_logits(self._h)), (B, T, self.cfg.padded_vocab_size),
                            torch.float32, self.ctx.device)

    def decode_step(self, tokens, B: int, pos: int):
        """tokens: CUDA int32 [B], standing at position pos.  Asynchronous; returns a view of the
        logits of that position, [B,Vp]."""
        import torch
        self.ctx.check(lib().b200_gpt2_decode_step(self._h, _ptr(tokens), B, pos), "gpt2_decode_step")
        return _view_device(int(lib().b200_gpt2_logits(self._h)), (B, self.cfg.padded_vocab_size),
                            torch.float32, self.ctx.device)

    def decode_step_host(self, tokens_host, B: int, pos: int, logits_host=None, argmax_host=None):
        self.ctx.check(lib().b200_gpt2_decode_step_host(self._h, _ptr(tokens_host), B, pos, _ptr(logits_host),
                                                        _ptr(argmax_host)), "gpt2_decode_step_host")

    def generate_greedy(self, prompt_host, B: int, T0: int, n_new: int, out_host):
        """Greedy continuation: prompt_host int32 [B,T0] -> out_host int32 [B,n_new]; synchronous."""
        self.ctx.check(lib().b200_gpt2_generate_greedy(self._h, _ptr(prompt_host), B, T0, n_new, _ptr(out_host)),
                       "gpt2_generate_greedy")

    def generate(self, prompt_host, B: int, T0: int, n_new: int, out_host, temperature: float = 1.0, seed: int = 0,
                 top_k: int = 0, top_p: float = 0.0):
        """Sampled continuation (temperature <= 0: greedy; top_k > 0: among the k most likely tokens);
        reproducible for a given seed."""
        self.ctx.check(lib().b200_gpt2_generate(self._h, _ptr(prompt_host), B, T0, n_new, float(temperature), int(top_k), float(top_p),
                                                int(seed) & 0xFFFFFFFF, _ptr(out_host)), "gpt2_generate")

    def set_profile(self, enabled: bool):
        self.ctx.check(lib().b200_gpt2_set_profile(self._h, int(enabled)), "set_profile")

    def read_profile(self) -> dict[str, tuple[float, int]]:
        """{operator: (milliseconds, launches)} since the previous read-out; synchronises."""
        ms = (C.c_double * len(PROF_NAMES))()
        n = (C.c_long * len(PROF_NAMES))()
        self.ctx.check(lib().b200_gpt2_read_profile(self._h, ms, n), "read_profile")
        return {name: (float(ms[k]), int(n[k])) for k, name in enumerate(PROF_NAMES)}

    def activation(self, name: str, shape, dtype=None):
        import torch
        p = lib().b200_gpt2_activation(self._h, name.encode())
        if not p:
            raise KeyError(name)
        return _view_device(int(p), shape, dtype or torch.float32, self.ctx.device)

    def close(self):
        if self._h:
            lib().b200_gpt2_destroy(self._h)
            self._h = C.c_void_p()


def gpt2_static_prepare(ctx: Context) -> int:
    """b200_gpt2_static_prepare: the one-time set-up of gpt2_forward_static on the context's device,
    to be called while device allocation is still allowed; returns the status code."""
    return int(lib().b200_gpt2_static_prepare(ctx._h))


def gpt2_forward_static(ctx: Context, cfg: GPT2Config, params, tokens, B: int, T: int, logits) -> int:
    """b200_gpt2_forward_static: the forward without any device allocation, for callers that may
    not allocate (see include/b200gpt2.h).  params / tokens / logits are CUDA tensors owned by the
    caller; returns the status code (0 = ok) without raising."""
    cc = cfg.c()
    return int(lib().b200_gpt2_forward_static(ctx._h, C.byref(cc), _ptr(params), _ptr(tokens), B, T, _ptr(logits)))


def _view_device(ptr: int, shape, dtype, device: int):
    """Zero-copy torch view over device memory owned by the library."""
    import torch

    n = 1
    for s in shape:
        n *= int(s)
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Holder:
        pass

    h = _Holder()
    typestr = {torch.float32: "<f4", torch.int32: "<i4"}[dtype]
    h.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                  "strides": None}
    t = torch.as_tensor(h, device=f"cuda:{device}")
    assert t.element_size() == itemsize
    return t.view(*shape)
