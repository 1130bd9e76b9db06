"""numpy/ctypes front-end of the CPU oracle (oracle/gpt2_oracle.c).

TEST INFRASTRUCTURE ONLY.  Only the tests, the smoke check and the benchmark's
CPU-baseline / reference legs may import this module; the product package never does.

Every function takes and returns C-contiguous numpy arrays (fp32 / int32) and mirrors the
reference's host-wrapper argument order (see the citations in gpt2_oracle.c).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libgpt2_oracle.so")
_lib = None

_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int32)


def build(force: bool = False) -> str:
    """Compile the oracle with `make` (gcc + OpenMP).  Returns the library path."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "gpt2_oracle.c"))
    ):
        subprocess.check_call(["make", "-C", _HERE, "libgpt2_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


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


GPT2_124M = GPT2Config()
GPT2_XL = GPT2Config(num_layers=48, num_heads=25, channels=1600)

PARAM_NAMES = ("wte", "wpe", "ln1w", "ln1b", "qkvw", "qkvb", "attprojw", "attprojb",
               "ln2w", "ln2b", "fcw", "fcb", "fcprojw", "fcprojb", "lnfw", "lnfb")


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_gpt2_param_offsets.restype = C.c_size_t
        _lib.oracle_gpt2_forward.restype = C.c_int
        _lib.oracle_num_threads.restype = C.c_int
        _lib.oracle_set_num_threads.restype = C.c_int
        _lib.oracle_set_num_threads.argtypes = [C.c_int]
    return _lib


def _p(a: np.ndarray | None, ty=_f):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(ty)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> int:
    """OpenMP team size for every later call (launchers such as torch.distributed.run export
    OMP_NUM_THREADS=1, which would otherwise put the whole forward on one core)."""
    return int(lib().oracle_set_num_threads(int(n)))


def use_all_host_threads() -> int:
    """Team size = the cores this process may run on; returns it."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return set_num_threads(max(1, n))


def fill_normal(shape, seed: int, stream: int = 0, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(shape, dtype=np.float32)
    lib().oracle_fill_normal(_p(out), C.c_size_t(out.size), C.c_uint64(seed), C.c_uint64(stream),
                             C.c_float(mean), C.c_float(std))
    return out


def fill_tokens(shape, seed: int, vocab: int = 50257) -> np.ndarray:
    out = np.empty(shape, dtype=np.int32)
    lib().oracle_fill_tokens(_p(out, _i), C.c_size_t(out.size), C.c_uint64(seed), C.c_int32(vocab))
    return out


def encoder_forward(inp, wte, wpe) -> np.ndarray:
    inp = np.ascontiguousarray(inp, dtype=np.int32)
    wte, wpe = _f32(wte), _f32(wpe)
    B, T = inp.shape
    Cc = wte.shape[1]
    out = np.empty((B, T, Cc), dtype=np.float32)
    lib().oracle_encoder_forward(_p(out), _p(inp, _i), _p(wte), _p(wpe), B, T, Cc)
    return out


def gelu_forward(inp, precise: bool = False) -> np.ndarray:
    inp = _f32(inp)
    out = np.empty_like(inp)
    lib().oracle_gelu_forward(_p(out), _p(inp), C.c_size_t(inp.size), int(precise))
    return out


def residual_forward(inp1, inp2) -> np.ndarray:
    inp1, inp2 = _f32(inp1), _f32(inp2)
    out = np.empty_like(inp1)
    lib().oracle_residual_forward(_p(out), _p(inp1), _p(inp2), C.c_size_t(inp1.size))
    return out


def layernorm_forward(inp, weight, bias, precise: bool = False):
    """inp [B,T,C] -> (out [B,T,C], mean [B,T], rstd [B,T])"""
    inp, weight, bias = _f32(inp), _f32(weight), _f32(bias)
    B, T, Cc = inp.shape
    out = np.empty_like(inp)
    mean = np.empty((B, T), dtype=np.float32)
    rstd = np.empty((B, T), dtype=np.float32)
    lib().oracle_layernorm_forward(_p(out), _p(mean), _p(rstd), _p(inp), _p(weight), _p(bias),
                                   B, T, Cc, int(precise))
    return out, mean, rstd


def fused_residual_layernorm_forward(inp1, inp2, weight, bias, precise: bool = False):
    """-> (res_out, layernorm_out, mean, rstd)"""
    inp1, inp2, weight, bias = _f32(inp1), _f32(inp2), _f32(weight), _f32(bias)
    B, T, Cc = inp1.shape
    res = np.empty_like(inp1)
    out = np.empty_like(inp1)
    mean = np.empty((B, T), dtype=np.float32)
    rstd = np.empty((B, T), dtype=np.float32)
    lib().oracle_fused_residual_layernorm_forward(_p(res), _p(out), _p(mean), _p(rstd), _p(inp1),
                                                  _p(inp2), _p(weight), _p(bias), B, T, Cc,
                                                  int(precise))
    return res, out, mean, rstd


def matmul_forward(inp, weight, bias=None, act: int = 0, residual=None, precise: bool = False):
    """inp [B,T,C], weight [OC,C], bias [OC]|None -> out [B,T,OC]; act 1 = tanh-GELU;
    residual [B,T,OC] is added after the activation."""
    inp, weight = _f32(inp), _f32(weight)
    bias = None if bias is None else _f32(bias)
    residual = None if residual is None else _f32(residual)
    B, T, Cc = inp.shape
    OC = weight.shape[0]
    assert weight.shape[1] == Cc
    out = np.empty((B, T, OC), dtype=np.float32)
    lib().oracle_matmul_forward_ex(_p(out), _p(inp), _p(weight), _p(bias), B, T, Cc, OC, int(act),
                                   _p(residual), int(precise))
    return out


def attention_forward(inp, NH: int, precise: bool = False):
    """inp [B,T,3C] packed (q|k|v, each [NH,HS]) -> (out [B,T,C], lse [B,NH,T])"""
    inp = _f32(inp)
    B, T, C3 = inp.shape
    Cc = C3 // 3
    out = np.empty((B, T, Cc), dtype=np.float32)
    lse = np.empty((B, NH, T), dtype=np.float32)
    lib().oracle_attention_forward(_p(out), _p(lse), _p(inp), B, T, Cc, NH, int(precise))
    return out, lse


def param_offsets(cfg: GPT2Config) -> list[int]:
    offs = (C.c_size_t * 17)()
    cc = cfg.c()
    lib().oracle_gpt2_param_offsets(C.byref(cc), offs)
    return [int(o) for o in offs]


def init_params(cfg: GPT2Config, seed: int = 1234) -> np.ndarray:
    n = param_offsets(cfg)[16]
    params = np.empty(n, dtype=np.float32)
    cc = cfg.c()
    lib().oracle_gpt2_init_params(_p(params), C.byref(cc), C.c_uint64(seed))
    return params


def param_views(params: np.ndarray, cfg: GPT2Config) -> dict[str, np.ndarray]:
    offs = param_offsets(cfg)
    Cc, L, Vp, mT = cfg.channels, cfg.num_layers, cfg.padded_vocab_size, cfg.max_seq_len
    shapes = [(Vp, Cc), (mT, Cc), (L, Cc), (L, Cc), (L, 3 * Cc, Cc), (L, 3 * Cc), (L, Cc, Cc), (L, Cc),
              (L, Cc), (L, Cc), (L, 4 * Cc, Cc), (L, 4 * Cc), (L, Cc, 4 * Cc), (L, Cc), (Cc,), (Cc,)]
    return {n: params[offs[i]:offs[i + 1]].reshape(shapes[i]) for i, n in enumerate(PARAM_NAMES)}


def gpt2_forward(params: np.ndarray, cfg: GPT2Config, tokens, precise: bool = False) -> np.ndarray:
    tokens = np.ascontiguousarray(tokens, dtype=np.int32)
    B, T = tokens.shape
    logits = np.empty((B, T, cfg.padded_vocab_size), dtype=np.float32)
    cc = cfg.c()
    rc = lib().oracle_gpt2_forward(_p(logits), _p(params), C.byref(cc), _p(tokens, _i), B, T,
                                   int(precise))
    if rc != 0:
        raise MemoryError("oracle_gpt2_forward: allocation failed")
    return logits
