"""Python faces of the CUDA kernels: argument checks, then one launch on the current stream.

The shared library is loaded with ctypes on first use (compiled first if stale).
Every wrapper checks dtype, device, contiguity and the sizes the kernel supports and
raises ``KernelError`` for what it cannot compute; there is no other implementation
to fall back to.  Tensors are passed as raw device pointers.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from .build import ensure_built


class KernelError(RuntimeError):
    pass


_lib = None
F32, BF16 = 0, 1


def lib():
    if _TIMER is not None and _lib is not None:
        return _TimedLib(_lib)
    return _load()


def _load():
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise KernelError("acorninfer_b200 needs a CUDA device (sm_100a); none is visible and there is no CPU path")
        path = ensure_built()
        _lib = ctypes.CDLL(str(path))
        for name in dir(_Sigs):
            if name.startswith("acorn_"):
                fn = getattr(_lib, name, None)
                if fn is None:
                    raise KernelError(f"{path} lacks the symbol {name}: stale build?")
                fn.argtypes = getattr(_Sigs, name)
                fn.restype = c_int
        _lib.acorn_uniform.restype = c_float
        _init_error_word(_lib)
    return _lib


_error_word: ctypes.c_int | None = None       # pinned host memory that kernels write when a bounded wait gives up
_KERNEL_NAMES = {1: "gemm_tcgen05", 2: "attention_prefill_tc", 3: "attention_decode_tma", 4: "gemm_tcgen05_pair", 9: "error-word self-test"}


def _init_error_word(library) -> None:
    global _error_word
    host, dev = c_void_p(), c_void_p()
    code = library.acorn_error_word_alloc(ctypes.byref(host), ctypes.byref(dev))
    if code != 0 or not host.value:
        raise KernelError(f"could not allocate the kernels' error word: CUDA error {code}")
    for setter in ("acorn_gemm_tc_set_error_word", "acorn_attention_tc_set_error_word",
                   "acorn_attention_decode_tma_set_error_word", "acorn_selftest_set_error_word",
                   "acorn_gemm_tc_pair_set_error_word"):
        code = getattr(library, setter)(dev)
        if code != 0:
            raise KernelError(f"{setter}: CUDA error {code}")
    _error_word = ctypes.c_int.from_address(host.value)


def raise_on_kernel_error() -> None:
    """Raises if a kernel of a step that has completed gave up a bounded wait (its results are not
    valid).  Costs a read of host memory: callers look after every step whose results they read."""
    if _error_word is None or _error_word.value == 0:
        return
    word = _error_word.value
    _error_word.value = 0
    for getter in (gemm_tc_error, attention_tc_error, attention_decode_tma_error, gemm_tc_pair_error):   # clear the kernels' own flags
        getter()
    raise KernelError(f"kernel {_KERNEL_NAMES.get(word // 100, word // 100)} gave up a bounded wait at point "
                      f"{word % 100}: the results of the step are not valid")


def error_word_selftest(point: int) -> None:
    """Launches a kernel that does nothing but report ``point`` the way a failing kernel would."""
    _ok(lib().acorn_error_word_selftest(point, _stream()), "error_word_selftest")


class _Sigs:
    acorn_embed = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    acorn_patch_tokens = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    acorn_add_rmsnorm = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]
    acorn_swiglu = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    acorn_add_layernorm = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                           c_int, c_void_p]
    acorn_add_into = [c_void_p, c_void_p, c_int64, c_int, c_void_p]
    acorn_head_gate = [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_int, c_void_p]
    acorn_ssm_prep = [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_void_p]
    acorn_silu_rows = [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p]
    acorn_linear_scan = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                         c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
    acorn_gated_norm = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_float, c_int,
                        c_float, c_int, c_void_p]
    acorn_cast = [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
    acorn_qk_rope_kv = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                        c_int, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_void_p,
                        c_void_p, c_void_p, c_int64, c_int, c_float, c_int, c_void_p]
    acorn_attention_plain = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                             c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_float, c_int, c_void_p]
    acorn_bigram_add = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                        c_int, c_int, c_int, c_int, c_void_p]
    acorn_rmsnorm_add = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]
    acorn_rmsnorm_add_norm = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int,
                              c_void_p]
    acorn_activation = [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    acorn_side_gate = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
    acorn_token_shift = [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_int, c_int, c_int, c_int, c_int, c_void_p]
    acorn_wkv_prep = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    acorn_latent_prep = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                         c_int, c_void_p, c_int64, c_void_p]
    acorn_latent_attention_tc = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    acorn_latent_attention_tc_supported = [c_int, c_int, c_int, c_int]
    acorn_head_linear = [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_int,
                         c_int, c_void_p]
    acorn_delta_prep = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    acorn_conv_state_update = [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_void_p, c_void_p]
    acorn_delta_rule = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                        c_void_p]
    acorn_delta_fold = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
    acorn_delta_out = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    acorn_moe_route = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    acorn_moe_plan = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    acorn_grouped_gemm = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_float, c_void_p]
    acorn_grouped_gemm_fuses_swiglu = [c_int, c_int, c_int64, c_int]
    acorn_grouped_gemm_tcgen05 = [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                  c_float, c_void_p]
    acorn_gather_rows = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    acorn_moe_combine = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                         c_void_p, c_void_p, c_float, c_void_p, c_void_p]
    acorn_diff_combine = [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_int,
                          c_void_p]
    acorn_pair_rows = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    acorn_add_row = [c_void_p, c_void_p, c_int, c_int, c_void_p]
    acorn_attention_decode = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                              c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    acorn_attention_decode_ex = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                 c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p]
    acorn_attention_decode_supported = [c_int, c_int, c_int]
    acorn_attention_decode_tma_main = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                       c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                       c_float, c_int, c_int, c_void_p, c_void_p, c_void_p]
    acorn_attention_decode_tma_supported = [c_int, c_int, c_int, c_int]
    acorn_attention_decode_tma_merges = [c_int, c_int]
    acorn_attention_decode_tma_error = []
    acorn_attention_decode_merge = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    acorn_attention_prefill = [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                               c_int, c_int, c_void_p, c_void_p, c_float, c_int, c_void_p]
    acorn_attention_prefill_supported = [c_int, c_int, c_int]
    acorn_gemm_tc = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                     c_void_p]
    acorn_attention_prefill_tc = [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                  c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p]
    acorn_attention_prefill_tc_supported = [c_int, c_int, c_int, c_int]
    acorn_attention_tc_error = []
    acorn_gemm_tc_ex = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                        c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
    acorn_gemm_tc_gelu_rows = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                               c_void_p, c_void_p, c_int64, c_int, c_void_p]
    acorn_gemm_tc_qkv_rope = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                              c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p]
    acorn_gemm_tc_supported = [c_int64, c_int64, c_int64, c_int64, c_int64]
    acorn_gemm_tc_pair = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
    acorn_gemm_tc_pair_qkv_rope = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int,
                                   c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                   c_void_p]
    acorn_rope_table = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]
    acorn_gemm_tc_pair_error = []
    acorn_gemm_tc_error = []
    acorn_gemm_f32 = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
    acorn_sample = [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_void_p, c_void_p]
    acorn_uniform = [ctypes.c_uint64, ctypes.c_uint64]
    acorn_random_fill = [c_void_p, c_int64, ctypes.c_uint64, ctypes.c_uint64, c_float, c_float, c_int, c_void_p]
    acorn_error_word_alloc = [c_void_p, c_void_p]
    acorn_error_word_selftest = [c_int, c_void_p]
    acorn_gemm_tc_set_error_word = [c_void_p]
    acorn_attention_tc_set_error_word = [c_void_p]
    acorn_attention_decode_tma_set_error_word = [c_void_p]
    acorn_selftest_set_error_word = [c_void_p]
    acorn_gemm_tc_pair_set_error_word = [c_void_p]


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index = None


def _stream() -> int:
    """The current CUDA stream's handle (also the capture stream while a graph is captured)."""
    global _device_index
    if _raw_stream is not None:
        if _device_index is None:
            _device_index = torch.cuda.current_device()      # the engine works on one device
        return _raw_stream(_device_index)
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _check(t: torch.Tensor, name: str, dtype=None, dims: int | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(t.shape)}")


LAUNCHES = 0      # kernels of this library launched so far (for reports)
COUNTS: dict[str, int] = {}    # the same by entry point: tests use it to see which kernel a path really took


class KernelTimer:
    """Per-launch device times of everything launched while it is active (``with kernel_timer() as t``):
    a CUDA event before and after every launch of this library, and around the library matrix products
    of ``linear``.  The events keep kernels from overlapping (no programmatic dependent launch across
    them) and nothing may be captured meanwhile, so the times are those of each kernel alone, in the
    order and with the data of a real step.  ``records()`` gives ``[(entry point, tag, microseconds)]``
    after a synchronize; the tag tells launches of one entry point apart (a product's M x N x K)."""

    def __init__(self):
        self._events: list = []
        self._open = None

    def begin(self) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._open = ev

    def end(self, what: str, tag: str = "") -> None:
        if self._open is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.append((what, tag, self._open, ev))
        self._open = None

    def records(self) -> list[tuple[str, str, float]]:
        torch.cuda.synchronize()
        return [(what, tag, a.elapsed_time(b) * 1e3) for what, tag, a, b in self._events]


_TIMER: KernelTimer | None = None


class kernel_timer:
    def __enter__(self) -> KernelTimer:
        global _TIMER
        if _TIMER is not None:
            raise KernelError("kernel_timer: already active")
        _load()
        _TIMER = KernelTimer()
        return _TIMER

    def __exit__(self, *exc) -> None:
        global _TIMER
        _TIMER = None


class _TimedLib:
    """The library while a timer is active: every entry point records the start event first (the end
    event is recorded where the wrapper reports the launch, ``_ok``)."""

    def __init__(self, library):
        self._library = library

    def __getattr__(self, name):
        fn = getattr(self._library, name)
        if not name.startswith("acorn_") or name.endswith(("_supported", "_error", "_merges")):
            return fn

        def timed(*args):
            if _TIMER is not None:
                _TIMER.begin()
            return fn(*args)
        return timed


def _ok(code: int, what: str, tag: str = "") -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        COUNTS[what] = COUNTS.get(what, 0) + 1
        if _TIMER is not None:
            _TIMER.end(what, tag)
        return
    if code == 10001:
        raise KernelError(f"{what}: sizes or dtypes not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------ elementwise / norm


def embed(ids: torch.Tensor, table: torch.Tensor, out32: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """out32[t] = table[ids[t]] * scale as float32.  ids int32 [T]; table [V, H]."""
    _check(ids, "ids", torch.int32, 1)
    _check(table, "table", None, 2)
    T, H = ids.numel(), table.shape[1]
    if out32 is None:
        out32 = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _check(out32, "out32", torch.float32, 2)
    _ok(lib().acorn_embed(ids.data_ptr(), table.data_ptr(), out32.data_ptr(), T, H, dtype_code(table.dtype),
                          float(scale), _stream()), "embed")
    return out32


def patch_tokens(token_ids: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, src_tokens: torch.Tensor) -> None:
    """token_ids[dst[i]] = src_tokens[src[i]] (all int32, on the device)."""
    for t, n in ((token_ids, "token_ids"), (dst, "dst"), (src, "src"), (src_tokens, "src_tokens")):
        _check(t, n, torch.int32, 1)
    if dst.numel() != src.numel():
        raise KernelError("patch_tokens: dst and src differ in length")
    _ok(lib().acorn_patch_tokens(token_ids.data_ptr(), dst.data_ptr(), src.data_ptr(), src_tokens.data_ptr(),
                                 dst.numel(), _stream()), "patch_tokens")


def add_rmsnorm(resid32: torch.Tensor, delta: torch.Tensor | None, weight32: torch.Tensor, eps: float,
                out_dtype: torch.dtype, row_idx: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """resid32 += delta (in place, unless row_idx is given); returns rmsnorm(resid32) * weight.

    With ``row_idx`` (int32 [R]) only those rows are normed, into rows 0..R-1 of the result,
    and the residual is left as it is.
    """
    _check(resid32, "resid32", torch.float32, 2)
    _check(weight32, "weight", torch.float32, 1)
    H = resid32.shape[1]
    if weight32.numel() != H:
        raise KernelError(f"norm weight has {weight32.numel()} elements, width is {H}")
    if delta is not None:
        _check(delta, "delta", out_dtype, 2)
        if delta.shape != resid32.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match the residual {tuple(resid32.shape)}")
    rows = resid32.shape[0]
    if row_idx is not None:
        _check(row_idx, "row_idx", torch.int32, 1)
        rows = row_idx.numel()
    if out is None:
        out = torch.empty((rows, H), dtype=out_dtype, device=resid32.device)
    _check(out, "out", out_dtype, 2)
    _ok(lib().acorn_add_rmsnorm(resid32.data_ptr(), _ptr(delta), weight32.data_ptr(), out.data_ptr(),
                                _ptr(row_idx), rows, H, float(eps), dtype_code(out_dtype), _stream()),
        "add_rmsnorm")
    return out


GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "capped_swish": 2}
GLU_EPILOGUE_ACTIVATIONS = ("silu", "gelu_tanh")       # those the tcgen05 products apply themselves


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int | None = None,
           activation: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """act(gate) * up, act silu or the tanh form of gelu; or the capped form (``capped_swish`` with ``limit`` L):
    ``g = min(gate, L), u = clamp(up, -L, L), g sigmoid(1.702 g) (u + 1)``.  A row holds, per block of ``block`` outputs, the gate values then the up
    values; the default (block = I) is the plain layout ``[gate | up]``."""
    _check(gate_up, "gate_up", None, 2)
    T, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even width")
    block = block or two_i // 2
    if (two_i // 2) % block:
        raise KernelError(f"swiglu: block {block} does not divide the width {two_i // 2}")
    if out is None:
        out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(out, "out", gate_up.dtype, 2)
    _ok(lib().acorn_swiglu(gate_up.data_ptr(), out.data_ptr(), T, two_i // 2, block, dtype_code(gate_up.dtype),
                           GLU_ACTIVATIONS[activation], float(limit), _stream()), "swiglu")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _check(x, "x")
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _ok(lib().acorn_cast(x.data_ptr(), out.data_ptr(), x.numel(), dtype_code(x.dtype), dtype_code(dtype),
                         _stream()), "cast")
    return out


# ------------------------------------------------------------------ attention pieces


def qk_rope_kv(qkv: torch.Tensor, q_weight32: torch.Tensor | None, k_weight32: torch.Tensor | None,
               inv_freq: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
               block_table: torch.Tensor, page_base: torch.Tensor, k_pages: torch.Tensor | None,
               v_pages: torch.Tensor | None, num_heads: int, num_kv_heads: int, head_dim: int,
               rotary_dim: int, interleaved: bool, eps: float, write_kv: bool = True,
               value_dim: int | None = None, values_from_keys: bool = False, bias32: torch.Tensor | None = None,
               conv: "ShortConv | None" = None, q_out: torch.Tensor | None = None, magnitude: float = 1.0,
               norm_after: bool = False) -> None:
    """Per-head q/k norm, rotary encoding, K/V page write; q is updated in place inside ``qkv``, or written
    to ``q_out`` [T, >= nq d] if that is given.  ``bias32`` (float32, one entry per channel of a row) is added to
    the row first; ``conv`` then runs a short causal convolution over time on every channel (``q_out`` is needed
    with it: a token's convolution reads its neighbours' rows as projected).
    ``value_dim``: width of a value head where it is not ``head_dim`` (the value pages then hold rows of
    that width).  ``values_from_keys``: the values are the keys as projected, before norm and rotation; a
    row of ``qkv`` is then ``[q | k]``.  A row may be wider than its heads (further columns are ignored).
    ``magnitude``: a factor on cos and sin.  ``norm_after``: q and k heads are brought to unit root mean square
    (``eps`` inside the root) after the rotation instead of before it, times their weight if one is given."""
    _check(qkv, "qkv", None, 2)
    T = qkv.shape[0]
    dv = head_dim if value_dim is None else int(value_dim)
    if values_from_keys and dv != head_dim:
        raise KernelError("qk_rope_kv: values taken from the keys have the keys' width")
    if qkv.shape[1] < (num_heads + num_kv_heads) * head_dim + (0 if values_from_keys else num_kv_heads * dv):
        raise KernelError(f"qkv width {qkv.shape[1]} < nq d + nkv d + nkv dv")
    if head_dim > 1024 or rotary_dim > head_dim or rotary_dim % 2:
        raise KernelError(f"head_dim {head_dim} / rotary_dim {rotary_dim} not supported (d <= 1024, even rotary_dim <= d)")
    _check(inv_freq, "inv_freq", torch.float32, 1)
    if inv_freq.numel() != rotary_dim // 2:
        raise KernelError("inv_freq must have rotary_dim / 2 entries")
    for t, n in ((positions, "positions"), (token_row, "token_row"), (page_base, "page_base")):
        _check(t, n, torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    for w, n in ((q_weight32, "q_norm weight"), (k_weight32, "k_norm weight")):
        if w is not None:
            _check(w, n, torch.float32, 1)
            if w.numel() != head_dim:
                raise KernelError(f"{n} must have head_dim entries")
    P = 0
    if write_kv:
        _check(k_pages, "k_pages", qkv.dtype, 4)
        _check(v_pages, "v_pages", qkv.dtype, 4)
        if k_pages.shape[1] != num_kv_heads or k_pages.shape[3] != head_dim or \
                tuple(v_pages.shape) != (*k_pages.shape[:3], dv):
            raise KernelError(f"cache pages {tuple(k_pages.shape)} / {tuple(v_pages.shape)} do not fit "
                              f"nkv={num_kv_heads}, d={head_dim}, dv={dv}")
        P = k_pages.shape[2]
    channels = (num_heads + num_kv_heads) * head_dim + (0 if values_from_keys else num_kv_heads * dv)
    if bias32 is not None:
        _check(bias32, "bias", torch.float32, 1)
        if bias32.numel() != channels:
            raise KernelError(f"qk_rope_kv: bias has {bias32.numel()} entries for {channels} channels")
    if conv is not None:
        _check(conv.weight32, "conv weight", torch.float32, 2)
        if conv.weight32.shape[0] != channels or q_out is None or values_from_keys or not write_kv:
            raise KernelError("qk_rope_kv: the convolution needs a weight row per channel, a query buffer, value "
                              "columns of their own and a run that writes its cache")
        if conv.state.shape[1] < conv.offset + (conv.weight32.shape[1] - 1) * channels:
            raise KernelError("qk_rope_kv: the state slot is too small for the convolution's memory")
    if q_out is not None:
        _check(q_out, "q_out", qkv.dtype, 2)
        if q_out.shape[0] != T or q_out.shape[1] < num_heads * head_dim:
            raise KernelError(f"qk_rope_kv: q_out {tuple(q_out.shape)} does not hold [{T}, {num_heads * head_dim}]")
    _ok(lib().acorn_qk_rope_kv(qkv.data_ptr(), _ptr(q_weight32), _ptr(k_weight32), inv_freq.data_ptr(),
                               positions.data_ptr(), token_row.data_ptr(), block_table.data_ptr(),
                               page_base.data_ptr(), block_table.stride(0), _ptr(k_pages), _ptr(v_pages), T,
                               num_heads, num_kv_heads, head_dim, rotary_dim, 1 if interleaved else 0,
                               max(P, 1), float(eps), 1 if write_kv else 0, dtype_code(qkv.dtype), qkv.stride(0), dv,
                               1 if values_from_keys else 0,
                               _ptr(conv.weight32) if conv is not None else None,
                               conv.weight32.shape[1] if conv is not None else 0, _ptr(bias32),
                               _ptr(conv.state) if conv is not None else None,
                               conv.state.stride(0) if conv is not None else 0, conv.offset if conv is not None else 0,
                               _ptr(conv.row_start) if conv is not None else None,
                               _ptr(conv.row_slot) if conv is not None else None,
                               _ptr(q_out), q_out.stride(0) if q_out is not None else 0,
                               1 if (conv is not None and conv.update_single) else 0, float(magnitude),
                               1 if norm_after else 0, _stream()),
        "qk_rope_kv")


class ShortConv:
    """What a short causal convolution over time needs of a step: the taps ``weight32`` [channels, taps]
    (float32, the last tap for the current token), the requests' state slots with the offset at which a
    slot keeps the last ``taps - 1`` inputs ([taps - 1, channels] float32 in time order), and the step's rows.
    ``update_single``: the kernel that convolves also shifts the memory of rows that bring a single token
    (``conv_state_update(skip_single=True)`` then does the longer rows, and need not run when there are none)."""

    def __init__(self, weight32: torch.Tensor, state: torch.Tensor, offset: int, row_start: torch.Tensor,
                 row_slot: torch.Tensor, update_single: bool = False):
        self.weight32, self.state, self.offset = weight32, state, int(offset)
        self.row_start, self.row_slot, self.update_single = row_start, row_slot, bool(update_single)


def attention_plain(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                    block_table: torch.Tensor, page_base: torch.Tensor, token_row: torch.Tensor,
                    positions: torch.Tensor, num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                    scale: float, window: int | None, out: torch.Tensor | None = None,
                    value_dim: int | None = None, sink32: torch.Tensor | None = None, chunk: int | None = None,
                    keep_first: int = 0, slopes32: torch.Tensor | None = None, softcap: float | None = None,
                    maps: int = 1) -> torch.Tensor:
    """Paged causal attention for any mix of rows; ``q`` may be the head of a wider buffer
    (row stride ``q_stride`` elements).  Returns [tokens, nq * value_dim].  ``value_dim`` (default
    ``head_dim``): the leading entries of a value row that are summed; ``v_pages`` may be ``k_pages``
    itself.  ``sink32`` (float32 [nq]): a learned term exp(sink) per query head in the softmax denominator.
    ``window`` / ``chunk`` / ``keep_first``: which earlier keys a query reads (the last ``window``
    positions; those of its own block of ``chunk`` positions; and always the request's first ``keep_first``).
    ``slopes32`` (float32 [nq]): ``slope_h * (query position - key position)`` is taken off every score.
    ``softcap`` c: the scaled score becomes ``c tanh(score / c)``.  ``maps`` n > 1: every head holds n score maps
    side by side (a query row is [head][map][head_dim / n], ``num_heads`` counts (head, map) pairs, a key row holds
    the maps' keys side by side, and pair (h, a) is scored against entries a of the key row only); the output
    is [tokens, num_heads (pairs), value_dim]."""
    _check_slopes(slopes32, num_heads)
    if maps < 1 or head_dim % maps:
        raise KernelError(f"attention: {maps} score maps do not divide a key row of {head_dim}")
    dv = head_dim if value_dim is None else int(value_dim)
    if not (1 <= dv <= v_pages.shape[3]):
        raise KernelError(f"value_dim must be in 1..{v_pages.shape[3]} (the value rows' width), got {dv}")
    if sink32 is not None:
        _check(sink32, "sink", torch.float32, 1)
        if sink32.numel() != num_heads:
            raise KernelError("sink must have one entry per query head")
    if head_dim > 1024:
        raise KernelError(f"plain attention supports head_dim <= 1024, got {head_dim}")
    if num_heads % num_kv_heads:
        raise KernelError("num_heads must be a multiple of num_kv_heads")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    _check(block_table, "block_table", torch.int32, 2)
    if out is None:
        out = torch.empty((num_tokens, num_heads * dv), dtype=q.dtype, device=q.device)
    _check(out, "out", q.dtype, 2)
    _ok(lib().acorn_attention_plain(q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(),
                                    v_pages.data_ptr(), block_table.data_ptr(), page_base.data_ptr(),
                                    block_table.stride(0), token_row.data_ptr(), positions.data_ptr(),
                                    num_tokens, num_heads, num_kv_heads, head_dim, k_pages.shape[2],
                                    float(scale), int(window or 0), dtype_code(q.dtype), dv, _ptr(sink32),
                                    int(chunk or 0), int(keep_first or 0), v_pages.shape[3], _ptr(slopes32),
                                    float(softcap or 0.0), int(maps), _stream()),
        "attention_plain")
    return out


def _check_sink(sink32: torch.Tensor | None, num_heads: int) -> None:
    if sink32 is not None:
        _check(sink32, "sink", torch.float32, 1)
        if sink32.numel() != num_heads:
            raise KernelError("sink must have one entry per query head")


def _check_slopes(slopes32: torch.Tensor | None, num_heads: int) -> None:
    if slopes32 is not None:
        _check(slopes32, "slopes", torch.float32, 1)
        if slopes32.numel() != num_heads:
            raise KernelError("slopes must have one entry per query head")


def attention_decode_supported(num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return bool(lib().acorn_attention_decode_supported(num_heads, num_kv_heads, head_dim))


def attention_prefill_supported(num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return bool(lib().acorn_attention_prefill_supported(num_heads, num_kv_heads, head_dim))


def attention_decode(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, page_base: torch.Tensor, token_row: torch.Tensor,
                     positions: torch.Tensor, num_tokens: int, num_heads: int, num_kv_heads: int, head_dim: int,
                     scale: float, window: int | None, num_splits: int, token_list: torch.Tensor | None = None,
                     out: torch.Tensor | None = None, scratch: tuple | None = None,
                     use_tma: bool | None = None, chunk: int | None = None, keep_first: int = 0,
                     slopes32: torch.Tensor | None = None, sink32: torch.Tensor | None = None,
                     softcap: float | None = None, maps: int = 1) -> torch.Tensor:
    """Split-K decode attention (bfloat16) for single-token rows: the tokens 0..num_tokens-1, or
    those listed in ``token_list``.  ``out`` is [all tokens of the step, nq * d]; rows of tokens
    not handled are left as they are.  ``scratch`` = (part_o float32 [n, nq, splits, d],
    part_lse float32 [n, nq, splits]) is made here when absent and the kernel needs it (the TMA
    kernel merges up to sixteen splits without; give ``scratch`` to force the separate merge pass).
    ``sink32``, ``softcap``, ``maps``: as for ``attention_plain`` (the cp.async kernel only)."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode takes bfloat16")
    _check_sink(sink32, num_heads)
    if not attention_decode_supported(num_heads, num_kv_heads, head_dim):
        raise KernelError(f"attention_decode does not take nq={num_heads}, nkv={num_kv_heads}, d={head_dim}")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    _check(block_table, "block_table", torch.int32, 2)
    n = num_tokens if token_list is None else token_list.numel()
    if n > 65535 or not (1 <= num_splits <= 32):
        raise KernelError(f"attention_decode: {n} tokens / {num_splits} splits beyond the grid limits")
    if out is None:
        out = torch.empty((num_tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    P = k_pages.shape[2]
    _check_slopes(slopes32, num_heads)
    if chunk or keep_first or slopes32 is not None or sink32 is not None or softcap or maps != 1:
        if use_tma:
            raise KernelError("attention_decode: the TMA kernel knows windows only")
        use_tma = False
    if use_tma is None:
        use_tma = bool(lib().acorn_attention_decode_tma_supported(num_heads, num_kv_heads, head_dim, P))
    # the TMA kernel merges up to sixteen splits itself (a cluster, through shared memory): no scratch
    limit = lib().acorn_attention_decode_tma_merges(num_heads, num_kv_heads) if use_tma and scratch is None else 1
    in_kernel_merge = num_splits > 1 and (num_splits <= min(limit, 8) or (num_splits == 16 and limit >= 16))
    part_o = part_lse = None
    if num_splits > 1 and not in_kernel_merge:
        if scratch is None:
            scratch = (torch.empty((n, num_heads, num_splits, head_dim), dtype=torch.float32, device=q.device),
                       torch.empty((n, num_heads, num_splits), dtype=torch.float32, device=q.device))
        part_o, part_lse = scratch
        if part_o.numel() < n * num_heads * num_splits * head_dim or part_lse.numel() < n * num_heads * num_splits:
            raise KernelError("attention_decode: scratch too small")
    if use_tma:
        # head size 128: K/V tiles by TMA (attention_decode_tma.cu); more than sixteen splits, or splits
        # with scratch given, end in the common merge pass
        _ok(lib().acorn_attention_decode_tma_main(
            q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0],
            block_table.data_ptr(), page_base.data_ptr(), block_table.stride(0), token_row.data_ptr(),
            positions.data_ptr(), _ptr(token_list), n, num_heads, num_kv_heads, head_dim, P, float(scale),
            int(window or 0), num_splits, _ptr(part_o), _ptr(part_lse), _stream()), "attention_decode_tma")
        if num_splits > 1 and not in_kernel_merge:
            _ok(lib().acorn_attention_decode_merge(part_o.data_ptr(), part_lse.data_ptr(), out.data_ptr(),
                                                   _ptr(token_list), n, num_heads, head_dim, num_splits, _stream()),
                "attention_decode_merge")
        return out
    _ok(lib().acorn_attention_decode_ex(q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                                        block_table.data_ptr(), page_base.data_ptr(), block_table.stride(0),
                                        token_row.data_ptr(), positions.data_ptr(), _ptr(token_list), n, num_heads,
                                        num_kv_heads, head_dim, P, float(scale), int(window or 0),
                                        num_splits, _ptr(part_o), _ptr(part_lse), int(chunk or 0), int(keep_first or 0),
                                        _ptr(slopes32), _ptr(sink32), float(softcap or 0.0), int(maps), _stream()),
        "attention_decode")
    return out


def attention_decode_tma_error() -> int:
    return int(lib().acorn_attention_decode_tma_error())


def attention_prefill(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, page_base: torch.Tensor, row_start: torch.Tensor,
                      row_pos: torch.Tensor, tiles: torch.Tensor, num_tokens: int, num_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: int | None,
                      out: torch.Tensor | None = None, chunk: int | None = None, keep_first: int = 0,
                      slopes32: torch.Tensor | None = None, sink32: torch.Tensor | None = None,
                      softcap: float | None = None, maps: int = 1) -> torch.Tensor:
    """Tensor-core prefill attention (bfloat16) for the query tiles listed in ``tiles``
    (int32 [n, 2]: row, first token within the row; 64 tokens a tile at most).  ``sink32``, ``softcap``,
    ``maps``: as for ``attention_plain``."""
    _check_slopes(slopes32, num_heads)
    _check_sink(sink32, num_heads)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill takes bfloat16")
    if not attention_prefill_supported(num_heads, num_kv_heads, head_dim):
        raise KernelError(f"attention_prefill does not take nq={num_heads}, nkv={num_kv_heads}, d={head_dim}")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    _check(block_table, "block_table", torch.int32, 2)
    _check(tiles, "tiles", torch.int32, 2)
    if out is None:
        out = torch.empty((num_tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _ok(lib().acorn_attention_prefill(q.data_ptr(), q_stride, out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                                      block_table.data_ptr(), page_base.data_ptr(), block_table.stride(0),
                                      row_start.data_ptr(), row_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0],
                                      num_heads, num_kv_heads, head_dim, k_pages.shape[2], float(scale),
                                      int(window or 0), int(chunk or 0), int(keep_first or 0), _ptr(slopes32),
                                      _ptr(sink32), float(softcap or 0.0), int(maps), _stream()),
        "attention_prefill")
    return out


def attention_prefill_tc_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return bool(lib().acorn_attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim, page_size))


def attention_prefill_tc(q: torch.Tensor, q_stride: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                         block_table: torch.Tensor, page_base: torch.Tensor, row_start: torch.Tensor,
                         row_pos: torch.Tensor, tiles: torch.Tensor, num_tokens: int, num_heads: int,
                         num_kv_heads: int, head_dim: int, scale: float, window: int | None,
                         out: torch.Tensor | None = None, chunk: int | None = None, keep_first: int = 0,
                         slopes32: torch.Tensor | None = None, sink32: torch.Tensor | None = None,
                         softcap: float | None = None) -> torch.Tensor:
    """tcgen05/TMA prefill attention (bfloat16, head size 128) for the query tiles listed in
    ``tiles`` (int32 [n, 2]: row, first token within the row; 128 tokens a tile at most).  CTAs
    start in the order of the list: give the tiles that read the most keys first."""
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc takes bfloat16")
    _check_slopes(slopes32, num_heads)
    _check_sink(sink32, num_heads)
    if (slopes32 is not None or softcap) and not scale > 0:
        raise KernelError("attention_prefill_tc: slopes and a cap need a positive scale")
    if slopes32 is not None and softcap:
        raise KernelError("attention_prefill_tc: a cap does not go with a distance penalty")
    _check(k_pages, "k_pages", q.dtype, 4)
    _check(v_pages, "v_pages", q.dtype, 4)
    if not attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim, k_pages.shape[2]):
        raise KernelError(f"attention_prefill_tc does not take nq={num_heads}, nkv={num_kv_heads}, d={head_dim}, "
                          f"page={k_pages.shape[2]}")
    if q_stride % 8 or q.data_ptr() % 16:
        raise KernelError("attention_prefill_tc: q rows must be 16-byte aligned")
    _check(block_table, "block_table", torch.int32, 2)
    _check(tiles, "tiles", torch.int32, 2)
    if out is None:
        out = torch.empty((num_tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _ok(lib().acorn_attention_prefill_tc(q.data_ptr(), q_stride, num_tokens, out.data_ptr(), k_pages.data_ptr(),
                                         v_pages.data_ptr(), k_pages.shape[0], block_table.data_ptr(),
                                         page_base.data_ptr(), block_table.stride(0), row_start.data_ptr(),
                                         row_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0], num_heads,
                                         num_kv_heads, head_dim, k_pages.shape[2], float(scale), int(window or 0),
                                         int(chunk or 0), int(keep_first or 0), _ptr(slopes32), _ptr(sink32),
                                         float(softcap or 0.0), _stream()),
        "attention_prefill_tc")
    return out


def attention_tc_error() -> int:
    """0, or where a bounded wait inside the tcgen05 attention kernel gave up since the last call."""
    return int(lib().acorn_attention_tc_error())


# ------------------------------------------------------------------ matrix products


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] @ w [N, K]^T in true float32 (CUDA cores)."""
    _check(w, "w", torch.float32, 2)
    if a.dtype != torch.float32 or a.dim() != 2 or a.stride(1) != 1:
        raise KernelError("a must be float32 [M, K] with contiguous K")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"inner sizes differ: a has K={K}, w has K={w.shape[1]}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _check(out, "out", torch.float32, 2)
    _ok(lib().acorn_gemm_f32(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                             out.stride(0), M, N, K, _stream()), "gemm_f32", f"{M}x{N}x{K}")
    return out


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] == w.shape[1]
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and bool(lib().acorn_gemm_tc_supported(x.shape[0], w.shape[0], x.shape[1], x.stride(0), w.stride(0))))


_SMS: dict = {}


def device_sms(device) -> int:
    """Multiprocessors of ``device`` (asked of the driver once)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _SMS:
        _SMS[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _SMS[key]


def gemm_tc_plan(M: int, N: int, K: int, num_sms: int = 148) -> tuple[int, int]:
    """(splits of the K range, CTAs to an SM) for a product on the tcgen05 kernel.

    Splits: a cluster of that many CTAs per output tile, a power of two, at most 8, chosen so that a
    matrix with few 128-row tiles still puts one to two CTAs on every SM.  CTAs to an SM: two, with
    a deep ring, or three with a short one (up to 32 rows).  ``num_sms`` defaults to a B200's 148;
    launches pass the device's own count.  An SM takes in about 66 GB/s, so the SM
    with the most tiles sets the time: 192 tiles on 148 SMs leave 44 SMs with two tiles (2.0 tiles'
    worth), while 384 half tiles, three to an SM, leave none with more than three halves (1.5).  The
    second form is taken for unsplit matrices with 1 to 1.5 tiles to an SM; where K is split
    already it gained nothing."""
    rows = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    tiles = -(-N // 128) * -(-M // rows)
    kblocks = -(-K // 64)
    splits = 1
    while splits < 8 and tiles * splits * 2 <= 2 * num_sms and kblocks // (splits * 2) >= 4:
        splits *= 2
    if rows <= 64 and splits == 1 and kblocks >= 8 and num_sms < tiles and tiles * 2 <= 3 * num_sms:
        return 2, 3                     # more tiles than SMs, fewer than 1.5 to an SM (measured: 36.0 -> 33.3 us)
    return splits, 2


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    return gemm_tc_plan(M, N, K)[0]


# At or below this many rows the tcgen05 kernel (weights on the 128-row side of the MMA) streams the
# weight matrix at least as fast as the library product; above it the library's larger tiles win.
GEMM_TC_MAX_ROWS = 32
# The paired kernel (256 x 256 tiles, a pair of SMs to a tile at a time, fused epilogues) is used from
# this many rows on, where its tiles fill the device: see ``pair_rows_ok``.
GEMM_PAIR_MIN_ROWS = 256
GEMM_PAIR_MAX_ROWS = 3072
GEMM_PAIR_MIN_FILL = 0.8          # for every product of a layer, when the whole layer is fused
GEMM_PAIR_MIN_FILL_ALONE = 0.6    # for the widest product taken alone (gate/up with SwiGLU) ...
GEMM_PAIR_ALONE_MAX_ROWS = 8192
GEMM_PAIR_ALONE_MIN_K = 2048      # ... whose K must be long enough for a tile's k-steps to hide its epilogue


def pair_fill(num_rows: int, width: int, num_sms: int = 148) -> float:
    """How full the paired kernel's rounds are for a product of ``num_rows`` rows and ``width`` output
    columns: its tiles of 256 x 256 are taken in rounds of one tile to a pair of SMs; the product's
    elements over those the rounds could hold (128 full tiles on 74 pairs: two rounds, 0.86; 96 tiles:
    two rounds, 0.65; 257 rows: every second tile holds one row)."""
    pairs = max(num_sms // 2, 1)
    tiles = -(-num_rows // 256) * -(-width // 256)
    return num_rows * width / (-(-tiles // pairs) * pairs * 65536)


def pair_rows_ok(num_rows: int, width: int, num_sms: int = 148, min_fill: float | None = None,
                 max_rows: int | None = None) -> bool:
    """Whether a product of ``num_rows`` rows and ``width`` output columns suits the paired kernel: its
    rounds must be filled to ``min_fill`` (``GEMM_PAIR_MIN_FILL`` if not given); below that the library's
    choice of tile shapes is faster.  Steps of more than ``max_rows`` rows (``GEMM_PAIR_MAX_ROWS`` if not
    given) run so long under the power cap that the library's kernel, which moves half the bytes from L2
    (multicast loads), keeps the higher clock: with every product of the layers on the paired kernel a step
    of 4,096 rows took 53.3 ms against 51.8 ms with the gate/up product alone on it, one of 6,144 rows 84.2
    against 80.9 (54.7 and 84.3 on the library alone); the gate/up product alone stops paying at about
    12,000 rows."""
    if num_rows < GEMM_PAIR_MIN_ROWS or num_rows > (GEMM_PAIR_MAX_ROWS if max_rows is None else max_rows):
        return False
    return pair_fill(num_rows, width, num_sms) >= (GEMM_PAIR_MIN_FILL if min_fill is None else min_fill)


@dataclass
class NormedRows:
    """Activations whose rows still lack their RMS factor: ``x = residual * norm weight`` and, per
    row, partial sums of ``residual^2`` (``ss`` [parts, rows]).  The matrix product that consumes
    them multiplies each output row by ``rsqrt(sum(ss) / width + eps)``: the norm costs no kernel."""

    x: torch.Tensor
    ss: torch.Tensor
    eps: float
    width: int


@dataclass
class AddNormEpilogue:
    """What the last product of a part does with its result instead of writing it: add it to the
    float32 residual stream (in place) and hand on ``NormedRows`` for the norm with this weight."""

    resid32: torch.Tensor
    weight32: torch.Tensor
    eps: float


@dataclass
class RopeKvEpilogue:
    """What the q/k/v product of an attention layer with head size 128 does with its result instead of
    writing it: per-head RMSNorm of the query and key heads (weights or None), rotation of the whole
    head in half pairing by ``position * inv_freq``, query heads to the output, keys and values to the
    token's slot in its cache pages (``k_pages`` None: they are dropped).  The same arithmetic as
    ``qk_rope_kv`` after a plain product, without the bfloat16 rounding in between."""

    positions: torch.Tensor
    token_row: torch.Tensor
    block_table: torch.Tensor
    page_base: torch.Tensor
    k_pages: torch.Tensor | None
    v_pages: torch.Tensor | None
    q_weight32: torch.Tensor | None
    k_weight32: torch.Tensor | None
    inv_freq: torch.Tensor
    num_heads: int
    num_kv_heads: int
    eps: float
    cos_sin: torch.Tensor | None = None      # [M, 128] float32 from ``rope_table``: spares the epilogue its sincosf


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """[tokens, 2 * len(inv_freq)] float32: cos, then sin, of position * inv_freq for every token."""
    _check(positions, "positions", torch.int32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    T, half = positions.numel(), inv_freq.numel()
    out = torch.empty((T, 2 * half), dtype=torch.float32, device=positions.device)
    _ok(lib().acorn_rope_table(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), T, half, _stream()), "rope_table")
    return out


def gemm_tc_qkv_rope(x, w: torch.Tensor, ep: RopeKvEpilogue, out: torch.Tensor | None = None) -> torch.Tensor:
    """The q/k/v product with ``RopeKvEpilogue``: returns [M, (nq + 2 nkv) * 128] bfloat16 whose first
    nq * 128 columns hold the finished query heads (the others are not written)."""
    rows = x if isinstance(x, NormedRows) else None
    xt = rows.x if rows is not None else x
    nq, nkv = ep.num_heads, ep.num_kv_heads
    M, K = xt.shape
    N = (nq + 2 * nkv) * 128
    if not gemm_tc_supported(xt, w) or w.shape[0] != N:
        raise KernelError(f"gemm_tc_qkv_rope does not take x {tuple(xt.shape)} {xt.dtype}, w {tuple(w.shape)} {w.dtype} "
                          f"for {nq}/{nkv} heads of 128")
    _check(ep.positions, "positions", torch.int32, 1)
    _check(ep.inv_freq, "inv_freq", torch.float32, 1)
    if ep.inv_freq.numel() != 64 or ep.positions.numel() < M:
        raise KernelError("gemm_tc_qkv_rope: inv_freq must have 64 entries and positions one per row")
    P = 1
    if ep.k_pages is not None:
        _check(ep.k_pages, "k_pages", torch.bfloat16, 4)
        _check(ep.v_pages, "v_pages", torch.bfloat16, 4)
        _check(ep.block_table, "block_table", torch.int32, 2)
        if tuple(ep.k_pages.shape[1:]) != (nkv, ep.k_pages.shape[2], 128) or ep.v_pages.shape != ep.k_pages.shape:
            raise KernelError("gemm_tc_qkv_rope: cache pages must be [pages, nkv, P, 128]")
        P = ep.k_pages.shape[2]
    for wt in (ep.q_weight32, ep.k_weight32):
        if wt is not None:
            _check(wt, "head norm weight", torch.float32, 1)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=xt.device)
    _check(out, "out", torch.bfloat16, 2)
    if M > GEMM_TC_MAX_ROWS:
        if ep.cos_sin is not None:
            _check(ep.cos_sin, "cos_sin", torch.float32, 2)
            if tuple(ep.cos_sin.shape) != (M, 128) or not ep.cos_sin.is_contiguous():
                raise KernelError("gemm_tc_qkv_rope: cos_sin must be contiguous [rows, 128]")
        pairs = device_sms(xt.device) // 2
        _ok(lib().acorn_gemm_tc_pair_qkv_rope(
            xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, K, pairs,
            rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
            rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
            ep.positions.data_ptr(), _ptr(ep.token_row), _ptr(ep.block_table), _ptr(ep.page_base),
            ep.block_table.stride(0) if ep.block_table is not None else 0, _ptr(ep.k_pages), _ptr(ep.v_pages),
            _ptr(ep.q_weight32), _ptr(ep.k_weight32), ep.inv_freq.data_ptr(), _ptr(ep.cos_sin), nq, nkv, P, float(ep.eps),
            _stream()), "gemm_tc_pair_qkv_rope", f"{M}x{N}x{K}")
        return out
    splits, per_sm = gemm_tc_plan(M, N, K, device_sms(xt.device))
    _ok(lib().acorn_gemm_tc_qkv_rope(
        xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, K, splits, per_sm,
        rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
        rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
        ep.positions.data_ptr(), _ptr(ep.token_row), _ptr(ep.block_table), _ptr(ep.page_base),
        ep.block_table.stride(0) if ep.block_table is not None else 0, _ptr(ep.k_pages), _ptr(ep.v_pages),
        _ptr(ep.q_weight32), _ptr(ep.k_weight32), ep.inv_freq.data_ptr(), nq, nkv, P, float(ep.eps), _stream()),
        "gemm_tc_qkv_rope", f"{M}x{N}x{K}")
    return out


def rope_kv_fusable(num_rows: int, dtype: torch.dtype, head_dim: int, rotary_dim: int, interleaved: bool) -> bool:
    """Whether the q/k/v product of such a layer can take ``RopeKvEpilogue`` (the row count is the
    caller's to check with ``fused_rows_ok``)."""
    return dtype == torch.bfloat16 and num_rows > 0 and head_dim == 128 and rotary_dim == 128 and not interleaved


TC_EPILOGUE_ACTS = {"relu_squared": 6, "tanh": 7}        # plain activations the one-CTA tcgen05 product applies itself (its mode)


def gemm_tc(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, splits: int | None = None,
            out: torch.Tensor | None = None, epilogue: AddNormEpilogue | None = None, swiglu: bool = False,
            activation: str = "silu",
            per_sm: int = 2, act: str | None = None):
    """x [M, K] @ w [N, K]^T on tcgen05 tensor cores (bfloat16 in, float32 accumulate).

    ``x`` may be ``NormedRows`` (at most 64 rows): the rows' RMS factors are applied to the product.
    ``epilogue``: see ``AddNormEpilogue`` (returns ``NormedRows``).  ``swiglu``: ``w`` holds blocks
    of 64 gate rows and 64 up rows; returns ``act(gate) * up`` [M, N / 2], ``act`` by ``activation`` (silu or the
    tanh form of gelu).  ``act`` (``"relu_squared"``, ``"tanh"``): a plain activation on the product, in its epilogue."""
    rows = x if isinstance(x, NormedRows) else None
    if act is not None and (act not in TC_EPILOGUE_ACTS or epilogue is not None or swiglu):
        raise KernelError(f"gemm_tc: activation {act!r} is not one of {sorted(TC_EPILOGUE_ACTS)}, or stands beside another epilogue")
    xt = rows.x if rows is not None else x
    if not gemm_tc_supported(xt, w):
        raise KernelError(f"gemm_tc does not take x {tuple(xt.shape)} {xt.dtype} stride {xt.stride()}, "
                          f"w {tuple(w.shape)} {w.dtype}: bf16, K contiguous, K and strides multiples of 8")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc writes bfloat16 or float32")
    M, K = xt.shape
    N = w.shape[0]
    if (rows is not None or epilogue is not None or swiglu) and M > 64:
        raise KernelError(f"gemm_tc: fused norm / SwiGLU epilogues take at most 64 rows, got {M}")
    if splits is None:
        splits, per_sm = gemm_tc_plan(M, N, K, device_sms(xt.device))
    mode, resid, ldr, norm_w, ss_out = 0, None, 0, None, None
    out_cols = N
    if epilogue is not None:
        if swiglu or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc: the add-norm epilogue writes bfloat16 and excludes SwiGLU")
        _check(epilogue.resid32, "resid32", torch.float32, 2)
        _check(epilogue.weight32, "norm weight", torch.float32, 1)
        if epilogue.resid32.shape != (M, N) or epilogue.weight32.numel() != N:
            raise KernelError("gemm_tc: residual / norm weight do not match the product's shape")
        mode, resid, ldr, norm_w = 1, epilogue.resid32, epilogue.resid32.stride(0), epilogue.weight32
        ss_out = torch.empty((-(-N // 128), M), dtype=torch.float32, device=xt.device)
    elif swiglu:
        if N % 128 or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc: SwiGLU epilogue needs N a multiple of 128 and bfloat16 output")
        mode, out_cols = (2, 5)[GLU_ACTIVATIONS[activation]], N // 2
    elif act is not None:
        mode = TC_EPILOGUE_ACTS[act]
    if out is None:
        out = torch.empty((M, out_cols), dtype=out_dtype, device=xt.device)
    _check(out, "out", out_dtype, 2)
    _ok(lib().acorn_gemm_tc_ex(
        xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
        1 if out_dtype == torch.float32 else 0, int(splits), int(per_sm), mode,
        rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
        rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
        _ptr(resid), ldr, _ptr(norm_w), _ptr(ss_out), _stream()), "gemm_tc", f"{M}x{N}x{K}")
    if epilogue is not None:
        return NormedRows(out, ss_out, epilogue.eps, N)
    return out


def gemm_tc_pair(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, out: torch.Tensor | None = None,
                 epilogue: AddNormEpilogue | None = None, swiglu: bool = False, pairs: int | None = None,
                 activation: str = "silu"):
    """x [M, K] @ w [N, K]^T in bfloat16 on pairs of CTAs (tcgen05 ``cta_group::2``), for many rows:
    tiles of 256 rows of ``x`` by 256 rows of ``w``, one pair of SMs to a tile at a time.  ``x`` as
    ``NormedRows``, ``epilogue`` and ``swiglu`` as in ``gemm_tc``."""
    rows = x if isinstance(x, NormedRows) else None
    xt = rows.x if rows is not None else x
    if not gemm_tc_supported(xt, w):
        raise KernelError(f"gemm_tc_pair does not take x {tuple(xt.shape)} {xt.dtype} stride {xt.stride()}, "
                          f"w {tuple(w.shape)} {w.dtype}: bf16, K contiguous, K and strides multiples of 8")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_tc_pair writes bfloat16 or float32")
    M, K = xt.shape
    N = w.shape[0]
    mode, resid, ldr, norm_w, ss_out = 0, None, 0, None, None
    out_cols = N
    if epilogue is not None:
        if swiglu or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc_pair: the add-norm epilogue writes bfloat16 and excludes SwiGLU")
        _check(epilogue.resid32, "resid32", torch.float32, 2)
        _check(epilogue.weight32, "norm weight", torch.float32, 1)
        if epilogue.resid32.shape != (M, N) or epilogue.weight32.numel() != N:
            raise KernelError("gemm_tc_pair: residual / norm weight do not match the product's shape")
        mode, resid, ldr, norm_w = 1, epilogue.resid32, epilogue.resid32.stride(0), epilogue.weight32
        ss_out = torch.empty((2 * -(-N // 256), M), dtype=torch.float32, device=xt.device)
    elif swiglu:
        if N % 128 or out_dtype != torch.bfloat16:
            raise KernelError("gemm_tc_pair: SwiGLU epilogue needs N a multiple of 128 and bfloat16 output")
        mode, out_cols = (2, 5)[GLU_ACTIVATIONS[activation]], N // 2
    if out is None:
        out = torch.empty((M, out_cols), dtype=out_dtype, device=xt.device)
    _check(out, "out", out_dtype, 2)
    if pairs is None:
        pairs = device_sms(xt.device) // 2
    _ok(lib().acorn_gemm_tc_pair(
        xt.data_ptr(), xt.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), M, N, K,
        1 if out_dtype == torch.float32 else 0, int(pairs), mode,
        rows.ss.data_ptr() if rows is not None else None, rows.ss.shape[0] if rows is not None else 0,
        rows.width if rows is not None else 0, float(rows.eps) if rows is not None else 0.0,
        _ptr(resid), ldr, _ptr(norm_w), _ptr(ss_out), _stream()), "gemm_tc_pair", f"{M}x{N}x{K}")
    if epilogue is not None:
        return NormedRows(out, ss_out, epilogue.eps, N)
    return out


def gemm_tc_pair_error() -> int:
    """0, or where a bounded wait inside the paired tcgen05 GEMM gave up since the last call (clears it)."""
    return int(lib().acorn_gemm_tc_pair_error())


def gemm_tc_error() -> int:
    """0, or where a bounded wait inside the tcgen05 GEMM gave up since the last call (clears it)."""
    return int(lib().acorn_gemm_tc_error())


def fused_rows_ok(num_rows: int, dtype: torch.dtype, widths=None, num_sms: int = 148) -> bool:
    """Whether products of this many rows run on a tcgen05 kernel of this library with fused epilogues:
    the one-CTA kernel up to ``GEMM_TC_MAX_ROWS`` rows; for more rows the paired kernel, where every
    product of the part (``widths``: their output columns, one number or several) fills the device
    (``pair_rows_ok``)."""
    if dtype != torch.bfloat16 or num_rows <= 0:
        return False
    if num_rows <= GEMM_TC_MAX_ROWS:
        return True
    if widths is None:
        return False
    widths = (widths,) if isinstance(widths, int) else tuple(widths)
    return all(pair_rows_ok(num_rows, w, num_sms) for w in widths)


def linear(x, w: torch.Tensor, out_dtype: torch.dtype | None = None, epilogue: AddNormEpilogue | None = None,
           swiglu: bool = False, residual32: torch.Tensor | None = None, activation: str = "silu",
           act: str | None = None):
    """x [T, K] times w [N, K] transposed.

    float32 operands: the CUDA-core kernel (no reduced-precision matrix mode).
    bfloat16 operands: up to GEMM_TC_MAX_ROWS rows the one-CTA tcgen05/TMA kernel of this library,
    above that the library matrix product (cuBLAS); float32 accumulation either way, and
    ``out_dtype=float32`` keeps the accumulator's precision (used for logits).
    A weight stored in float32 under a bfloat16 engine is multiplied in float32.
    ``x`` as ``NormedRows``, ``epilogue`` and ``swiglu`` exist on the tcgen05 kernels only: the one-CTA
    kernel up to GEMM_TC_MAX_ROWS rows, the paired kernel above (``activation``: the gate's function under
    ``swiglu``; callers ask ``fused_rows_ok`` whether
    that pays for their sizes); asking for them with other operands is an error, not a silent detour.
    ``residual32`` ([T, N] float32) is an offer: where the product goes to the library it is
    added to ``residual32`` in place, in float32 (the library's C operand: the product is not
    rounded first), and None is returned; elsewhere the offer is ignored and the product returned.
    ``act`` (a name of ``ACTIVATIONS``): a plain activation on the product: in the epilogue of the one-CTA
    tcgen05 kernel where that runs and knows it, by the activation kernel after the product elsewhere.
    """
    if act is not None:
        if epilogue is not None or swiglu or residual32 is not None or isinstance(x, NormedRows):
            raise KernelError("linear: a plain activation stands alone")
        if (act in TC_EPILOGUE_ACTS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.shape[0] <= GEMM_TC_MAX_ROWS and gemm_tc_supported(x, w) and (out_dtype or x.dtype) == torch.bfloat16):
            return gemm_tc(x, w, torch.bfloat16, act=act)
        return activation_rows(linear(x, w, out_dtype), act)
    fused = isinstance(x, NormedRows) or epilogue is not None or swiglu
    xt = x.x if isinstance(x, NormedRows) else x
    out_dtype = out_dtype or xt.dtype
    if fused:
        if not (xt.dtype == torch.bfloat16 and gemm_tc_supported(xt, w)):
            raise KernelError(f"linear: fused epilogues need a tcgen05 path (bf16, K a multiple of 8); got "
                              f"{tuple(xt.shape)} {xt.dtype} x {tuple(w.shape)} {w.dtype}")
        if xt.shape[0] > GEMM_TC_MAX_ROWS:
            return gemm_tc_pair(x, w, out_dtype, epilogue=epilogue, swiglu=swiglu, activation=activation)
        return gemm_tc(x, w, out_dtype, epilogue=epilogue, swiglu=swiglu, activation=activation)
    if w.dtype == torch.float32:
        y = gemm_f32(cast(x, torch.float32) if x.dtype != torch.float32 else x, w)
        return y if out_dtype == torch.float32 else cast(y, out_dtype)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtypes x={x.dtype}, w={w.dtype}")
    if x.shape[0] <= GEMM_TC_MAX_ROWS and gemm_tc_supported(x, w):
        return gemm_tc(x, w, out_dtype)
    if _TIMER is not None:
        _TIMER.begin()
    try:
        if residual32 is not None and residual32.dtype == torch.float32 and residual32.is_contiguous() \
                and tuple(residual32.shape) == (x.shape[0], w.shape[0]):
            torch.addmm(residual32, x, w.t(), out_dtype=torch.float32, out=residual32)
            return None
        if out_dtype == torch.float32:
            return torch.mm(x, w.t(), out_dtype=torch.float32)
        return torch.mm(x, w.t())
    finally:
        if _TIMER is not None:
            _TIMER.end("library_gemm", f"{x.shape[0]}x{w.shape[0]}x{x.shape[1]}")



# ------------------------------------------------------------------ hashed bigram rows, output norms


def bigram_add(resid32: torch.Tensor, token_ids: torch.Tensor, token_row: torch.Tensor, row_start: torch.Tensor,
               row_pos: torch.Tensor, row_slot: torch.Tensor, prev_state: torch.Tensor, table: torch.Tensor,
               buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """resid32[t] += table[(prev * mul_prev + cur * mul_cur) mod buckets], row ``buckets`` for a request's
    first token.  ``prev_state`` (int32 [slots]) holds every request's last token between steps and is
    updated."""
    _check(resid32, "resid32", torch.float32, 2)
    _check(table, "table", None, 2)
    _check(prev_state, "prev_state", torch.int32, 1)
    for t, n in ((token_ids, "token_ids"), (token_row, "token_row"), (row_start, "row_start"), (row_pos, "row_pos"),
                 (row_slot, "row_slot")):
        _check(t, n, torch.int32, 1)
    T, H = resid32.shape
    if table.shape != (buckets + 1, H):
        raise KernelError(f"bigram table {tuple(table.shape)} is not [buckets + 1, width] = [{buckets + 1}, {H}]")
    _ok(lib().acorn_bigram_add(resid32.data_ptr(), token_ids.data_ptr(), token_row.data_ptr(), row_start.data_ptr(),
                               row_pos.data_ptr(), row_slot.data_ptr(), prev_state.data_ptr(), table.data_ptr(), T, H,
                               int(buckets), int(mul_prev), int(mul_cur), dtype_code(table.dtype), _stream()), "bigram_add")
    return resid32


class RoundedRows:
    """The residual stream as the next sublayer reads it (rounded to the activation dtype; the float32
    stream itself under a float32 engine), with nothing left to add: what a block hands on when it has
    already added its last result."""

    def __init__(self, x: torch.Tensor):
        self.x = x


def rmsnorm_add(resid32: torch.Tensor, y: torch.Tensor, weight32: torch.Tensor, eps: float,
                rounded: bool = True) -> torch.Tensor | None:
    """resid32 += rmsnorm(y) * weight (in place, float32).  Returns the new residual rows rounded to
    ``y``'s dtype if that is not float32 and ``rounded`` is set (else None)."""
    _check(resid32, "resid32", torch.float32, 2)
    _check(y, "y", None, 2)
    _check(weight32, "weight", torch.float32, 1)
    if y.shape != resid32.shape or weight32.numel() != y.shape[1]:
        raise KernelError(f"rmsnorm_add: y {tuple(y.shape)}, residual {tuple(resid32.shape)}, weight {weight32.numel()}")
    out = torch.empty_like(y) if (rounded and y.dtype != torch.float32) else None
    _ok(lib().acorn_rmsnorm_add(resid32.data_ptr(), y.data_ptr(), weight32.data_ptr(), _ptr(out), y.shape[0], y.shape[1],
                                float(eps), dtype_code(y.dtype), _stream()), "rmsnorm_add")
    return out


def rmsnorm_add_norm(resid32: torch.Tensor, y: torch.Tensor, weight32: torch.Tensor, eps: float,
                     next_weight32: torch.Tensor, next_eps: float) -> torch.Tensor:
    """resid32 += rmsnorm(y) * weight (in place, float32), then the RMS norm of the new rows with
    ``next_weight32``, in ``y``'s dtype: a sublayer's output norm and the next sublayer's input norm at once."""
    _check(resid32, "resid32", torch.float32, 2)
    _check(y, "y", None, 2)
    _check(weight32, "weight", torch.float32, 1)
    _check(next_weight32, "next weight", torch.float32, 1)
    H = y.shape[1]
    if y.shape != resid32.shape or weight32.numel() != H or next_weight32.numel() != H:
        raise KernelError(f"rmsnorm_add_norm: y {tuple(y.shape)}, residual {tuple(resid32.shape)}, weights "
                          f"{weight32.numel()} / {next_weight32.numel()}")
    out = torch.empty_like(y)
    _ok(lib().acorn_rmsnorm_add_norm(resid32.data_ptr(), y.data_ptr(), weight32.data_ptr(), next_weight32.data_ptr(),
                                     out.data_ptr(), y.shape[0], H, float(eps), float(next_eps), dtype_code(y.dtype),
                                     _stream()), "rmsnorm_add_norm")
    return out


class NormedPending:
    """A sublayer's result whose RMS norm is still to be added to the stream: ``resid32 += rmsnorm(y) * weight32``.
    A block hands it on so that the next block's first norm can be taken in the same kernel
    (``rmsnorm_add_norm``); ``settle`` adds it where nobody takes it."""

    def __init__(self, y: torch.Tensor, weight32: torch.Tensor, eps: float):
        self.y, self.weight32, self.eps = y, weight32, float(eps)

    def settle(self, resid32: torch.Tensor) -> None:
        rmsnorm_add(resid32, self.y, self.weight32, self.eps, rounded=False)


RMSNORM_ADD_NORM_MAX_WIDTH = 12288          # the updated row waits in shared memory (48 KB of float32)


# ------------------------------------------------------------------ attention through a latent


def latent_prep(proj: torch.Tensor, qcat: torch.Tensor, c_weight32: torch.Tensor | None, inv_freq: torch.Tensor,
                magnitude: float, positions: torch.Tensor, token_row: torch.Tensor, block_table: torch.Tensor,
                page_base: torch.Tensor, pages: torch.Tensor | None, num_heads: int, dim: int, rot: int, rank: int,
                rot_dims: int, eps: float, kv_rows: torch.Tensor | None = None) -> None:
    """Rotates the rotated part of every head's query into ``qcat[t, h, rank:]`` and, with ``pages``
    ([pages, 1, P, rank + rot]), writes the token's cache row: the RMS-normed latent and the rotated
    shared key part.  ``proj`` [T, H (dim + rot) (+ rank + rot)]; with ``kv_rows`` [T, rank + rot] the latent and
    the shared key part are read from there and ``proj`` holds the queries only."""
    _check(proj, "proj", None, 2)
    _check(qcat, "qcat", proj.dtype, 3)
    T = proj.shape[0]
    write = pages is not None
    want = num_heads * (dim + rot) + (rank + rot if write and kv_rows is None else 0)
    if kv_rows is not None:
        _check(kv_rows, "kv_rows", proj.dtype, 2)
        if kv_rows.shape != (T, rank + rot) or kv_rows.stride(1) != 1:
            raise KernelError(f"latent_prep: kv_rows {tuple(kv_rows.shape)} is not [T, rank + rot]")
    if proj.shape[1] != want or qcat.shape != (T, num_heads, rank + rot):
        raise KernelError(f"latent_prep: proj {tuple(proj.shape)} / qcat {tuple(qcat.shape)} do not fit H={num_heads}, "
                          f"dim={dim}, rot={rot}, rank={rank}")
    _check(inv_freq, "inv_freq", torch.float32, 1)
    if inv_freq.numel() != rot_dims // 2:
        raise KernelError("inv_freq must have rot_dims / 2 entries")
    P = 1
    if write:
        _check(pages, "pages", proj.dtype, 4)
        _check(c_weight32, "latent norm weight", torch.float32, 1)
        if pages.shape[1] != 1 or pages.shape[3] != rank + rot or c_weight32.numel() != rank:
            raise KernelError(f"latent_prep: cache pages {tuple(pages.shape)} do not fit rank + rot = {rank + rot}")
        P = pages.shape[2]
    _ok(lib().acorn_latent_prep(proj.data_ptr(), proj.stride(0), qcat.data_ptr(), _ptr(c_weight32), inv_freq.data_ptr(),
                                float(magnitude), positions.data_ptr(), token_row.data_ptr(), block_table.data_ptr(),
                                page_base.data_ptr(), block_table.stride(0), _ptr(pages), T, num_heads, dim, rot, rank,
                                rot_dims, P, float(eps), 1 if write else 0, dtype_code(proj.dtype), _ptr(kv_rows),
                                kv_rows.stride(0) if kv_rows is not None else 0, _stream()), "latent_prep")


LATENT_TILE_ROWS = 64          # (token, head) pairs a block of the tensor-core kernel takes


def latent_attention_tc_supported(dtype: torch.dtype, num_heads: int, head_dim: int, value_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and bool(lib().acorn_latent_attention_tc_supported(num_heads, head_dim, value_dim, page_size))


def latent_attention_tc(q: torch.Tensor, pages: torch.Tensor, block_table: torch.Tensor, page_base: torch.Tensor,
                        row_start: torch.Tensor, row_pos: torch.Tensor, tiles: torch.Tensor, sink32: torch.Tensor | None,
                        scale: float, window: int | None, value_dim: int, splits: int | None = None) -> torch.Tensor:
    """Attention of q [T, H, d] (bfloat16) over one cached row of d per token (pages [pages, 1, P, d]) whose
    first ``value_dim`` entries are the values: returns [T, H, value_dim].  ``tiles`` int32 [n, 2]: (row, first
    token within the row) of every group of ``LATENT_TILE_ROWS // H`` tokens.  ``splits``: blocks that share a
    tile's keys (None: as many as fill the device when tiles are few, by the table's width and the window, so
    that a captured step keeps its grid)."""
    _check(q, "q", torch.bfloat16, 3)
    _check(pages, "pages", torch.bfloat16, 4)
    _check(tiles, "tiles", torch.int32, 2)
    T, H, d = q.shape
    if pages.shape[1] != 1 or pages.shape[3] != d:
        raise KernelError(f"latent_attention_tc: pages {tuple(pages.shape)} do not fit one row of {d} per token")
    if sink32 is not None:
        _check(sink32, "sink", torch.float32, 1)
    out = torch.empty((T, H, value_dim), dtype=torch.bfloat16, device=q.device)
    n = tiles.shape[0]
    if splits is None:
        bound = block_table.shape[1] * pages.shape[2]
        if window:
            bound = min(bound, int(window) + LATENT_TILE_ROWS)
        splits = max(1, min(-(-device_sms(q.device) // max(n, 1)), -(-bound // 64), 32)) if n * 2 <= device_sms(q.device) else 1
    part = torch.empty((n, splits, LATENT_TILE_ROWS, value_dim + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
    _ok(lib().acorn_latent_attention_tc(q.data_ptr(), out.data_ptr(), pages.data_ptr(), block_table.data_ptr(),
                                        page_base.data_ptr(), block_table.stride(0), row_start.data_ptr(), row_pos.data_ptr(),
                                        tiles.data_ptr(), n, _ptr(sink32), float(scale), int(window or 0), H, d,
                                        int(value_dim), pages.shape[2], int(splits), _ptr(part), _stream()), "latent_attention_tc")
    return out


def head_linear(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """y[t, h, :] = w[h] x[t, h, :] for every head.  x [T, H, I] and y [T, H, O] may be views with any
    token and head strides (innermost contiguous); w [H, O, I] contiguous."""
    _check(w, "w", x.dtype, 3)
    H, O, I = w.shape
    if x.dim() != 3 or y.dim() != 3 or x.shape[1:] != (H, I) or y.shape != (x.shape[0], H, O) or y.dtype != x.dtype:
        raise KernelError(f"head_linear: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)} do not fit")
    if x.stride(2) != 1 or y.stride(2) != 1 or not x.is_cuda or not y.is_cuda:
        raise KernelError("head_linear: innermost dimensions must be contiguous CUDA memory")
    if x.dtype == torch.bfloat16 and x.shape[0] > GEMM_TC_MAX_ROWS:
        # many rows: the library's batched product (one batch entry a head), as the plain products of such steps
        if _TIMER is not None:
            _TIMER.begin()
        torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=y.transpose(0, 1))
        if _TIMER is not None:
            _TIMER.end("library_bmm", f"{x.shape[0]}x{H}x{O}x{I}")
        return y
    _ok(lib().acorn_head_linear(x.data_ptr(), x.stride(0), x.stride(1), w.data_ptr(), y.data_ptr(), y.stride(0), y.stride(1),
                                x.shape[0], H, O, I, dtype_code(x.dtype), _stream()), "head_linear", f"{x.shape[0]}x{H}x{O}x{I}")
    return y


# ------------------------------------------------------------------ gated delta rule


def delta_prep(main: torch.Tensor, up32: torch.Tensor, conv_w32: torch.Tensor, state: torch.Tensor, conv_off: int,
               a_log32: torch.Tensor, dt_bias32: torch.Tensor, token_row: torch.Tensor, row_start: torch.Tensor,
               row_slot: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, taps: int):
    """Convolution + silu of the q, k, v channels, unit norms, write strength, decays and output gate of
    every token: returns float32 (q [T, KH, dim], k [T, KH, dim], v [T, H, vdim], beta [T, H],
    g [T, H, dim], gate [T, H, vdim])."""
    _check(main, "main", None, 2)
    _check(up32, "up", torch.float32, 2)
    _check(state, "state", torch.float32, 2)
    _check(conv_w32, "conv weights", torch.float32, 2)
    T = main.shape[0]
    C = 2 * kv_heads * dim + heads * vdim
    if main.shape[1] != C + heads or up32.shape != (T, heads * dim + heads * vdim) or conv_w32.shape != (C, taps):
        raise KernelError(f"delta_prep: main {tuple(main.shape)}, up {tuple(up32.shape)}, conv {tuple(conv_w32.shape)} do not fit")
    if state.shape[1] < conv_off + (taps - 1) * C or a_log32.numel() != heads or dt_bias32.numel() != heads * dim:
        raise KernelError("delta_prep: state or decay parameters do not fit")
    dev = main.device
    f = lambda *shape: torch.empty(shape, dtype=torch.float32, device=dev)
    q, k, v = f(T, kv_heads, dim), f(T, kv_heads, dim), f(T, heads, vdim)
    beta, g, gate = f(T, heads), f(T, heads, dim), f(T, heads, vdim)
    _ok(lib().acorn_delta_prep(main.data_ptr(), main.stride(0), up32.data_ptr(), up32.stride(0), conv_w32.data_ptr(),
                               state.data_ptr(), state.stride(0), int(conv_off), a_log32.data_ptr(), dt_bias32.data_ptr(),
                               token_row.data_ptr(), row_start.data_ptr(), row_slot.data_ptr(), q.data_ptr(), k.data_ptr(),
                               v.data_ptr(), beta.data_ptr(), g.data_ptr(), gate.data_ptr(), T, heads, kv_heads, dim, vdim,
                               taps, dtype_code(main.dtype), _stream()), "delta_prep")
    return q, k, v, beta, g, gate


def conv_state_update(main: torch.Tensor, state: torch.Tensor, conv_off: int, row_start: torch.Tensor,
                      row_slot: torch.Tensor, num_rows: int, channels: int, taps: int, skip_single: bool = False,
                      bias32: torch.Tensor | None = None) -> None:
    """The last ``taps - 1`` convolution inputs of every row's request into its state.  ``skip_single``: rows of
    one token are left alone (the kernel before has shifted their memory: ``ssm_prep(update_single=True)``).
    ``bias32`` (float32 [channels]): added to the inputs as they are kept."""
    if bias32 is not None:
        _check(bias32, "bias", torch.float32, 1)
        if bias32.numel() != channels:
            raise KernelError("conv_state_update: one bias entry per channel")
    if main.shape[1] < channels or state.shape[1] < conv_off + (taps - 1) * channels:
        raise KernelError("conv_state_update: rows or state slots too small for the channels")
    _ok(lib().acorn_conv_state_update(main.data_ptr(), main.stride(0), state.data_ptr(), state.stride(0), int(conv_off),
                                      row_start.data_ptr(), row_slot.data_ptr(), num_rows, channels, taps,
                                      dtype_code(main.dtype), 1 if skip_single else 0, _ptr(bias32), _stream()),
        "conv_state_update")


DELTA_MIN_SEGMENT = 64              # tokens: shorter segments are not worth a second pass
DELTA_MAX_SEGMENTS = 16
DELTA_WAVE_BLOCKS = 296             # blocks of the segmented passes that run at once (148 SMs x 2: their shared memory)


def delta_segments(longest_row: int, num_rows: int, heads: int, dim: int, vdim: int) -> tuple[int, int]:
    """(tokens a segment, segments a row) for the form of ``delta_rule`` that reads the state first; (0, 1): rows in
    one piece.  Rows run side by side with heads and tiles of columns; where those are too few to fill the device
    and a row is long, rows are cut into segments that run side by side, at the price of a second pass: as many
    as still run at once (a second wave of blocks would wait for the first)."""
    cols = 64 if dim <= 128 else 16                                     # columns a block of the segmented passes takes
    blocks = num_rows * heads * -(-vdim // cols)
    nseg = min(DELTA_MAX_SEGMENTS, longest_row // DELTA_MIN_SEGMENT, DELTA_WAVE_BLOCKS // max(blocks, 1))
    if nseg < 2:
        return 0, 1
    return -(-longest_row // nseg), nseg


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor | None, g: torch.Tensor,
               state: torch.Tensor, row_start: torch.Tensor, row_slot: torch.Tensor, num_rows: int,
               bonus32: torch.Tensor | None = None, longest_row: int | None = None) -> torch.Tensor:
    """The recurrence over every row's tokens from the state in its slot (updated in place): float32
    o [T, H, vdim].  With ``bonus32`` (float32 [H, dim]) and no ``beta`` the form without the delta correction
    whose output reads the state before the token's decay and write and sees the token itself through the
    bonus: ``o = S^T q + (sum_d q_d bonus_d k_d) v;  S = diag(g) S + k v^T``.  In that form, with ``longest_row``
    (the most tokens a row of the step brings, a host value), long rows of a step with few rows run in segments
    side by side (``delta_segments``)."""
    T, H, vdim = v.shape
    KH, dim = q.shape[1], q.shape[2]
    if (beta is None) == (bonus32 is None):
        raise KernelError("delta_rule: give beta (the delta rule) or bonus32 (the form that reads the state first)")
    if bonus32 is not None:
        _check(bonus32, "bonus", torch.float32, 2)
        if bonus32.shape != (H, dim):
            raise KernelError(f"delta_rule: bonus {tuple(bonus32.shape)} is not [H, dim] = [{H}, {dim}]")
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (g, "g")) + (((beta, "beta"),) if beta is not None else ()):
        _check(t, n, torch.float32)
    _check(state, "state", torch.float32, 2)
    if state.shape[1] < H * dim * vdim or g.shape != (T, H, dim) or dim > 256:
        raise KernelError(f"delta_rule: sizes do not fit (state {tuple(state.shape)}, H={H}, dim={dim}, vdim={vdim})")
    out = torch.empty((T, H, vdim), dtype=torch.float32, device=v.device)
    seg_len, nseg = delta_segments(longest_row, num_rows, H, dim, vdim) if (bonus32 is not None and longest_row) else (0, 1)

    def run(pass_, seg_state=None, seg_decay=None):
        _ok(lib().acorn_delta_rule(q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(beta), g.data_ptr(), state.data_ptr(),
                                   state.stride(0), row_start.data_ptr(), row_slot.data_ptr(), out.data_ptr(), num_rows, H,
                                   KH, dim, vdim, _ptr(bonus32), pass_, nseg, max(seg_len, 1), _ptr(seg_state),
                                   _ptr(seg_decay), _stream()), "delta_rule", f"pass {pass_}")

    if nseg == 1:
        run(0)
        return out
    seg_state = torch.empty((num_rows * nseg, H, dim, vdim), dtype=torch.float32, device=v.device)
    seg_decay = torch.empty((num_rows * nseg, H, dim), dtype=torch.float32, device=v.device)
    run(1, seg_state, seg_decay)
    _ok(lib().acorn_delta_fold(state.data_ptr(), state.stride(0), row_slot.data_ptr(), seg_state.data_ptr(),
                               seg_decay.data_ptr(), num_rows, nseg, H, dim, vdim, _stream()), "delta_fold")
    run(2, seg_state, seg_decay)
    return out


def delta_out(o32: torch.Tensor, gate32: torch.Tensor, weight32: torch.Tensor, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """Per token and head o / rms(o) * weight * gate -> [T, H * vdim] in ``dtype``.  ``weight32``: [vdim],
    shared by the heads, or [H * vdim], a weight per head."""
    T, H, vdim = o32.shape
    _check(o32, "o", torch.float32, 3)
    _check(gate32, "gate", torch.float32, 3)
    _check(weight32, "weight", torch.float32, 1)
    if weight32.numel() not in (vdim, H * vdim):
        raise KernelError(f"delta_out: weight of {weight32.numel()} entries for heads of {vdim} ({H} heads)")
    y = torch.empty((T, H * vdim), dtype=dtype, device=o32.device)
    _ok(lib().acorn_delta_out(o32.data_ptr(), gate32.data_ptr(), weight32.data_ptr(), y.data_ptr(), T, H, vdim, float(eps),
                              dtype_code(dtype), 1 if (weight32.numel() == H * vdim and H > 1) else 0, _stream()), "delta_out")
    return y


# ------------------------------------------------------------------ time mixing with a matrix state


def token_shift(h: torch.Tensor, mu32: torch.Tensor, state: torch.Tensor, prev_off: int, token_row: torch.Tensor,
                row_start: torch.Tensor, row_slot: torch.Tensor, update_single: bool = False) -> torch.Tensor:
    """``out[s, t] = h[t] + (prev[t] - h[t]) * mu32[s]`` for every blend s: ``prev`` is the row before ``t`` in its
    request, for a step's first token the float32 row kept in the request's state slot at ``prev_off`` (which
    ``conv_state_update`` with two taps keeps; with ``update_single`` this kernel keeps it for rows of a single
    token, which that one then skips: ``skip_single``).  h [T, W]; mu32 [n, W]; returns [n, T, W] in h's dtype."""
    if not h.is_cuda or h.dim() != 2:
        raise KernelError("token_shift: h must be CUDA rows [T, W]")
    _check(mu32, "mu", torch.float32, 2)
    _check(state, "state", torch.float32, 2)
    T, W = h.shape
    n = mu32.shape[0]
    if mu32.shape[1] != W or not mu32.is_contiguous() or state.shape[1] < prev_off + W or h.stride(1) != 1:
        raise KernelError(f"token_shift: h {tuple(h.shape)}, mu {tuple(mu32.shape)}, state {tuple(state.shape)} do not fit")
    out = torch.empty((n, T, W), dtype=h.dtype, device=h.device)
    _ok(lib().acorn_token_shift(h.data_ptr(), h.stride(0), mu32.data_ptr(), state.data_ptr(), state.stride(0), int(prev_off),
                                token_row.data_ptr(), row_start.data_ptr(), row_slot.data_ptr(), out.data_ptr(), T, W, n,
                                dtype_code(h.dtype), 1 if update_single else 0, _stream()), "token_shift")
    return out


def wkv_prep(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, z32: torch.Tensor, w0_32: torch.Tensor,
             heads: int):
    """For the recurrence, float32 [T, H, dim] each: r, k, v as they are, the decay ``exp(-exp(z + w0))`` and the
    gate ``silu(g)``.  r, k, v, g: [T, H dim] of the activation dtype with one row stride; z32 [T, H dim] float32."""
    T, C = r.shape
    for t, n in ((r, "r"), (k, "k"), (v, "v"), (g, "g")):
        if not t.is_cuda or t.dtype != r.dtype or t.dim() != 2:
            raise KernelError(f"wkv_prep: {n} must be CUDA rows of one dtype")
        if t.shape != (T, C) or t.stride(0) != r.stride(0) or t.stride(1) != 1:
            raise KernelError("wkv_prep: r, k, v, g must have one shape and row stride")
    _check(z32, "z", torch.float32, 2)
    _check(w0_32, "w0", torch.float32, 1)
    if z32.shape != (T, C) or w0_32.numel() != C or C % heads:
        raise KernelError(f"wkv_prep: z {tuple(z32.shape)} / w0 {w0_32.numel()} do not fit [{T}, {C}]")
    outs = torch.empty((5, T, heads, C // heads), dtype=torch.float32, device=r.device)
    _ok(lib().acorn_wkv_prep(r.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), r.stride(0), z32.data_ptr(),
                             z32.stride(0), w0_32.data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(),
                             outs[3].data_ptr(), outs[4].data_ptr(), T, C, dtype_code(r.dtype), _stream()), "wkv_prep")
    return outs[0], outs[1], outs[2], outs[3], outs[4]


# ------------------------------------------------------------------ plain activations, a token's side rows

ACTIVATIONS = {"relu_squared": 0, "tanh": 1, "gelu_tanh": 2, "silu": 3}


def activation_rows(x: torch.Tensor, kind: str) -> torch.Tensor:
    return activation(x, kind)


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """``act(x)`` elementwise over rows [T, n] (a row stride is allowed); float32 arithmetic, one rounding."""
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation must be one of {sorted(ACTIVATIONS)}, got {kind!r}")
    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("activation: x must be CUDA rows [T, n] with contiguous entries")
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    _ok(lib().acorn_activation(x.data_ptr(), x.stride(0), out.data_ptr(), x.shape[0], x.shape[1], ACTIVATIONS[kind],
                               dtype_code(x.dtype), _stream()), "activation")
    return out


def side_gate_linear(x: torch.Tensor, w: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, col0: int) -> torch.Tensor:
    """``gelu_tanh(x w^T)[t] * table[token_ids[t], col0 : col0 + n]`` for x [T, K], w [n, K]: the gate as the epilogue
    of the one-CTA tcgen05 product where that runs (bfloat16, at most GEMM_TC_MAX_ROWS rows: the product is not
    rounded before the gate), else the product followed by ``side_gate``."""
    _check(table, "table", x.dtype, 2)
    _check(token_ids, "token_ids", torch.int32, 1)
    T, n = x.shape[0], w.shape[0]
    if table.stride(1) != 1 or col0 < 0 or col0 + n > table.shape[1] or token_ids.numel() != T:
        raise KernelError(f"side_gate_linear: x {tuple(x.shape)} / w {tuple(w.shape)} / table {tuple(table.shape)} / "
                          f"first column {col0} do not fit")
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and T <= GEMM_TC_MAX_ROWS and gemm_tc_supported(x, w)):
        return side_gate(linear(x, w, out_dtype=x.dtype), token_ids, table, col0)
    K = x.shape[1]
    splits, per_sm = gemm_tc_plan(T, n, K, device_sms(x.device))
    out = torch.empty((T, n), dtype=torch.bfloat16, device=x.device)
    _ok(lib().acorn_gemm_tc_gelu_rows(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
                                      T, n, K, int(splits), int(per_sm), token_ids.data_ptr(), table.data_ptr(),
                                      table.stride(0), int(col0), _stream()), "gemm_tc_side_gate", f"{T}x{n}x{K}")
    return out


def side_gate(z: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, col0: int) -> torch.Tensor:
    """``gelu_tanh(z[t]) * table[token_ids[t], col0 : col0 + n]`` for z [T, n]."""
    _check(z, "z", None, 2)
    _check(table, "table", z.dtype, 2)
    _check(token_ids, "token_ids", torch.int32, 1)
    T, n = z.shape
    if not z.is_contiguous() or table.stride(1) != 1 or col0 < 0 or col0 + n > table.shape[1]:
        raise KernelError(f"side_gate: z {tuple(z.shape)} / table {tuple(table.shape)} / first column {col0} do not fit")
    out = torch.empty_like(z)
    _ok(lib().acorn_side_gate(z.data_ptr(), token_ids.data_ptr(), table.data_ptr(), table.stride(0), int(col0),
                              out.data_ptr(), T, n, dtype_code(z.dtype), _stream()), "side_gate")
    return out


# ------------------------------------------------------------------ layer norm, sums, head gates


def add_layernorm(resid32: torch.Tensor, delta, weight32: torch.Tensor, bias32: torch.Tensor | None, eps: float,
                  out_dtype: torch.dtype, row_idx: torch.Tensor | None = None,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """resid32 += delta (in place, unless row_idx is given); returns the layer norm of it,
    ``(x - mean) / sqrt(var + eps) * weight + bias``.  ``delta``: None, a tensor, or a ``DeltaPair`` (both are added)."""
    _check(resid32, "resid32", torch.float32, 2)
    _check(weight32, "weight", torch.float32, 1)
    H = resid32.shape[1]
    if weight32.numel() != H or (bias32 is not None and bias32.numel() != H):
        raise KernelError(f"norm weight / bias do not have the width {H}")
    d1, d2 = (delta.a, delta.b) if isinstance(delta, DeltaPair) else (delta, None)
    for d in (d1, d2):
        if d is not None:
            _check(d, "delta", out_dtype, 2)
            if d.shape != resid32.shape:
                raise KernelError(f"delta {tuple(d.shape)} does not match the residual {tuple(resid32.shape)}")
    rows = resid32.shape[0]
    if row_idx is not None:
        _check(row_idx, "row_idx", torch.int32, 1)
        rows = row_idx.numel()
    if out is None:
        out = torch.empty((rows, H), dtype=out_dtype, device=resid32.device)
    _check(out, "out", out_dtype, 2)
    _ok(lib().acorn_add_layernorm(resid32.data_ptr(), _ptr(d1), _ptr(d2), weight32.data_ptr(), _ptr(bias32),
                                  out.data_ptr(), _ptr(row_idx), rows, H, float(eps), dtype_code(out_dtype), _stream()),
        "add_layernorm")
    return out


class DeltaPair:
    """Two results that are both still to be added to the residual stream (the mixer's and the
    feed-forward's of a block whose sublayers read the same normed rows)."""

    def __init__(self, a: torch.Tensor, b: torch.Tensor):
        self.a, self.b = a, b


def add_into(resid32: torch.Tensor, delta: torch.Tensor) -> None:
    """resid32 += delta (float32 sum, in place)."""
    _check(resid32, "resid32", torch.float32)
    _check(delta, "delta")
    if delta.shape != resid32.shape:
        raise KernelError(f"add_into: {tuple(delta.shape)} onto {tuple(resid32.shape)}")
    _ok(lib().acorn_add_into(resid32.data_ptr(), delta.data_ptr(), resid32.numel(), dtype_code(delta.dtype), _stream()),
        "add_into")


def fold_pair(resid32: torch.Tensor, delta):
    """A ``DeltaPair`` as one pending result: the first is added to the stream now, the second handed on."""
    if isinstance(delta, DeltaPair):
        add_into(resid32, delta.a)
        return delta.b
    return delta


def head_gate(x: torch.Tensor, gate: torch.Tensor | None, heads: int, scale: float = 1.0,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, heads * d] times scale * sigmoid(gate[:, h]) per head, in place or into ``out`` (rows of another
    buffer).  ``gate`` [T, >= heads] may be a slice of a wider buffer; None: x * scale."""
    _check(x, "x", None, 2)
    out = x if out is None else out
    _rows2(out, "out", x.dtype)
    if out.shape != x.shape:
        raise KernelError(f"head_gate: out {tuple(out.shape)} for x {tuple(x.shape)}")
    if gate is not None and (gate.dtype != x.dtype or gate.dim() != 2 or gate.stride(1) != 1
                             or gate.shape[0] != x.shape[0] or gate.shape[1] < heads):
        raise KernelError(f"head_gate: gate {tuple(gate.shape)} {gate.dtype} does not fit x {tuple(x.shape)} {x.dtype}")
    if x.shape[1] % heads:
        raise KernelError("head_gate: the row is not a whole number of heads")
    _ok(lib().acorn_head_gate(x.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(),
                              out.stride(0), x.shape[0], heads, x.shape[1] // heads, float(scale), dtype_code(x.dtype),
                              _stream()), "head_gate")
    return out


# ------------------------------------------------------------------ linear recurrences (state space, linear attention)


def _rows2(t: torch.Tensor, name: str, dtype=None):
    """A [T, W] view whose rows may be strided (a slice of a wider buffer)."""
    if t.dim() != 2 or t.stride(1) != 1 or (dtype is not None and t.dtype != dtype) or not t.is_cuda:
        raise KernelError(f"{name}: expected a 2-d {dtype or ''} device tensor with unit column stride, got "
                          f"{tuple(t.shape)} {t.dtype} strides {t.stride()}")


def ssm_prep(proj: torch.Tensor, conv_col: int, dt_col: int, conv_w32: torch.Tensor, conv_b32: torch.Tensor | None,
             state: torch.Tensor, conv_off: int, a_log32: torch.Tensor, dt_bias32: torch.Tensor,
             token_row: torch.Tensor, row_start: torch.Tensor, row_slot: torch.Tensor, taps: int,
             update_single: bool = False):
    """Of a projection ``proj`` [T, W]: the short causal convolution (``taps`` weights per channel, the last for
    the current token; inputs before the step from the request's state at ``conv_off``) with bias and silu of the
    ``C`` channels from column ``conv_col``, and of the ``H`` columns from ``dt_col`` the step sizes
    ``softplus(. + dt_bias)`` and the decays ``exp(-exp(A_log) dt)``.  Returns float32 (act [T, C], dt [T, H], decay [T, H]).
    ``update_single``: the convolution's memory of rows of one token is shifted here as well (rows of more tokens
    need ``conv_state_update(skip_single=True)`` after this)."""
    _rows2(proj, "proj")
    _check(state, "state", torch.float32, 2)
    _check(conv_w32, "conv weights", torch.float32, 2)
    T = proj.shape[0]
    C, H = conv_w32.shape[0], a_log32.numel()
    if conv_w32.shape[1] != taps or (conv_b32 is not None and conv_b32.numel() != C) or dt_bias32.numel() != H:
        raise KernelError("ssm_prep: convolution or step-size parameters do not fit")
    if conv_col + C > proj.shape[1] or dt_col + H > proj.shape[1] or state.shape[1] < conv_off + (taps - 1) * C:
        raise KernelError("ssm_prep: columns beyond the projection, or a state too small for the convolution's memory")
    f = lambda *shape: torch.empty(shape, dtype=torch.float32, device=proj.device)
    act, dt, decay = f(T, C), f(T, H), f(T, H)
    _ok(lib().acorn_ssm_prep(proj.data_ptr(), proj.stride(0), int(conv_col), int(dt_col), conv_w32.data_ptr(),
                             _ptr(conv_b32), state.data_ptr(), state.stride(0), int(conv_off), a_log32.data_ptr(),
                             dt_bias32.data_ptr(), token_row.data_ptr(), row_start.data_ptr(), row_slot.data_ptr(),
                             act.data_ptr(), dt.data_ptr(), decay.data_ptr(), T, C, H, taps, dtype_code(proj.dtype),
                             1 if update_single else 0, _stream()), "ssm_prep")
    return act, dt, decay


def silu_rows(x: torch.Tensor) -> torch.Tensor:
    """silu(x) as float32 [T, W]; ``x`` may be a column slice of a wider buffer."""
    _rows2(x, "x")
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _ok(lib().acorn_silu_rows(x.data_ptr(), x.stride(0), out.data_ptr(), x.shape[0], x.shape[1], dtype_code(x.dtype),
                              _stream()), "silu_rows")
    return out


SCAN_MIN_SEGMENT = 64             # tokens: shorter segments are not worth a second pass
SCAN_MAX_SEGMENTS = 16
SCAN_ENOUGH_BLOCKS = 2400         # blocks of 128 threads that fill the device (148 SMs, 16 a piece)
SCAN_SCRATCH_BYTES = 1 << 30


def scan_segments(longest_row: int, num_rows: int, heads: int, n: int, v: int) -> tuple[int, int]:
    """(tokens a segment, segments a row) for ``linear_scan``, (0, 1) for rows in one piece.  Rows run
    side by side with heads and tiles of columns; where those are too few to fill the device and a row is
    long, rows are cut into segments that run side by side (at the price of a second pass)."""
    lanes = 1
    while lanes * 16 < n:
        lanes *= 2
    blocks = num_rows * heads * -(-v // (128 // lanes))
    nseg = min(SCAN_MAX_SEGMENTS, longest_row // SCAN_MIN_SEGMENT, -(-SCAN_ENOUGH_BLOCKS // blocks), 65535 // max(1, num_rows),
               SCAN_SCRATCH_BYTES // (4 * num_rows * heads * n * v) - 1)
    if nseg < 2:
        return 0, 1
    return -(-longest_row // nseg), nseg


def linear_scan(b: torch.Tensor, c: torch.Tensor, x: torch.Tensor, decay: torch.Tensor, w: torch.Tensor | None,
                skip32: torch.Tensor | None, state: torch.Tensor, state_off: int, row_start: torch.Tensor,
                row_slot: torch.Tensor, num_rows: int, heads: int, groups: int, n: int, v: int,
                longest_row: int = 1) -> torch.Tensor:
    """Per head ``S <- a S + b (w x)^T; y = S^T c + skip x`` over every row's tokens, from the state in the
    row's slot (``[heads, v, n]`` float32 at ``state_off``, updated in place).  ``b``, ``c`` [T, groups * n],
    ``x`` [T, heads * v] float32 (column slices allowed); ``decay`` [T, heads] per token or [heads] for all;
    ``w`` [T, heads] or None.  Returns float32 y [T, heads * v].  ``longest_row``: a bound on the tokens of a row
    (a host number); long rows of a step with few rows are run in segments side by side (``scan_segments``)."""
    for t, name in ((b, "b"), (c, "c"), (x, "x")):
        _rows2(t, name, torch.float32)
    _check(state, "state", torch.float32, 2)
    T = x.shape[0]
    if b.shape != (T, groups * n) or c.shape != (T, groups * n) or x.shape[1] != heads * v:
        raise KernelError(f"linear_scan: b {tuple(b.shape)}, c {tuple(c.shape)}, x {tuple(x.shape)} do not fit "
                          f"heads={heads}, groups={groups}, n={n}, v={v}")
    if heads % groups or n > 512 or state.shape[1] < state_off + heads * n * v:
        raise KernelError("linear_scan: sizes not supported (groups must divide heads, n <= 512) or state too small")
    if decay.dtype != torch.float32 or (decay.dim() == 1 and decay.numel() != heads) or \
            (decay.dim() == 2 and (decay.shape != (T, heads) or decay.stride(1) != 1)):
        raise KernelError(f"linear_scan: decay {tuple(decay.shape)} is neither [T, heads] nor [heads]")
    if w is not None:
        _rows2(w, "w", torch.float32)
    if skip32 is not None:
        _check(skip32, "skip", torch.float32, 1)
    y = torch.empty((T, heads * v), dtype=torch.float32, device=x.device)
    seg, nseg = scan_segments(int(longest_row), num_rows, heads, n, v)
    seg_state = seg_decay = None
    if seg:
        seg_state = torch.empty((num_rows, nseg + 1, heads * n * v), dtype=torch.float32, device=x.device)
        seg_decay = torch.empty((num_rows, nseg, heads), dtype=torch.float32, device=x.device)
    _ok(lib().acorn_linear_scan(b.data_ptr(), b.stride(0), c.data_ptr(), c.stride(0), x.data_ptr(), x.stride(0),
                                decay.data_ptr(), decay.stride(0) if decay.dim() == 2 else 0, _ptr(w),
                                w.stride(0) if w is not None else 0, _ptr(skip32), state.data_ptr(), state.stride(0),
                                int(state_off), y.data_ptr(), row_start.data_ptr(), row_slot.data_ptr(), num_rows, heads,
                                groups, n, v, seg, nseg, _ptr(seg_state), _ptr(seg_decay), _stream()), "linear_scan")
    return y


def gated_norm(y32: torch.Tensor, gate: torch.Tensor, weight32: torch.Tensor, eps: float, groups: int, gate_first: bool,
               out: torch.Tensor, out_scale: float = 1.0) -> torch.Tensor:
    """RMS norm of ``y32`` [T, W] in ``groups`` equal parts times ``weight32``, with a gate ``z`` [T, W]:
    ``gate_first``: ``norm(y silu(z))``; else ``norm(y) sigmoid(z)``.  Times ``out_scale``, rounded once into ``out``
    [T, W] (a column slice of a wider buffer is allowed, as for ``gate``)."""
    _check(y32, "y", torch.float32, 2)
    _rows2(gate, "gate")
    _rows2(out, "out", gate.dtype)
    _check(weight32, "weight", torch.float32, 1)
    T, W = y32.shape
    if gate.shape != (T, W) or out.shape != (T, W) or weight32.numel() != W or W % groups:
        raise KernelError(f"gated_norm: y {tuple(y32.shape)}, gate {tuple(gate.shape)}, out {tuple(out.shape)}, groups {groups}")
    _ok(lib().acorn_gated_norm(y32.data_ptr(), gate.data_ptr(), gate.stride(0), weight32.data_ptr(), out.data_ptr(),
                               out.stride(0), T, W, groups, float(eps), 0 if gate_first else 1, float(out_scale),
                               dtype_code(gate.dtype), _stream()), "gated_norm")
    return out


# ------------------------------------------------------------------ routed experts


def moe_route(z32: torch.Tensor, correction32: torch.Tensor, top: int, groups: int, keep: int, normalize: bool = False):
    """(chosen [T, top] int32, weights [T, top] float32) from router logits z [T, N].  ``normalize``: the
    chosen outputs' scores are divided by their sum (+ 1e-20)."""
    _check(z32, "router logits", torch.float32, 2)
    _check(correction32, "correction", torch.float32, 1)
    T, N = z32.shape
    if correction32.numel() != N:
        raise KernelError("moe_route: correction must have one entry per router output")
    idx = torch.empty((T, top), dtype=torch.int32, device=z32.device)
    wts = torch.empty((T, top), dtype=torch.float32, device=z32.device)
    _ok(lib().acorn_moe_route(z32.data_ptr(), correction32.data_ptr(), idx.data_ptr(), wts.data_ptr(), T, N, int(top),
                              int(groups), int(keep), 1 if normalize else 0, _stream()), "moe_route")
    return idx, wts


def moe_plan(idx: torch.Tensor, num_outputs: int):
    """Groups the (token, choice) pairs by chosen output: (offsets [N + 1], slot_of [T, top], slot_token
    [T * top]), all int32."""
    _check(idx, "idx", torch.int32, 2)
    T, top = idx.shape
    dev = idx.device
    offsets = torch.empty(num_outputs + 1, dtype=torch.int32, device=dev)
    slot_of = torch.empty((T, top), dtype=torch.int32, device=dev)
    slot_token = torch.empty(T * top, dtype=torch.int32, device=dev)
    _ok(lib().acorn_moe_plan(idx.data_ptr(), offsets.data_ptr(), slot_of.data_ptr(), slot_token.data_ptr(), T * top,
                             num_outputs, top, _stream()), "moe_plan")
    return offsets, slot_of, slot_token


GROUPED_TCGEN05_MIN_ROWS = 64      # rows an expert on average from which the grouped product takes the tcgen05 kernel


def grouped_gemm(a: torch.Tensor, a_rows: torch.Tensor | None, w: torch.Tensor, offsets: torch.Tensor, slots: int,
                 swiglu_pairs: bool = False, activation: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """out[slot] = a[a_rows[slot]] @ w[e]^T for the slots offsets[e] .. offsets[e + 1] - 1 of every
    expert e (w [E, N, K]); rows of other slots are left unwritten.  ``swiglu_pairs``: rows 2i and 2i + 1 of
    ``w[e]`` are the gate and the up row of output i, and what is returned is ``silu(gate) * up``
    [slots, N / 2]: inside the product's epilogue on the tensor-core kernel, by the SwiGLU kernel after it
    otherwise.  ``activation="capped_swish"`` with ``limit`` L: the capped form instead of silu (see ``swiglu``)."""
    if activation not in ("silu", "capped_swish") or (activation == "capped_swish" and not limit > 0):
        raise KernelError(f"grouped_gemm: activation {activation!r} with limit {limit}")
    glu_limit = float(limit) if activation == "capped_swish" else 0.0
    _check(a, "a", None, 2)
    _check(w, "w", a.dtype, 3)
    E, N, K = w.shape
    if a.shape[1] != K:
        raise KernelError(f"grouped_gemm: a {tuple(a.shape)} against w {tuple(w.shape)}")
    fused = swiglu_pairs and a.data_ptr() % 16 == 0 and bool(
        lib().acorn_grouped_gemm_fuses_swiglu(N, K, a.stride(0), dtype_code(a.dtype)))
    if (a.dtype == torch.bfloat16 and slots >= GROUPED_TCGEN05_MIN_ROWS * E and K % 8 == 0 and a.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and (N % 2 == 0 or not swiglu_pairs)):
        # many rows an expert (a prompt's step): tiles of 128 rows on the tcgen05 kernel, operand tiles by TMA, which
        # wants an expert's rows next to one another: the tokens' rows are first copied into slot order
        if a_rows is not None:
            rows_in = torch.empty((slots, K), dtype=a.dtype, device=a.device)
            _ok(lib().acorn_gather_rows(a.data_ptr(), a_rows.data_ptr(), rows_in.data_ptr(), slots, K, dtype_code(a.dtype),
                                        _stream()), "gather_rows")
        else:
            rows_in = a
        out = torch.empty((slots, N // 2 if swiglu_pairs else N), dtype=a.dtype, device=a.device)
        _ok(lib().acorn_grouped_gemm_tcgen05(rows_in.data_ptr(), rows_in.stride(0), w.data_ptr(), out.data_ptr(), out.stride(0),
                                             offsets.data_ptr(), slots, E, N, K, 1 if swiglu_pairs else 0, glu_limit, _stream()),
            "grouped_gemm_tcgen05", f"{slots}x{N}x{K}")
        return out
    out = torch.empty((slots, N // 2 if fused else N), dtype=a.dtype, device=a.device)
    _ok(lib().acorn_grouped_gemm(a.data_ptr(), a.stride(0), _ptr(a_rows), w.data_ptr(), out.data_ptr(), out.stride(0),
                                 offsets.data_ptr(), slots, E, N, K, dtype_code(a.dtype), 1 if fused else 0, glu_limit, _stream()),
        "grouped_gemm", f"{slots}x{N}x{K}")
    if swiglu_pairs and not fused:
        return swiglu(out, block=1, activation=activation, limit=limit)
    return out


def moe_combine(y: torch.Tensor, x: torch.Tensor, slot_of: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor,
                num_experts: int, resid32: torch.Tensor | None = None, weight32: torch.Tensor | None = None,
                eps: float = 0.0, extra: torch.Tensor | None = None) -> torch.Tensor | None:
    """out[t] = sum_k wts[t, k] * (idx[t, k] >= num_experts ? x[t] : y[slot_of[t, k]]).  With ``resid32`` the
    float32 sum is not returned but RMS-normed (``weight32``, ``eps``) and added to ``resid32`` in place; what
    is returned is then the new stream rounded to ``x``'s dtype (None if that is float32).  ``extra`` [T, H]: added
    to every token's sum (what all tokens take beside their choices: a shared expert)."""
    _check(y, "y", x.dtype, 2)
    if extra is not None:
        _check(extra, "extra", x.dtype, 2)
        if extra.shape != x.shape:
            raise KernelError("moe_combine: extra does not fit")
    _check(x, "x", None, 2)
    T, H = x.shape
    fused = resid32 is not None
    if fused:
        _check(resid32, "resid32", torch.float32, 2)
        _check(weight32, "norm weight", torch.float32, 1)
        if resid32.shape != x.shape or weight32.numel() != H:
            raise KernelError("moe_combine: residual or norm weight do not fit")
    out = None if (fused and x.dtype == torch.float32) else torch.empty_like(x)
    _ok(lib().acorn_moe_combine(y.data_ptr(), x.data_ptr(), slot_of.data_ptr(), idx.data_ptr(), wts.data_ptr(), _ptr(out),
                                T, H, idx.shape[1], int(num_experts), dtype_code(x.dtype), _ptr(resid32), _ptr(weight32),
                                float(eps), _ptr(extra), _stream()), "moe_combine")
    return out



def diff_combine(a: torch.Tensor, gate: torch.Tensor | None, heads: int, value_dim: int, lam: float, scale: float,
                 eps: float) -> torch.Tensor:
    """a [T, heads * 2 * value_dim]: per head the outputs a1, a2 of its two score maps.  Returns
    ``unit_rms(a1 - lam a2) * scale * sigmoid(gate)`` [T, heads * value_dim] (``gate`` [T, >= heads * value_dim], a
    slice of a wider buffer, or None); float32 arithmetic, one rounding."""
    _check(a, "a", None, 2)
    T = a.shape[0]
    if a.shape[1] != heads * 2 * value_dim:
        raise KernelError(f"diff_combine: a {tuple(a.shape)} is not [T, {heads} * 2 * {value_dim}]")
    if gate is not None and (gate.dtype != a.dtype or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[0] != T
                             or gate.shape[1] < heads * value_dim):
        raise KernelError(f"diff_combine: gate {tuple(gate.shape)} {gate.dtype} does not fit")
    out = torch.empty((T, heads * value_dim), dtype=a.dtype, device=a.device)
    _ok(lib().acorn_diff_combine(a.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(), T,
                                 heads, value_dim, float(lam), float(scale), float(eps), dtype_code(a.dtype), _stream()),
        "diff_combine")
    return out


def pair_rows(a32: torch.Tensor, b32: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """``[a | b]`` of two float32 streams [T, H], rounded to ``dtype``: [T, 2 H]."""
    _check(a32, "a", torch.float32, 2)
    _check(b32, "b", torch.float32, 2)
    if a32.shape != b32.shape:
        raise KernelError("pair_rows: the streams differ in shape")
    out = torch.empty((a32.shape[0], 2 * a32.shape[1]), dtype=dtype, device=a32.device)
    _ok(lib().acorn_pair_rows(a32.data_ptr(), b32.data_ptr(), out.data_ptr(), a32.shape[0], a32.shape[1], dtype_code(dtype),
                              _stream()), "pair_rows")
    return out


def add_row(x32: torch.Tensor, row32: torch.Tensor) -> torch.Tensor:
    """x32 [T, H] += row32 [H], in place (float32)."""
    _check(x32, "x", torch.float32, 2)
    _check(row32, "row", torch.float32, 1)
    if row32.numel() != x32.shape[1]:
        raise KernelError("add_row: the row does not fit")
    _ok(lib().acorn_add_row(x32.data_ptr(), row32.data_ptr(), x32.shape[0], x32.shape[1], _stream()), "add_row")
    return x32

# ------------------------------------------------------------------ sampling


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, counter: torch.Tensor, want_logprobs: bool = False):
    """One token per row of float32 logits.  Per-row parameters are device tensors:
    temperature/top_p float32, top_k int32, seed/counter int64 (used as unsigned)."""
    _check(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _check(temperature, "temperature", torch.float32, 1)
    _check(top_p, "top_p", torch.float32, 1)
    _check(top_k, "top_k", torch.int32, 1)
    _check(seed, "seed", torch.int64, 1)
    _check(counter, "counter", torch.int64, 1)
    for t in (temperature, top_k, top_p, seed, counter):
        if t.numel() != R:
            raise KernelError("per-row sampling parameters must have one entry per logits row")
    tokens = torch.empty(R, dtype=torch.int32, device=logits.device)
    logprobs = torch.empty(R, dtype=torch.float32, device=logits.device) if want_logprobs else None
    _ok(lib().acorn_sample(logits.data_ptr(), logits.stride(0), R, V, temperature.data_ptr(), top_k.data_ptr(),
                           top_p.data_ptr(), seed.data_ptr(), counter.data_ptr(), tokens.data_ptr(),
                           _ptr(logprobs), _stream()), "sample")
    return tokens, logprobs


def random_fill(out: torch.Tensor, key: int, first: int, scale: float, offset: float, kind: int) -> torch.Tensor:
    """Fills ``out`` (flat, contiguous) with elements ``first ..`` of the counter-based random tensor
    ``key``: ``offset + lane_sum * scale`` (kind 0 float32, 1 bfloat16) or 15-bit integers (kind 2)."""
    _check(out, "out", {0: torch.float32, 1: torch.bfloat16, 2: torch.int32}[kind])
    _ok(lib().acorn_random_fill(out.data_ptr(), out.numel(), ctypes.c_uint64(key), ctypes.c_uint64(first),
                                float(scale), float(offset), kind, _stream()), "random_fill")
    return out


def uniform(seed: int, counter: int) -> float:
    """The uniform number the sampling kernel draws for (seed, counter), computed on the host."""
    return float(lib_host().acorn_uniform(ctypes.c_uint64(seed & (2 ** 64 - 1)), ctypes.c_uint64(counter & (2 ** 64 - 1))))


def lib_host():
    """The library for its host-only helpers (no device needed)."""
    global _lib
    if _lib is not None:
        return _lib
    h = ctypes.CDLL(str(ensure_built()))
    h.acorn_uniform.argtypes = _Sigs.acorn_uniform
    h.acorn_uniform.restype = c_float
    return h
