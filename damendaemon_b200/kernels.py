"""Python face of the hand-written CUDA kernels (ctypes over the extern "C" launchers).

Every function takes CUDA tensors and launches on the current stream. There is no CPU
path and no library stand-in: a tensor that is not on a CUDA device, or a library that
cannot be built or loaded, raises ``KernelError``.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from .csrc import build

F32, BF16 = 0, 1
ACTIVATIONS = {None: 0, "none": 0, "gelu_new": 1, "gelu": 2, "relu2": 3}
GATED_FORMS = {"clamped_swish": 0, "silu": 1, "gelu_tanh": 2}     # the forms of a gated unit (csrc/common.cuh)

_c_int, _c_float, _c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "core": {
        "dd_device_arch": [],
        "dd_copy_to_device": [_c_void, _c_void, ctypes.c_longlong, _c_void],
        "dd_embed": [_c_void] * 5 + [_c_int] * 5 + [_c_float, _c_void, _c_void],
        "dd_layernorm": [_c_void] * 5 + [_c_int, _c_int, _c_float, _c_int, _c_void],
        "dd_rmsnorm": [_c_void] * 4 + [_c_int, _c_int, _c_float, _c_float, _c_int, _c_void],
        "dd_rmsnorm_groups": [_c_void] * 4 + [_c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_void],
        "dd_rmsnorm_shift": [_c_void] * 8 + [_c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_void],
        "dd_weighted_sum": [_c_void, ctypes.c_longlong, _c_void, _c_int, _c_void, _c_void],
        "dd_blend_rows": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_void],
        "dd_delta_state_rows": [_c_int],
        "dd_delta_prepare": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_void, _c_int] + [_c_void] * 11 + [_c_int] * 6 + [_c_void],
        "dd_conv_state_update": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
        "dd_delta_rule": [_c_void] * 7 + [_c_int, _c_void, _c_void] + [_c_int] * 4 + [_c_void],
        "dd_delta_finish": [_c_void] * 4 + [_c_int] * 4 + [_c_float, _c_int, _c_void],
        "dd_latent_prepare": [_c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_int, _c_int, _c_void, _c_float, _c_void, _c_int,
                              _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void],
        "dd_per_head_linear": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_int, _c_int] + [_c_int] * 6 + [_c_void],
        "dd_rotary": [_c_void, _c_void, _c_int, _c_void, _c_void, _c_float] + [_c_int] * 7 + [_c_void],
        "dd_gemm_simt_group_tile": [],
        "dd_gemm_simt_grouped": [_c_void, _c_int, _c_void, _c_int, ctypes.c_longlong, _c_void, _c_void, _c_int] + [_c_int] * 6 + [_c_void],
        "dd_route_by_table": [_c_void, _c_void] + [_c_int] * 6 + [_c_void] * 5,
        "dd_gather_rows": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
        "dd_gated_unit": [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_float, _c_float, _c_int, _c_void, _c_int, _c_void],
        "dd_combine_rows": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_int, _c_float, _c_void, _c_void],
        "dd_route_by_score": [_c_void, _c_int, _c_void, _c_int] + [_c_int] * 6 + [_c_float, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void],
        "dd_head_norm_rotary": [_c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_float] + [_c_int] * 7 + [_c_void],
        "dd_retention": [_c_void, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_void,
                         _c_float, _c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int, _c_void],
        "dd_retention_finish": [_c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void],
        "dd_gemm_simt": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int] + [_c_int] * 6 + [_c_void],
        "dd_kv_store": [_c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_void] + [_c_int] * 7 + [_c_void, _c_void],
        "dd_attention_rows": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_void, _c_void]
                             + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void, _c_void],
        "dd_attention_rows_masked": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_void, _c_void]
                                    + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int],
        "dd_attention_rows_sinks": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int, _c_void, _c_void]
                                   + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int,
                                      _c_int, _c_float, _c_void, _c_int],
        "dd_embed_pairs": [_c_void] * 9 + [_c_int] * 4 + [ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_void, _c_void],
        "dd_tanh_norm": [_c_void] * 6 + [_c_int, _c_int, _c_int, _c_void],
        "dd_add_rows": [_c_void, _c_void, _c_void, _c_int, _c_int, _c_void],
        "dd_norm_pair_add": [_c_void] * 5 + [_c_float, _c_float, _c_int, _c_int, _c_void],
        "dd_wide_norm_rotary": [_c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_float] + [_c_int] * 7 + [_c_void],
        "dd_sigmoid_gate": [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_int, _c_void],
        "dd_tanh_cap": [_c_void, ctypes.c_longlong, _c_float, _c_void],
        "dd_state_space_rows": [_c_int],
        "dd_conv_channels": [_c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int,
                             _c_int, _c_int, _c_int, _c_int, _c_void],
        "dd_state_space_scan": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_void]
                               + [_c_int] * 5 + [_c_void, _c_int],
        "dd_gated_group_norm": [_c_void, _c_void, _c_int, _c_void, _c_float, _c_void, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void],
        "dd_recurrence_gates": [_c_void] * 6 + [_c_float, _c_void, _c_void, _c_int, _c_int, _c_int, _c_void],
        "dd_linear_scan": [_c_void, _c_void, _c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void, _c_int, _c_int, _c_int,
                           _c_int, _c_void],
        "dd_sample": [_c_void, _c_int, _c_int, _c_int] + [_c_void] * 6,
        "dd_adjust_logits": [_c_void, _c_int, _c_int] + [_c_void] * 8 + [_c_int, _c_void],
    },
    "tensor": {
        "dd_gemm_tcgen05_plan": [_c_int, _c_int, _c_int, _c_int, _c_void, _c_void],
        "dd_gemm_grouped_tcgen05": [_c_void, _c_int, _c_void, _c_int, _c_int, _c_int, _c_void, _c_void, _c_int] + [_c_int] * 5
                                   + [_c_float, _c_float, _c_int, _c_void, _c_void, _c_int],
        "dd_wait_probe": [ctypes.c_ulonglong, _c_void, _c_void, _c_void],
        "dd_attention_decode_supported": [_c_int] * 4,
        "dd_attention_prefill_supported": [_c_int] * 4,
        "dd_attention_prefill": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int]
                                + [_c_int] * 6 + [_c_float, _c_void, _c_void, _c_int, _c_void, _c_int],
        "dd_attention_prefill_sinks": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int]
                                      + [_c_int] * 6 + [_c_float, _c_void, _c_void, _c_int, _c_void, _c_int, _c_int, _c_float, _c_void, _c_int],
        "dd_attention_latent_supported": [_c_int] * 3,
        "dd_attention_latent_tile": [_c_int] * 3,
        "dd_attention_latent": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int,
                                _c_void, _c_void] + [_c_int] * 5 + [_c_float, _c_int, _c_void, _c_void, _c_void],
        "dd_per_head_mma_supported": [_c_int] * 6,
        "dd_per_head_mma": [_c_void, _c_int, _c_int, _c_void, _c_void, _c_int, _c_int] + [_c_int] * 5 + [_c_void],
        "dd_attention_prefill_tcgen05_supported": [_c_int] * 5,
        "dd_attention_prefill_tcgen05": [_c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int]
                                        + [_c_int] * 6 + [_c_float, _c_void, _c_void, _c_int, _c_void, _c_int],
        "dd_attention_prefill_tcgen05_sink": [_c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_void, _c_void, _c_int, _c_int, _c_void, _c_int, _c_void, _c_int]
                                             + [_c_int] * 6 + [_c_float, _c_void, _c_void, _c_int, _c_void, _c_int, _c_void],
        "dd_attention_decode_pages_supported": [_c_int] * 5,
        "dd_attention_decode_pages_splits": [_c_int] * 5,
        "dd_attention_decode_pages": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int,
                                      _c_void, _c_void, _c_void] + [_c_int] * 7 + [_c_float, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int],
        "dd_attention_decode": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int,
                                _c_void, _c_void, _c_void] + [_c_int] * 7 + [_c_float, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int],
        "dd_attention_decode_sinks": [_c_void, _c_int, _c_void, _c_void, _c_void, _c_void, _c_void, _c_void, _c_int, _c_void, _c_int,
                                      _c_void, _c_void, _c_void] + [_c_int] * 7 + [_c_float, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int,
                                      _c_int, _c_float, _c_void, _c_int],
        "dd_gemm_tcgen05": [_c_void, _c_int, _c_void, _c_int, _c_void, _c_void, _c_int, _c_void, _c_int] + [_c_int] * 8
                           + [_c_void, _c_void, _c_int, _c_void, ctypes.c_longlong, _c_void, _c_void],
    },
}

_libs, _lock = {}, threading.Lock()


def library(name):
    """Load (building first if needed) one of the kernel libraries."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    with _lock:
        if name in _libs:
            return _libs[name]
        try:
            path = build.build_library(name)
            lib = ctypes.CDLL(str(path))
        except (build.BuildError, OSError) as error:
            raise KernelError(f"the '{name}' CUDA kernels are not available ({error}); "
                              "this engine has no CPU or library fallback") from error
        lib.dd_last_error.restype = ctypes.c_char_p
        lib.dd_set_pdl.argtypes, lib.dd_set_pdl.restype = [_c_int], _c_int
        lib.dd_set_pdl(1 if _pdl else 0)
        for fn, args in _SIGNATURES[name].items():
            f = getattr(lib, fn)
            f.argtypes, f.restype = args, _c_int
        _libs[name] = lib
        return lib


launches = 0          # kernels launched through this module (what the bench reports as gpu_launches)


def set_pdl(enabled):
    """Programmatic dependent launch for every kernel of both libraries (on by default)."""
    for name in list(_libs):
        _libs[name].dd_set_pdl(1 if enabled else 0)
    global _pdl
    _pdl = bool(enabled)


_pdl = True


class pdl_scope:
    """Kernels launched inside run with programmatic dependent launch on or off; the setting that was in force comes
    back afterwards. The float32 engine turns it off: its kernels (hundreds of blocks of CUDA-core work, no prologue
    worth starting early) were measured to run a decode step of 12 GPT-2 XL layers in 2.2 ms without it and in 2.6
    to 4.3 ms with it, while the bfloat16 kernels gain from it everywhere (1.78 against 2.34 ms for 48 layers)."""

    def __init__(self, enabled):
        self.enabled = bool(enabled)

    def __enter__(self):
        self.before = _pdl
        if self.enabled != self.before:
            set_pdl(self.enabled)

    def __exit__(self, *exc):
        if _pdl != self.before:
            set_pdl(self.before)
        return False


def _call(lib, fn, *args, n_kernels=1):
    global launches
    launches += n_kernels
    code = getattr(lib, fn)(*args)
    if code:
        raise KernelError(lib.dd_last_error().decode())


_scoped_stream = None


def _stream():
    return _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream


class stream_scope:
    """Every kernel launched inside the scope goes to the stream that was current when the scope was entered, looked
    up once: asking torch for the current stream costs a few microseconds, and a step launches hundreds of kernels.
    (Enter it inside a graph capture, not around it: the capture switches streams.)"""

    def __enter__(self):
        global _scoped_stream
        self.outer, _scoped_stream = _scoped_stream, torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self.outer
        return False


def _dt(t):
    if t is torch.float32 or t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t}")


def _ptr(t, name="tensor", dtype=None):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA only (no CPU fallback)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    return t.data_ptr()


def _rows(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with contiguous rows, has shape {tuple(t.shape)} strides {t.stride()}")
    return t


_error_flags = {}


def error_flag(device):
    """One int32 per device that kernels OR error bits into (1 bad token/position, 2 bad page
    on store, 4 bad page on read, 8 a bounded wait ran out)."""
    key = torch.device(device).index or 0
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def copy_to_device(dst, src, n_bytes):
    """One asynchronous host-to-device copy on the current stream, from pinned memory (src) into dst: the step's
    metadata. Not counted as a kernel launch."""
    global launches
    _call(library("core"), "dd_copy_to_device", dst.data_ptr(), src.data_ptr(), int(n_bytes), _stream(), n_kernels=0)


def read_error_flag(device):
    flag = error_flag(device)
    value = int(flag.item())
    if value:
        clear_after_error(device, value)
    return value


def clear_after_error(device, bits):
    """Zero the device's error word (in stream order) and, after a wait that ran out (bit 8), the split counters:
    a kernel that gave up may have left one short of its reset."""
    error_flag(device).zero_()
    key = torch.device(device).index or 0
    if bits & 8 and key in _counters:
        _counters[key].zero_()


def wait_probe(limit_ns, device):
    """Launch the block whose barrier nobody arrives at (csrc/wait_probe.cu) with a wait limit of limit_ns and
    return how long its two waiting warps waited, in ns. The device's error word then has bit 8 set, as after a
    wait that ran out in a pipelined kernel; read_error_flag reads and clears it."""
    waited = torch.zeros(2, dtype=torch.int64, device=device)
    _call(library("tensor"), "dd_wait_probe", int(limit_ns), _ptr(error_flag(device)), waited.data_ptr(), _stream())
    return waited.tolist()


# ---------------------------------------------------------------- kernels

def embed(ids, positions, token_table, position_table=None, out=None, scale=1.0):
    """x[t] = token_table[ids[t]] * scale (+ position_table[positions[t]]), float32."""
    n, width = ids.numel(), token_table.shape[1]
    if out is None:
        out = torch.empty((n, width), dtype=torch.float32, device=ids.device)
    if position_table is not None and position_table.dtype != token_table.dtype:
        raise KernelError("token and position tables must have one dtype")
    _call(library("core"), "dd_embed", _ptr(ids, "ids", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(token_table, "token table"), _ptr(position_table, "position table"), _ptr(out, "out", torch.float32),
          n, width, token_table.shape[0], 0 if position_table is None else position_table.shape[0],
          _dt(token_table.dtype), float(scale), _ptr(error_flag(ids.device)), _stream())
    return out


def embed_pairs(ids, positions, token_entry, entry_start, entry_slot, token_table, pair_table, last_id, mul_prev, mul_cur, out=None):
    """x[t] = token_table[ids[t]] + pair_table[row(t)], float32; row(t) = (id before * mul_prev + ids[t] * mul_cur) mod buckets
    with buckets = rows of pair_table - 1, and the table's last row for a token at position 0. ``last_id``: int32 [slots], the
    id before an entry's first token (read), replaced by the entry's last id."""
    n, width = ids.numel(), token_table.shape[1]
    if pair_table.dtype != token_table.dtype or pair_table.shape[1] != width or pair_table.shape[0] < 2 or \
            not pair_table.is_contiguous() or not token_table.is_contiguous():
        raise KernelError("embed_pairs: the pair table must have the token table's dtype and width")
    if last_id.dtype != torch.int32 or last_id.dim() != 1 or not last_id.is_contiguous():
        raise KernelError("embed_pairs: the state must be int32 [slots]")
    if out is None:
        out = torch.empty((n, width), dtype=torch.float32, device=ids.device)
    _call(library("core"), "dd_embed_pairs", _ptr(ids, "ids", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(token_entry, "token_entry", torch.int32), _ptr(entry_start, "entry_start", torch.int32),
          _ptr(entry_slot, "entry_slot", torch.int32), _ptr(token_table, "token table"), _ptr(pair_table, "pair table"),
          _ptr(last_id), _ptr(out, "out", torch.float32), n, width, token_table.shape[0], pair_table.shape[0] - 1, int(mul_prev),
          int(mul_cur), _dt(token_table.dtype), _ptr(error_flag(ids.device)), _stream())
    return out


def tanh_norm(x, alpha, weight, bias, out_dtype, row_index=None, out=None):
    """tanh(alpha * x) * weight + bias over float32 rows (alpha: float32, one number on the device), float32 inside."""
    _rows(x, "x")
    rows = x.shape[0] if row_index is None else row_index.numel()
    width = x.shape[1]
    if not x.is_contiguous():
        raise KernelError("tanh_norm input must be contiguous")
    for v, name, size in ((alpha, "alpha", 1), (weight, "weight", width), (bias, "bias", width)):
        if v.numel() != size or v.dtype != torch.float32 or not v.is_contiguous():
            raise KernelError(f"tanh_norm: {name} must be float32 with {size} element(s)")
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=x.device)
    _call(library("core"), "dd_tanh_norm", _ptr(x, "x", torch.float32), _ptr(row_index, "row_index", torch.int32), _ptr(alpha),
          _ptr(weight), _ptr(bias), _ptr(out, "out", out_dtype), rows, width, _dt(out_dtype), _stream())
    return out


def add_rows(x, other=None, vec=None):
    """x += other + vec in place: x float32 [N, width] contiguous, other the same shape or None, vec float32 [width] or None."""
    _rows(x, "x")
    if x.dtype != torch.float32 or not x.is_contiguous() or \
            (other is not None and (other.shape != x.shape or other.dtype != torch.float32 or not other.is_contiguous())) or \
            (vec is not None and (vec.numel() != x.shape[1] or vec.dtype != torch.float32 or not vec.is_contiguous())):
        raise KernelError("add_rows: float32 rows of one shape and a float32 vector of their width wanted")
    _call(library("core"), "dd_add_rows", _ptr(x), _ptr(other), _ptr(vec), x.shape[0], x.shape[1], _stream())
    return x


def norm_pair_add(x, left, right, left_weight, right_weight, eps, factor=0.5):
    """x += factor * (left / rms(left) * left_weight + right / rms(right) * right_weight), all float32 [N, width]."""
    for t in (x, left, right):
        if t.dtype != torch.float32 or not t.is_contiguous() or t.shape != x.shape or t.dim() != 2:
            raise KernelError("norm_pair_add: three contiguous float32 tensors of one shape wanted")
    for w in (left_weight, right_weight):
        if w.numel() != x.shape[1] or w.dtype != torch.float32 or not w.is_contiguous():
            raise KernelError("norm_pair_add: a weight must be float32 [width]")
    _call(library("core"), "dd_norm_pair_add", _ptr(x), _ptr(left), _ptr(right), _ptr(left_weight), _ptr(right_weight), float(eps),
          float(factor), x.shape[0], x.shape[1], _stream())
    return x


def wide_norm_rotary(q, k, positions, q_weight, k_weight, eps, q_heads, k_heads, head_dim, freqs=None, interleaved=True):
    """In place: q (and k, a row view of the same buffer, or None with k_heads 0) becomes x / sqrt(mean(x^2) + eps) * weight
    with the mean over the WHOLE projection (all heads at once) and a weight per element (float32 [heads * head_dim]; None:
    that kind is not normed); then the first 2 * len(freqs) dimensions of every head are rotated by position * freqs as in
    ``rotary``. All float32 inside."""
    if k is not None and (q.stride(0) != k.stride(0) or k.stride(1) != 1 or q.dtype != k.dtype or k.shape[1] != k_heads * head_dim):
        raise KernelError("wide_norm_rotary: q and k must be row views of one buffer")
    if q.stride(1) != 1 or q.shape[1] != q_heads * head_dim or (k is None) != (k_heads == 0):
        raise KernelError("wide_norm_rotary: shapes do not fit the heads")
    for w, heads in ((q_weight, q_heads), (k_weight, k_heads)):
        if w is not None and (w.numel() != heads * head_dim or w.dtype != torch.float32 or not w.is_contiguous()):
            raise KernelError("wide_norm_rotary: a weight must be float32 [heads * head_dim]")
    n_pairs = 0 if freqs is None else freqs.numel()
    _call(library("core"), "dd_wide_norm_rotary", _ptr(q, "q"), _ptr(k, "k"), q.stride(0), _ptr(positions, "positions", torch.int32),
          _ptr(freqs, "freqs", torch.float32), _ptr(q_weight, "q_weight"), _ptr(k_weight, "k_weight"), float(eps), q.shape[0],
          q_heads, k_heads, head_dim, n_pairs, 1 if interleaved else 0, _dt(q.dtype), _stream())
    return q, k


def sigmoid_gate(x, gate):
    """x *= sigmoid(gate) in place, element by element (float32 inside); x and gate row views of one shape and dtype."""
    if x.shape != gate.shape or x.dim() != 2 or x.stride(1) != 1 or gate.stride(1) != 1 or x.dtype != gate.dtype:
        raise KernelError("sigmoid_gate: two row views of one shape and dtype wanted")
    _call(library("core"), "dd_sigmoid_gate", _ptr(x, "x"), x.stride(0), _ptr(gate, "gate"), gate.stride(0), x.shape[0], x.shape[1],
          _dt(x.dtype), _stream())
    return x


def tanh_cap(x, cap):
    """x = cap * tanh(x / cap) in place; x float32 contiguous."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("tanh_cap: contiguous float32 wanted")
    _call(library("core"), "dd_tanh_cap", _ptr(x), x.numel(), float(cap), _stream())
    return x


def conv_channels(x, taps, bias, conv_state, token_entry, entry_start, entry_slot, activation=None, out=None):
    """A short causal convolution over time per channel: out[t, c] = act(bias[c] + sum_j taps[c, j] * x[t - (n - 1 - j), c]),
    float32 [N, channels]. x: a row view [N, channels]; taps float32 [channels, n]; bias float32 [channels] or None; the n - 1
    inputs before an entry's first token come from conv_state float32 [slots, n - 1, channels] (``conv_state_update`` leaves
    them there afterwards). activation: None or 'silu'."""
    n, channels = x.shape
    n_taps = taps.shape[1]
    if x.stride(1) != 1 or taps.shape[0] != channels or taps.dtype != torch.float32 or not taps.is_contiguous() or \
            conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or tuple(conv_state.shape[1:]) != (n_taps - 1, channels) or \
            (bias is not None and (bias.numel() != channels or bias.dtype != torch.float32 or not bias.is_contiguous())):
        raise KernelError("conv_channels: shapes do not fit")
    if out is None:
        out = torch.empty((n, channels), dtype=torch.float32, device=x.device)
    _call(library("core"), "dd_conv_channels", _ptr(x, "x"), x.stride(0), _ptr(taps), _ptr(bias), n_taps, _ptr(conv_state),
          _ptr(token_entry, "token_entry", torch.int32), _ptr(entry_start, "entry_start", torch.int32),
          _ptr(entry_slot, "entry_slot", torch.int32), _ptr(out), out.stride(0), n, channels, {None: 0, "silu": 1}[activation],
          _dt(x.dtype), _stream())
    return out


def state_space_state_shape(heads, state, value_dim):
    """Shape of one request's state-space state (float32): per head the columns of S one after the other, each padded to
    what the lanes of a column hold."""
    if not 0 < state <= 256 or value_dim <= 0:
        raise KernelError(f"state space: a state of {state} by {value_dim} is not supported (at most 256 rows)")
    lanes = 1
    while lanes * 8 < state:
        lanes *= 2
    return (int(heads), int(value_dim), 8 * lanes)          # what dd_state_space_rows answers


def state_space_scan(xbc, dt, dt_bias, a_log, skip, entry_start, entry_slot, state, heads, groups, n_state, value_dim, out=None):
    """The state-space recurrence of a step: per entry and head h, from the state in row entry_slot[e] of ``state`` (float32
    [slots, *state_space_state_shape(...)], read and written), token by token: step = softplus(dt + dt_bias[h]);
    S = exp(-exp(a_log[h]) * step) * S + step * B x^T; y = S^T C + skip[h] * x. xbc: float32 [N, heads * value_dim + 2 * groups *
    n_state] rows [x | B | C]; dt: a row view [N, heads]. Returns y float32 [N, heads * value_dim]."""
    n = xbc.shape[0]
    inner = heads * value_dim
    if xbc.dtype != torch.float32 or xbc.stride(1) != 1 or xbc.shape[1] != inner + 2 * groups * n_state or dt.shape != (n, heads) or \
            dt.stride(1) != 1 or state.dtype != torch.float32 or not state.is_contiguous() or \
            tuple(state.shape[1:]) != state_space_state_shape(heads, n_state, value_dim):
        raise KernelError("state_space_scan: shapes do not fit the state")
    for v in (dt_bias, a_log, skip):
        if v.numel() != heads or v.dtype != torch.float32 or not v.is_contiguous():
            raise KernelError("state_space_scan: the per-head parameters must be float32 [heads]")
    if out is None:
        out = torch.empty((n, inner), dtype=torch.float32, device=xbc.device)
    _call(library("core"), "dd_state_space_scan", _ptr(xbc), xbc.stride(0), _ptr(dt, "dt"), dt.stride(0), _ptr(dt_bias), _ptr(a_log),
          _ptr(skip), _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_slot, "entry_slot", torch.int32), entry_slot.numel(),
          _ptr(state), _ptr(out), heads, groups, n_state, value_dim, _dt(dt.dtype), _stream(), n)
    return out


def gated_group_norm(y, z, weight, groups, eps, out_dtype, out=None):
    """out = (y * silu(z)) in ``groups`` equal stretches, each divided by its root mean square (eps inside the root), times
    weight. y float32 [N, inner] contiguous; z a row view [N, inner] in out_dtype; weight float32 [inner]."""
    n, inner = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or z.shape != y.shape or z.stride(1) != 1 or z.dtype != out_dtype or \
            weight.numel() != inner or weight.dtype != torch.float32 or not weight.is_contiguous() or inner % groups:
        raise KernelError("gated_group_norm: shapes do not fit")
    if out is None:
        out = torch.empty((n, inner), dtype=out_dtype, device=y.device)
    _call(library("core"), "dd_gated_group_norm", _ptr(y), _ptr(z, "z"), z.stride(0), _ptr(weight), float(eps), _ptr(out), out.stride(0),
          n, int(groups), inner, _dt(out_dtype), _stream())
    return out


def recurrence_gates(u, wa, ba, wi, bi, lam, gain):
    """The gates of a gated linear recurrence, float32: with the channels of u [N, width] in ``blocks`` equal parts (wa, wi:
    float32 [blocks, part, part], [out, in]; ba, bi, lam: float32 [width]), r = sigmoid(wa u + ba), i = sigmoid(wi u + bi),
    a = exp(-gain * r * softplus(lam)). Returns (1 - a, sqrt(1 - a^2) * i * u), both float32 [N, width]: the decay travels as
    its distance from one, which float32 holds far more exactly for a slow channel than the decay itself."""
    n, width = u.shape
    blocks = wa.shape[0]
    ok = all(t.dtype == torch.float32 and t.is_contiguous() for t in (u, wa, ba, wi, bi, lam))
    if not ok or width % blocks or tuple(wa.shape) != (blocks, width // blocks, width // blocks) or wi.shape != wa.shape or \
            any(v.numel() != width for v in (ba, bi, lam)):
        raise KernelError("recurrence_gates: shapes do not fit")
    a = torch.empty_like(u)
    drive = torch.empty_like(u)
    _call(library("core"), "dd_recurrence_gates", _ptr(u), _ptr(wa), _ptr(ba), _ptr(wi), _ptr(bi), _ptr(lam), float(gain), _ptr(a),
          _ptr(drive), n, width, blocks, _stream())
    return a, drive


def linear_scan(a, drive, y, entry_start, entry_slot, state, activation=None, out=None):
    """S = S - a[t] * S + drive[t] (a holds 1 - decay, as ``recurrence_gates`` leaves it) per channel and entry, from row entry_slot[e] of ``state`` (float32 [slots, width], read and
    written), token by token; out[t] = S * act(y[t]) rounded once to y's dtype. activation: None or 'gelu_tanh'."""
    n, width = a.shape
    if a.dtype != torch.float32 or drive.dtype != torch.float32 or not a.is_contiguous() or not drive.is_contiguous() or \
            drive.shape != a.shape or y.shape != a.shape or y.stride(1) != 1 or state.dtype != torch.float32 or \
            not state.is_contiguous() or tuple(state.shape[1:]) != (width,):
        raise KernelError("linear_scan: shapes do not fit the state")
    if out is None:
        out = torch.empty((n, width), dtype=y.dtype, device=a.device)
    _call(library("core"), "dd_linear_scan", _ptr(a), _ptr(drive), _ptr(y, "y"), y.stride(0),
          _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_slot, "entry_slot", torch.int32), entry_slot.numel(), _ptr(state),
          _ptr(out), out.stride(0), width, {None: 0, "gelu_tanh": 1}[activation], _dt(y.dtype), _stream())
    return out


def layernorm(x, gamma, beta, eps, out_dtype, row_index=None, out=None):
    _rows(x, "x")
    rows = x.shape[0] if row_index is None else row_index.numel()
    width = x.shape[1]
    if not x.is_contiguous():
        raise KernelError("layernorm input must be contiguous")
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=x.device)
    _call(library("core"), "dd_layernorm", _ptr(x, "x", torch.float32), _ptr(row_index, "row_index", torch.int32),
          _ptr(gamma, "gamma", torch.float32), _ptr(beta, "beta", torch.float32), _ptr(out, "out", out_dtype),
          rows, width, float(eps), _dt(out_dtype), _stream())
    return out


def rmsnorm(x, weight, eps, out_dtype, row_index=None, offset=0.0, out=None, groups=1):
    """x / sqrt(mean(x^2) + eps) * (offset + weight) over float32 rows; offset 1 for a weight stored around zero.
    groups > 1: the row in that many equal consecutive stretches, each divided by its own root mean square."""
    _rows(x, "x")
    rows = x.shape[0] if row_index is None else row_index.numel()
    width = x.shape[1]
    if not x.is_contiguous():
        raise KernelError("rmsnorm input must be contiguous")
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=x.device)
    if groups != 1:
        _call(library("core"), "dd_rmsnorm_groups", _ptr(x, "x", torch.float32), _ptr(row_index, "row_index", torch.int32),
              _ptr(weight, "weight", torch.float32), _ptr(out, "out", out_dtype), rows, width, int(groups), float(eps),
              float(offset), _dt(out_dtype), _stream())
        return out
    _call(library("core"), "dd_rmsnorm", _ptr(x, "x", torch.float32), _ptr(row_index, "row_index", torch.int32),
          _ptr(weight, "weight", torch.float32), _ptr(out, "out", out_dtype), rows, width, float(eps), float(offset),
          _dt(out_dtype), _stream())
    return out


def rmsnorm_shift(x, weight, eps, out_dtype, shift, state, token_entry, entry_start, entry_slot, offset=0.0, groups=1, out=None):
    """The RMS norm (in ``groups`` stretches) of float32 rows, each blended with the normed row of the token before it in its
    sequence: out[t] = n[t] + (n[t-1] - n[t]) * shift, float32 inside. ``state`` float32 [slots, width] holds the normed row
    of every request's last token (zeros for a new request): read for an entry's first token, then replaced by the entry's
    last normed row."""
    _rows(x, "x")
    rows, width = x.shape
    if not x.is_contiguous() or state.dtype != torch.float32 or not state.is_contiguous() or state.shape[1:] != (width,):
        raise KernelError("rmsnorm_shift: contiguous float32 rows and a float32 state [slots, width] wanted")
    for v, name in ((weight, "weight"), (shift, "shift")):
        if v.numel() != width or v.dtype != torch.float32 or not v.is_contiguous():
            raise KernelError(f"rmsnorm_shift: {name} must be float32 [width]")
    if out is None:
        out = torch.empty((rows, width), dtype=out_dtype, device=x.device)
    _call(library("core"), "dd_rmsnorm_shift", _ptr(x, "x", torch.float32), _ptr(weight), _ptr(shift), _ptr(state),
          _ptr(token_entry, "token_entry", torch.int32), _ptr(entry_start, "entry_start", torch.int32),
          _ptr(entry_slot, "entry_slot", torch.int32), _ptr(out, "out", out_dtype), rows, width, int(groups), float(eps),
          float(offset), _dt(out_dtype), _stream())
    return out


def weighted_sum(stack, weights, n, out):
    """out = sum over j < n of weights[j] * stack[j], float32, j ascending. stack: float32 [planes, ...] contiguous;
    weights: float32 [>= n] on the device; out: float32 of a plane's shape (it may be a later plane of the stack)."""
    if stack.dtype != torch.float32 or out.dtype != torch.float32 or not stack.is_contiguous() or not out.is_contiguous() or \
            weights.dtype != torch.float32 or weights.numel() < n or n > stack.shape[0] or out.numel() != stack[0].numel():
        raise KernelError("weighted_sum: float32 contiguous planes and at least n weights wanted")
    _call(library("core"), "dd_weighted_sum", _ptr(stack, "stack"), out.numel(), _ptr(weights, "weights"), int(n), _ptr(out, "out"),
          _stream())
    return out


def blend_rows(v, other, weight):
    """In place: v <- (1 - weight) * v + weight * other, float32 inside. v, other: row views [N, width] of one element type;
    weight: one float32 on the device."""
    if v.shape != other.shape or v.dtype != other.dtype or v.stride(1) != 1 or other.stride(1) != 1 or \
            weight.dtype != torch.float32 or weight.numel() != 1:
        raise KernelError("blend_rows: two row views of one shape and type and one float32 weight wanted")
    _call(library("core"), "dd_blend_rows", _ptr(v, "v"), v.stride(0), _ptr(other, "other"), other.stride(0), _ptr(weight, "weight"),
          v.shape[0], v.shape[1], _dt(v.dtype), _stream())
    return v


def delta_state_shape(heads, head_dim, value_dim):
    """Shape of one request's delta-rule state (float32): per head the columns of S one after the other, each padded to the
    rows the kernel's lanes hold (eight a lane, a power of two of lanes); zeros for a new request."""
    rows = 0
    if 0 < head_dim <= 256:
        lanes = 1
        while lanes * 8 < head_dim:
            lanes *= 2
        rows = 8 * lanes          # what dd_delta_state_rows answers
    if not rows or value_dim <= 0:
        raise KernelError(f"delta rule: heads of {head_dim} by {value_dim} are not supported (keys of at most 256)")
    return (int(heads), int(value_dim), rows)


def delta_prepare(proj, beta_in, step_in, conv_w, conv_state, a_log, dt_bias, token_entry, entry_start, entry_slot, heads,
                  kv_heads, head_dim, value_dim):
    """The delta rule's operands of a step, float32: (q, k [N, kv_heads*head_dim], v [N, heads*value_dim], decay
    [N, heads*head_dim], beta [N, heads]). proj: rows whose first elements are the q, k and v projections (a row view);
    beta_in: a [N, heads] view of the same type; step_in: float32 [N, heads*head_dim] (the decay's low-rank projection);
    conv_w: float32 [channels, taps]; conv_state: float32 [slots, taps - 1, channels] (read only here). q, k and v pass the
    causal convolution and silu; q and k become unit vectors per head, q times head_dim^-1/2; beta = sigmoid(beta_in);
    decay = exp(-exp(a_log[head]) * softplus(step_in + dt_bias))."""
    n = proj.shape[0]
    qk, vw = kv_heads * head_dim, heads * value_dim
    channels, taps = conv_w.shape
    if channels != 2 * qk + vw or proj.shape[1] < channels or proj.stride(1) != 1 or beta_in.shape != (n, heads) or \
            beta_in.dtype != proj.dtype or beta_in.stride(1) != 1 or step_in.dtype != torch.float32 or not step_in.is_contiguous() or \
            step_in.shape != (n, heads * head_dim) or conv_w.dtype != torch.float32 or not conv_w.is_contiguous() or \
            conv_state.dtype != torch.float32 or not conv_state.is_contiguous() or tuple(conv_state.shape[1:]) != (taps - 1, channels) or \
            a_log.numel() != heads or dt_bias.numel() != heads * head_dim:
        raise KernelError("delta_prepare: shapes do not fit the heads")
    dev = proj.device
    f32 = lambda w: torch.empty((n, w), dtype=torch.float32, device=dev)
    q, k, v, decay, beta = f32(qk), f32(qk), f32(vw), f32(heads * head_dim), f32(heads)
    _call(library("core"), "dd_delta_prepare", _ptr(proj, "proj"), proj.stride(0), _ptr(beta_in, "beta_in"), beta_in.stride(0),
          _ptr(step_in), _ptr(conv_w), int(taps), _ptr(conv_state), _ptr(a_log, "a_log", torch.float32),
          _ptr(dt_bias, "dt_bias", torch.float32), _ptr(token_entry, "token_entry", torch.int32),
          _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_slot, "entry_slot", torch.int32), _ptr(q), _ptr(k), _ptr(v),
          _ptr(decay), _ptr(beta), n, heads, kv_heads, head_dim, value_dim, _dt(proj.dtype), _stream())
    return q, k, v, decay, beta


def conv_state_update(proj, conv_state, entry_start, entry_slot):
    """Leave in conv_state [slots, taps - 1, channels] (float32) the last taps - 1 input rows of every entry: what the
    state held, followed by the step's rows of proj (a row view whose first ``channels`` elements are the inputs)."""
    keep, channels = conv_state.shape[1], conv_state.shape[2]
    if proj.shape[1] < channels or proj.stride(1) != 1 or conv_state.dtype != torch.float32 or not conv_state.is_contiguous():
        raise KernelError("conv_state_update: shapes do not fit")
    _call(library("core"), "dd_conv_state_update", _ptr(proj, "proj"), proj.stride(0), _ptr(conv_state), keep + 1,
          _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_slot, "entry_slot", torch.int32), entry_slot.numel(), channels,
          _dt(proj.dtype), _stream())


def delta_rule(q, k, v, decay, beta, entry_start, entry_slot, state, heads, kv_heads, head_dim, value_dim, out=None):
    """The gated delta rule of a step: per entry and head, from the state in row entry_slot[e] of ``state`` (float32
    [slots, *delta_state_shape(...)], read and written), token by token: S = decay[:, None] * S; u = beta * (v - S^T k);
    S = S + k u^T; o = S^T q. Operands float32 as ``delta_prepare`` leaves them. Returns o float32 [N, heads*value_dim]."""
    n = q.shape[0]
    ok = all(t.dtype == torch.float32 and t.is_contiguous() for t in (q, k, v, decay, beta, state))
    if not ok or q.shape != (n, kv_heads * head_dim) or k.shape != q.shape or v.shape != (n, heads * value_dim) or \
            decay.shape != (n, heads * head_dim) or beta.shape != (n, heads) or \
            tuple(state.shape[1:]) != delta_state_shape(heads, head_dim, value_dim):
        raise KernelError("delta_rule: shapes do not fit the state")
    if out is None:
        out = torch.empty((n, heads * value_dim), dtype=torch.float32, device=q.device)
    _call(library("core"), "dd_delta_rule", _ptr(q), _ptr(k), _ptr(v), _ptr(decay), _ptr(beta),
          _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_slot, "entry_slot", torch.int32), entry_slot.numel(),
          _ptr(state), _ptr(out), heads, kv_heads, head_dim, value_dim, _stream())
    return out


def delta_finish(o, gate, weight, heads, eps, out_dtype, out=None):
    """out[t, head] = o[t, head] / sqrt(mean(o[t, head]^2) + eps) * weight * sigmoid(gate[t, head]); o, gate float32
    [N, heads*dv] contiguous, weight float32 [dv]."""
    n, total = o.shape
    if gate.shape != o.shape or gate.dtype != torch.float32 or o.dtype != torch.float32 or not o.is_contiguous() or \
            not gate.is_contiguous() or total % heads or weight.numel() != total // heads or weight.dtype != torch.float32:
        raise KernelError("delta_finish: the gate or the weight does not fit the read-out")
    if out is None:
        out = torch.empty((n, total), dtype=out_dtype, device=o.device)
    _call(library("core"), "dd_delta_finish", _ptr(o), _ptr(gate), _ptr(weight), _ptr(out, "out", out_dtype), out.stride(0), n,
          heads, total // heads, float(eps), _dt(out_dtype), _stream())
    return out


def latent_prepare(q, down, weight, eps, freqs, token_entry, positions, block_table, cache, heads, head_dim, rot_dim, rank):
    """A step's latent rows into the cache, and its queries rotated. down: [N, rank + rot_dim] row view; the cache row of a
    token becomes [rms(down[:rank]) * weight | down[rank:] rotated by its position] (cache [pages, page_size * (rank +
    rot_dim)]); the last rot_dim elements of every query head (q [N, heads * (head_dim + rot_dim)], a row view) are rotated
    in place. Neighbouring dimensions pair; the first 2 * len(freqs) of the rot_dim turn. float32 inside."""
    n = q.shape[0]
    row = rank + rot_dim
    if q.shape[1] != heads * (head_dim + rot_dim) or q.stride(1) != 1 or down.shape != (n, row) or down.stride(1) != 1 or \
            q.dtype != down.dtype or cache.dtype != q.dtype or cache.dim() != 2 or cache.shape[1] % row or not cache.is_contiguous() or \
            weight.numel() != rank or weight.dtype != torch.float32 or freqs.dtype != torch.float32 or 2 * freqs.numel() > rot_dim:
        raise KernelError("latent_prepare: shapes do not fit")
    _call(library("core"), "dd_latent_prepare", _ptr(q, "q"), q.stride(0), heads, head_dim, rot_dim, _ptr(down, "down"),
          down.stride(0), rank, _ptr(weight), float(eps), _ptr(freqs), freqs.numel(), _ptr(token_entry, "token_entry", torch.int32),
          _ptr(positions, "positions", torch.int32), _ptr(block_table, "block_table", torch.int32), block_table.shape[1],
          _ptr(cache), cache.shape[0], cache.shape[1] // row, n, _dt(q.dtype), _ptr(error_flag(q.device)), _stream())


def per_head_linear(x, w, in_head, out_head=None, tail=0, out=None, kernel=None):
    """out[t, h, :J] = w[h] @ x[t, h, :I], out[t, h, J:J+tail] = x[t, h, I:I+tail]: every head's piece of a row times the
    head's own matrix. x: a row view whose head h starts at h * in_head; w: [heads, J, I] contiguous, x's type; out: rows
    whose head h starts at h * out_head (default J + tail, packed). float32 sums in an order that does not depend on the
    batch. kernel: 'mma' (bfloat16 on the tensor cores, tiles of 64 tokens x 128 outputs), 'plain', or None for 'mma'
    where the sizes allow it."""
    heads, J, I = w.shape
    out_head = J + tail if out_head is None else out_head
    n = x.shape[0]
    if x.stride(1) != 1 or w.dtype != x.dtype or not w.is_contiguous() or x.shape[1] < (heads - 1) * in_head + I + tail:
        raise KernelError("per_head_linear: shapes do not fit")
    if out is None:
        out = torch.empty((n, heads * out_head), dtype=x.dtype, device=x.device)
    if kernel is None:
        kernel = "mma" if x.dtype == torch.bfloat16 and bool(library("tensor").dd_per_head_mma_supported(
            x.stride(0), int(in_head), out.stride(0), int(out_head), I, BF16)) else "plain"
    if kernel == "mma":
        _call(library("tensor"), "dd_per_head_mma", _ptr(x, "x"), x.stride(0), int(in_head), _ptr(w, "w"), _ptr(out, "out"),
              out.stride(0), int(out_head), n, heads, I, J, int(tail), _stream())
        return out
    _call(library("core"), "dd_per_head_linear", _ptr(x, "x"), x.stride(0), int(in_head), _ptr(w, "w"), _ptr(out, "out"),
          out.stride(0), int(out_head), n, heads, I, J, int(tail), _dt(x.dtype), _stream())
    return out


def attention_latent_supported(row, v_dim, dtype):
    return dtype == torch.bfloat16 and bool(library("tensor").dd_attention_latent_supported(row, v_dim, BF16))


def attention_latent_splits(n_tokens, n_entries, n_heads, context, device):
    """Into how many pieces a step of single tokens cuts its keys so that its tiles fill the GPU about twice (a piece is
    at least one key tile of 64); 1 for a step with portions of prompts."""
    if n_tokens != n_entries:
        return 1
    tile = int(library("tensor").dd_attention_latent_tile(n_tokens, n_entries, n_heads))
    tiles = n_entries * -(-n_heads // tile)
    return max(1, min(-(-2 * sm_count(device) // tiles), -(-context // 64), 32))


def attention_latent(q, cache, entry_start, entry_pos0, block_table, n_heads, v_dim, scale, n_splits=1, sink=None, out=None):
    """Tensor-core causal attention of runs of consecutive tokens over cached latent rows: the cache
    ([pages, page_size * row] bfloat16) holds one row a token, which is every head's key, and whose first v_dim elements
    are the value. q: [N, n_heads * row] row view; entry_start int32 [E+1], entry_pos0 int32 [E]; block_table row e is
    entry e's pages. sink: float32 [n_heads], exp(sink) joins the softmax's denominator. n_splits: into how many pieces
    a row's keys are cut (partial sums merged by a second kernel). Returns [N, n_heads * v_dim]. The softmax weights meet
    the values as two bfloat16 terms. See attention_latent_supported for the sizes."""
    n, n_entries = q.shape[0], entry_pos0.numel()
    row = q.shape[1] // n_heads
    if q.shape[1] != n_heads * row or q.stride(1) != 1 or q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or \
            cache.dim() != 2 or cache.shape[1] % row or not cache.is_contiguous() or entry_start.numel() != n_entries + 1:
        raise KernelError("attention_latent: q or the entry arrays do not fit the cache")
    if sink is not None and (sink.numel() != n_heads or sink.dtype != torch.float32 or not sink.is_contiguous()):
        raise KernelError("attention: the sink must be float32 [heads]")
    if out is None:
        out = torch.empty((n, n_heads * v_dim), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((n * n_heads * n_splits * v_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_heads * n_splits * 2,), dtype=torch.float32, device=q.device)
    _call(library("tensor"), "dd_attention_latent", _ptr(q, "q"), q.stride(0), _ptr(cache, "cache"),
          _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_pos0, "entry_pos0", torch.int32), n_entries, n,
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(out, "out"), out.stride(0),
          _ptr(part_o), _ptr(part_ml), n_heads, row, int(v_dim), cache.shape[1] // row, cache.shape[0], float(scale),
          int(n_splits), _ptr(error_flag(q.device)), _ptr(sink, "sink"), _stream(), n_kernels=2 if n_splits > 1 else 1)
    return out


def rotary(q, k, positions, freqs, magnitude, q_heads, k_heads, head_dim, interleaved=True):
    """Rotate, in place, the first 2 * len(freqs) dimensions of every head of q and k (row views of one buffer) by
    position * freqs; cosine and sine are multiplied by magnitude. interleaved: pairs are neighbours (2i, 2i+1);
    else the two halves of the rotated dimensions (i, i + len(freqs))."""
    if q.stride(0) != k.stride(0) or q.stride(1) != 1 or k.stride(1) != 1 or q.dtype != k.dtype:
        raise KernelError("rotary: q and k must be row views of one buffer")
    if q.shape[1] != q_heads * head_dim or k.shape[1] != k_heads * head_dim or 2 * freqs.numel() > head_dim:
        raise KernelError("rotary: shapes do not fit the heads")
    _call(library("core"), "dd_rotary", _ptr(q, "q"), _ptr(k, "k"), q.stride(0), _ptr(positions, "positions", torch.int32),
          _ptr(freqs, "freqs", torch.float32), float(magnitude), q.shape[0], q_heads, k_heads, head_dim, freqs.numel(),
          1 if interleaved else 0, _dt(q.dtype), _stream())
    return q, k


def head_norm_rotary(q, k, positions, q_weight, k_weight, eps, q_heads, k_heads, head_dim, freqs=None, interleaved=True):
    """In place and in one pass: every head of q (and of k, a row view of the same buffer, or None with k_heads 0)
    becomes x / sqrt(mean(x^2) + eps) * weight (q_weight for query heads, k_weight for key heads, float32 [head_dim];
    None: that kind is not normed), then the first 2 * len(freqs) dimensions of the head are rotated by position * freqs
    as in ``rotary`` (freqs None: no rotation). All float32 inside."""
    if k is not None and (q.stride(0) != k.stride(0) or k.stride(1) != 1 or q.dtype != k.dtype or k.shape[1] != k_heads * head_dim):
        raise KernelError("head_norm_rotary: q and k must be row views of one buffer")
    if q.stride(1) != 1 or q.shape[1] != q_heads * head_dim or (k is None) != (k_heads == 0):
        raise KernelError("head_norm_rotary: shapes do not fit the heads")
    for w in (q_weight, k_weight):
        if w is not None and (w.numel() != head_dim or w.dtype != torch.float32 or not w.is_contiguous()):
            raise KernelError("head_norm_rotary: a weight must be float32 [head_dim]")
    n_pairs = 0 if freqs is None else freqs.numel()
    _call(library("core"), "dd_head_norm_rotary", _ptr(q, "q"), _ptr(k, "k"), q.stride(0), _ptr(positions, "positions", torch.int32),
          _ptr(freqs, "freqs", torch.float32), _ptr(q_weight, "q_weight"), _ptr(k_weight, "k_weight"), float(eps), q.shape[0],
          q_heads, k_heads, head_dim, n_pairs, 1 if interleaved else 0, _dt(q.dtype), _stream())
    return q, k


def retention_state_shape(heads, head_dim, value_dim):
    """Shape of one request's retention state (float32): per head the columns of S one after the other, each padded to a
    multiple of four rows (a thread of the kernel holds four rows as one 16-byte piece); zeros for a new request."""
    if not 0 < head_dim <= 256 or value_dim <= 0:
        raise KernelError(f"retention: heads of {head_dim} by {value_dim} are not supported (keys of at most 256)")
    return (int(heads), int(value_dim), -(-int(head_dim) // 4) * 4)


def retention(q, k, v, positions, entry_start, entry_slot, decay, key_scale, state, head_dim, value_dim, freqs=None,
              interleaved=True, out=None):
    """The retention recurrence of a step: per entry (rows entry_start[e] .. entry_start[e+1]) and head, from the
    state in row entry_slot[e] of ``state`` (float32 [slots, *retention_state_shape(heads, head_dim, value_dim)], read and
    written), token by token: S = decay * S + k' v^T, o = S^T q', with q', k' rotated by position * freqs (None: not
    rotated) and k' times key_scale. q, k [N, heads*head_dim], v [N, heads*value_dim]: row views of one buffer. Returns o
    float32 [N, heads*value_dim]."""
    n_slots, heads = state.shape[0], state.shape[1]
    dk, dv = int(head_dim), int(value_dim)
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1 or \
            not (q.dtype == k.dtype == v.dtype):
        raise KernelError("retention: q, k and v must be row views of one buffer")
    if q.shape[1] != heads * dk or k.shape[1] != heads * dk or v.shape[1] != heads * dv or state.dtype != torch.float32 or \
            not state.is_contiguous() or decay.numel() != heads or tuple(state.shape[1:]) != retention_state_shape(heads, dk, dv):
        raise KernelError("retention: shapes do not fit the state")
    n, n_entries = q.shape[0], entry_slot.numel()
    if out is None:
        out = torch.empty((n, heads * dv), dtype=torch.float32, device=q.device)
    # a step with portions: rotated q and k and v as float32 rows, written once for all the blocks of the recurrence
    scratch = None
    if n > n_entries:
        scratch = torch.empty((n * heads * (2 * (-(-dk // 4) * 4) + -(-dv // 4) * 4),), dtype=torch.float32, device=q.device)
    _call(library("core"), "dd_retention", _ptr(q, "q"), _ptr(k, "k"), _ptr(v, "v"), q.stride(0),
          _ptr(positions, "positions", torch.int32), _ptr(entry_start, "entry_start", torch.int32),
          _ptr(entry_slot, "entry_slot", torch.int32), entry_slot.numel(), _ptr(freqs, "freqs", torch.float32),
          0 if freqs is None else freqs.numel(), 1 if interleaved else 0, _ptr(decay, "decay", torch.float32), float(key_scale),
          _ptr(state, "state"), n_slots, _ptr(out, "out", torch.float32), heads, dk, dv, _dt(q.dtype),
          _ptr(error_flag(q.device)), _stream(), n, _ptr(scratch), n_kernels=2 if scratch is not None else 1)
    return out


def retention_finish(o, gate, heads, eps, out_dtype, out=None):
    """out[t, head] = o[t, head] / sqrt(mean(o[t, head]^2) + eps) * silu(gate[t, head]); o float32 [N, heads*dv], gate a
    row view [N, heads*dv] in out_dtype."""
    n, total = o.shape
    if gate.shape != (n, total) or gate.stride(1) != 1 or gate.dtype != out_dtype or not o.is_contiguous() or total % heads:
        raise KernelError("retention_finish: the gate does not fit the read-out")
    if out is None:
        out = torch.empty((n, total), dtype=out_dtype, device=o.device)
    _call(library("core"), "dd_retention_finish", _ptr(o, "o", torch.float32), _ptr(gate, "gate"), gate.stride(0), _ptr(out, "out"),
          out.stride(0), n, heads, total // heads, float(eps), _dt(out_dtype), _stream())
    return out


def gemm_simt(a, w, bias=None, residual=None, activation=None, out_dtype=None, out=None):
    """act(a @ w.T + bias) (+ residual) with CUDA-core float32 multiply-add. a [M,K], w [N,K]."""
    _rows(a, "a"), _rows(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or a.dtype != w.dtype:
        raise KernelError(f"gemm: a {tuple(a.shape)} {a.dtype} does not fit w {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or a.dtype
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _rows(out, "out")
    if residual is not None:
        _rows(residual, "residual")
    _call(library("core"), "dd_gemm_simt", _ptr(a, "a"), a.stride(0), _ptr(w, "w"), w.stride(0),
          _ptr(bias, "bias", torch.float32), _ptr(residual, "residual", torch.float32),
          0 if residual is None else residual.stride(0), _ptr(out, "out", out_dtype), out.stride(0),
          M, N, K, ACTIVATIONS[activation], _dt(a.dtype), _dt(out_dtype), _stream())
    return out


def cache_geometry(cache, kv_heads=None, head_dim=None, v_dim=None):
    """(pages, kv_heads, page_size, head_dim, v_dim) of a layer's cache: [pages, 2, kv_heads, page, head_dim], or, where
    a value head has another size than a key head, [pages, kv_heads * page * (head_dim + v_dim)] (a page's key plane
    followed by its value plane), whose sizes the caller names."""
    if cache.dim() == 5:
        return cache.shape[0], cache.shape[2], cache.shape[3], cache.shape[4], cache.shape[4]
    if cache.dim() != 2 or not kv_heads or not head_dim or not v_dim or cache.shape[1] % (kv_heads * (head_dim + v_dim)):
        raise KernelError(f"a cache of shape {tuple(cache.shape)} needs its head count and head sizes named")
    return cache.shape[0], kv_heads, cache.shape[1] // (kv_heads * (head_dim + v_dim)), head_dim, v_dim


def kv_store(k, v, token_entry, positions, block_table, cache, n_tokens=None, kv_heads=None, head_dim=None, v_dim=None):
    """k: [N, kv_heads*head_dim], v: [N, kv_heads*v_dim] views (row stride free); cache: see cache_geometry."""
    n_pages, kv_heads, page_size, head_dim, v_dim = cache_geometry(cache, kv_heads, head_dim, v_dim)
    if k.stride(0) != v.stride(0) or k.stride(1) != 1 or v.stride(1) != 1 or k.dtype != cache.dtype:
        raise KernelError("kv_store: k and v must be row views of one buffer in the cache dtype")
    if k.shape[1] != kv_heads * head_dim or v.shape[1] != kv_heads * v_dim or not cache.is_contiguous():
        raise KernelError("kv_store: shapes do not fit the cache")
    _call(library("core"), "dd_kv_store", _ptr(k, "k"), _ptr(v, "v"), k.stride(0),
          _ptr(token_entry, "token_entry", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(cache, "cache"),
          n_pages, kv_heads, page_size, head_dim, v_dim, k.shape[0] if n_tokens is None else n_tokens, _dt(cache.dtype),
          _ptr(error_flag(k.device)), _stream())


def attention_rows(q, cache, token_entry, positions, block_table, n_heads, scale, window=None, n_splits=1, out=None,
                   chunk=None, gate=None, kv_heads=None, v_dim=None, keep_first=0, softcap=None, sink=None,
                   values_in_keys=False):
    """General paged causal attention. q: [N, n_heads*head_dim] view; returns [N, n_heads*v_dim]. chunk: positions
    are cut into chunks of this many from the start of the sequence and nothing is seen across a border. gate:
    [N, n_heads] view, a head's output is multiplied by the logistic function of its entry. kv_heads and v_dim name the
    sizes of a cache whose value heads differ from its key heads (see cache_geometry). keep_first: behind a window, the
    first so many keys of the sequence stay visible. softcap c: a scaled score s becomes c * tanh(s / c). sink: float32
    [n_heads], exp(sink) joins the softmax's denominator. values_in_keys: the cache holds key rows only
    ([pages, kv_heads * page_size * head_dim]) and a value is the first v_dim elements of its key row."""
    head_dim = q.shape[1] // n_heads
    if values_in_keys:
        kv_heads = kv_heads or 1
        if cache.dim() != 2 or cache.shape[1] % (kv_heads * head_dim) or not v_dim or v_dim > head_dim:
            raise KernelError("attention: a cache of key rows that hold the values needs [pages, kv_heads * page * head_dim]")
        n_pages, page_size = cache.shape[0], cache.shape[1] // (kv_heads * head_dim)
    else:
        n_pages, kv_heads, page_size, head_dim, v_dim = cache_geometry(cache, kv_heads, head_dim, v_dim)
    if sink is not None and (sink.numel() != n_heads or sink.dtype != torch.float32 or not sink.is_contiguous()):
        raise KernelError("attention: the sink must be float32 [heads]")
    n = q.shape[0]
    if q.shape[1] != n_heads * head_dim or q.stride(1) != 1 or q.dtype != cache.dtype or not cache.is_contiguous():
        raise KernelError("attention: q does not fit the cache")
    if gate is not None and (gate.shape != (n, n_heads) or gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise KernelError("attention: the gate must be a [tokens, heads] row view in q's dtype")
    if out is None:
        out = torch.empty((n, n_heads * v_dim), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = torch.empty((n * n_heads * n_splits * v_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_heads * n_splits * 2,), dtype=torch.float32, device=q.device)
    _call(library("core"), "dd_attention_rows_sinks", _ptr(q, "q"), q.stride(0), _ptr(cache, "cache"),
          _ptr(token_entry, "token_entry", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(out, "out"), out.stride(0),
          _ptr(part_o), _ptr(part_ml), n, n_heads, kv_heads, head_dim, page_size, n_pages,
          0 if window is None else int(window), float(scale), int(n_splits), _dt(q.dtype),
          _ptr(error_flag(q.device)), _stream(), v_dim, 0 if chunk is None else int(chunk), _ptr(gate, "gate"),
          0 if gate is None else gate.stride(0), int(keep_first or 0), float(softcap or 0.0), _ptr(sink, "sink"),
          1 if values_in_keys else 0, n_kernels=2 if n_splits > 1 else 1)
    return out


# ---- experts chosen by a table: routing, the grouped product, the gated unit, the weighted sum ----

def grouped_rows(n_tokens, top, n_experts, tile):
    """Rows of the buffer in which every expert's (token, choice) pairs start on a multiple of tile."""
    pairs = n_tokens * top
    return -(-(pairs + min(n_experts, pairs) * (tile - 1)) // tile) * tile


def route_by_table(ids, table, n_experts, tile):
    """ids int32 [N], table int32 [vocab, K] -> (pair_row [N*K], row_token [rows], tile_group [rows/tile]). ids None:
    token t reads row t of the table (the step's own choices, [N, K], as ``route_by_score`` leaves them)."""
    vocab, top = table.shape
    n = vocab if ids is None else ids.numel()
    rows = grouped_rows(n, top, n_experts, tile)
    pair_row = torch.empty((n * top,), dtype=torch.int32, device=table.device)
    row_token = torch.empty((rows,), dtype=torch.int32, device=table.device)
    tile_group = torch.empty((rows // tile,), dtype=torch.int32, device=table.device)
    _call(library("core"), "dd_route_by_table", _ptr(ids, "ids", torch.int32), _ptr(table, "table", torch.int32), n, vocab, top,
          n_experts, tile, rows, _ptr(pair_row), _ptr(row_token), _ptr(tile_group), _ptr(error_flag(table.device)), _stream())
    return pair_row, row_token, tile_group


def route_by_score(y, router, n_experts, top, groups=1, keep=1, weight_scale=1.0, shared_gate=False):
    """Normed rows y [N, width] and the router's matrix [n_experts (+ 1), width] (one storage type) -> (chosen int32
    [N, top], pair_weight float32 [N, top], shared_scale float32 [N] or None). logit = y . router row as float32 sums of
    exact products, score = sigmoid(logit); the experts form ``groups`` equal runs of neighbours, a run's worth is the sum
    of its two largest scores, only the ``keep`` worthiest runs stay eligible; the ``top`` largest eligible scores win, each
    weighing score * weight_scale. shared_gate: the router's last row is a shared unit's gate vector, whose sigmoid is
    returned as shared_scale."""
    _rows(y, "y"), _rows(router, "router")
    n, width = y.shape
    if router.shape != (n_experts + (1 if shared_gate else 0), width) or router.dtype != y.dtype:
        raise KernelError(f"route_by_score: router {tuple(router.shape)} {router.dtype} does not fit {n_experts} experts over y {tuple(y.shape)} {y.dtype}")
    chosen = torch.empty((n, top), dtype=torch.int32, device=y.device)
    weight = torch.empty((n, top), dtype=torch.float32, device=y.device)
    shared = torch.empty((n,), dtype=torch.float32, device=y.device) if shared_gate else None
    _call(library("core"), "dd_route_by_score", _ptr(y, "y"), y.stride(0), _ptr(router, "router"), router.stride(0), width, n,
          n_experts, top, groups, keep, float(weight_scale), n_experts if shared_gate else -1, _ptr(chosen), _ptr(weight),
          _ptr(shared), _dt(y.dtype), _stream())
    return chosen, weight, shared


def gather_rows(x, row_token):
    """out[r] = x[row_token[r]], zeros where row_token[r] < 0."""
    _rows(x, "x")
    out = torch.empty((row_token.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    if not x.is_contiguous():
        raise KernelError("gather_rows input must be contiguous")
    _call(library("core"), "dd_gather_rows", _ptr(x, "x"), _ptr(row_token, "row_token", torch.int32), _ptr(out), row_token.numel(),
          x.shape[1], _dt(x.dtype), _stream())
    return out


def simt_group_tile():
    return int(library("core").dd_gemm_simt_group_tile())


def gemm_simt_grouped(a, w, tile_group, activation=None, out_dtype=None):
    """a [rows, K] in tiles of simt_group_tile() rows; w [groups, N, K]; tile i is multiplied with w[tile_group[i]]
    (skipped where that is negative). CUDA-core float32 multiply-add, k ascending."""
    _rows(a, "a")
    if w.dim() != 3 or not w.is_contiguous() or w.shape[2] != a.shape[1] or w.dtype != a.dtype:
        raise KernelError(f"grouped gemm: a {tuple(a.shape)} {a.dtype} does not fit w {tuple(w.shape)} {w.dtype}")
    M, K = a.shape
    N = w.shape[1]
    out_dtype = out_dtype or a.dtype
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _call(library("core"), "dd_gemm_simt_grouped", _ptr(a, "a"), a.stride(0), _ptr(w, "w"), w.stride(1), w.stride(0),
          _ptr(tile_group, "tile_group", torch.int32), _ptr(out), out.stride(0), M, N, K, ACTIVATIONS[activation],
          _dt(a.dtype), _dt(out_dtype), _stream())
    return out


GROUPED_TCGEN05_TILES = (16, 32, 64, 128)


def gemm_grouped_tcgen05(a, w, tile_group, tile, gated=None, out_dtype=None):
    """a [rows, K] bfloat16 in tiles of ``tile`` rows (one of GROUPED_TCGEN05_TILES); w [groups, N, K] bfloat16; tile i
    is multiplied with w[tile_group[i]] on the tensor cores (skipped where that is negative). gated=(limit, alpha) or
    (limit, alpha, form): w holds gate rows then up rows ([groups, 2 * inner, K]) and the result is the gated unit (form:
    one of GATED_FORMS, the clamped one by default) of the two products, [rows, inner], computed in float32 in the
    product's epilogue."""
    _rows(a, "a")
    if w.dim() != 3 or not w.is_contiguous() or w.shape[2] != a.shape[1] or w.dtype != torch.bfloat16 or a.dtype != torch.bfloat16:
        raise KernelError(f"grouped gemm: a {tuple(a.shape)} {a.dtype} does not fit w {tuple(w.shape)} {w.dtype}")
    rows, K = a.shape
    groups, per_group = w.shape[0], w.shape[1]
    N = per_group // 2 if gated else per_group
    out_dtype = out_dtype or torch.bfloat16
    out = torch.empty((rows, N), dtype=out_dtype, device=a.device)
    limit, alpha, form = (tuple(gated) + ("clamped_swish",))[:3] if gated else (0.0, 0.0, "clamped_swish")
    _call(library("tensor"), "dd_gemm_grouped_tcgen05", _ptr(a, "a"), a.stride(0), _ptr(w, "w"), w.stride(1), groups, per_group,
          _ptr(tile_group, "tile_group", torch.int32), _ptr(out), out.stride(0), rows, N, K, int(tile), 1 if gated else 0,
          float(limit), float(alpha), _dt(out_dtype), _ptr(error_flag(a.device)), _stream(), GATED_FORMS[form])
    return out


def gated_unit(gate_up, limit, alpha, out=None, form="clamped_swish", row_scale=None):
    """rows of [gate | up] halves -> the gated unit's value. form 'clamped_swish': min(gate, limit) * sigmoid(alpha *
    min(gate, limit)) * (clamp(up, -limit, limit) + 1); 'silu': gate * sigmoid(gate) * up; 'gelu_tanh': gelu_new(gate) * up.
    row_scale: float32 [rows], multiplies a row's values (in float32, before they are rounded)."""
    _rows(gate_up, "gate_up")
    rows, inner = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inner), dtype=gate_up.dtype, device=gate_up.device)
    if row_scale is not None and (row_scale.numel() != rows or row_scale.dtype != torch.float32 or not row_scale.is_contiguous()):
        raise KernelError("gated_unit: row_scale must be float32 [rows]")
    _call(library("core"), "dd_gated_unit", _ptr(gate_up, "gate_up"), gate_up.stride(0), _ptr(out), out.stride(0), rows, inner,
          float(limit), float(alpha), _dt(gate_up.dtype), _stream(), GATED_FORMS[form], _ptr(row_scale, "row_scale"))
    return out


def combine_rows(y, pair_row, stream_rows, top, weight, pair_weight=None):
    """stream_rows[t] += weight * sum over k of (pair_weight[t*top + k] *) y[pair_row[t*top + k]] (float32, k ascending),
    in place. pair_weight: float32 [N * top] or None."""
    if y.dtype != torch.float32 or stream_rows.dtype != torch.float32 or not y.is_contiguous() or not stream_rows.is_contiguous():
        raise KernelError("combine_rows: float32 contiguous rows wanted")
    if pair_weight is not None and (pair_weight.numel() != stream_rows.shape[0] * top or pair_weight.dtype != torch.float32
                                    or not pair_weight.is_contiguous()):
        raise KernelError("combine_rows: pair_weight must be float32 [tokens * top]")
    _call(library("core"), "dd_combine_rows", _ptr(y), _ptr(pair_row, "pair_row", torch.int32), _ptr(stream_rows),
          stream_rows.shape[0], stream_rows.shape[1], int(top), float(weight), _stream(), _ptr(pair_weight, "pair_weight"))
    return stream_rows


def sample(logits, temperature=None, uniform=None, top_k=None, top_p=None, out=None):
    """Row-wise token choice: argmax where temperature is 0 (or None), else an inverse-CDF draw
    with the given uniform numbers over the tokens that top_k and top_p keep. Returns int32 ids,
    -1 for rows without a finite maximum."""
    _rows(logits, "logits")
    rows, vocab = logits.shape
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    if temperature is not None and uniform is None:
        raise KernelError("sampling with a temperature needs uniform draws")
    _call(library("core"), "dd_sample", _ptr(logits, "logits", torch.float32), logits.stride(0), rows, vocab,
          _ptr(temperature, "temperature", torch.float32), _ptr(top_k, "top_k", torch.int32),
          _ptr(top_p, "top_p", torch.float32), _ptr(uniform, "uniform", torch.float64),
          _ptr(out, "out", torch.int32), _stream())
    return out


def adjust_logits(logits, item_row, item_token, item_count, item_bias, item_seen, repetition, frequency, presence):
    """In place: penalties and bias on the listed (row, token) pairs (each pair listed once)."""
    _rows(logits, "logits")
    _call(library("core"), "dd_adjust_logits", _ptr(logits, "logits", torch.float32), logits.stride(0), logits.shape[1],
          _ptr(item_row, "item_row", torch.int32), _ptr(item_token, "item_token", torch.int32),
          _ptr(item_count, "item_count", torch.float32), _ptr(item_bias, "item_bias", torch.float32),
          _ptr(item_seen, "item_seen", torch.int32), _ptr(repetition, "repetition", torch.float32),
          _ptr(frequency, "frequency", torch.float32), _ptr(presence, "presence", torch.float32),
          item_row.numel(), _stream())
    return logits


_counters = {}
_sm_count = {}


def _tile_counters(device, n):
    key = torch.device(device).index or 0
    if key not in _counters or _counters[key].numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError(f"{n} split counters are needed during a graph capture; size them before (kernels._tile_counters)")
        _counters[key] = torch.zeros(max(n, 8192), dtype=torch.int32, device=device)
    return _counters[key]


def sm_count(device):
    key = torch.device(device).index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[key]


_plans = {}


def gemm_tcgen05(a, w, bias=None, residual=None, activation=None, out_dtype=None, out=None, splits=None, token_tile=None,
                 cluster=None, prefetch=None):
    """act(a @ w.T + bias) (+ residual) on the tcgen05 tensor cores. a [M,K] and w [N,K] bfloat16,
    bias/residual float32, out bfloat16 or float32. K and the row strides must be multiples of 8.
    splits/token_tile/cluster override the kernel's own plan (cluster 1: reduce the K splits inside a
    thread-block cluster instead of through a workspace; 3: the same with rings of 10 stages, one block per SM,
    token tiles of 16 only; 2: two SMs on a tile of 256 tokens). prefetch: a tensor that a later kernel will
    stream (the next weight matrix of a decode step); this kernel asks L2 to fetch it meanwhile."""
    _rows(a, "a"), _rows(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != K:
        raise KernelError(f"gemm_tcgen05: needs bfloat16 a [M,K] and w [N,K]; got {tuple(a.shape)} {a.dtype}, {tuple(w.shape)} {w.dtype}")
    out_dtype = out_dtype or torch.bfloat16
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _rows(out, "out")
    lib = library("tensor")
    plan = _plans.get((M, N, K))
    if plan is None:
        tile, mode = ctypes.c_int(0), ctypes.c_int(0)
        planned = lib.dd_gemm_tcgen05_plan(M, N, K, sm_count(a.device), ctypes.byref(tile), ctypes.byref(mode))
        plan = _plans[(M, N, K)] = (planned, tile.value, mode.value)
    if splits is not None and cluster is None:
        cluster = 0
    splits = plan[0] if splits is None else splits
    token_tile = plan[1] if token_tile is None else token_tile
    cluster = plan[2] if cluster is None else int(cluster)
    workspace = counters = None
    n_counters = 0
    if splits > 1 and not cluster:
        workspace = torch.empty((splits * M * N,), dtype=torch.float32, device=a.device)
        n_counters = ((N + 127) // 128) * ((M + token_tile - 1) // token_tile)
        counters = _tile_counters(a.device, n_counters)
    _call(lib, "dd_gemm_tcgen05", _ptr(a, "a"), a.stride(0), _ptr(w, "w"), w.stride(0),
          _ptr(bias, "bias", torch.float32), _ptr(residual, "residual", torch.float32),
          0 if residual is None else residual.stride(0), _ptr(out, "out", out_dtype), out.stride(0), M, N, K,
          ACTIVATIONS[activation], _dt(out_dtype), splits, token_tile, cluster, _ptr(workspace), _ptr(counters), n_counters,
          None if prefetch is None else prefetch.data_ptr(),
          0 if prefetch is None else prefetch.numel() * prefetch.element_size(), _ptr(error_flag(a.device)), _stream())
    return out


def attention_decode_supported(n_heads, kv_heads, head_dim, dtype):
    return dtype == torch.bfloat16 and bool(library("tensor").dd_attention_decode_supported(n_heads, kv_heads, head_dim, BF16))


def attention_decode_pages_supported(n_heads, kv_heads, head_dim, page_size, dtype):
    return dtype == torch.bfloat16 and bool(
        library("tensor").dd_attention_decode_pages_supported(n_heads, kv_heads, head_dim, page_size, BF16))


def attention_decode_pages_splits(n_tokens, n_heads, page_size, context, device):
    """The key split count the page-streaming decode kernel wants for this many tokens and this longest context."""
    return int(library("tensor").dd_attention_decode_pages_splits(n_tokens, n_heads, page_size, context, sm_count(device)))


def _gate_args(gate, q, n_heads, chunk):
    """(chunk, gate pointer, gate row stride) as the attention launchers take them."""
    if gate is not None and (gate.shape != (q.shape[0], n_heads) or gate.stride(1) != 1 or gate.dtype != q.dtype):
        raise KernelError("attention: the gate must be a [tokens, heads] row view in q's dtype")
    return 0 if chunk is None else int(chunk), _ptr(gate, "gate"), 0 if gate is None else gate.stride(0)


def attention_decode(q, cache, token_entry, positions, block_table, n_heads, scale, window=None, n_splits=1, out=None,
                     k_new=None, v_new=None, kernel="rows", chunk=None, gate=None, keep_first=0, softcap=None, sink=None,
                     exact_weights=False):
    """Decode attention (one query per token) over a bfloat16 cache. kernel 'rows': a warp copies key rows 16 bytes
    at a time (see attention_decode_supported); 'pages': whole pages of a group of heads by TMA (see
    attention_decode_pages_supported). With k_new/v_new (row views of the buffer q lives in) the step's own keys and
    values are used from there and written into the cache by this kernel; otherwise they must be in the cache already.
    token_entry None: token t belongs to entry t (a step of single tokens in entry order). n_splits: into how many
    pieces a token's keys are cut; for 'pages' the most a token may get (the kernel deals them out by context length).
    chunk, gate, keep_first, softcap, sink: as attention_rows; the last three, and exact_weights (the softmax weights
    meet the values as two bfloat16 terms instead of one rounded to bfloat16), only with kernel 'rows'."""
    if kernel not in ("rows", "pages"):
        raise KernelError(f"attention_decode: unknown kernel {kernel!r}")
    more = ()
    if keep_first or softcap or sink is not None or exact_weights:
        if kernel != "rows":
            raise KernelError("attention_decode: kept first keys, capped scores, a sink and exact weights need the kernel 'rows'")
        if sink is not None and (sink.numel() != n_heads or sink.dtype != torch.float32 or not sink.is_contiguous()):
            raise KernelError("attention: the sink must be float32 [heads]")
        more = (int(keep_first or 0), float(softcap or 0.0), _ptr(sink, "sink"), int(bool(exact_weights)))
    n_pages, _, kv_heads, page_size, head_dim = cache.shape
    n = q.shape[0]
    if q.shape[1] != n_heads * head_dim or q.stride(1) != 1 or q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 \
            or not cache.is_contiguous():
        raise KernelError("attention_decode: q does not fit the cache")
    if (k_new is None) != (v_new is None):
        raise KernelError("attention_decode: k_new and v_new come together")
    if k_new is not None and (k_new.stride(0) != q.stride(0) or v_new.stride(0) != q.stride(0) or k_new.stride(1) != 1
                              or v_new.stride(1) != 1 or k_new.dtype != q.dtype or k_new.shape != q.shape):
        raise KernelError("attention_decode: k_new and v_new must be row views like q")
    if out is None:
        out = torch.empty((n, n_heads * head_dim), dtype=q.dtype, device=q.device)
    part_o = part_ml = counters = None
    if n_splits > 1:
        part_o = torch.empty((n * n_heads * n_splits * head_dim,), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n * n_heads * n_splits * 2,), dtype=torch.float32, device=q.device)
        counters = _tile_counters(q.device, n * n_heads)
    _call(library("tensor"), "dd_attention_decode" + ("_pages" if kernel == "pages" else "_sinks" if more else ""), _ptr(q, "q"), q.stride(0),
          _ptr(k_new, "k_new"), _ptr(v_new, "v_new"),
          _ptr(cache, "cache"), _ptr(token_entry, "token_entry", torch.int32), _ptr(positions, "positions", torch.int32),
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(out, "out"), out.stride(0),
          _ptr(part_o), _ptr(part_ml), _ptr(counters), n, n_heads, kv_heads, head_dim, page_size, n_pages,
          0 if window is None else int(window), float(scale), int(n_splits), _ptr(error_flag(q.device)), _stream(),
          *_gate_args(gate, q, n_heads, chunk), *more)
    return out


def attention_prefill_supported(n_heads, kv_heads, head_dim, dtype):
    return dtype == torch.bfloat16 and bool(library("tensor").dd_attention_prefill_supported(n_heads, kv_heads, head_dim, BF16))


def attention_prefill_tcgen05_supported(n_heads, kv_heads, head_dim, page_size, dtype):
    return dtype == torch.bfloat16 and bool(
        library("tensor").dd_attention_prefill_tcgen05_supported(n_heads, kv_heads, head_dim, page_size, BF16))


ATTENTION_PREFILL_TCGEN05_KEY_BLOCK = 128       # keys per block of the tcgen05 prompt attention


def attention_prefill(q, cache, entry_start, entry_pos0, block_table, n_heads, scale, window=None, out=None, kernel="mma",
                      k_new=None, v_new=None, store_new=False, chunk=None, gate=None, keep_first=0, softcap=None, sink=None,
                      exact_weights=False):
    """Tensor-core attention for runs of consecutive tokens (prompt portions; a decoded token is a run of one)
    over a bfloat16 cache. entry_start: int32 [E+1], entry_pos0: int32 [E]. kernel: 'mma' (mma.sync tiles of 64
    queries, see attention_prefill_supported) or 'tcgen05' (tiles of 128 queries with TMA and TMEM accumulators,
    see attention_prefill_tcgen05_supported). The cache must hold this step's keys and values already; k_new/v_new
    (row views of the buffer q lives in, the same values) let the tcgen05 kernel read the key blocks that lie wholly
    in this step from there, in one piece per block instead of page by page. store_new: the tcgen05 kernel writes
    k_new/v_new into the cache itself (no kv_store before it); only for steps whose entries all start at a position
    that is a multiple of ATTENTION_PREFILL_TCGEN05_KEY_BLOCK (an entry that does not sets error bit 2).
    chunk, gate, keep_first, softcap, sink: as attention_rows; keep_first, softcap and exact_weights (the softmax weights
    meet the values as two bfloat16 terms instead of one rounded to bfloat16) only with kernel 'mma'; a sink alone also with
    'tcgen05'."""
    n_pages, _, kv_heads, page_size, head_dim = cache.shape
    n, n_entries = q.shape[0], entry_pos0.numel()
    more = ()
    if kernel == "tcgen05" and sink is not None and not (keep_first or softcap or exact_weights):
        # the tcgen05 kernel takes a sink (one more term in a row's denominator), none of the other three
        if sink.numel() != n_heads or sink.dtype != torch.float32 or not sink.is_contiguous():
            raise KernelError("attention: the sink must be float32 [heads]")
        more, kernel = (_ptr(sink, "sink"),), "tcgen05_sink"
    elif keep_first or softcap or sink is not None or exact_weights:
        if kernel != "mma":
            raise KernelError("attention_prefill: kept first keys, capped scores, a sink and exact weights need the kernel 'mma'")
        if sink is not None and (sink.numel() != n_heads or sink.dtype != torch.float32 or not sink.is_contiguous()):
            raise KernelError("attention: the sink must be float32 [heads]")
        more = (int(keep_first or 0), float(softcap or 0.0), _ptr(sink, "sink"), int(bool(exact_weights)))
    if q.shape[1] != n_heads * head_dim or q.stride(1) != 1 or q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 \
            or not cache.is_contiguous() or entry_start.numel() != n_entries + 1:
        raise KernelError("attention_prefill: q or the entry arrays do not fit the cache")
    if out is None:
        out = torch.empty((n, n_heads * head_dim), dtype=q.dtype, device=q.device)
    if kernel not in ("mma", "tcgen05", "tcgen05_sink"):
        raise KernelError(f"attention_prefill: unknown kernel {kernel!r}")
    tensor_memory = kernel != "mma"
    if (k_new is None) != (v_new is None) or (k_new is not None and (
            not tensor_memory or k_new.stride(0) != q.stride(0) or v_new.stride(0) != q.stride(0) or k_new.stride(1) != 1
            or v_new.stride(1) != 1 or k_new.dtype != q.dtype or v_new.dtype != q.dtype
            or k_new.shape != (n, kv_heads * head_dim) or v_new.shape != k_new.shape)):
        raise KernelError("attention_prefill: k_new and v_new come together, as row views like q, for the tcgen05 kernel")
    if store_new and k_new is None:
        raise KernelError("attention_prefill: store_new needs k_new and v_new")
    new_rows = (_ptr(k_new, "k_new"), _ptr(v_new, "v_new"), int(bool(store_new))) if tensor_memory else ()
    _call(library("tensor"), "dd_attention_prefill" + ("_" + kernel if tensor_memory else "_sinks" if more else ""), _ptr(q, "q"), q.stride(0), *new_rows,
          _ptr(cache, "cache"),
          _ptr(entry_start, "entry_start", torch.int32), _ptr(entry_pos0, "entry_pos0", torch.int32), n_entries, n,
          _ptr(block_table, "block_table", torch.int32), block_table.shape[1], _ptr(out, "out"), out.stride(0),
          n_heads, kv_heads, head_dim, page_size, n_pages, 0 if window is None else int(window), float(scale),
          _ptr(error_flag(q.device)), _stream(), *_gate_args(gate, q, n_heads, chunk), *more)
    return out
