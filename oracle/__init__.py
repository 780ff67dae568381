"""CPU oracle for the ug hot path -- TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers over the two C restatements in this directory
(``ug_cpu_ops.c``: ug-llama's hand-written CPU operators with Rust
arithmetic rules; ``ug_cpu_gen.c``: the C that ug-core's CPU backend emits,
built with the reference's own gcc flags).  Nothing in the shipped package
imports this module: only the tests, the smoke check and the CPU-baseline
leg of the benchmark do, and only as the checker / the timed baseline.
"""
import ctypes as C

import numpy as np

from . import build as _build

_gen_path, _ops_path = _build.build()
_gen = C.CDLL(_gen_path)
_ops = C.CDLL(_ops_path)

_ops.ug_set_threads.restype = C.c_int
_ops.ug_set_threads.argtypes = [C.c_int]


# "Long-run" mode, for oracle runs of thousands of positions (a 2048-position prompt through the
# 22-layer model) that the strict forms would spend minutes on: the GEMM stand-in becomes numpy's
# blocked sgemm (the accumulation order of crate gemm is unpinned either way) and rms_norm computes
# each row's sum of squares once instead of once per element (the same value, O(cols) instead of
# O(cols^2)).  Everything else -- rope, cat, masks, softmax, silu, adds -- stays on the C restatements.
_long_run = False


class long_run_mode:
    """Context manager that switches the oracle to its long-run forms (see above)."""

    def __enter__(self):
        global _long_run
        self._prev, _long_run = _long_run, True
        return self

    def __exit__(self, *exc):
        global _long_run
        _long_run = self._prev
        return False


def set_threads(n=0):
    """Threads of the oracle's row loops and GEMM stand-in (0 = leave as is); returns the count in force."""
    return int(_ops.ug_set_threads(int(n)))


_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_u16p = C.POINTER(C.c_uint16)


def _p(a, t=_f32p):
    return a.ctypes.data_as(t)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


for _name, _args in {
    "ug_custom_softmax_f32": [_f32p, _f32p, C.c_size_t, C.c_size_t],
    "ug_causal_mask_f32": [_f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t],
    "ug_rope_f32": [_f32p, _f32p, _f32p, _i32p, _f32p] + [C.c_size_t] * 4,
    "ug_rope_i_f32": [_f32p, _f32p, _f32p, _i32p, _f32p] + [C.c_size_t] * 4,
    "ug_cat_f32": [_f32p, _f32p, _f32p] + [C.c_size_t] * 3,
    "ug_index_select_f32": [_f32p, _i32p, _f32p, C.c_size_t, C.c_size_t],
    "ug_gemm_f32": [_f32p, _f32p, _f32p] + [C.c_size_t] * 4
    + [C.c_ssize_t, C.c_ssize_t, C.c_size_t, C.c_ssize_t, C.c_ssize_t, C.c_size_t],
    "ug_round_to_bf16_f32": [_f32p, _f32p, C.c_size_t],
    "ug_f32_to_bf16": [_f32p, _u16p, C.c_size_t],
}.items():
    getattr(_ops, _name).argtypes = _args
    getattr(_ops, _name).restype = None

for _name, _args in {
    "ug_gen_softmax_exp": [_f32p, _f32p] + [C.c_int] * 4,
    "ug_gen_softmax_div": [_f32p, _f32p] + [C.c_int] * 4,
    "ug_gen_rms_norm": [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int,
                        C.c_int],
    "ug_gen_rms_norm_silu_gate": [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_float,
                                  C.c_float, C.c_int, C.c_int],
    "ug_gen_silu_mul": [_f32p, _f32p, _f32p, C.c_int],
    "ug_gen_add": [_f32p, _f32p, _f32p, C.c_int],
}.items():
    getattr(_gen, _name).argtypes = _args
    getattr(_gen, _name).restype = None


# ---------------------------------------------------------------- custom ops
def custom_softmax(x):
    """ug-llama/src/cpu_ops.rs:6-31 over the last dimension."""
    x = _f32(x)
    y = np.empty_like(x)
    n_cols = x.shape[-1]
    _ops.ug_custom_softmax_f32(_p(x), _p(y), x.size // max(n_cols, 1), n_cols)
    return y


def causal_mask(x):
    """ug-llama/src/cpu_ops.rs:33-56 on [b, h, s1, s2]."""
    x = _f32(x)
    b, h, s1, s2 = x.shape
    y = np.empty_like(x)
    _ops.ug_causal_mask_f32(_p(x), _p(y), b * h, s1, s2)
    return y


def _rope(fn, x, cos, sin, pos):
    x, cos, sin = _f32(x), _f32(cos), _f32(sin)
    pos = np.ascontiguousarray(pos, dtype=np.int32).reshape(-1)
    b, h, t, d = x.shape
    y = np.empty_like(x)
    fn(_p(x), _p(cos), _p(sin), _p(pos, _i32p), _p(y), b, h, t, d)
    return y


def rope(x, cos, sin, pos):
    """ug-llama/src/cpu_ops.rs:91-127 (half rotation)."""
    return _rope(_ops.ug_rope_f32, x, cos, sin, pos)


def rope_i(x, cos, sin, pos):
    """ug-llama/src/cpu_ops.rs:58-89 (interleaved pairs)."""
    return _rope(_ops.ug_rope_i_f32, x, cos, sin, pos)


def cat(lhs, rhs, axis):
    """ug-llama/src/cpu_ops.rs:129-167."""
    lhs, rhs = _f32(lhs), _f32(rhs)
    if axis >= lhs.ndim or lhs.ndim != rhs.ndim:
        raise ValueError(f"unexpected shapes for cat {lhs.shape} {rhs.shape} axis: {axis}")
    for i, (l, r) in enumerate(zip(lhs.shape, rhs.shape)):
        if i != axis and l != r:
            raise ValueError(f"unexpected shapes for cat {lhs.shape} {rhs.shape} axis: {axis}")
    dims = list(lhs.shape)
    dims[axis] = lhs.shape[axis] + rhs.shape[axis]
    d1 = int(np.prod(lhs.shape[:axis], dtype=np.int64))
    d2_l = int(np.prod(lhs.shape[axis:], dtype=np.int64))
    d2_r = int(np.prod(rhs.shape[axis:], dtype=np.int64))
    y = np.empty(dims, dtype=np.float32)
    _ops.ug_cat_f32(_p(lhs), _p(rhs), _p(y), d1, d2_l, d2_r)
    return y


def index_select(emb, ids):
    """ug-llama/src/model.rs:32-63: dst[b, t, :] = emb[ids[b, t], :]."""
    emb = _f32(emb)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    y = np.empty(ids.shape + (emb.shape[1],), dtype=np.float32)
    _ops.ug_index_select_f32(_p(emb), _p(ids, _i32p), _p(y), ids.size, emb.shape[1])
    return y


def matmul(lhs, rhs, transpose_rhs=False):
    """Stand-in for crate gemm 0.18.0 behind ug-core/src/cpu_runtime.rs:551-619.

    ``lhs`` is [b, m, k] (or [m, k]); ``rhs`` is [b, k, n], or [b, n, k] when
    ``transpose_rhs`` (LazyBuffer::matmul_t); a rank-2 rhs is shared by every
    batch step (batch skip 0).
    """
    lhs, rhs = _f32(lhs), _f32(rhs)
    if _long_run:
        r = np.swapaxes(rhs, -1, -2) if transpose_rhs else rhs
        return np.matmul(lhs, r)
    squeeze = lhs.ndim == 2
    if squeeze:
        lhs = lhs[None]
    b, m, k = lhs.shape
    shared = rhs.ndim == 2
    r = rhs if not shared else rhs[None]
    if transpose_rhs:
        n = r.shape[1]
        assert r.shape[2] == k
        rs, cs = 1, k
    else:
        n = r.shape[2]
        assert r.shape[1] == k
        rs, cs = n, 1
    y = np.empty((b, m, n), dtype=np.float32)
    _ops.ug_gemm_f32(_p(y), _p(lhs), _p(r), b, m, n, k, k, 1, m * k, rs, cs,
                     0 if shared else n * k)
    return y[0] if squeeze else y


def round_bf16(x):
    """f32 -> bf16 (round to nearest even) -> f32, as half 2.3.1 does."""
    x = _f32(x)
    y = np.empty_like(x)
    _ops.ug_round_to_bf16_f32(_p(x), _p(y), x.size)
    return y


def to_bf16_bits(x):
    x = _f32(x)
    y = np.empty(x.shape, dtype=np.uint16)
    _ops.ug_f32_to_bf16(_p(x), _p(y, _u16p), x.size)
    return y


# ----------------------------------------------- emitted-C (lazy graph) forms
def gen_softmax(x, rows=None):
    """model.rs:94-101 through the CPU backend: two kernels, O(rows*cols^2)."""
    x = _f32(x)
    n_cols = x.shape[-1]
    n_rows = x.size // n_cols
    lo, hi = (0, n_rows) if rows is None else rows
    e = np.zeros_like(x)
    y = np.zeros_like(x)
    _gen.ug_gen_softmax_exp(_p(x), _p(e), n_rows, n_cols, lo, hi)
    _gen.ug_gen_softmax_div(_p(e), _p(y), n_rows, n_cols, lo, hi)
    return y


def gen_rms_norm(x, alpha, eps, rows=None):
    """model.rs:65-78 through the CPU backend."""
    x, alpha = _f32(x), _f32(alpha)
    n_cols = x.shape[-1]
    n_rows = x.size // n_cols
    lo, hi = (0, n_rows) if rows is None else rows
    inv_d = np.float32(1.0) / np.float32(n_cols)
    if _long_run and rows is None:
        ss = np.sum(x * x, axis=-1, keepdims=True, dtype=np.float32)
        return (x / np.sqrt(ss * inv_d + np.float32(eps)) * alpha).astype(np.float32)
    y = np.zeros_like(x)
    _gen.ug_gen_rms_norm(_p(x), _p(alpha), _p(y), n_rows, n_cols, inv_d, np.float32(eps), lo, hi)
    return y


def gen_rms_norm_silu_gate(x, alpha, gate, eps, rows=None):
    """rms_norm(x) * alpha * silu(gate) as one CPU-backend kernel."""
    x, alpha, gate = _f32(x), _f32(alpha), _f32(gate)
    n_cols = x.shape[-1]
    n_rows = x.size // n_cols
    lo, hi = (0, n_rows) if rows is None else rows
    y = np.zeros_like(x)
    inv_d = np.float32(1.0) / np.float32(n_cols)
    _gen.ug_gen_rms_norm_silu_gate(_p(x), _p(alpha), _p(gate), _p(y), n_rows, n_cols, inv_d,
                                   np.float32(eps), lo, hi)
    return y


def gen_silu_mul(gate, up):
    gate, up = _f32(gate), _f32(up)
    y = np.empty_like(gate)
    _gen.ug_gen_silu_mul(_p(gate), _p(up), _p(y), gate.size)
    return y


def gen_add(a, b):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    _gen.ug_gen_add(_p(a), _p(b), _p(y), a.size)
    return y


# ------------------------------------------------- CPU backend as a host-layer device
class CpuOps:
    """ug-llama's CPU operators (ug-llama/src/cpu_ops.rs) on slices of the oracle CPU device."""

    def __init__(self, lib):
        self._lib = lib

    def _arr(self, raw, n, dtype=np.float32):
        p = self._lib.oracle_cpu_slice_ptr(raw)
        if not p:
            raise ValueError("not a CPU slice")
        ct = C.c_float if dtype == np.float32 else C.c_int32
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=(max(n, 1),))[:n]

    def softmax(self, src, dst, n_rows, n_cols):
        n = n_rows * n_cols
        _ops.ug_custom_softmax_f32(_p(self._arr(src, n)), _p(self._arr(dst, n)), n_rows, n_cols)

    def causal_mask(self, src, dst, bh, s1, s2):
        n = bh * s1 * s2
        _ops.ug_causal_mask_f32(_p(self._arr(src, n)), _p(self._arr(dst, n)), bh, s1, s2)

    def rope(self, interleaved, src, cos, sin, pos, dst, b, h, t, d):
        n = b * h * t * d
        fn = _ops.ug_rope_i_f32 if interleaved else _ops.ug_rope_f32
        from ug_b200.lazy import host
        nc = host.ugh_slice_len(cos)
        fn(_p(self._arr(src, n)), _p(self._arr(cos, nc)), _p(self._arr(sin, nc)),
           _p(self._arr(pos, 1, np.int32), _i32p), _p(self._arr(dst, n)), b, h, t, d)

    def cat(self, lhs, rhs, dst, d1, d2_l, d2_r):
        _ops.ug_cat_f32(_p(self._arr(lhs, d1 * d2_l)), _p(self._arr(rhs, d1 * d2_r)),
                        _p(self._arr(dst, d1 * (d2_l + d2_r))), d1, d2_l, d2_r)


def cpu_host_device():
    """ug-core's CPU backend (oracle/cpu_device.cpp) as a ``ug_b200.lazy.HostDevice``."""
    from ug_b200 import lazy
    lib = C.CDLL(_build.build_cpu_device())
    lib.oracle_cpu_device_new.restype = C.c_void_p
    lib.oracle_cpu_slice_ptr.restype = C.c_void_p
    lib.oracle_cpu_slice_ptr.argtypes = [C.c_void_p]
    dev = lazy.HostDevice.adopt(lib.oracle_cpu_device_new(), CpuOps(lib))
    dev._cpu_lib = lib
    return dev


# ------------------------------------- the reference's own CUDA kernels (oracle/_ref)
def reference_cuda():
    """ctypes handle on oracle/_ref/libugref_cuda.so (the reference's softmax.cu / rope.cu / cat.cu
    compiled where they lie by oracle/build_ref.py), or None when it was not built."""
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libugref_cuda.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    vp, ci, cu = C.c_void_p, C.c_int, C.c_uint
    lib.ugref_softmax_f32.argtypes = [vp, vp, ci, ci, vp]
    lib.ugref_rope_f32.argtypes = [vp, vp, vp, vp, vp, cu, cu, cu, cu, vp]
    lib.ugref_cat_f32.argtypes = [vp, vp, vp, cu, cu, cu, vp]
    return lib
