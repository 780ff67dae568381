"""Host-side mirror of ``ug::Device`` / ``ug::Slice`` and of ug-llama's
``Device`` operator trait, over the C ABI.

Names, argument meaning and error behaviour follow the reference:
ug-core/src/lib.rs:29-73 (traits), ug-cuda/src/runtime.rs (CUDA device),
ug-llama/src/main.rs:22-28 and ug-llama/src/cuda_ops.rs (operators).
Errors surface as :class:`UgError` carrying the status code and the message
the library recorded, the counterpart of ``ug::Error``.
"""
import ctypes as C
import enum

import numpy as np

from ._lib import lib


class DType(enum.IntEnum):
    """ug::DType (ug-core/src/dtype.rs:4-11)."""
    BF16 = 0
    F16 = 1
    F32 = 2
    I32 = 3
    I64 = 4

    @property
    def size_in_bytes(self):
        return {0: 2, 1: 2, 2: 4, 3: 4, 4: 8}[int(self)]


# numpy has no bfloat16: bf16 buffers cross the host boundary as uint16 bit patterns.
_NP = {DType.BF16: np.uint16, DType.F16: np.float16, DType.F32: np.float32,
       DType.I32: np.int32, DType.I64: np.int64}


def np_dtype(dt):
    return _NP[DType(dt)]


def dtype_of(arr, bf16=False):
    if bf16:
        if arr.dtype != np.uint16:
            raise UgError(2, "bf16 host data must be uint16 bit patterns")
        return DType.BF16
    for k, v in _NP.items():
        if k != DType.BF16 and arr.dtype == v:
            return k
    raise UgError(2, f"unsupported host dtype {arr.dtype}")


class UgError(RuntimeError):
    """Counterpart of ug::Error: status code + message."""

    def __init__(self, code, msg):
        super().__init__(f"[ugb status {code}] {msg}")
        self.code = code
        self.msg = msg


class Slice:
    """ug::Slice (ug-core/src/lib.rs:29-47) over a ``ugb_slice`` handle."""

    def __init__(self, device, handle):
        self.device = device
        self._h = handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None and getattr(self.device, "_h", None) and not getattr(self, "_borrowed", False):
            lib.ugb_free(h)

    @property
    def dtype(self):
        return DType(lib.ugb_slice_dtype(self._h))

    def __len__(self):
        return lib.ugb_slice_len(self._h)

    len = property(__len__)

    def is_empty(self):
        return len(self) == 0

    @property
    def device_ptr(self):
        return lib.ugb_slice_ptr(self._h) or 0

    def copy_host_to_device(self, src, bf16=False):
        """Slice::copy_host_to_device: dtype and length must match the slice."""
        src = np.ascontiguousarray(src)
        dt = dtype_of(src, bf16 or self.dtype == DType.BF16 and src.dtype == np.uint16)
        self.device._check(lib.ugb_h2d(self._h, src.ctypes.data, src.size, int(dt)))

    def copy_device_to_host(self, dst):
        dst_dt = DType.BF16 if (self.dtype == DType.BF16 and dst.dtype == np.uint16) else dtype_of(dst)
        if not dst.flags.c_contiguous:
            raise UgError(1, "destination must be contiguous")
        self.device._check(lib.ugb_d2h(self._h, dst.ctypes.data, dst.size, int(dst_dt)))

    def to_vec(self):
        """Slice::to_vec: a fresh host array with the slice's contents."""
        out = np.empty(len(self), dtype=np_dtype(self.dtype))
        self.copy_device_to_host(out)
        return out


class Func:
    """ug::Device::Func: a compiled SSA kernel with its launch configuration."""

    def __init__(self, device, handle):
        self.device, self._h = device, handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None and getattr(self.device, "_h", None):
            lib.ugb_func_free(h)

    @property
    def source(self):
        return (lib.ugb_func_source(self._h) or b"").decode()

    def launch3(self, s1, s2, s3):
        """Func.launch3 of the reference's Python module (ug-pyo3/src/lib.rs:27-50): three slices of one
        length, the last one written."""
        if len(s1) != len(s3):
            raise UgError(3, f"length mismatch {len(s1)} <> {len(s3)}")
        if len(s2) != len(s3):
            raise UgError(3, f"length mismatch {len(s2)} <> {len(s3)}")
        self.device.run(self, [s1, s2, s3])


class Device:
    """ug::Device (ug-core/src/lib.rs:49-73) + ug-llama's operator trait."""

    def __init__(self, ordinal=0):
        h = C.c_void_p()
        rc = lib.ugb_device_create(ordinal, C.byref(h))
        if rc != 0:
            raise UgError(rc, (lib.ugb_last_error(None) or b"").decode())
        self._h = h
        self.ordinal = ordinal

    def close(self):
        h, self._h = self._h, None
        if h:
            lib.ugb_device_destroy(h)

    def _check(self, rc):
        if rc != 0:
            raise UgError(rc, (lib.ugb_last_error(self._h) or b"").decode())

    # ---- ug::Device -------------------------------------------------------
    @staticmethod
    def use_grid():
        return bool(lib.ugb_use_grid())

    def allocate_uninit(self, dtype, length):
        h = C.c_void_p()
        self._check(lib.ugb_alloc(self._h, int(dtype), length, C.byref(h)))
        return Slice(self, h)

    def slice_from_values(self, values, bf16=False):
        """ug_cuda::Device::slice_from_values (ug-cuda/src/runtime.rs:198-202)."""
        values = np.ascontiguousarray(values)
        s = self.allocate_uninit(dtype_of(values, bf16), values.size)
        s.copy_host_to_device(values, bf16)
        return s

    def synchronize(self):
        self._check(lib.ugb_sync(self._h))

    def compile(self, instrs, grid_dim=1, block_dim=1, shared_mem=0, name=None):
        """ug::Device::compile: ``instrs`` is a list of ``ug_b200.lazy.SsaInstr`` (ssa::Instr in wire
        form); the launch shape is the kernel's LaunchConfig (ug-core/src/lang.rs:34-45)."""
        from .lazy import SsaInstr
        arr = (SsaInstr * max(len(instrs), 1))(*instrs)
        h = C.c_void_p()
        self._check(lib.ugb_compile(self._h, arr, len(instrs), grid_dim, block_dim, shared_mem,
                                    name.encode() if name else None, C.byref(h)))
        return Func(self, h)

    def compile_cu(self, cu_code, func_name, grid_dim=1, block_dim=1, shared_mem=0):
        """ug_cuda::Device::compile_cu (runtime.rs:179-186): caller-written CUDA C, pointer parameters only."""
        h = C.c_void_p()
        self._check(lib.ugb_compile_cu(self._h, cu_code.encode(), func_name.encode(), grid_dim, block_dim,
                                       shared_mem, C.byref(h)))
        return Func(self, h)

    def compile_ptx(self, ptx_code, func_name, grid_dim=1, block_dim=1, shared_mem=0):
        """ug_cuda::Device::compile_ptx (runtime.rs:188-193)."""
        h = C.c_void_p()
        self._check(lib.ugb_compile_ptx(self._h, ptx_code.encode(), func_name.encode(), grid_dim, block_dim,
                                        shared_mem, C.byref(h)))
        return Func(self, h)

    def zeros(self, length):
        """ug_cuda::Device::zeros (runtime.rs:195-198): an f32 slice of zeros."""
        return self.slice_from_values(np.zeros(length, np.float32))

    def run(self, func, args):
        """ug::Device::run: one slice per pointer argument of the kernel."""
        arr = (C.c_void_p * max(len(args), 1))(*[a._h for a in args])
        self._check(lib.ugb_run(self._h, func._h, arr, len(args)))

    @property
    def launch_count(self):
        return lib.ugb_launch_count(self._h)

    def matmul(self, dst, lhs, rhs, bmnk, lhs_l, rhs_l):
        """ug::Device::matmul; a layout is (dims, strides, offset) in elements."""
        b, m, n, k = bmnk
        (ld, ls, lo), (rd, rs, ro) = lhs_l, rhs_l
        if len(ld) != len(rd):
            raise UgError(3, f"matmul: operand ranks differ {ld} {rd}")
        rank = len(ld)
        arr = C.c_size_t * rank
        self._check(lib.ugb_matmul(self._h, dst._h, lhs._h, rhs._h, b, m, n, k, rank,
                                   C.cast(arr(*ld), C.c_void_p), C.cast(arr(*ls), C.c_void_p), lo,
                                   C.cast(arr(*rd), C.c_void_p), C.cast(arr(*rs), C.c_void_p), ro))

    # ---- timing on the device's own stream --------------------------------
    def timer_begin(self):
        self._check(lib.ugb_timer_begin(self._h))

    def timer_end(self):
        self._check(lib.ugb_timer_end(self._h))

    def timer_elapsed_ms(self):
        ms = C.c_float()
        self._check(lib.ugb_timer_elapsed_ms(self._h, C.byref(ms)))
        return ms.value

    # ---- ug_llama::Device (ug-llama/src/main.rs:22-28) ---------------------
    def custom_softmax(self, src, dst, n_rows, n_cols):
        self._check(lib.ugb_softmax(self._h, src._h, dst._h, n_rows, n_cols))

    def causal_mask(self, src, dst, bh, s1, s2):
        self._check(lib.ugb_causal_mask(self._h, src._h, dst._h, bh, s1, s2))

    def rope(self, src, cos, sin, pos, dst, b, h, t, d):
        self._check(lib.ugb_rope(self._h, src._h, cos._h, sin._h, pos._h, dst._h, b, h, t, d))

    def rope_i(self, src, cos, sin, pos, dst, b, h, t, d):
        self._check(lib.ugb_rope_i(self._h, src._h, cos._h, sin._h, pos._h, dst._h, b, h, t, d))

    def cat(self, lhs, rhs, dst, d1, d2_l, d2_r):
        self._check(lib.ugb_cat(self._h, lhs._h, rhs._h, dst._h, d1, d2_l, d2_r))

    # ---- fused row / map operators -----------------------------------------
    def rms_norm(self, x, alpha, dst, n_rows, n_cols, eps):
        self._check(lib.ugb_rms_norm(self._h, x._h, alpha._h, dst._h, n_rows, n_cols, eps))

    def rms_norm_silu_gate(self, x, alpha, gate, dst, n_rows, n_cols, eps):
        self._check(lib.ugb_rms_norm_silu_gate(self._h, x._h, alpha._h, gate._h, dst._h, n_rows,
                                               n_cols, eps))

    def silu_mul(self, gate, up, dst, n):
        self._check(lib.ugb_silu_mul(self._h, gate._h, up._h, dst._h, n))

    def add(self, a, b, dst, n):
        self._check(lib.ugb_add(self._h, a._h, b._h, dst._h, n))

    def index_select(self, emb, ids, dst, n_ids, h, vocab):
        self._check(lib.ugb_index_select(self._h, emb._h, ids._h, dst._h, n_ids, h, vocab))

    def set_option(self, name, value):
        """Tuning switch of the device handle (ugb_device_set_option), e.g. gemm_cta_pairs = 0 / 1."""
        self._check(lib.ugb_device_set_option(self._h, name.encode(), int(value)))

    def causal_attention(self, q, k, v, out, b, t, pos0, n_heads, n_kv, t_max):
        """Fused causal grouped-query attention for a block of t new positions per sequence over the
        cache (Attention::fwd with seq_len > 1, model.rs:231-245)."""
        self._check(lib.ugb_causal_attention(self._h, q._h, k._h, v._h, out._h, b, t, pos0, n_heads, n_kv, t_max))

    def decode_attention(self, q, k, v, pos, out, b, n_heads, n_kv, t_max, n_slices=2):
        """Fused grouped-query attention for one new position per sequence (model.rs:231-245)."""
        self._check(lib.ugb_decode_attention(self._h, q._h, k._h, v._h, pos._h, out._h, b, n_heads, n_kv,
                                             t_max, n_slices))
