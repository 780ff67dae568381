"""Host-side mirror of ug-core's lazy graph API over ``libughost.so``.

``LazyBuffer`` (``LB``), ``Schedule``, ``CompiledSchedule`` and
``CompilationCache`` follow ug-core/src/lazy_buffer.rs, schedule.rs and
cache.rs: the same builder names, argument meaning and error behaviour
(errors surface as :class:`ug_b200.UgError`).  The graph, the scheduler and
the lowering run in C++ (``ug_b200/csrc/host``); this module only marshals.
"""
import ctypes as C
import enum
import os
import re

import numpy as np

from . import _lib
from .device import DType, UgError, np_dtype

HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB = os.path.join(HERE, "libughost.so")
HOST_HEADER = os.path.join(HERE, "..", "include", "ughost.h")

CUSTOM_FN = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.POINTER(C.c_void_p), C.c_size_t)


def _load():
    if not os.path.exists(HOST_LIB):
        raise ImportError(f"{HOST_LIB} is missing: build it with `python -m ug_b200.build`")
    _ = _lib.lib          # libugb200.so first (libughost.so links against it)
    h = C.CDLL(HOST_LIB)
    for name, (ret, params) in _lib.parse_header(HOST_HEADER).items():
        fn = getattr(h, name)
        fn.restype = _lib._ctype(ret)
        fn.argtypes = [CUSTOM_FN if "ugh_custom_fn" in p else _lib._param_type(p) for p in params]
    return h


_lib._CTYPES.setdefault("int64_t", C.c_int64)
host = _load()


def _err():
    return (host.ugh_last_error() or b"").decode()


def _ptr(h):
    if not h:
        raise UgError(1, _err())
    return h


def _chk(rc):
    if rc != 0:
        raise UgError(rc, _err())


def _dims(shape):
    shape = tuple(int(d) for d in (shape if hasattr(shape, "__len__") else (shape,)))
    return (C.c_size_t * max(len(shape), 1))(*shape), len(shape)


class UnaryOp(enum.IntEnum):
    """ug::lang::UnaryOp (ug-core/src/lang.rs:12-21); casts go through ``LazyBuffer.cast``."""
    Id = 0
    Exp = 1
    Sin = 2
    Cos = 3
    Neg = 4
    Sqrt = 5


class BinaryOp(enum.IntEnum):
    """ug::lang::BinaryOp (lang.rs:23-32)."""
    Add = 0
    Sub = 1
    Mul = 2
    Div = 3
    Mod = 4
    Min = 5
    Max = 6


class ReduceOp(enum.IntEnum):
    """ug::lang::ReduceOp (lang.rs:5-10)."""
    Sum = 0
    Max = 1
    Min = 2


class SsaInstr(C.Structure):
    class Arg(C.Structure):
        _fields_ = [("is_var", C.c_int32), ("dtype", C.c_int32), ("value", C.c_int64)]

    _fields_ = [("kind", C.c_int32), ("dtype", C.c_int32), ("op", C.c_int32), ("reserved", C.c_int32),
                ("index", C.c_int64), ("v0", C.c_int64), ("a0", Arg), ("a1", Arg), ("cst", Arg)]


class ssa:
    """Builders for hand-written SSA kernels (ug-core/src/lang.rs:690-709); a variable is the line
    number of the instruction that defines it."""
    KINDS = ["DefineAcc", "DefineGlobal", "DefineLocal", "Special", "Const", "Unary", "Binary", "Range", "Load",
             "Assign", "EndRange", "If", "EndIf", "Store", "Barrier", "ReduceLocal"]

    @staticmethod
    def var(v):
        return SsaInstr.Arg(1, 0, int(v))

    @staticmethod
    def i32(v):
        return SsaInstr.Arg(0, int(DType.I32), int(v))

    @staticmethod
    def f32(v):
        return SsaInstr.Arg(0, int(DType.F32), int(np.float32(v).view(np.uint32)))

    @staticmethod
    def _a(x):
        return x if isinstance(x, SsaInstr.Arg) else ssa.var(x)

    @staticmethod
    def instr(kind, dtype=DType.F32, op=0, index=0, v0=0, a0=None, a1=None, cst=None):
        i = SsaInstr()
        i.kind, i.dtype, i.op, i.index, i.v0 = ssa.KINDS.index(kind), int(dtype), int(op), int(index), int(v0)
        if a0 is not None:
            i.a0 = ssa._a(a0)
        if a1 is not None:
            i.a1 = ssa._a(a1)
        if cst is not None:
            i.cst = cst
        return i


class HostDevice:
    """A device handle of the host layer.  ``HostDevice(ug_b200.Device(0))`` wraps the B200 backend;
    ``HostDevice.adopt(ptr, ops)`` takes a C++ ``ug::Device*`` created elsewhere (the tests plug the
    CPU oracle in this way) together with the object that implements ug-llama's operators for it."""

    def __init__(self, dev=None, _handle=None, ops=None):
        if _handle is not None:
            self._h, self.b200, self.ops = _handle, None, ops
        else:
            self._h = _ptr(host.ugh_device_b200(dev._h))
            self.b200 = dev
            self.ops = B200Ops(dev)
        self._keep = []          # ctypes callbacks must outlive the graph nodes that hold them

    @classmethod
    def adopt(cls, cpp_device_ptr, ops):
        return cls(_handle=_ptr(host.ugh_device_adopt(cpp_device_ptr)), ops=ops)

    def set_launch_policy(self, reference):
        """True: the reference's grid heuristic (ug-core/src/schedule.rs:162-188); False: this backend's."""
        _chk(host.ugh_device_set_launch_policy(self._h, 0 if reference else 1))

    def synchronize(self):
        _chk(host.ugh_device_synchronize(self._h))


class B200Ops:
    """ug-llama's Device operators (ug-llama/src/main.rs:22-28) on B200 slices."""

    def __init__(self, dev):
        self.dev = dev

    def _s(self, raw):
        from .device import Slice
        s = Slice.__new__(Slice)
        s.device, s._h, s._borrowed = self.dev, C.c_void_p(host.ugh_slice_b200(raw)), True
        if not s._h:
            raise UgError(1, "custom op received a slice of another device")
        return s

    def softmax(self, src, dst, n_rows, n_cols):
        self.dev.custom_softmax(self._s(src), self._s(dst), n_rows, n_cols)

    def causal_mask(self, src, dst, bh, s1, s2):
        self.dev.causal_mask(self._s(src), self._s(dst), bh, s1, s2)

    def rope(self, interleaved, src, cos, sin, pos, dst, b, h, t, d):
        f = self.dev.rope_i if interleaved else self.dev.rope
        f(self._s(src), self._s(cos), self._s(sin), self._s(pos), self._s(dst), b, h, t, d)

    def cat(self, lhs, rhs, dst, d1, d2_l, d2_r):
        self.dev.cat(self._s(lhs), self._s(rhs), self._s(dst), d1, d2_l, d2_r)


class LazyBuffer:
    """ug::LazyBuffer (ug-core/src/lazy_buffer.rs)."""

    def __init__(self, handle, device):
        self._h, self.device = handle, device

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            host.ugh_lb_free(h)

    def _new(self, h):
        return LazyBuffer(_ptr(h), self.device)

    # ---- constructors
    @staticmethod
    def cst(value, shape, device):
        d, r = _dims(shape)
        if isinstance(value, (int, np.integer)) and not isinstance(value, bool):
            return LazyBuffer(_ptr(host.ugh_lb_cst_i32(int(value), d, r, device._h)), device)
        return LazyBuffer(_ptr(host.ugh_lb_cst_f32(float(value), d, r, device._h)), device)

    @staticmethod
    def copy(data, shape, device, bf16=False):
        data = np.ascontiguousarray(data)
        dt = DType.BF16 if bf16 else {np.dtype(np.float32): DType.F32, np.dtype(np.int32): DType.I32,
                                      np.dtype(np.int64): DType.I64, np.dtype(np.float16): DType.F16}[data.dtype]
        d, r = _dims(shape)
        return LazyBuffer(_ptr(host.ugh_lb_copy(data.ctypes.data, data.size, int(dt), d, r, device._h)), device)

    @staticmethod
    def alloc_uninit(dtype, shape, device):
        d, r = _dims(shape)
        return LazyBuffer(_ptr(host.ugh_lb_alloc_uninit(int(dtype), d, r, device._h)), device)

    @staticmethod
    def custom(f, args, shape, dtype, device):
        """``f(slices)`` receives opaque slice handles, arguments in call order and the destination last."""
        cb = _make_cb(f)
        device._keep.append(cb)
        arr = (C.c_void_p * max(len(args), 1))(*[a._h for a in args])
        d, r = _dims(shape)
        return LazyBuffer(_ptr(host.ugh_lb_custom(cb, None, arr, len(args), d, r, int(dtype), device._h)), device)

    def custom_ip(self, f, args):
        cb = _make_cb(f)
        self.device._keep.append(cb)
        arr = (C.c_void_p * max(len(args), 1))(*[a._h for a in args])
        return self._new(host.ugh_lb_custom_ip(self._h, cb, None, arr, len(args)))

    @staticmethod
    def ssa(instrs, args, shape, dtype, device):
        ins = (SsaInstr * len(instrs))(*instrs)
        arr = (C.c_void_p * max(len(args), 1))(*[a._h for a in args])
        d, r = _dims(shape)
        return LazyBuffer(_ptr(host.ugh_lb_ssa(ins, len(instrs), arr, len(args), d, r, int(dtype), device._h)), device)

    @staticmethod
    def cat(args, dim):
        arr = (C.c_void_p * len(args))(*[a._h for a in args])
        return LazyBuffer(_ptr(host.ugh_lb_cat(arr, len(args), dim)), args[0].device)

    # ---- builders
    def unary(self, op):
        return self._new(host.ugh_lb_unary(self._h, int(op)))

    def cast(self, dtype):
        return self._new(host.ugh_lb_cast(self._h, int(dtype)))

    def binary(self, op, rhs):
        return self._new(host.ugh_lb_binary(self._h, int(op), rhs._h))

    def reduce(self, op, dim):
        return self._new(host.ugh_lb_reduce(self._h, int(op), dim))

    def matmul(self, rhs):
        return self._new(host.ugh_lb_matmul(self._h, rhs._h, 0))

    def matmul_t(self, rhs):
        return self._new(host.ugh_lb_matmul(self._h, rhs._h, 1))

    def broadcast(self, shape):
        d, r = _dims(shape)
        return self._new(host.ugh_lb_broadcast(self._h, d, r))

    def reshape(self, shape):
        d, r = _dims(shape)
        return self._new(host.ugh_lb_reshape(self._h, d, r))

    def transpose(self, dim1, dim2):
        return self._new(host.ugh_lb_transpose(self._h, dim1, dim2))

    def split_dim(self, dim, size1, size2):
        return self._new(host.ugh_lb_split_dim(self._h, dim, size1, size2))

    def merge_dims(self, dim):
        return self._new(host.ugh_lb_merge_dims(self._h, dim))

    def narrow(self, dim, offset, length):
        return self._new(host.ugh_lb_narrow(self._h, dim, offset, length))

    def squeeze(self, dim):
        return self._new(host.ugh_lb_squeeze(self._h, dim))

    def unsqueeze(self, dim):
        return self._new(host.ugh_lb_unsqueeze(self._h, dim))

    def set(self, values):
        return self._new(host.ugh_lb_set(self._h, values._h))

    def set_l(self, values, dims, strides=None, offset=0):
        dims = tuple(dims) if hasattr(dims, "__len__") else (dims,)
        if strides is None:          # Layout::from_shape
            strides, acc = [], 1
            for d in reversed(dims):
                strides.append(acc)
                acc *= d
            strides = tuple(reversed(strides))
        n = len(dims)
        return self._new(host.ugh_lb_set_l(self._h, values._h, (C.c_size_t * n)(*dims), (C.c_size_t * n)(*strides), n, offset))

    # ---- queries
    def dims(self):
        r = host.ugh_lb_rank(self._h)
        out = (C.c_size_t * max(r, 1))()
        host.ugh_lb_dims(self._h, out)
        return tuple(out[i] for i in range(r))

    shape = dims

    def rank(self):
        return host.ugh_lb_rank(self._h)

    def dtype(self):
        return DType(host.ugh_lb_dtype(self._h))

    def elem_count(self):
        return int(np.prod(self.dims(), dtype=np.int64))

    def realized(self):
        return bool(host.ugh_lb_realized(self._h))

    def realize(self):
        _chk(host.ugh_lb_realize(self._h))

    def data_vec(self):
        """LazyBuffer::data_vec: realize, then read back (bf16 comes back as uint16 bit patterns)."""
        out = np.empty(self.elem_count(), dtype=np_dtype(self.dtype()))
        _chk(host.ugh_lb_data(self._h, out.ctypes.data, out.size, int(self.dtype())))
        return out

    def write(self, data):
        """Overwrite the realized storage (what the reference's tests do through ``data()``)."""
        data = np.ascontiguousarray(data, dtype=np_dtype(self.dtype()))
        _chk(host.ugh_lb_write(self._h, data.ctypes.data, data.size, int(self.dtype())))


LB = LazyBuffer


def _make_cb(f):
    def cb(_user, slices, n):
        try:
            f([slices[i] for i in range(n)])
            return 0
        except Exception as e:      # noqa: BLE001 -- reported through the C status, never raised across the ABI
            import sys
            print(f"custom op failed: {e!r}", file=sys.stderr)
            return 1
    return CUSTOM_FN(cb)


class CompilationCache:
    """ug::cache::CompilationCache (ug-core/src/cache.rs:73-101)."""

    def __init__(self):
        self._h = host.ugh_cache_create()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            host.ugh_cache_free(h)

    @property
    def hits(self):
        return host.ugh_cache_hits(self._h)

    @property
    def misses(self):
        return host.ugh_cache_misses(self._h)

    @property
    def poly_hits(self):
        """Hits served by a shape-generic kernel (the same kernel seen before at another size)."""
        return host.ugh_cache_poly_hits(self._h)

    def set_polymorphic(self, on):
        host.ugh_cache_set_polymorphic(self._h, int(bool(on)))


class CompiledSchedule:
    def __init__(self, h, buffers):
        self._h, self._buffers = h, buffers

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            host.ugh_compiled_free(h)

    def run(self):
        _chk(host.ugh_compiled_run(self._h))

    def __len__(self):
        return host.ugh_compiled_n_funcs(self._h)

    def origins(self):
        """Per function: "matmul", "custom", "ssa", or the generated vectorised shape it runs on."""
        out = []
        for i in range(len(self)):
            buf = C.create_string_buffer(64)
            _chk(host.ugh_compiled_func_origin(self._h, i, buf, len(buf)))
            out.append(buf.value.decode())
        return out


class Schedule:
    """ug::Schedule (ug-core/src/schedule.rs:62-207)."""
    KINDS = ("Kernel", "MatMul", "Custom", "Ssa")

    def __init__(self, h, buffers):
        self._h, self._buffers = h, buffers

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            host.ugh_schedule_free(h)

    @staticmethod
    def create(buffers):
        arr = (C.c_void_p * len(buffers))(*[b._h for b in buffers])
        return Schedule(_ptr(host.ugh_schedule_create(arr, len(buffers))), list(buffers))

    @staticmethod
    def create_one(buffer):
        return Schedule.create([buffer])

    def items(self):
        return [self.KINDS[host.ugh_schedule_item_kind(self._h, i)] for i in range(host.ugh_schedule_n_items(self._h))]

    def ssa_text(self, i, policy=-1):
        """SSA listing of kernel item ``i``: policy -1 default Opts, 0 reference grid, 1 this backend's."""
        buf = C.create_string_buffer(1 << 20)
        _chk(host.ugh_schedule_item_ssa_text(self._h, i, policy, buf, len(buf)))
        return buf.value.decode()

    def fast_source(self, i):
        """CUDA C generated for kernel item ``i`` when it is a row or map kernel ("" otherwise)."""
        buf = C.create_string_buffer(1 << 20)
        _chk(host.ugh_schedule_item_fast_source(self._h, i, buf, len(buf)))
        return buf.value.decode()

    def compile(self, cache=None):
        return CompiledSchedule(_ptr(host.ugh_schedule_compile(self._h, cache._h if cache else None)), self._buffers)

    compile_with_cache = compile
