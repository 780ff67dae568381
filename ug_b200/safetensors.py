"""ug::safetensors::MmapedSafetensors (ug-core/src/safetensors.rs:10-318) over the C ABI."""
import ctypes as C

from ._lib import lib
from .device import DType, Slice, UgError


class MmapedSafetensors:
    """Memory-mapped .safetensors file(s); ``MmapedSafetensors(path)`` is ``::new``, a list of paths
    is ``::multi`` (a name present in several files resolves to the last one)."""

    def __init__(self, paths, dev):
        if isinstance(paths, (str, bytes)) or hasattr(paths, "__fspath__"):
            paths = [paths]
        self.dev = dev
        enc = [str(p).encode() for p in paths]
        arr = (C.c_char_p * len(enc))(*enc)
        h = C.c_void_p()
        dev._check(lib.ugb_st_open(dev._h, arr, len(enc), C.byref(h)))
        self._h = h

    @classmethod
    def multi(cls, paths, dev):
        return cls(list(paths), dev)

    def close(self):
        h, self._h = self._h, None
        if h:
            lib.ugb_st_close(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def names(self):
        return [lib.ugb_st_name(self._h, i).decode() for i in range(lib.ugb_st_count(self._h))]

    def get(self, name):
        """(dtype, shape) of a tensor; dtype is None for a safetensors dtype ug has no DType for."""
        dt, rank = C.c_int32(), C.c_int32()
        dims = (C.c_size_t * 8)()
        self.dev._check(lib.ugb_st_info(self.dev._h, self._h, name.encode(), C.byref(dt), C.byref(rank), dims, 8))
        return (DType(dt.value) if dt.value >= 0 else None), tuple(dims[i] for i in range(rank.value))

    def tensors(self):
        return [(n, *self.get(n)) for n in self.names()]

    def load_slice(self, name, dev=None):
        """(shape, Slice) with the tensor's own dtype (safetensors.rs:83-118)."""
        dev = dev or self.dev
        h = C.c_void_p()
        dev._check(lib.ugb_st_load_slice(dev._h, self._h, name.encode(), C.byref(h)))
        return self.get(name)[1], Slice(dev, h)

    def load_slice_with_cast(self, name, dtype, dev=None):
        """(shape, Slice) converted to ``dtype`` on the host (safetensors.rs:120-271)."""
        dev = dev or self.dev
        h = C.c_void_p()
        dev._check(lib.ugb_st_load_slice_with_cast(dev._h, self._h, name.encode(), int(dtype), C.byref(h)))
        return self.get(name)[1], Slice(dev, h)
