"""ug_b200 -- B200 (sm_100a) execution backend for ug's hot path.

Python host mirror of the reference's backend interface (``ug::Device`` /
``ug::Slice`` and ug-llama's operator trait) over the C ABI of
``libugb200.so``.  The CUDA library is the implementation; this package only
marshals arguments.  Attributes resolve lazily so that ``ug_b200.build`` can
run before the shared library exists; touching anything else without the
library raises ImportError.
"""

_EXPORTS = {"DType": "device", "Device": "device", "Slice": "device", "UgError": "device"}


def __getattr__(name):
    if name in _EXPORTS:
        import importlib
        return getattr(importlib.import_module(f".{_EXPORTS[name]}", __name__), name)
    raise AttributeError(name)
