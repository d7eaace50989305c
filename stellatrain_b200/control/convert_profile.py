"""Offline converter: a scikit-optimize result pickle -> the plain ``.npz`` / ``.json`` profile that ``GPProfile`` reads.

The reference's controller loads its convergence profiles with ``skopt.load`` (joblib) and calls the last model's
``predict`` (backend/src/engine/batch_rate_alloc_optim.py:139-172).  Such a file is a pickle: loading it the normal way
imports and runs whatever it names.  This converter never does that.  It walks the pickle with the pure-Python
unpickler and an allow-list: numpy's array, dtype and scalar constructors are real, ``copyreg._reconstructor`` is real
(it only allocates an instance of a class this module supplies), and EVERY other name in the file, whether class or
function, becomes an inert record that stores its arguments and state.  Nothing of scikit-optimize, scikit-learn,
scipy or joblib is imported.  joblib stores array payloads as raw bytes behind a small wrapper object; those are read
here by hand.

What is taken from the record tree: the training inputs, the dual coefficients, the kernel's constant, length scales
and smoothness, the target normalisation of the last Gaussian-process model, and the ``metadata`` dictionary the
authors attached to the result.

    python -m stellatrain_b200.control.convert_profile profile.pkl profile.npz
"""
from __future__ import annotations

import argparse
import io
import pickle
import zlib
from pathlib import Path
from typing import Any, Optional

import numpy as np

from .gp_profile import GPProfile, ProfileMeta

_MAX_BYTES = 256 << 20


class Record(dict):
    """Inert stand-in for any object of a class that is not on the allow-list: keeps constructor arguments, state
    and, for mapping-like classes, items."""

    _name = "?"
    args: tuple = ()          # class-level defaults: most instances are allocated without a constructor call
    kwargs: dict = {}
    state: Any = None

    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__()
        self.args, self.kwargs, self.state = args, kwargs, None

    def __setstate__(self, state: Any) -> None:
        self.state = state

    def attr(self, name: str, default: Any = None) -> Any:
        """Attribute as the original object would have it: from a ``__dict__`` state or from the mapping items."""
        st = self.state
        if isinstance(st, tuple) and len(st) == 2 and isinstance(st[0], dict):   # (dict state, slots state)
            st = st[0]
        if isinstance(st, dict) and name in st:
            return st[name]
        return self.get(name, default)

    def __reduce__(self):  # records are never pickled again
        raise TypeError("a profile record cannot be pickled")


def _record_class(module: str, name: str) -> type:
    return type(name, (Record,), {"_name": f"{module}.{name}"})


class _ArrayWrapper:
    """joblib's marker in front of an array payload (fields arrive through BUILD)."""

    def __setstate__(self, state: dict) -> None:
        self.__dict__.update(state)


_NUMPY_OK = {
    ("numpy.core.multiarray", "_reconstruct"), ("numpy._core.multiarray", "_reconstruct"),
    ("numpy.core.multiarray", "scalar"), ("numpy._core.multiarray", "scalar"),
    ("numpy", "ndarray"), ("numpy", "dtype"),
}


class _SafeUnpickler(pickle._Unpickler):  # the pure-Python implementation: its dispatch table can be extended
    def __init__(self, file: io.BufferedIOBase) -> None:
        super().__init__(file)
        self._file = file

    def find_class(self, module: str, name: str) -> Any:
        if (module, name) in _NUMPY_OK:
            mod = np.core.multiarray if "multiarray" in module else np
            return getattr(mod, name)
        if (module, name) == ("copyreg", "_reconstructor"):
            import copyreg

            return copyreg._reconstructor
        if (module, name) in (("builtins", "object"), ("builtins", "dict"), ("builtins", "list"), ("builtins", "tuple"),
                              ("builtins", "set"), ("builtins", "frozenset"), ("collections", "OrderedDict")):
            import builtins
            import collections

            return getattr(collections if module == "collections" else builtins, name)
        if (module, name) == ("joblib.numpy_pickle", "NumpyArrayWrapper"):
            return _ArrayWrapper
        return _record_class(module, name)

    def persistent_load(self, pid: Any) -> Any:
        raise pickle.UnpicklingError("persistent ids are not supported")

    # joblib writes the array's bytes right behind the wrapper object: replace the wrapper by the array
    def load_build(self) -> None:
        pickle._Unpickler.load_build(self)
        top = self.stack[-1]
        if isinstance(top, _ArrayWrapper):
            self.stack[-1] = self._read_array(top)

    dispatch = dict(pickle._Unpickler.dispatch)
    dispatch[pickle.BUILD[0]] = load_build

    def _read_array(self, w: _ArrayWrapper) -> np.ndarray:
        dtype = np.dtype(w.dtype)
        shape = tuple(int(s) for s in w.shape)
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if dtype.hasobject:
            arr = _SafeUnpickler(self._file).load()       # an object array is a nested pickle, read under the same rules
            return np.asarray(arr, dtype=object)
        if count * dtype.itemsize > _MAX_BYTES:
            raise pickle.UnpicklingError("array payload too large")
        if getattr(w, "numpy_array_alignment_bytes", None) is not None:
            pad = self._file.read(1)
            if len(pad) != 1:
                raise pickle.UnpicklingError("truncated array padding")
            self._file.read(pad[0])
        data = self._file.read(count * dtype.itemsize)
        if len(data) != count * dtype.itemsize:
            raise pickle.UnpicklingError("truncated array payload")
        arr = np.frombuffer(data, dtype=dtype, count=count).copy()
        order = getattr(w, "order", "C")
        return arr.reshape(shape[::-1]).T if order == "F" and len(shape) > 1 else arr.reshape(shape)


def read_records(path: str) -> Any:
    """The object tree of a (possibly zlib-compressed) pickle as inert records and numpy arrays."""
    raw = Path(path).read_bytes()
    if len(raw) > _MAX_BYTES:
        raise ValueError("file too large for a profile")
    if raw[:1] == b"x":                      # joblib's zlib container
        raw = zlib.decompressobj().decompress(raw, _MAX_BYTES)
    return _SafeUnpickler(io.BytesIO(raw)).load()
