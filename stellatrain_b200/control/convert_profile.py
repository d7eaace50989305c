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


def _safe_scalar(dtype: Any, data: Any) -> Any:
    """numpy's scalar constructor, refused for object dtypes: for those numpy itself unpickles ``data`` with the
    ordinary, unrestricted unpickler."""
    dt = np.dtype(dtype)
    if dt.hasobject or not isinstance(data, (bytes, bytearray)):
        raise pickle.UnpicklingError("object-typed numpy scalars are not read")
    import numpy._core.multiarray as multiarray

    return multiarray.scalar(dt, bytes(data))


class _SafeUnpickler(pickle._Unpickler):  # the pure-Python implementation: its dispatch table can be extended
    def __init__(self, file: io.BufferedIOBase) -> None:
        super().__init__(file)
        self._file = file

    def find_class(self, module: str, name: str) -> Any:
        if (module, name) in _NUMPY_OK:
            if name == "scalar":
                return _safe_scalar
            if "multiarray" in module:
                import numpy._core.multiarray as multiarray

                return getattr(multiarray, name)
            return getattr(np, name)
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


def _find_kernel_parts(kernel: Any) -> dict:
    """Constant, length scales and smoothness of ``Constant * Matern [+ White]`` (any nesting order)."""
    out: dict = {}

    def walk(k: Any) -> None:
        if not isinstance(k, Record):
            return
        leaf = k._name.rsplit(".", 1)[-1]
        if leaf in ("Sum", "Product"):
            walk(k.attr("k1"))
            walk(k.attr("k2"))
        elif leaf == "ConstantKernel":
            out["constant"] = float(k.attr("constant_value"))
        elif leaf == "Matern":
            out["length_scale"] = np.atleast_1d(np.asarray(k.attr("length_scale"), dtype=float))
            out["nu"] = float(k.attr("nu"))
        elif leaf == "RBF":
            out["length_scale"] = np.atleast_1d(np.asarray(k.attr("length_scale"), dtype=float))
            out["nu"] = float("inf")
        elif leaf == "WhiteKernel":
            out["noise"] = float(k.attr("noise_level", 0.0))
        else:
            raise ValueError(f"unsupported kernel component {k._name}")

    walk(kernel)
    if "length_scale" not in out:
        raise ValueError("no Matern or RBF component in the kernel")
    out.setdefault("constant", 1.0)
    return out


def profile_from_records(result: Any) -> GPProfile:
    """Build a ``GPProfile`` from the record tree of a scikit-optimize result."""
    if not isinstance(result, Record) or "models" not in result:
        raise ValueError("not a scikit-optimize result: no 'models' entry")
    models = result["models"]
    if not models:
        raise ValueError("the result holds no fitted model")
    gp = models[-1]
    x_train = np.asarray(gp.attr("X_train_"), dtype=float)
    alpha = np.asarray(gp.attr("alpha_"), dtype=float).reshape(-1)
    if x_train.ndim != 2 or x_train.shape[1] != 2 or x_train.shape[0] != alpha.shape[0]:
        raise ValueError(f"unexpected training set: X {x_train.shape}, alpha {alpha.shape}")
    parts = _find_kernel_parts(gp.attr("kernel_"))
    ls = parts["length_scale"]
    ls = np.repeat(ls, 2) if ls.shape[0] == 1 else ls
    y_mean = gp.attr("_y_train_mean", gp.attr("y_train_mean_", 0.0))
    y_std = gp.attr("_y_train_std", gp.attr("y_train_std_", 1.0))
    md = result.get("metadata") or {}
    if isinstance(md, Record):
        md = dict(md)
    known = {k: md[k] for k in ("batch_size", "max_batch_size", "min_batch_size", "bandwidth", "compression") if k in md}
    meta = ProfileMeta(**{k: float(v) for k, v in known.items()}, model=str(md.get("model", "")))
    return GPProfile(x_train, alpha, ls, parts["constant"], parts["nu"], float(np.asarray(y_mean)), float(np.asarray(y_std)), meta)


def convert(src: str, dst: Optional[str] = None) -> GPProfile:
    prof = profile_from_records(read_records(src))
    if dst:
        if dst.endswith(".json"):
            import json

            Path(dst).write_text(json.dumps({
                "x_train": prof.x_train.tolist(), "alpha": prof.alpha.tolist(), "length_scale": prof.length_scale.tolist(),
                "constant": prof.constant, "nu": prof.nu, "y_mean": prof.y_mean, "y_std": prof.y_std,
                "metadata": prof.meta.__dict__}))
        else:
            prof.save(dst)
    return prof


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("src", help="scikit-optimize result written by skopt.dump / joblib.dump")
    ap.add_argument("dst", help=".npz or .json profile for MODEL_PROFILE")
    a = ap.parse_args()
    prof = convert(a.src, a.dst)
    print(f"{a.dst}: {len(prof.alpha)} training points, kernel {prof.constant:.4g} * Matern(nu={prof.nu}, "
          f"length_scale={prof.length_scale.tolist()}), metadata {prof.meta.__dict__}")


if __name__ == "__main__":
    main()
