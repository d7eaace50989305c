"""Offline convergence profile h(total batch, bandwidth) used by the controller.

The reference loads scikit-optimize pickles whose last model is a Gaussian process with kernel
Constant x Matern + White over (total batch / max batch, bandwidth / reference bandwidth) and uses the
posterior mean as a multiplicative "iterations needed" penalty, ``1 + 50 h``
(backend/src/engine/batch_rate_alloc_optim.py:139-172, 190).  Those pickles are foreign code-bearing
files and are never loaded by the controller.  Instead:

* ``python -m stellatrain_b200.control.convert_profile in.pkl out.npz`` turns such a pickle into plain arrays
  offline, reading it with an allow-list unpickler that runs nothing the file names;
* ``GPProfile`` evaluates the posterior mean of a Matern GP from plain arrays (``.npz`` or JSON):
  ``mean(x) = K(x, X) @ alpha * y_std + y_mean``;
* ``fit_profile`` builds such a profile from measured (batch, bandwidth, penalty) points;
* ``AnalyticProfile`` is the default when no profile is given.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Sequence, Union

import numpy as np


def matern(d: np.ndarray, nu: float) -> np.ndarray:
    """Matern correlation for scaled distances d >= 0 (nu in {0.5, 1.5, 2.5, inf})."""
    if nu == 0.5:
        return np.exp(-d)
    if nu == 1.5:
        k = math.sqrt(3.0) * d
        return (1.0 + k) * np.exp(-k)
    if nu == 2.5:
        k = math.sqrt(5.0) * d
        return (1.0 + k + k * k / 3.0) * np.exp(-k)
    if math.isinf(nu):
        return np.exp(-0.5 * d * d)
    raise ValueError("nu must be 0.5, 1.5, 2.5 or inf")


@dataclass
class ProfileMeta:
    batch_size: float = 256.0        # operating point the profile was taken at
    max_batch_size: float = 1024.0
    min_batch_size: float = 32.0
    bandwidth: float = 1.0           # reference bandwidth unit (Gbps)
    compression: float = 0.9
    model: str = ""


@dataclass
class GPProfile:
    x_train: np.ndarray               # (n, 2) in scaled coordinates
    alpha: np.ndarray                 # (n,)
    length_scale: np.ndarray          # (2,)
    constant: float = 1.0
    nu: float = 2.5
    y_mean: float = 0.0
    y_std: float = 1.0
    meta: ProfileMeta = field(default_factory=ProfileMeta)

    def _k(self, x: np.ndarray) -> np.ndarray:
        diff = (x[:, None, :] - self.x_train[None, :, :]) / self.length_scale[None, None, :]
        return self.constant * matern(np.sqrt((diff * diff).sum(-1)), self.nu)

    def h(self, total_batch: Union[float, np.ndarray], bandwidth: Union[float, np.ndarray]) -> np.ndarray:
        tb = np.atleast_1d(np.asarray(total_batch, dtype=float)) / self.meta.max_batch_size
        bw = np.atleast_1d(np.asarray(bandwidth, dtype=float)) / self.meta.bandwidth
        tb, bw = np.broadcast_arrays(tb, bw)
        x = np.stack([tb, bw], axis=-1)
        return self._k(x) @ self.alpha * self.y_std + self.y_mean

    def save(self, path: Union[str, Path]) -> None:
        np.savez(path, x_train=self.x_train, alpha=self.alpha, length_scale=self.length_scale, constant=self.constant,
                 nu=self.nu, y_mean=self.y_mean, y_std=self.y_std, meta=json.dumps(self.meta.__dict__))

    @classmethod
    def load(cls, path: Union[str, Path]) -> "GPProfile":
        path = Path(path)
        if path.suffix == ".json":
            d = json.loads(path.read_text())
            meta = ProfileMeta(**d.get("metadata", {}))
        else:
            with np.load(path, allow_pickle=False) as z:
                d = {k: z[k] for k in z.files}
            meta = ProfileMeta(**json.loads(str(d["meta"])))
        return cls(np.asarray(d["x_train"], float), np.asarray(d["alpha"], float),
                   np.asarray(d["length_scale"], float).reshape(-1), float(d.get("constant", 1.0)),
                   float(d.get("nu", 2.5)), float(d.get("y_mean", 0.0)), float(d.get("y_std", 1.0)), meta)


def fit_profile(total_batch: Sequence[float], bandwidth: Sequence[float], penalty: Sequence[float],
                meta: Optional[ProfileMeta] = None, length_scale=(0.3, 0.3), nu: float = 2.5,
                noise: float = 1e-4) -> GPProfile:
    """GP regression with fixed kernel hyper-parameters (enough for a smooth two-dimensional profile)."""
    meta = meta or ProfileMeta()
    x = np.stack([np.asarray(total_batch, float) / meta.max_batch_size, np.asarray(bandwidth, float) / meta.bandwidth], -1)
    y = np.asarray(penalty, float)
    y_mean, y_std = float(y.mean()), float(y.std() or 1.0)
    ls = np.asarray(length_scale, float)
    prof = GPProfile(x, np.zeros(len(y)), ls, 1.0, nu, y_mean, y_std, meta)
    k = prof._k(x) + noise * np.eye(len(y))
    prof.alpha = np.linalg.solve(k, (y - y_mean) / y_std)
    return prof


@dataclass
class AnalyticProfile:
    """Default surrogate: extra iterations grow once the total batch passes the critical batch and when
    little bandwidth forces heavy compression.  Smooth, monotone, cheap."""

    meta: ProfileMeta = field(default_factory=ProfileMeta)
    critical_batch: float = 512.0

    def h(self, total_batch, bandwidth) -> np.ndarray:
        tb = np.atleast_1d(np.asarray(total_batch, dtype=float))
        bw = np.maximum(np.atleast_1d(np.asarray(bandwidth, dtype=float)), 1e-6)
        tb, bw = np.broadcast_arrays(tb, bw)
        batch_term = np.log1p(tb / self.critical_batch) / 50.0
        bw_term = 0.02 / (1.0 + bw / self.meta.bandwidth)
        return batch_term + bw_term


# Profiles that ship with the package, by a substring of the device name a client reports: (file, parameters of the
# model it was taken for).  The reference ships one profile per model too (bayesian/profile/*.pkl).
SHIPPED_PROFILES = {"B200": [("b200_gpt2_small.json", 124.4e6), ("b200_resnet152.json", 58.3e6), ("b200_resnet50.json", 23.7e6),
                             ("b200_vitb16.json", 85.9e6), ("b200_swinb.json", 87.0e6)]}


def shipped_profile_path(gpu_name: Optional[str], n_params: Optional[float] = None) -> Optional[Path]:
    """The fitted profile that ships for this kind of GPU (``sweep_profile.py`` produced it), or None.  Of several, the
    one taken for the model closest in size (ratio of parameter counts); the first one while the size is unknown.
    Models of nearly the same size (ViT-B/16 and Swin-B) cannot be told apart this way: name the profile then
    (``--profile`` / ``MODEL_PROFILE``, as the reference requires for every run)."""
    import math

    for needle, entries in SHIPPED_PROFILES.items():
        if gpu_name and needle in gpu_name:
            present = [(f, n) for f, n in entries if (Path(__file__).parent / "profiles" / f).exists()]
            if not present:
                return None
            if n_params and n_params > 0:
                present.sort(key=lambda e: abs(math.log(e[1] / float(n_params))))
            return Path(__file__).parent / "profiles" / present[0][0]
    return None


def load_profile(path: Optional[str], gpu_name: Optional[str] = None, n_params: Optional[float] = None):
    """``path`` (or, without one, the profile that ships for ``gpu_name`` and a model of ``n_params`` parameters; the
    analytic surrogate when there is none)."""
    if not path:
        shipped = shipped_profile_path(gpu_name, n_params)
        if shipped is None:
            return AnalyticProfile()
        return GPProfile.load(shipped)
    p = Path(path)
    if p.suffix in (".pkl", ".pickle"):
        raise ValueError("pickled scikit-optimize profiles are not loaded here; convert them once with "
                         "`python -m stellatrain_b200.control.convert_profile in.pkl out.npz`")
    return GPProfile.load(p)
