"""Plain-PyTorch restatement of the sparse path: the correctness oracle of the kernels.

Every function works on one tensor (one segment) in fp32 on any device and states the rule the CUDA
and CPU kernels implement, with the reference's algorithm cited next to each:

* error feedback            backend/src/engine/modules/compress.cpp:139-188
* top-k (intended rule)     backend/src/compress/topk.cpp:28-46
* threshold-v               backend/src/compress/thresholdv.cpp:40-83
* threshold-v16             backend/src/compress/thresholdv16.cpp:78-295
* merge                     backend/src/engine/modules/cpu_optimize.cpp:40-72
* sparse SGD / Adam         backend/src/optim/sgd.cpp:221-262, backend/src/optim/adam.cpp:19-87

Deliberate differences from the shipped reference, all stated where they apply: ties are broken by the
lowest index; the first threshold is the smallest selected key followed by the reference's first AIMD
step; a tail block of threshold-v16 is a zero-padded full block; a NaN is dropped.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

SENTINEL = 0xFFFFFFFF


@dataclass
class ThresholdState:
    tau: float = 0.0
    tau_inc: float = 0.0
    inited: bool = False


def f32(x: float) -> float:
    return float(torch.tensor(x, dtype=torch.float32))


def ef_accumulate(grad: torch.Tensor, resid: torch.Tensor) -> torch.Tensor:
    """a = g + r with NaNs dropped."""
    a = grad.float() + resid.float()
    return torch.where(torch.isnan(a), torch.zeros_like(a), a)


def _top_indices(keys: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest keys, equal keys by ascending index; result in rank order."""
    order = torch.sort(keys, descending=True, stable=True).indices
    return order[:k]


def select_topk(a: torch.Tensor, k: int) -> torch.Tensor:
    return _top_indices(a.abs(), k)


def select_thresholdv(a: torch.Tensor, k: int, st: ThresholdState) -> torch.Tensor:
    """Indices (ascending) of the elements sent; may be fewer than k. Updates ``st``."""
    mag = a.abs()
    mx = float(mag.max()) if a.numel() else 0.0
    if not st.inited:
        idx = _top_indices(mag, k)
        t0 = float(mag[idx[-1]])
        st.tau = f32(f32(t0) + f32(f32(f32(0.01) * f32((k + 1) / k)) * f32(mx)))
        st.tau_inc = 0.0
        st.inited = True
        return idx
    tau = torch.tensor(st.tau, dtype=torch.float32, device=a.device)
    mask = mag >= tau
    found = int(mask.sum())
    idx = torch.nonzero(mask).flatten()[:k]
    if k > found:
        st.tau = f32(f32(st.tau) * f32(0.99))
    elif k < found:
        st.tau = f32(f32(st.tau) + f32(f32(f32(0.01) * f32(f32(found) / f32(k))) * f32(mx)))
    return idx


def block_scores(a_pad: torch.Tensor) -> torch.Tensor:
    """L1 norm of each aligned 16-block with the kernels' fixed reduction tree."""
    m = a_pad.abs().view(-1, 4, 4)
    lane = (m[:, :, 0] + m[:, :, 1]) + (m[:, :, 2] + m[:, :, 3])
    return (lane[:, 0] + lane[:, 1]) + (lane[:, 2] + lane[:, 3])


def select_thresholdv16(a: torch.Tensor, k: int, st: ThresholdState, one_pass: bool = False) -> torch.Tensor:
    """Element indices sent (k of them; some may point into the zero padding of the last block).

    ``one_pass`` states the rule of the one-pass kernel chain for a tensor that already has a threshold: the
    blocks at or over the threshold go first, in index order; when they fall short of the budget, the best of
    the others complete it (the reference's heap fill, backend/src/compress/thresholdv16.cpp:261-293), but a
    block that holds nothing is never sent, so a tensor with fewer non-zero blocks than the budget yields
    fewer than k indices (the rest of its stream says "no entry").  The two-pass chain sends such blocks."""
    n = a.numel()
    n_pad = (n + 15) // 16 * 16
    a_pad = torch.zeros(n_pad, dtype=torch.float32, device=a.device)
    a_pad[:n] = a
    score = block_scores(a_pad)
    kb = (k + 15) // 16
    last_len = k - 16 * (kb - 1)

    def expand(blocks: torch.Tensor) -> torch.Tensor:
        if blocks.numel() < kb:         # short stream: whole blocks only
            return (blocks[:, None] * 16 + torch.arange(16, device=a.device)[None, :]).flatten()
        full = (blocks[:-1, None] * 16 + torch.arange(16, device=a.device)[None, :]).flatten()
        tail = blocks[-1] * 16 + torch.arange(last_len, device=a.device)
        return torch.cat([full, tail])

    if not st.inited:
        blocks = _top_indices(score, kb)
        t0 = float(score[blocks[-1]])
        st.tau_inc = f32(f32(0.01) * f32(t0))
        st.tau = f32(f32(t0) + f32(st.tau_inc))
        st.inited = True
        return expand(blocks)
    tau = torch.tensor(st.tau, dtype=torch.float32, device=a.device)
    flagged = score >= tau
    nf = int(flagged.sum())
    if nf * 16 >= k:
        blocks = torch.nonzero(flagged).flatten()[:kb]
        st.tau = f32(f32(st.tau) + f32(st.tau_inc))
    else:
        blocks = _top_indices(score, kb)
        if one_pass:
            blocks = blocks[score[blocks] > 0]
        st.tau = f32(f32(st.tau) * f32(0.99))
    return expand(blocks)


def compress_step(kind: str, grad: torch.Tensor, resid: torch.Tensor, k: int,
                  st: Optional[ThresholdState] = None, one_pass: bool = False) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """One error-feedback compression of one tensor: returns (idx, val, new_residual).

    For threshold-v16 the residual and the indices refer to the zero-padded tensor."""
    a = ef_accumulate(grad, resid)
    if kind == "topk":
        idx = select_topk(a, k)
    elif kind == "thresholdv":
        idx = select_thresholdv(a, k, st)
    elif kind == "thresholdv16":
        n = a.numel()
        n_pad = (n + 15) // 16 * 16
        if n_pad != n:
            a = torch.cat([a, torch.zeros(n_pad - n, dtype=a.dtype, device=a.device)])
        idx = select_thresholdv16(a[:n], k, st, one_pass=one_pass)
    else:
        raise ValueError(kind)
    val = a[idx]
    new_r = a.clone()
    new_r[idx] = 0
    return idx, val, new_r


def merge_streams(n: int, streams: list[tuple[torch.Tensor, torch.Tensor]], weights: list[float]):
    """Dense merged gradient and the mask of touched indices (union over sources)."""
    dev = streams[0][1].device
    dense = torch.zeros(n, dtype=torch.float64, device=dev)
    touched = torch.zeros(n, dtype=torch.bool, device=dev)
    for (idx, val), w in zip(streams, weights):
        keep = idx.long() != SENTINEL
        i = idx.long()[keep]
        dense.index_add_(0, i, val[keep].double() * f32(w))
        touched[i] = True
    return dense.float(), touched


@dataclass
class SGDConfig:
    lr: float = 1e-3
    momentum: float = 0.0
    dampening: float = 0.0
    weight_decay: float = 0.0
    nesterov: bool = False
    maximize: bool = False
    smart_momentum: bool = False


@dataclass
class SGDState:
    b: Optional[torch.Tensor] = None
    last: Optional[torch.Tensor] = None
    first: bool = True
    m_iter: int = 0


def sparse_sgd(param: torch.Tensor, g: torch.Tensor, touched: torch.Tensor, cfg: SGDConfig, st: SGDState) -> None:
    """Lazy SGD on the touched indices only; ``m_iter`` advances once per step."""
    if st.b is None:
        st.b = torch.zeros_like(param)
        st.last = torch.zeros_like(param, dtype=torch.int64)
    i = torch.nonzero(touched).flatten()
    x = param[i]
    gg = g[i].clone()
    mu = torch.full_like(gg, cfg.momentum)
    if cfg.smart_momentum and st.m_iter != 0:
        mu = torch.pow(torch.full_like(gg, cfg.momentum), (st.m_iter - st.last[i]).float())
    if cfg.weight_decay != 0:
        gg = gg + cfg.weight_decay * x
    if cfg.momentum != 0:
        b = gg.clone() if st.first else st.b[i] * mu + (1 - cfg.dampening) * gg
        gg = gg + mu * b if cfg.nesterov else b
        st.b[i] = b
    lr = -cfg.lr if cfg.maximize else cfg.lr
    param[i] = x - lr * gg
    if cfg.smart_momentum:
        st.last[i] = st.m_iter
    st.first = False
    st.m_iter += 1


@dataclass
class AdamConfig:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    amsgrad: bool = False
    maximize: bool = False


@dataclass
class AdamState:
    m: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    vmax: Optional[torch.Tensor] = None
    tick: int = 1


def sparse_adam(param: torch.Tensor, g: torch.Tensor, touched: torch.Tensor, cfg: AdamConfig, st: AdamState) -> None:
    """Lazy Adam on the touched indices; the step counter advances once per call (per tensor per
    step). AMSGrad keeps a per-element maximum (the reference keeps one scalar per tensor,
    backend/src/optim/adam.cpp:70-72, which is not the published algorithm)."""
    if st.m is None:
        st.m = torch.zeros_like(param)
        st.v = torch.zeros_like(param)
        st.vmax = torch.zeros_like(param)
    i = torch.nonzero(touched).flatten()
    x = param[i].double()
    gg = g[i].double()
    if cfg.maximize:
        gg = -gg
    if cfg.weight_decay != 0:
        gg = gg + cfg.weight_decay * x
    m = cfg.beta1 * st.m[i].double() + (1 - cfg.beta1) * gg
    v = cfg.beta2 * st.v[i].double() + (1 - cfg.beta2) * gg * gg
    mh = m / (1 - cfg.beta1 ** st.tick)
    vh = v / (1 - cfg.beta2 ** st.tick)
    if cfg.amsgrad:
        vh = torch.maximum(st.vmax[i].double(), vh)
        st.vmax[i] = vh.float()
    param[i] = (x - cfg.lr * mh / (vh.sqrt() + cfg.eps)).float()
    st.m[i] = m.float()
    st.v[i] = v.float()
    st.tick += 1


@dataclass
class DenseReference:
    """Dense-update reference for the flat-gradient benchmark: the same optimiser fed with the full
    gradient (no sparsification), against which the compressed run is compared."""

    param: torch.Tensor
    adam: AdamConfig = field(default_factory=AdamConfig)
    state: AdamState = field(default_factory=AdamState)

    def step(self, grad: torch.Tensor) -> None:
        sparse_adam(self.param, grad, torch.ones_like(grad, dtype=torch.bool), self.adam, self.state)
