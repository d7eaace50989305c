"""Selections of this package's CPU compressors against the reference's own compiled code on the same input.

Needs the out-of-tree build of the unmodified reference (``baseline/build_reference.sh`` -> ``baseline/_ref``) and its
source tree for the headers; skipped otherwise.  ``baseline/reference_cpu_flat.cpp`` calls the reference's compressor
classes and writes the input of the first step and what each of them selected from it."""
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
# the upstream tree: named by the environment, else a checkout called "reference" beside this repository
REF_TREE = Path(os.environ.get("STELLATRAIN_REFERENCE") or ROOT.parent / "reference")


@pytest.fixture(scope="module")
def dump(tmp_path_factory):
    if not (ROOT / "baseline" / "_ref" / "libfasterdp_core.so").exists() or not (REF_TREE / "backend" / "src").exists():
        pytest.skip("the reference is not built or its tree is not at hand")
    out = tmp_path_factory.mktemp("refdump")
    env = dict(os.environ, TMPDIR=str(out))
    run = subprocess.run(["bash", str(ROOT / "baseline" / "run_reference_cpu_flat.sh"), str(REF_TREE), "200000", "8", str(out)],
                         capture_output=True, text=True, timeout=600, env=env)
    if run.returncode != 0:
        pytest.skip("the harness did not build here: " + run.stderr[-300:])
    return out


def _load(dump, method):
    x = np.fromfile(dump / "input.f32", dtype=np.float32)
    ri = np.fromfile(dump / f"{method}.idx.u32", dtype=np.uint32).astype(np.int64)
    rv = np.fromfile(dump / f"{method}.val.f32", dtype=np.float32)
    return x, ri, rv


def _ours(x, method):
    from stellatrain_b200 import cpu_tier

    k = len(x) // 100
    oi, ov = cpu_tier.compress(f"parity-{method}-{os.getpid()}", torch.from_numpy(x.copy()), k, method)
    return oi.numpy().astype(np.int64), ov.numpy()


def test_threshold_v16_selects_the_reference_blocks(dump):
    x, ri, rv = _load(dump, "thresholdv16")
    oi, ov = _ours(x, "thresholdv16")
    assert len(ri) == len(oi) == len(x) // 100 and np.array_equal(x[ri], rv)
    both, either = len(set(ri.tolist()) & set(oi.tolist())), len(set(ri.tolist()) | set(oi.tolist()))
    # the reference takes the blocks over its first threshold in scan order and can miss the best of two blocks at the
    # threshold; this package takes the best blocks: at most one block of 125 differs, never to this package's loss
    assert both / either >= 0.97
    assert np.abs(ov).sum() >= np.abs(rv).sum() * (1 - 1e-6)
    assert all(len({i // 16 for i in sel}) * 16 == len(sel) for sel in (ri.tolist(), oi.tolist()))   # whole blocks both


def test_threshold_v_selects_the_reference_elements(dump):
    x, ri, rv = _load(dump, "thresholdv")
    oi, ov = _ours(x, "thresholdv")
    assert np.array_equal(x[ri], rv)
    both, either = len(set(ri.tolist()) & set(oi.tolist())), len(set(ri.tolist()) | set(oi.tolist()))
    assert both / either >= 0.995                   # the reference's first threshold admits k + 1 elements, index order drops one
    assert np.abs(ov).sum() >= np.abs(rv).sum() * (1 - 1e-6)


def test_top_k_is_exact_where_the_reference_is_not(dump):
    x, ri, rv = _load(dump, "topk")
    oi, ov = _ours(x, "topk")
    want = torch.topk(torch.from_numpy(np.abs(x)), len(oi)).values.numpy()
    assert np.array_equal(np.sort(np.abs(ov)), np.sort(want)) and np.array_equal(x[oi], ov)
    # the reference copies n bytes instead of n floats and reports positions of its partitioned copy as indices
    # (backend/src/compress/topk.cpp:28-46): its values are not the input's values at its indices and carry less mass
    assert not np.array_equal(x[ri], rv)
    assert np.abs(rv).sum() < np.abs(ov).sum()


def test_sparse_optimisers_match_the_reference_numerically(dump):
    """Two calls of the reference's sparse Adam (lr 1e-3) and SGD (lr 0.1, momentum 0.9) on one selection, from zero
    parameters, against this package's CPU optimisers on the same (index, value) pairs."""
    from stellatrain_b200 import cpu_tier

    x, ri, rv = _load(dump, "thresholdv")
    idx = torch.from_numpy(ri.astype(np.int32)).contiguous()
    val = torch.from_numpy(rv.copy())
    for kind, options, file, tol in (("adam", {"lr": 1e-3}, "adam.param.f32", 2e-6), ("sgd", {"lr": 0.1, "momentum": 0.9}, "sgd.param.f32", 1e-6)):
        want = np.fromfile(dump / file, dtype=np.float32)
        opt = cpu_tier.make_optimizer(kind)
        for k, v in options.items():
            opt.configure(k, v)
        param = torch.zeros(len(x))
        for _ in range(2):
            opt.optimize(param.data_ptr(), len(x), "parity", val.data_ptr(), idx.data_ptr(), len(ri))
        got = param.numpy()[ri]
        assert np.abs(want).max() > 0
        np.testing.assert_allclose(got, want, rtol=tol, atol=1e-9)
        assert float(param.abs().sum()) == pytest.approx(float(np.abs(got).sum()), rel=1e-6)      # nothing else moved


def test_eight_steps_of_error_feedback_and_sparse_adam_track_the_reference(dump):
    """The whole per-tensor pipeline (accumulate with the residual, threshold-v16 with its adapting threshold, residual
    save, sparse Adam) for eight steps on the reference's gradients: selections may differ by a block per step, so the
    comparison is on what matters downstream."""
    from stellatrain_b200 import cpu_tier

    n, steps = 200000, 8
    grads = np.fromfile(dump / "grads.f32", dtype=np.float32).reshape(steps, n)
    want_p = np.fromfile(dump / "thresholdv16.final_param.f32", dtype=np.float32)
    want_r = np.fromfile(dump / "thresholdv16.final_resid.f32", dtype=np.float32)
    opt = cpu_tier.make_optimizer("adam")
    opt.configure("lr", 1e-3)
    param, resid, k = torch.zeros(n), torch.zeros(n), n // 100
    name = f"parity-pipeline-{os.getpid()}"
    for s in range(steps):
        idx, val = cpu_tier.compress_with_feedback(name, torch.from_numpy(grads[s].copy()), resid, k, "thresholdv16")
        assert idx.numel() == k
        opt.optimize(param.data_ptr(), n, "pipeline", val.data_ptr(), idx.data_ptr(), idx.numel())
    got_p, got_r = param.numpy(), resid.numpy()
    cos = float(np.dot(got_p, want_p) / (np.linalg.norm(got_p) * np.linalg.norm(want_p)))
    assert cos > 0.97, cos
    touched_both = np.count_nonzero((got_p != 0) & (want_p != 0)) / max(1, np.count_nonzero((got_p != 0) | (want_p != 0)))
    assert touched_both > 0.95
    # nothing is lost in either: what was not sent sits in the residual
    total = grads.astype(np.float64).sum()
    assert abs(float(got_r.astype(np.float64).sum()) - float(want_r.astype(np.float64).sum())) < 0.05 * abs(total) + 1.0
    assert np.linalg.norm(got_r - want_r) / np.linalg.norm(want_r) < 0.1
