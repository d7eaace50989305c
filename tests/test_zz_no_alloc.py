"""The allocation-free top-k entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory at the moment they need a selection (fixed
memory pools, plugins inside a process that owns the device memory, latency paths); for them the
library carries its working memory inside its own device image.  This test checks that the entry point
returns the same selection as the engine's ordinary path, twice in a row (the second call reuses the
working memory the first one dirtied), and that it refuses oversized inputs.

Collected last on purpose: a failure here must not hide failures elsewhere under ``pytest -x``.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from stellatrain_b200 import _build

    _build.load_extension("_C")
    lib = ctypes.CDLL(str(_build.so_path("_C")))
    lib.st_topk_select_noalloc.restype = ctypes.c_int
    lib.st_topk_select_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p,
                                           ctypes.c_void_p]
    lib.st_noalloc_last_error.restype = ctypes.c_char_p
    lib.st_noalloc_status.restype = ctypes.c_int
    lib.st_noalloc_status.argtypes = [ctypes.POINTER(ctypes.c_uint32), ctypes.c_void_p]
    return lib


def _call(lib, values: torch.Tensor, k: int):
    out = torch.empty(k, 2, dtype=torch.int32, device=values.device)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.st_topk_select_noalloc(values.data_ptr(), values.numel(), k, out.data_ptr(), stream)
    assert rc == 0, lib.st_noalloc_last_error().decode()
    status = ctypes.c_uint32(99)
    assert lib.st_noalloc_status(ctypes.byref(status), stream) == 0, lib.st_noalloc_last_error().decode()
    assert status.value == 0, "the kernels must report success on the device as well"
    torch.cuda.synchronize()
    idx = out[:, 0].cpu().numpy().view(np.uint32).astype(np.int64)
    val = out[:, 1].contiguous().view(torch.float32).cpu().numpy()
    order = np.argsort(idx, kind="stable")
    return idx[order], val[order]


def _existing(values: torch.Tensor, k: int, tag: str):
    from stellatrain_b200.ops.select import compress_tensor

    ratio = 1.0 - (k + 0.5) / values.numel()
    idx, val = compress_tensor(f"noalloc-check-{tag}", values, ratio, "topk")
    assert idx.numel() == k
    idx = idx.cpu().numpy().astype(np.int64)
    val = val.cpu().numpy()
    order = np.argsort(idx, kind="stable")
    return idx[order], val[order]


def test_noalloc_topk_matches_engine_path_twice():
    lib = _lib()
    g = torch.Generator(device="cuda").manual_seed(99)
    for call, (n, k) in enumerate([(300_001, 3000), (70_000, 123)]):
        values = torch.randn(n, device="cuda", generator=g)
        values[::997] = values[5]          # some exact ties
        got_idx, got_val = _call(lib, values, k)
        want_idx, want_val = _existing(values, k, str(call))
        assert np.array_equal(got_idx, want_idx)
        np.testing.assert_allclose(got_val, want_val, rtol=0, atol=0)
        assert np.array_equal(values[torch.from_numpy(got_idx).cuda()].cpu().numpy(), got_val), "input must stay intact"


def _plain_topk(values: torch.Tensor, k: int):
    """Independent oracle in plain PyTorch: largest magnitudes, equal ones towards the lower index, NaN as 0."""
    clean = torch.where(torch.isnan(values), torch.zeros_like(values), values)
    order = torch.sort(clean.abs(), descending=True, stable=True).indices[:k]
    idx = np.sort(order.cpu().numpy().astype(np.int64), kind="stable")
    return idx, clean.cpu().numpy()[idx]


def test_noalloc_topk_matches_plain_pytorch_with_odd_sizes_ties_and_nan():
    lib = _lib()
    g = torch.Generator(device="cuda").manual_seed(5)
    for n, k in [(100_003, 1001), (17, 5), (65_537, 7)]:        # none a multiple of 16
        values = torch.randn(n, device="cuda", generator=g)
        values[::13] = values[1]                                 # exact ties, some of them across the k-th place
        values[3] = float("nan")
        values[n - 1] = float("nan")
        before = values.clone()
        got_idx, got_val = _call(lib, values, k)
        want_idx, want_val = _plain_topk(values, k)
        assert np.array_equal(got_idx, want_idx), (n, k)
        np.testing.assert_array_equal(got_val, want_val)
        assert torch.equal(torch.nan_to_num(values), torch.nan_to_num(before)) and bool(torch.isnan(values[3])), "input must stay intact"


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib = _lib()
    small = torch.zeros(16, device="cuda")
    out = torch.empty(4, 2, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert lib.st_topk_select_noalloc(small.data_ptr(), (1 << 20) + 1, 4, out.data_ptr(), s) == 1
    assert b"limit" in lib.st_noalloc_last_error()
    assert lib.st_topk_select_noalloc(small.data_ptr(), 16, 0, out.data_ptr(), s) == 2
    assert lib.st_topk_select_noalloc(small.data_ptr(), 16, 17, out.data_ptr(), s) == 2
    assert lib.st_topk_select_noalloc(None, 16, 4, out.data_ptr(), s) == 2
    torch.cuda.synchronize()
