"""Property tests (hypothesis) of the CPU-tier kernels: invariants that must hold for every input, not
just for the sizes the example-based tests pick."""
import numpy as np
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st   # noqa: E402

from stellatrain_b200 import cpu_tier   # noqa: E402

ext = cpu_tier._load()

values = st.one_of(
    st.floats(min_value=-4.0, max_value=4.0, allow_nan=False, width=32),
    st.sampled_from([0.0, -0.0, 1.0, -1.0, 0.5, 1e-38, -1e-38, 3.0e38]),      # ties, zeros, a denormal-range and a huge value
)


@st.composite
def problem(draw, max_n=3000):
    n = draw(st.integers(min_value=1, max_value=max_n))
    k = draw(st.integers(min_value=1, max_value=n))
    seed = draw(st.integers(min_value=0, max_value=2**31 - 1))
    special = draw(st.lists(values, min_size=0, max_size=min(n, 40)))
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * 1e-2).astype(np.float32)
    if draw(st.booleans()):
        x = np.round(x * 200) / 200                      # heavy ties
    pos = rng.permutation(n)[: len(special)]
    x[pos] = np.array(special, dtype=np.float32)
    return torch.from_numpy(x.astype(np.float32)), k


def _compress(method, name, grad, resid, k):
    n = grad.numel()
    comp = ext.Compressor(method)
    idx = torch.full((k,), -1, dtype=torch.int32)
    val = torch.zeros(k)
    out = []
    for _ in range(2):        # second call runs with the adapted threshold
        g = grad.clone()
        before = resid.clone()
        cnt = comp.compress_with_feedback(name, g.data_ptr(), resid.data_ptr(), n, k, idx.data_ptr(), val.data_ptr())
        out.append((cnt, idx[:cnt].long().clone(), val[:cnt].clone(), before, resid.clone()))
    return out


@settings(max_examples=60, deadline=None)
@given(problem())
def test_selection_invariants(p):
    grad, k = p
    n = grad.numel()
    for method in ("topk", "thresholdv", "thresholdv16"):
        resid = torch.zeros(n)
        for cnt, idx, val, before, after in _compress(method, "t", grad, resid, k):
            a = grad + before
            assert 0 <= cnt <= k
            assert idx.numel() == idx.unique().numel(), "an index was sent twice"
            assert bool((idx >= 0).all()) and bool((idx < n).all())
            assert torch.equal(val, a[idx]), "sent values are the accumulated gradient at the sent indices"
            # mass conservation: every element is either sent or kept, bit for bit
            kept = a.clone()
            kept[idx] = 0.0
            assert torch.equal(after, kept)
            if method == "topk":
                assert cnt == k
                rest = kept.abs()
                assert float(val.abs().min()) >= float(rest.max()), "something larger than a sent element stayed behind"
            if method == "thresholdv16":
                # whole blocks are taken; only the zero padding of the tensor's last block is left out
                assert k - 15 <= cnt <= k, "threshold-v16 fills the stream"


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 5), st.integers(1, 400), st.integers(0, 2**31 - 1))
def test_merge_equals_dense_sum(world, n, seed):
    rng = np.random.default_rng(seed)
    idxs, vals, cnts, dense = [], [], [], np.zeros(n, dtype=np.float64)
    weights = rng.random(world).astype(np.float32)
    for w in range(world):
        c = int(rng.integers(0, n + 1))
        i = torch.from_numpy(rng.permutation(n)[:c].astype(np.int32))
        v = torch.from_numpy(rng.standard_normal(c).astype(np.float32))
        idxs.append(i); vals.append(v); cnts.append(c)
        dense[i.numpy()] += (v.numpy() * weights[w]).astype(np.float32)
    keep = [t if t.numel() else torch.zeros(1, dtype=t.dtype) for t in idxs + vals]          # valid pointers for empty streams
    got_i, got_v = ext.merge_streams([t.data_ptr() for t in keep[:world]], [t.data_ptr() for t in keep[world:]], cnts,
                                     [float(x) for x in weights], n)
    touched = sorted(set(np.concatenate([i.numpy() for i in idxs]).tolist())) if sum(cnts) else []
    assert sorted(got_i) == touched, "the merge returns the union of the indices, each once"
    for i, v in zip(got_i, got_v):
        assert v == pytest.approx(dense[i], rel=1e-5, abs=1e-6)


@settings(max_examples=40, deadline=None)
@given(st.lists(st.integers(0, 65535), min_size=1, max_size=300), st.lists(values, min_size=1, max_size=300))
def test_wire_casts_roundtrip(indices, vals):
    idx = torch.tensor(indices, dtype=torch.int32)
    n16 = torch.empty(len(indices), dtype=torch.int16); back = torch.empty(len(indices), dtype=torch.int32)
    ext.narrow_u32_to_u16(idx.data_ptr(), n16.data_ptr(), len(indices))
    ext.widen_u16_to_u32(n16.data_ptr(), back.data_ptr(), len(indices))
    assert torch.equal(idx, back)
    x = torch.tensor(vals, dtype=torch.float32)
    h = torch.empty(len(vals), dtype=torch.int16); y = torch.empty(len(vals))
    ext.f32_to_bf16(x.data_ptr(), h.data_ptr(), len(vals)); ext.bf16_to_f32(h.data_ptr(), y.data_ptr(), len(vals))
    assert torch.equal(y, x.bfloat16().float())
    ext.f32_to_f16(x.data_ptr(), h.data_ptr(), len(vals)); ext.f16_to_f32(h.data_ptr(), y.data_ptr(), len(vals))
    assert torch.equal(y, x.half().float())


@st.composite
def sparse_stream(draw):
    """Unique indices with a mix of whole aligned blocks of 16, runs that only look like blocks and loose entries."""
    numel = draw(st.sampled_from([40, 4096, 65536, 70000, 1 << 20, (1 << 20) + 64, 5_000_000]))
    n_blocks = draw(st.integers(min_value=0, max_value=min(12, numel // 16)))
    blocks = draw(st.lists(st.integers(min_value=0, max_value=numel // 16 - 1), min_size=n_blocks, max_size=n_blocks, unique=True))
    used = set()
    idx = []
    for b in blocks:
        keep = draw(st.sampled_from([16, 16, 16, 15, 9]))          # some blocks arrive truncated
        run = list(range(16 * b, 16 * b + keep))
        if draw(st.booleans()) and keep == 16:
            run = run[1:] + run[:1]                                # all 16 present, but not in counting order
        idx += run
        used.update(run)
        for j in draw(st.lists(st.integers(min_value=0, max_value=numel - 1), max_size=3)):
            if j not in used:
                idx.append(j)
                used.add(j)
    seed = draw(st.integers(min_value=0, max_value=2**31 - 1))
    val = np.random.default_rng(seed).standard_normal(len(idx)).astype(np.float32).tolist()
    return numel, idx, val, draw(st.booleans()), draw(st.sampled_from([0, 1, 2])), draw(st.booleans())


@settings(max_examples=150, deadline=None)
@given(sparse_stream())
def test_wire_payload_round_trip_for_any_mix_of_blocks_and_loose_entries(case):
    numel, idx, val, allow_u16, value_format, allow_blocks = case
    flags, payload = ext.encode_sparse(idx, val, numel, allow_u16, value_format, allow_blocks)
    got_idx, got_val = ext.decode_sparse(flags, payload, numel)
    want = torch.tensor(val, dtype=torch.float32)
    if value_format == 1:
        want = want.half().float()
    elif value_format == 2:
        want = want.bfloat16().float()
    assert sorted(zip(got_idx, got_val)) == sorted(zip(idx, want.tolist()))
    pairs = 4 + len(idx) * ((2 if (flags & 1) else 4) + (2 if value_format else 4))
    assert len(payload) <= pairs + 4                       # the block form is only chosen when a block exists
    if not allow_blocks:
        assert not flags & 0x08


@settings(max_examples=300, deadline=None)
@given(st.integers(min_value=0, max_value=31), st.binary(max_size=200), st.sampled_from([0, 100, 70000]))
def test_wire_decoder_refuses_or_decodes_arbitrary_bytes(flags, payload, numel):
    """What arrives from the network is untrusted: the decoder either returns entries inside the tensor or raises."""
    try:
        idx, val = ext.decode_sparse(flags, payload, numel)
    except ValueError:
        return
    assert len(idx) == len(val)
    if numel:
        assert all(i < numel or i == 0xFFFFFFFF for i in idx)


@settings(max_examples=10, deadline=None)
@given(st.lists(st.integers(1, 3000), min_size=2, max_size=7), st.sampled_from([64, 512, 2048, 1 << 16]),
       st.sampled_from(["topk", "thresholdv", "thresholdv16"]), st.integers(0, 2**20))
def test_bundles_train_bit_for_bit_like_one_task_per_tensor(sizes, bundle_elems, method, seed):
    """Any mix of tensor sizes, any bundle limit, any compressor: laying small tensors end to end in one task changes
    nothing in what is selected, merged and applied (selection stays per tensor, under the tensor's own threshold)."""
    import torch.nn as nn

    class Bag(nn.Module):
        def __init__(self):
            super().__init__()
            g = torch.Generator().manual_seed(seed)
            self.ps = nn.ParameterList([nn.Parameter(torch.randn(n, generator=g)) for n in sizes])

        def forward(self, coeffs):
            return sum((p * c).sum() for p, c in zip(self.ps, coeffs))

    def run(be):
        model = Bag()
        eng = cpu_tier.CpuOffloadEngine(model, method=method, ratio=0.8, optimizer="adam", optimizer_options={"lr": 1e-2},
                                        staleness=1, data_bytes=4 << 20, workers=2, bundle_elems=be)
        g = torch.Generator().manual_seed(seed + 1)
        for _ in range(4):
            model([torch.randn(n, generator=g) for n in sizes]).backward()
        eng.synchronize()
        out = [p.detach().clone() for p in model.parameters()], eng.engine.num_params()
        eng.close()
        return out

    want, n_plain = run(0)
    got, n_units = run(bundle_elems)
    assert n_plain == len(sizes) and n_units <= n_plain
    for a, b in zip(got, want):
        assert torch.equal(a, b)
