"""CPU-tier kernels (native `_Ccpu`) against the PyTorch oracle."""
import numpy as np
import pytest
import torch

from stellatrain_b200 import cpu_tier
from stellatrain_b200.ops import oracle as O

ext = cpu_tier._load()
SIZES = [1, 15, 16, 17, 1000, 65535, 65536, 70001, 300007]


def _states(comp, name):
    st = comp.state().get(name)
    return O.ThresholdState(*st) if st else O.ThresholdState()


@pytest.mark.parametrize("method", ["topk", "thresholdv", "thresholdv16"])
@pytest.mark.parametrize("n", SIZES)
def test_compressors_match_oracle(method, n):
    g = torch.Generator().manual_seed(n)
    comp = ext.Compressor(method)
    name = f"t{n}"
    k = max(1, n // 100)
    resid = torch.zeros(n)
    resid_ref = torch.zeros(n)
    for step in range(4):
        grad = torch.randn(n, generator=g) * 1e-2
        if step == 2:
            grad = torch.round(grad * 300) / 300        # many exact ties
        st = _states(comp, name)
        idx = torch.empty(k, dtype=torch.int32)
        val = torch.empty(k, dtype=torch.float32)
        cnt = comp.compress_with_feedback(name, grad.data_ptr(), resid.data_ptr(), n, k, idx.data_ptr(), val.data_ptr())
        want_idx, want_val, new_r = O.compress_step(method, grad, resid_ref, k, st)
        keep = want_idx < n
        want_idx, want_val = want_idx[keep], want_val[keep]
        got = idx[:cnt].long()
        order_g, order_w = torch.argsort(got, stable=True), torch.argsort(want_idx, stable=True)
        assert torch.equal(got[order_g], want_idx[order_w]), (method, n, step)
        assert torch.equal(val[:cnt][order_g], want_val[order_w])
        resid_ref = new_r[:n].clone()
        assert torch.equal(resid, resid_ref)
        if method != "topk":
            tau = comp.state()[name][0]
            assert tau == pytest.approx(st.tau, rel=1e-6, abs=1e-30)


def test_threshold_state_roundtrip():
    comp = ext.Compressor("thresholdv16")
    x = torch.randn(4096)
    idx = torch.empty(40, dtype=torch.int32); val = torch.empty(40)
    comp.compress("a", x.data_ptr(), 4096, 40, idx.data_ptr(), val.data_ptr())
    st = comp.state()
    other = ext.Compressor("thresholdv16")
    other.set_state(st)
    assert other.state() == st


def test_randomk_distinct_and_in_range():
    comp = ext.Compressor("randomk")
    x = torch.randn(5000)
    idx = torch.empty(500, dtype=torch.int32); val = torch.empty(500)
    n1 = comp.compress("r", x.data_ptr(), 5000, 500, idx.data_ptr(), val.data_ptr())
    first = idx.clone()
    assert n1 == 500 and len(set(idx.tolist())) == 500 and int(idx.max()) < 5000
    assert torch.equal(val, x[idx.long()])
    comp.compress("r", x.data_ptr(), 5000, 500, idx.data_ptr(), val.data_ptr())
    assert not torch.equal(first, idx), "a new call must draw a new sample"
    s = ext.sample_without_replacement(10, 10, 7)
    assert sorted(s) == list(range(10))


def test_xorshift_streams():
    a = ext.xorshift_stream(1, 1000)
    b = ext.xorshift_stream(2, 1000)
    assert a != b and len(set(a)) == 1000
    lanes = ext.xorshift_lanes8(1, 100)
    assert lanes[0] == a[0], "lane 0 continues the scalar stream"
    per_lane = [lanes[i::8] for i in range(8)]
    assert all(per_lane[0] != per_lane[i] for i in range(1, 8))
    bits = np.unpackbits(np.array(a, dtype=np.uint64).view(np.uint8))
    assert abs(bits.mean() - 0.5) < 0.01


@pytest.mark.parametrize("kind", ["sgd", "adam"])
def test_sparse_optimizers_match_oracle(kind):
    g = torch.Generator().manual_seed(0)
    n = 10007
    param = torch.randn(n, generator=g)
    ref = param.clone()
    if kind == "sgd":
        opt = ext.SGD(); opt.configure("lr", 0.1); opt.configure("momentum", 0.9); opt.configure("weight_decay", 1e-4)
        cfg, st = O.SGDConfig(lr=0.1, momentum=0.9, weight_decay=1e-4), O.SGDState()
    else:
        opt = ext.Adam(); opt.configure("lr", 1e-3); opt.configure("weight_decay", 1e-2)
        cfg, st = O.AdamConfig(lr=1e-3, weight_decay=1e-2), O.AdamState()
    for step in range(5):
        idx = torch.randperm(n, generator=g)[:777].to(torch.int32)
        val = torch.randn(777, generator=g)
        opt.optimize(param.data_ptr(), n, "p", val.data_ptr(), idx.data_ptr(), 777)
        dense = torch.zeros(n); dense[idx.long()] = val
        touched = torch.zeros(n, dtype=torch.bool); touched[idx.long()] = True
        (O.sparse_sgd if kind == "sgd" else O.sparse_adam)(ref, dense, touched, cfg, st)
        torch.testing.assert_close(param, ref, rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError, match="NO OPTION"):
        opt.configure("no_such_option", 1.0)


def test_sgd_options_and_dense_oracle():
    g = torch.Generator().manual_seed(3)
    n = 513
    param = torch.randn(n, generator=g); ref = param.clone()
    opt = ext.SGD()
    for k, v in (("lr", 0.05), ("momentum", 0.8), ("dampening", 0.1), ("nestrov", True), ("smart_momentum", True)):
        opt.configure(k, v)
    cfg, st = O.SGDConfig(lr=0.05, momentum=0.8, dampening=0.1, nesterov=True, smart_momentum=True), O.SGDState()
    for step in range(6):
        idx = torch.randperm(n, generator=g)[:100].to(torch.int32); val = torch.randn(100, generator=g)
        opt.optimize(param.data_ptr(), n, "p", val.data_ptr(), idx.data_ptr(), 100)
        dense = torch.zeros(n); dense[idx.long()] = val
        touched = torch.zeros(n, dtype=torch.bool); touched[idx.long()] = True
        O.sparse_sgd(ref, dense, touched, cfg, st)
        torch.testing.assert_close(param, ref, rtol=1e-4, atol=1e-6)
    # the dense variant equals torch.optim.SGD when every index is touched
    p2 = torch.randn(n, generator=g); q = torch.nn.Parameter(p2.clone())
    naive = ext.SGDNaive(); naive.configure("lr", 0.1); naive.configure("momentum", 0.9)
    topt = torch.optim.SGD([q], lr=0.1, momentum=0.9)
    allidx = torch.arange(n, dtype=torch.int32)
    for _ in range(3):
        gr = torch.randn(n, generator=g)
        naive.optimize(p2.data_ptr(), n, "q", gr.data_ptr(), allidx.data_ptr(), n)
        q.grad = gr.clone(); topt.step()
    torch.testing.assert_close(p2, q.detach(), rtol=1e-5, atol=1e-6)


def test_merge_streams_union_and_weights():
    a_i = torch.tensor([1, 5, 9], dtype=torch.int32); a_v = torch.tensor([1.0, 2.0, 3.0])
    b_i = torch.tensor([5, 7, -1], dtype=torch.int32); b_v = torch.tensor([10.0, 20.0, 0.0])   # -1 = padding
    idx, val = ext.merge_streams([a_i.data_ptr(), b_i.data_ptr()], [a_v.data_ptr(), b_v.data_ptr()], [3, 3], [0.5, 0.5], 16)
    got = dict(zip(idx, val))
    assert got == {1: 0.5, 5: 6.0, 9: 1.5, 7: 10.0}


def test_casts_and_add():
    idx = torch.tensor([0, 1, 32767, 32768, 65535], dtype=torch.int32)
    n16 = torch.empty(5, dtype=torch.int16); back = torch.empty(5, dtype=torch.int32)
    ext.narrow_u32_to_u16(idx.data_ptr(), n16.data_ptr(), 5)
    ext.widen_u16_to_u32(n16.data_ptr(), back.data_ptr(), 5)
    assert torch.equal(idx, back), "indices above 32767 must survive the 16-bit wire form"
    x = torch.randn(1003) * 10
    h = torch.empty(1003, dtype=torch.int16); y = torch.empty(1003)
    ext.f32_to_f16(x.data_ptr(), h.data_ptr(), 1003); ext.f16_to_f32(h.data_ptr(), y.data_ptr(), 1003)
    assert torch.equal(y, x.half().float())
    ext.f32_to_bf16(x.data_ptr(), h.data_ptr(), 1003); ext.bf16_to_f32(h.data_ptr(), y.data_ptr(), 1003)
    assert torch.equal(y, x.bfloat16().float())
    a = torch.randn(1003); b = torch.randn(1003); want = a + b
    ext.add_arrays(a.data_ptr(), b.data_ptr(), 1003)
    assert torch.equal(a, want)
    sc = torch.empty(63); xs = torch.randn(1003)
    ext.block_l1_norms(xs.data_ptr(), 1003, sc.data_ptr())
    pad = torch.zeros(1008); pad[:1003] = xs
    assert torch.equal(sc, O.block_scores(pad))


def test_thread_pool_ordering_and_task_model():
    assert ext.pool_order_probe([5, 1, 3, 1, 0]) == [4, 1, 3, 2, 0]
    assert ext.parallel_sum_probe(100000, 7) == sum(range(100000))
    key, pkey, prio = ext.task_keys(12, 3, "conv1.weight")
    assert (key, pkey, prio) == ("12@3@conv1.weight", "3@conv1.weight", 12003)
    with pytest.raises(RuntimeError):
        ext.task_keys(0, 0, "x" * 80)
    CREATED, COPYIN, GATHER, COMPRESS, EXCHANGE, OPTIMIZE, WAIT, COPYOUT, FINISHED, FAILED = range(10)
    assert ext.task_transition_allowed(CREATED, COPYIN) and ext.task_transition_allowed(COMPRESS, OPTIMIZE)
    assert ext.task_transition_allowed(EXCHANGE, EXCHANGE) and ext.task_transition_allowed(GATHER, FAILED)
    assert not ext.task_transition_allowed(CREATED, OPTIMIZE) and not ext.task_transition_allowed(FINISHED, FAILED)


def test_flat_gradient_benchmark_small():
    """Scaled-down form of the flat-gradient configuration: compressed + error feedback + sparse Adam
    tracks the dense-update reference; the full size runs in stellatrain_b200.bench_cpu_flat."""
    from stellatrain_b200.bench_cpu_flat import run

    for method in ("topk", "thresholdv"):
        out = run(numel=200_000, steps=10, method=method, seed=0)
        assert out["sent_fraction"] == pytest.approx(0.01, rel=0.15)
        assert out["rel_l2_to_dense"] < 1.0 and out["cos_to_dense"] > 0.1
        assert out["residual_mass_conserved"]


@pytest.mark.parametrize("method", ["topk", "thresholdv", "thresholdv16"])
def test_nan_gradients_are_dropped(method):
    """A NaN in the gradient is neither sent nor kept: the accumulate step writes zero in its place."""
    n, k = 1003, 50
    g = torch.Generator().manual_seed(3)
    grad = torch.randn(n, generator=g)
    bad = torch.tensor([0, 15, 16, 17, 500, 1001, 1002])
    grad[bad] = float("nan")
    resid = torch.randn(n, generator=g) * 0.1
    want = resid + grad
    want[bad] = 0.0
    comp = ext.Compressor(method)
    idx = torch.empty(k, dtype=torch.int32); val = torch.empty(k)
    cnt = comp.compress_with_feedback("t", grad.data_ptr(), resid.data_ptr(), n, k, idx.data_ptr(), val.data_ptr())
    assert not torch.isnan(resid).any() and not torch.isnan(val[:cnt]).any()
    rebuilt = resid.clone()
    rebuilt[idx[:cnt].long()] = val[:cnt]
    assert torch.equal(rebuilt, want)          # sent + kept = g + r with the NaN positions at zero
