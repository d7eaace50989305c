"""Several ranks of the sparse exchange emulated on ONE GPU: every rank is a GpuBucket of its own, wired to the
others' receive areas through ordinary device pointers, and all kernels run on one stream in an order in which
every flag is set before the kernel that waits for it is launched (select of all ranks, then scatter+apply of all
ranks, then the parameter copy of all ranks).  Covers the replicated and the partitioned optimiser state."""
import pytest
import torch

pytestmark = pytest.mark.gpu

NUMELS = [5000, 70000, 130, 40000, 16, 9000]


def _make_ranks(world, numels, compressor, optimizer, partition, ratio, dev, lr=1e-2, narrow=False, debug=False,
                deterministic=False):
    from stellatrain_b200.parallel import buckets as B
    from stellatrain_b200.parallel.gpu_bucket import CandidateScratch, GpuBucket, Wiring

    scratch = CandidateScratch(dev)
    ranks = []
    for r in range(world):
        layout = B.BucketLayout([f"t{i}" for i in range(len(numels))], list(numels), chunk_elems=1024, narrow_wire=narrow)
        ranks.append(GpuBucket(0, layout, dev, compressor=compressor, ratio=ratio, world=world, rank=r,
                               optimizer=optimizer, scratch=scratch, timeout_s=1.0, partition_state=partition,
                               deterministic_merge=deterministic, divide_k_by_world=not deterministic))
    nbytes = ranks[0].recv_bytes()
    mk8 = lambda: torch.zeros(nbytes, dtype=torch.uint8, device=dev)       # noqa: E731
    mkf = lambda: torch.zeros(2 * world, dtype=torch.int64, device=dev)    # noqa: E731
    recv, wb = [mk8() for _ in ranks], [mk8() for _ in ranks]
    flag, ack, pflag = [mkf() for _ in ranks], [mkf() for _ in ranks], [mkf() for _ in ranks]
    cks = [torch.zeros(2 * world, dtype=torch.int32, device=dev) for _ in ranks]
    ptrs = lambda ts: [t.data_ptr() for t in ts]                           # noqa: E731
    for r, b in enumerate(ranks):
        dbg = dict(cksum_local=cks[r], peer_cksum=ptrs(cks), poison=True) if debug else {}
        b.wire(Wiring(world, r, recv[r], ptrs(recv), flag[r], ptrs(flag), ack[r], ptrs(ack), use_flags=True,
                      use_acks=True, wb_local=wb[r], peer_wb=ptrs(wb), pflag_local=pflag[r], peer_pflag=ptrs(pflag), **dbg))
        b.set_optimizer_options(lr=lr, momentum=0.9)
    init = torch.randn(ranks[0].layout.n_total, device=dev, generator=torch.Generator(device=dev).manual_seed(7))
    for b in ranks:
        b.param.copy_(init)
    return ranks


def _step(ranks, grads):
    for b, g in zip(ranks, grads):
        b.grad.copy_(g)
    for b in ranks:
        b.select()
    for b in ranks:
        b.apply(phase=1)
    for b in ranks:
        b.apply(phase=2)


def _grads(world, layout, step, dev):
    """One flat gradient per rank; the padding behind every tensor stays zero, as the engine keeps it."""
    n = layout.n_total
    g = torch.Generator(device=dev).manual_seed(1000 * step + 1)
    valid = torch.zeros(n, device=dev)
    for s in layout.segments:
        valid[s.off : s.off + s.numel] = 1.0
    return [torch.randn(n, device=dev, generator=g) * 1e-2 * valid for _ in range(world)]


@pytest.mark.parametrize("narrow", [False, True])
@pytest.mark.parametrize("partition", [False, True])
def test_topk_adam_matches_dense_restatement(partition, narrow):
    """narrow: tensors below 65536 elements travel as (u16 index, bf16 value); the sender keeps the rounding
    error in its residual."""
    dev = torch.device("cuda:0")
    world, ratio, lr = 4, 0.9, 1e-2
    ranks = _make_ranks(world, NUMELS, "topk", "adam", partition, ratio, dev, lr, narrow=narrow)
    L = LAY = ranks[0].layout
    n = L.n_total
    x = ranks[0].param.double().clone()
    resid = [torch.zeros(n, device=dev) for _ in range(world)]    # fp32 like the device: selection must see equal keys
    m = torch.zeros(n, dtype=torch.float64, device=dev)
    v = torch.zeros(n, dtype=torch.float64, device=dev)
    for step in range(1, 6):
        grads = _grads(world, LAY, step, dev)
        _step(ranks, grads)
        merged = torch.zeros(n, dtype=torch.float64, device=dev)
        touched = torch.zeros(n, dtype=torch.bool, device=dev)
        for r in range(world):
            a = resid[r] + grads[r]
            for s in L.segments:
                seg = a[s.off : s.off + s.numel]
                idx = torch.topk(seg.abs(), s.k).indices + s.off
                sent = a[idx]
                if narrow and s.n_pad < 65536:
                    sent = sent.bfloat16().float()
                merged[idx] += sent.double() / world
                touched[idx] = True
                a[idx] = a[idx] - sent
            resid[r] = a
        g = merged[touched]
        m[touched] = 0.9 * m[touched] + 0.1 * g
        v[touched] = 0.999 * v[touched] + 0.001 * g * g
        x[touched] -= lr * (m[touched] / (1 - 0.9 ** step)) / ((v[touched] / (1 - 0.999 ** step)).sqrt() + 1e-8)
    torch.cuda.synchronize()
    for b in ranks:
        b.check_status()
        assert float((b.param.double() - x).abs().max()) < 2e-5
    for r, b in enumerate(ranks):
        assert torch.equal(b.resid, resid[r])
        lo, hi = b.state_lo, b.state_hi
        assert float((b.m[: hi - lo].double() - m[lo:hi]).abs().max()) < 1e-6
        if partition:
            assert torch.equal(b.param, ranks[0].param)         # owners' values are copied, not recomputed
            assert b.m.numel() < n and (hi - lo) <= n
    if partition:
        assert sum(b.state_hi - b.state_lo for b in ranks) == n   # the ranges tile the bucket
    if narrow:
        L0 = ranks[0].layout
        assert L0.wire_bytes() < 8 * L0.cap and any(L0.is_narrow(s) for s in L0.segments) and not L0.is_narrow(L0.segments[1])
        idx, val = ranks[0].stream_of(1, 2)          # epoch 5 sits in slot 1; decode rank 2's stream
        if not partition:
            s3 = L0.segments[3]
            got = idx[s3.out_off : s3.out_off + s3.k]
            assert bool(((got >= s3.off) & (got < s3.off + s3.numel)).all())


@pytest.mark.parametrize("compressor", ["thresholdv16", "thresholdv", "randomk"])
@pytest.mark.parametrize("optimizer", ["adam", "sgd"])
def test_partitioned_state_equals_replicated(compressor, optimizer):
    dev = torch.device("cuda:0")
    world = 4
    rep = _make_ranks(world, NUMELS, compressor, optimizer, False, 0.9, dev)
    par = _make_ranks(world, NUMELS, compressor, optimizer, True, 0.9, dev)
    LAY = rep[0].layout
    for step in range(1, 9):
        grads = _grads(world, LAY, step, dev)
        _step(rep, grads)
        _step(par, grads)
        if step == 4:                       # a change of the compression ratio moves the owners' entry ranges
            torch.cuda.synchronize()
            for b in rep + par:
                b.set_ratio(0.95)
    torch.cuda.synchronize()
    for b in rep + par:
        b.check_status()
    for r in range(world):
        assert torch.equal(par[r].param, par[0].param)
        assert float((par[r].param - rep[r].param).abs().max()) < 1e-5
        assert torch.equal(par[r].resid, rep[r].resid)          # selection does not depend on where the state lives


def test_ranks_that_own_nothing():
    dev = torch.device("cuda:0")
    world = 4
    numels = [100000, 50]
    rep = _make_ranks(world, numels, "topk", "adam", False, 0.9, dev)
    par = _make_ranks(world, numels, "topk", "adam", True, 0.9, dev)
    owners = [s.owner for s in par[0].layout.segments]
    assert len(set(owners)) < world
    LAY = rep[0].layout
    for step in range(1, 5):
        grads = _grads(world, LAY, step, dev)
        _step(rep, grads)
        _step(par, grads)
    torch.cuda.synchronize()
    for r in range(world):
        par[r].check_status()
        assert torch.equal(par[r].param, par[0].param)
        assert float((par[r].param - rep[r].param).abs().max()) < 1e-5


def test_full_state_loads_into_partitioned_buckets():
    """A checkpoint that holds the whole bucket's moments (replicated state, or a gathered file) restores ranks that
    keep only their own range; training then continues exactly as the replicated ranks do."""
    dev = torch.device("cuda:0")
    world = 4
    rep = _make_ranks(world, NUMELS, "topk", "adam", False, 0.9, dev)
    LAY = rep[0].layout
    for step in range(1, 4):
        _step(rep, _grads(world, LAY, step, dev))
    torch.cuda.synchronize()
    par = _make_ranks(world, NUMELS, "topk", "adam", True, 0.9, dev)
    for r in range(world):
        par[r].load_state_dict(rep[r].state_dict())
        lo, hi = par[r].state_lo, par[r].state_hi
        assert torch.equal(par[r].m[: hi - lo], rep[r].m[lo:hi]) and torch.equal(par[r].v[: hi - lo], rep[r].v[lo:hi])
    # flags, acknowledgements and write-back flags restart from the restored epoch
    e = int(par[0].counters[0]) - 1
    for b in par:
        for t in (b.wiring.flag_local, b.wiring.ack_local, b.wiring.pflag_local):
            t.fill_(e)
    for step in range(4, 8):
        grads = _grads(world, LAY, step, dev)
        _step(rep, grads)
        _step(par, grads)
    torch.cuda.synchronize()
    for r in range(world):
        par[r].check_status()
        assert torch.equal(par[r].param, par[0].param)
        assert float((par[r].param - rep[r].param).abs().max()) < 1e-5


@pytest.mark.parametrize("compressor", ["topk", "thresholdv16"])
@pytest.mark.parametrize("partition,narrow", [(False, False), (True, False), (False, True)])
def test_debug_checks_accept_good_streams_and_catch_a_corrupted_one(partition, narrow, compressor):
    """Debug checks: every stream carries the sum of a hash over its entries; the receiver recomputes it.  Clean
    steps pass and give the same parameters as without the checks; one flipped bit in one received entry is reported by
    the rank that received it (status 6) and by nobody else."""
    dev = torch.device("cuda:0")
    world = 4
    plain = _make_ranks(world, NUMELS, compressor, "adam", partition, 0.9, dev, narrow=narrow)
    dbg = _make_ranks(world, NUMELS, compressor, "adam", partition, 0.9, dev, narrow=narrow, debug=True)
    LAY = dbg[0].layout
    for step in range(1, 5):
        grads = _grads(world, LAY, step, dev)
        _step(plain, grads)
        _step(dbg, grads)
    torch.cuda.synchronize()
    for r in range(world):
        dbg[r].check_status()
        assert torch.equal(dbg[r].param, plain[r].param) or float((dbg[r].param - plain[r].param).abs().max()) < 1e-6
    # step 5 (slot 1): corrupt what rank 1 received from rank 2, between the selects and the applies
    grads = _grads(world, LAY, 5, dev)
    for b, g in zip(dbg, grads):
        b.grad.copy_(g)
    for b in dbg:
        b.select()
    victim, src = dbg[1], 2
    cap = LAY.cap
    words = victim.wiring.recv_local.view(torch.int32)[: 2 * world * cap * 2].view(2, world, cap, 2)
    pos = LAY.owner_bounds(world)[1] if partition else LAY.segments[1].out_off     # an entry of the 70000-element tensor: wide format
    words[1, src, pos, 1] ^= 0x00010000
    for b in dbg:
        b.apply(phase=1)
    for b in dbg:
        b.apply(phase=2)
    torch.cuda.synchronize()
    codes = [int(b.status.item()) for b in dbg]
    assert codes[1] == 6, codes
    # with partitioned state the owner that found the mismatch withholds its parameter values, so the others'
    # bounded wait for them runs out (status 2) instead of reading values computed from a corrupted stream
    allowed = (0, 2) if partition else (0,)
    assert all(c in allowed for i, c in enumerate(codes) if i != 1), codes


def test_deterministic_merge_keeps_replicas_bit_equal():
    """Every rank keeps half of every tensor (k is not divided by the world size here), so most elements receive three or
    four contributions; added in rank order they round the same way on every replica."""
    dev = torch.device("cuda:0")
    world = 4
    ranks = _make_ranks(world, NUMELS, "topk", "adam", False, 0.5, dev, deterministic=True)
    LAY = ranks[0].layout
    for step in range(1, 7):
        _step(ranks, _grads(world, LAY, step, dev))
    torch.cuda.synchronize()
    for b in ranks:
        b.check_status()
        assert torch.equal(b.param, ranks[0].param) and torch.equal(b.m, ranks[0].m) and torch.equal(b.v, ranks[0].v)
    assert float((ranks[0].param - torch.randn(LAY.n_total, device=dev, generator=torch.Generator(device=dev).manual_seed(7))).abs().max()) > 0
