"""CPU tier between nodes: the whole host pipeline of W "nodes" on one machine over a paced loopback link.

    python -m stellatrain_b200.bench_cpu_ring                       # 2 nodes, 1 Gbit/s, ResNet-18-sized parameters
    python -m stellatrain_b200.bench_cpu_ring --gbps 0 --nodes 4    # unpaced loopback

Every node is a process with its own shared-memory session and its own native engine (one local rank); the nodes
exchange their sparse streams over the TCP ring and each sender is paced to ``--gbps`` by the comm manager's token
bucket, which stands in for the slow links the reference was written for (about 1 Gbit/s between machines,
README.md:21-29; the reference itself needs real machines for this, backend/test/test_end_to_end.py:15-34).  Gradients
are synthetic host tensors, so no GPU takes part: what is timed is gather, compress, exchange, merge and the sparse
optimiser, with staleness 1, for each wire format:

* ``pairs``: (index, value) entries, fp32 values (what the reference sends);
* ``blocks``: whole aligned runs of 16 indices as one block id;
* ``blocks+bf16``: the same with bf16 values whose rounding error stays in the sender's residual.

Prints one JSON line per wire format: milliseconds per step (max over nodes) and bytes a node sends per step.
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import socket
import time

# parameter tensors of torchvision's ResNet-18 above 100k elements (the small ones do not matter for bandwidth)
RESNET18_LARGE = [2359296] * 3 + [1179648, 589824, 589824, 589824, 294912, 147456, 147456, 147456, 131072, 512000]
WIRE = {"pairs": (False, 0), "blocks": (True, 0), "blocks+bf16": (True, 2)}


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _node(q, port: int, session: int, world: int, node: int, sizes: list, steps: int, warmup: int, method: str,
          ratio: float, wire: str, bytes_per_s: float) -> None:
    try:
        import torch

        from stellatrain_b200 import cpu_tier

        ext = cpu_tier._load()
        ext.set_log_level(3)
        torch.set_num_threads(1)
        eng = ext.CpuEngine()
        data_bytes = int(sum(sizes) * 4 * 4 * 1.25) + (16 << 20)
        eng.configure("127.0.0.1", port, world, node, session + node, 1, 0, method, 1, 1, ratio, data_bytes, 60000, 8, False,
                      False, False)
        eng.configure_wire(*WIRE[wire])
        eng.set_optimizer("adam")
        eng.configure_optimizer("lr", 1e-3)
        if bytes_per_s > 0:
            eng.set_tx_rate_limit(bytes_per_s, 256 << 10)
        params = [torch.zeros(n) for n in sizes]
        idxs = [eng.pre_train_init(i, f"p{i}", p.numel(), p.data_ptr()) for i, p in enumerate(params)]
        gen = torch.Generator().manual_seed(17 + node)
        grads = [[torch.randn(n, generator=gen) * 1e-2 for n in sizes] for _ in range(2)]

        def step(s: int) -> None:
            for i in idxs:
                eng.pre_forward_process(i)
            for i in reversed(idxs):
                eng.post_backward_process(i, grads[s % 2][i].data_ptr())

        for s in range(warmup):
            step(s)
        eng.synchronize()
        eng.barrier()
        tx0 = eng.comm_bytes()[0]
        t0 = time.perf_counter()
        for s in range(steps):
            step(s)
        eng.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        tx = eng.comm_bytes()[0] - tx0
        eng.barrier()
        q.put((node, "ok", ms / steps, tx / steps))
        del eng
    except Exception as e:  # noqa: BLE001 - reported to the parent
        q.put((node, "error", f"{type(e).__name__}: {e}", 0))


def run(nodes: int = 2, gbps: float = 1.0, steps: int = 10, warmup: int = 3, method: str = "thresholdv16", ratio: float = 0.99,
        wire: str = "blocks", sizes: list | None = None) -> dict:
    from stellatrain_b200 import cpu_tier

    sizes = sizes or RESNET18_LARGE
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, session = _free_port(), (os.getpid() % 10000) * 1000 + 100
    procs = [ctx.Process(target=_node, args=(q, port, session, nodes, r, sizes, steps, warmup, method, ratio, wire, gbps * 1e9 / 8))
             for r in range(nodes)]
    for p in procs:
        p.start()
    results = []
    deadline = time.time() + 600
    while len(results) < nodes and time.time() < deadline:
        try:
            results.append(q.get(timeout=0.5))
        except Exception:  # noqa: BLE001 - queue.Empty
            if not any(p.is_alive() for p in procs) and q.empty():
                break
    for p in procs:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
    ext = cpu_tier._load()
    for r in range(nodes):
        ext.ShmManager.unlink_session(session + r)
    bad = [r for r in results if r[1] != "ok"]
    if bad or len(results) != nodes:
        raise RuntimeError(f"ring benchmark failed: {bad or 'a node did not report'}")
    return {"config": "CPU tier, one process per node on one host, paced loopback TCP ring, staleness 1, sparse Adam",
            "nodes": nodes, "link_gbps": gbps or None, "method": method, "kept_fraction": 1 - ratio, "wire": wire,
            "params": sum(sizes), "tensors": len(sizes), "steps": steps,
            "ms_per_step": max(r[2] for r in results), "tx_bytes_per_step_per_node": max(r[3] for r in results)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", type=int, default=2)
    ap.add_argument("--gbps", type=float, default=1.0, help="pace of every node's sends; 0: unpaced")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--method", default="thresholdv16")
    ap.add_argument("--ratio", type=float, default=0.99)
    ap.add_argument("--wire", default="all", choices=["all", *WIRE])
    a = ap.parse_args()
    for w in (WIRE if a.wire == "all" else [a.wire]):
        print(json.dumps(run(a.nodes, a.gbps, a.steps, a.warmup, a.method, a.ratio, w)), flush=True)


if __name__ == "__main__":
    main()
