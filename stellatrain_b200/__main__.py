"""``python -m stellatrain_b200``: what is built and what this machine offers.

The reference ships a ``fasterdp_engine`` executable that prints a banner, constructs the engine and blocks
(backend/src/engine/entry.cpp:5-12).  This entry point reports instead: package version, whether the two native
extensions are built for the current sources, the GPUs, their peer access and whether NVLink multicast (NVLS) is
available to the symmetric-memory pool.  ``--build`` compiles what is stale first.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def report(build: bool = False) -> dict:
    from . import __version__, _build

    out: dict = {"package": "stellatrain_b200", "version": __version__, "extensions": {}}
    if build:
        _build.build_all()
    for name in _build.EXTENSIONS:
        so = _build.so_path(name)
        out["extensions"][name] = {"path": str(so), "built": so.exists(), "current": _build.is_current(name)}
    try:
        import torch

        out["torch"] = torch.__version__
        out["cuda_available"] = bool(torch.cuda.is_available())
        gpus = []
        if torch.cuda.is_available():
            n = torch.cuda.device_count()
            for i in range(n):
                p = torch.cuda.get_device_properties(i)
                gpus.append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                             "memory_gb": round(p.total_memory / 2**30, 1),
                             "peers": [j for j in range(n) if j != i and torch.cuda.can_device_access_peer(i, j)]})
        out["gpus"] = gpus
        out["nccl"] = ".".join(map(str, torch.cuda.nccl.version())) if torch.cuda.is_available() else None
    except Exception as e:  # noqa: BLE001 - a report must not fail because one probe did
        out["torch_error"] = repr(e)
    try:
        from . import cpu_tier

        ext = cpu_tier._load()
        out["cpu_simd"] = ext.best_isa()
        # the reference's transports (ZeroMQ sockets, protobuf messages) are options that need a libzmq at run time
        lib = os.environ.get("STELLATRAIN_LIBZMQ") or cpu_tier.bundled_libzmq()
        try:
            import zmq

            pyzmq = zmq.__version__
        except ImportError:
            pyzmq = None
        out["zeromq"] = {"pyzmq": pyzmq, "libzmq": lib or None}
    except Exception as e:  # noqa: BLE001
        out["cpu_tier_error"] = repr(e)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(prog="python -m stellatrain_b200", description=__doc__.split("\n\n")[0])
    ap.add_argument("--build", action="store_true", help="compile stale extensions first")
    args = ap.parse_args()
    json.dump(report(args.build), sys.stdout, indent=2)
    sys.stdout.write("\n")


if __name__ == "__main__":
    main()
