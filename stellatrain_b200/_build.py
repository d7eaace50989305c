"""In-tree build of the native extensions.

Two shared objects are produced next to this file:

* ``_C``    the sm_100a CUDA kernels plus their pybind11 surface (``csrc/cuda``)
* ``_Ccpu`` the CPU-offload tier: SIMD compressors and sparse optimisers, thread pool, task model,
            shared-memory pool, TCP comm manager, telemetry (``csrc/cpu``, ``csrc/core``,
            ``csrc/comm``, ``csrc/telemetry``)

The reference builds its single ``fasterdp`` module with CMake for the host CPU only
(backend/CMakeLists.txt:3-6, 28-29); here the device code is compiled for exactly one target,
``-gencode arch=compute_100a,code=sm_100a``.

A build is skipped when the recorded hash of the sources and flags matches, so importing the package on
a machine that received pre-built objects does not recompile.
"""
from __future__ import annotations

import hashlib
import importlib.machinery
import importlib.util
import json
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ_DIR = ROOT / "build"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
# -ffp-contract=off: vector and scalar variants of a kernel must round identically, so that replicas
# that process an element on different paths stay bit-equal
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function", "-pthread",
             "-ffp-contract=off"]


def _pybind_includes() -> list[str]:
    import pybind11

    return [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}"]


EXTENSIONS = {
    "_C": {
        "cu": ["cuda/select_kernels.cu", "cuda/apply_kernels.cu", "cuda/aux_kernels.cu", "cuda/noalloc_entry.cu"],
        "cpp": ["cuda/bindings.cpp"],
        # compiled against the torch headers and linked with the torch libraries: the native step engine registers
        # C++ hooks on autograd's accumulation nodes (the reference links its engine against torch the same way,
        # backend/CMakeLists.txt:12-16, 84-100)
        "torch_cpp": ["cuda/native_engine.cpp"],
        "link": "nvcc",
    },
    "_Ccpu": {
        "cu": [],
        "cpp": [
            "cpu/compressors.cpp", "cpu/optimizers.cpp", "cpu/array_util.cpp", "cpu/xorshift.cpp",
            "core/threadpool.cpp", "core/task.cpp", "core/shm_manager.cpp", "core/engine.cpp", "core/cuda_api.cpp", "core/fake_cuda.cpp",
            "core/stages.cpp", "comm/comm_manager.cpp", "comm/net_util.cpp", "comm/zmq_link.cpp",
            "telemetry/telemetry.cpp", "telemetry/proto_wire.cpp", "bindings_cpu.cpp",
        ],
        "link": "g++",
    },
}


def _torch_paths() -> dict:
    """Include and library directories of the installed torch (found without importing it)."""
    spec = importlib.util.find_spec("torch")
    if spec is None or not spec.submodule_search_locations:
        raise RuntimeError("the native step engine needs torch's headers and libraries")
    root = Path(list(spec.submodule_search_locations)[0])
    version = (root / "version.py").read_text() if (root / "version.py").exists() else ""
    return {"include": [root / "include", root / "include" / "torch" / "csrc" / "api" / "include"], "lib": root / "lib",
            "version": version}


def _existing(name: str) -> dict:
    spec = EXTENSIONS[name]
    return {
        "cu": [s for s in spec["cu"] if (CSRC / s).exists()],
        "cpp": [s for s in spec["cpp"] if (CSRC / s).exists()],
        "torch_cpp": [s for s in spec.get("torch_cpp", []) if (CSRC / s).exists()],
        "link": spec["link"],
    }


def _source_hash(name: str) -> str:
    spec = _existing(name)
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    files = [CSRC / s for s in spec["cu"] + spec["cpp"] + spec["torch_cpp"]]
    if spec["torch_cpp"]:
        h.update(_torch_paths()["version"].encode())
    files += sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")) + sorted(CSRC.rglob("*.hpp"))
    for f in files:
        h.update(str(f.relative_to(CSRC)).encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def so_path(name: str) -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return ROOT / f"{name}{suffix}"


def _stamp_path(name: str) -> Path:
    return OBJ_DIR / f"{name}.stamp.json"


def is_current(name: str) -> bool:
    so, stamp = so_path(name), _stamp_path(name)
    if not so.exists() or not stamp.exists():
        return False
    try:
        return json.loads(stamp.read_text()).get("hash") == _source_hash(name)
    except (OSError, ValueError):
        return False


def _run(cmd: list[str]) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return proc.stdout + proc.stderr


def build_extension(name: str, force: bool = False, verbose: bool = False) -> Path:
    """Compile and link one extension; returns the path of the shared object.

    Several ranks of one job may find the extension stale at the same moment (sources newer than the shipped
    objects): one of them builds while the others wait on a lock file and then find the result current.  Objects go
    to a directory of the building process and the shared object is renamed into place, so nobody ever loads a
    half-written file."""
    if not force and is_current(name):
        return so_path(name)
    import fcntl

    OBJ_DIR.mkdir(exist_ok=True)
    with open(OBJ_DIR / f"{name}.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and is_current(name):
                return so_path(name)
            return _build_locked(name, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(name: str, verbose: bool) -> Path:
    spec = _existing(name)
    if not spec["cu"] and not spec["cpp"]:
        raise RuntimeError(f"extension {name} has no sources")
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = str(CUDA_HOME / "bin" / "nvcc")
    inc = [f"-I{CSRC}", f"-I{CSRC / 'cuda'}", f"-I{CUDA_HOME / 'include'}"] + _pybind_includes()
    jobs, objs = [], []
    for s in spec["cu"]:
        obj = OBJ_DIR / (name + "_" + s.replace("/", "_") + ".o")
        extra = ["-Xptxas", "-v"] if verbose else []
        jobs.append([nvcc, *NVCC_FLAGS, *extra, *inc, "-c", str(CSRC / s), "-o", str(obj)])
        objs.append(obj)
    for s in spec["cpp"]:
        obj = OBJ_DIR / (name + "_" + s.replace("/", "_") + ".o")
        jobs.append(["g++", *CXX_FLAGS, *inc, "-c", str(CSRC / s), "-o", str(obj)])
        objs.append(obj)
    link_extra = []
    if spec["torch_cpp"]:
        tp = _torch_paths()
        tinc = [f"-I{CSRC}", f"-I{CSRC / 'cuda'}", *[f"-I{d}" for d in tp["include"]], f"-I{sysconfig.get_paths()['include']}",
                f"-I{CUDA_HOME / 'include'}"]
        for s in spec["torch_cpp"]:
            obj = OBJ_DIR / (name + "_" + s.replace("/", "_") + ".o")
            jobs.append(["g++", *[f for f in CXX_FLAGS if f != "-Wall"], "-D_GLIBCXX_USE_CXX11_ABI=1", *tinc, "-c", str(CSRC / s),
                         "-o", str(obj)])
            objs.append(obj)
        link_extra = [f"-L{tp['lib']}", "-ltorch_python", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10_cuda", "-lc10",
                      "-Xlinker", f"-rpath={tp['lib']}"]
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        outs = list(ex.map(_run, jobs))
    if verbose:
        for o in outs:
            if o.strip():
                print(o)
    so = so_path(name)
    tmp = so.with_name(so.name + f".tmp{os.getpid()}")
    if spec["link"] == "nvcc":
        _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), *link_extra])
    else:
        _run(["g++", "-shared", "-o", str(tmp), *map(str, objs), "-pthread", "-lrt", "-ldl"])
    os.replace(tmp, so)
    _stamp_path(name).write_text(json.dumps({"hash": _source_hash(name)}))
    return so


def load_extension(name: str, build_if_missing: bool = True):
    """Import an in-tree extension by file path (never from site-packages)."""
    full = f"{__package__}.{name}"
    if full in sys.modules:
        return sys.modules[full]
    so = so_path(name)
    if not is_current(name):
        if not build_if_missing and not so.exists():
            raise ImportError(f"{so} is missing; run `python -m stellatrain_b200._build`")
        if build_if_missing:
            build_extension(name)
    loader = importlib.machinery.ExtensionFileLoader(full, str(so))
    spec = importlib.util.spec_from_file_location(full, str(so), loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules[full] = mod
    return mod


def build_selftest(sanitizer: str = "thread", out_dir: Path | None = None) -> Path:
    """Stand-alone exerciser of the CPU tier (``csrc/selftest/cpu_selftest.cpp``) linked with a sanitizer runtime:
    ``thread`` (TSAN), ``address`` (ASAN + UBSAN) or ``none``.  The reference has no such target."""
    out_dir = Path(out_dir) if out_dir is not None else OBJ_DIR
    out_dir.mkdir(parents=True, exist_ok=True)
    flags = {"thread": ["-fsanitize=thread"], "address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"],
             "none": []}[sanitizer]
    srcs = [s for s in EXTENSIONS["_Ccpu"]["cpp"] if not s.startswith("bindings")]
    srcs.append("selftest/cpu_selftest.cpp")
    exe = out_dir / f"cpu_selftest_{sanitizer}"
    base = [f for f in CXX_FLAGS if f not in ("-O3", "-fvisibility=hidden")] + ["-O1", "-g", "-fno-omit-frame-pointer"]
    objs, jobs = [], []
    for s in srcs:
        obj = out_dir / (f"selftest_{sanitizer}_" + s.replace("/", "_") + ".o")
        jobs.append(["g++", *base, *flags, f"-I{CSRC}", "-c", str(CSRC / s), "-o", str(obj)])
        objs.append(obj)
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        list(ex.map(_run, jobs))
    _run(["g++", *flags, "-o", str(exe), *map(str, objs), "-pthread", "-lrt", "-ldl"])
    return exe


def build_all(force: bool = False, verbose: bool = False) -> None:
    for name in EXTENSIONS:
        if _existing(name)["cu"] or _existing(name)["cpp"]:
            build_extension(name, force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for n in EXTENSIONS:
        print(n, so_path(n), "ok" if so_path(n).exists() else "absent")
