"""Build the native library: every ``.cu``/``.cpp`` in this directory → ``jaxpp_b200/_native/libjaxpp_b200.so``.

Plain ``nvcc`` invocations (no torch headers: the library has a C ABI and is loaded with ctypes), all for
``sm_100a``; object files are rebuilt only when their source or a header is newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(os.path.dirname(HERE), "_native")
LIB = os.path.join(OUT_DIR, "libjaxpp_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nccl_paths():
    try:
        import nvidia.nccl as n

        root = os.path.dirname(n.__file__) if getattr(n, "__file__", None) else list(n.__path__)[0]
        return os.path.join(root, "include"), os.path.join(root, "lib")
    except Exception:
        return None, None


STAMP = os.path.join(OUT_DIR, "libjaxpp_b200.stamp")


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cu", ".cpp")))


def source_hash() -> str:
    """Hash of everything the library is built from; written next to the library after a successful link so
    that a loader can tell a stale binary from a current one."""
    import hashlib

    h = hashlib.sha256()
    for f in sorted(os.listdir(HERE)):
        if f.endswith((".cu", ".cpp", ".cuh", ".h", ".hpp")):
            h.update(f.encode())
            with open(os.path.join(HERE, f), "rb") as fh:
                h.update(fh.read())
    return h.hexdigest()


def is_current() -> bool:
    try:
        with open(STAMP) as f:
            return os.path.exists(LIB) and f.read().strip() == source_hash()
    except OSError:
        return False


def build(verbose: bool = False, force: bool = False) -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(OUT_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h", ".hpp"))]
    newest_header = max([os.path.getmtime(h) for h in headers] + [os.path.getmtime(__file__)])
    inc, libdir = _nccl_paths()
    extra = ["-I" + inc] if inc else []
    jobs = []
    objs = []
    for src in sources():
        obj = os.path.join(obj_dir, src.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        path = os.path.join(HERE, src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), newest_header):
            continue
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-x", "cu", "-c", path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        jobs.append((src, cmd))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            results = list(pool.map(lambda j: (j[0], subprocess.run(j[1], capture_output=True, text=True)), jobs))
        for src, res in results:
            if verbose or res.returncode != 0:
                sys.stderr.write(f"--- {src}\n{res.stdout}{res.stderr}\n")
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}")
    if jobs or not os.path.exists(LIB):
        link = [nvcc, "-shared", "-o", LIB, *objs, "-lcudart", "-ldl"]
        res = subprocess.run(link, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    with open(STAMP, "w") as f:
        f.write(source_hash())
    return LIB


def ensure_current() -> str:
    """Build if the library is missing or older than its sources; safe to call from several processes."""
    import fcntl

    if is_current():
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    with open(os.path.join(OUT_DIR, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not is_current():
                build()
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
