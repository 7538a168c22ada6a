"""Builds libgq.so — the CUDA backend behind include/gq.h — in-tree with nvcc
for sm_100a only. Run as ``python -m grilly2_b200.build`` (add ``-v`` for the
ptxas resource report)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "_lib", "libgq.so")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def stale() -> bool:
    if not os.path.exists(OUT):
        return True
    built = os.path.getmtime(OUT)
    deps = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    deps.append(os.path.join(ROOT, "include", "gq.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def _headers() -> list[str]:
    return [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))] + [os.path.join(ROOT, "include", "gq.h")]


def build(force: bool = False, verbose: bool = False) -> str:
    """Each source is compiled to an object of its own (in parallel, and only when it or a header is newer), then linked."""
    if not force and not stale():
        return OUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libgq.so cannot be built (there is no CPU fallback)")
    obj_dir = os.path.join(HERE, "_lib", "obj")
    os.makedirs(obj_dir, exist_ok=True)
    common = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-ccbin", "g++", f"-I{os.path.join(ROOT, 'include')}",
              f"-I{CSRC}", "-DGQ_BUILD", "-I/usr/include"]
    if verbose:
        common.insert(1, "-Xptxas=-v")
    newest_header = max(os.path.getmtime(h) for h in _headers())
    jobs, objects = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), newest_header):
            jobs.append(common + ["-c", src, "-o", obj])
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=min(8, max(len(jobs), 1))) as pool:
        for done in pool.map(lambda c: subprocess.run(c, capture_output=not verbose, text=True), jobs):
            if done.returncode != 0:
                raise RuntimeError(f"nvcc failed: {' '.join(done.args)}\n{done.stdout or ''}{done.stderr or ''}")
            if verbose and done.stderr:
                sys.stderr.write(done.stderr)
    subprocess.run([nvcc, "-shared", "-ccbin", "g++", "-o", OUT] + objects + ["-ldl"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv))
