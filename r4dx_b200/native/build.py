"""Builds the two in-tree native libraries.

``libr4dxb_host.so``  plain C++17 (container, quantizers, sampler, planners); needs no CUDA.
``libr4dxb_cuda.so``  every sm_100a kernel, compiled by nvcc with
                      ``-gencode arch=compute_100a,code=sm_100a``.

Both expose a plain C ABI (raw pointers + a stream handle) and are loaded with ctypes, so no
torch header is compiled and a full rebuild takes well under a minute.  Objects are cached by
a hash of the source, the headers and the flags.

Run ``python -m r4dx_b200.native.build`` (add ``--force`` to ignore the cache, ``--verbose`` to
print ptxas register/spill figures).
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC_CUDA = HERE / "src" / "cuda"
SRC_HOST = HERE / "src" / "host"
INCLUDE = HERE / "include"
LIB = HERE / "lib"
OBJ = HERE / "build"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", shutil.which("g++") or "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "-Xptxas", "-v",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-Xcompiler", "-fPIC",
    "-I", str(INCLUDE), "-I", str(SRC_CUDA),
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-march=x86-64-v3", "-pthread", "-fno-math-errno",
             "-I", str(INCLUDE), "-I", str(SRC_HOST)]


def _hash(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(str(p.name).encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _headers():
    hs = list(INCLUDE.glob("*.h")) + list(SRC_CUDA.glob("*.cuh")) + list(SRC_CUDA.glob("*.h"))
    hs += list(SRC_HOST.glob("*.h")) + list(SRC_HOST.glob("*.hpp"))
    return hs


def _compile_one(src: Path, cuda: bool, verbose: bool, force: bool):
    OBJ.mkdir(exist_ok=True)
    flags = NVCC_FLAGS if cuda else CXX_FLAGS
    key = _hash([src] + _headers(), " ".join(flags))
    obj = OBJ / f"{src.stem}.{key}.o"
    if obj.exists() and not force:
        return obj, ""
    for old in OBJ.glob(f"{src.stem}.*.o"):
        old.unlink()
    for old in OBJ.glob(f"{src.stem}.*.ptxas"):
        old.unlink()
    if cuda:
        cmd = [NVCC] + flags + ["-c", str(src), "-o", str(obj)]
    else:
        cmd = [CXX] + flags + ["-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if cuda:
        obj.with_suffix(".ptxas").write_text(r.stderr)      # registers / spills / shared memory of every kernel
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False, cuda: bool = True, host: bool = True) -> dict:
    """Compile what changed and link the shared libraries; returns their paths."""
    LIB.mkdir(exist_ok=True)
    out = {}
    jobs = []
    if host:
        jobs += [(p, False) for p in sorted(SRC_HOST.glob("*.cpp"))]
    if cuda:
        jobs += [(p, True) for p in sorted(SRC_CUDA.glob("*.cu"))]
    objs = {True: [], False: []}
    logs = []
    with cf.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        futs = {ex.submit(_compile_one, p, c, verbose, force): (p, c) for p, c in jobs}
        for f in cf.as_completed(futs):
            p, c = futs[f]
            obj, log = f.result()
            objs[c].append(obj)
            if log and verbose:
                logs.append(f"== {p.name}\n{log}")
    if host and objs[False]:
        so = LIB / "libr4dxb_host.so"
        stamp = _hash(objs[False], "host")
        if force or not so.exists() or _read_stamp(so) != stamp:
            cmd = [CXX, "-shared", "-pthread", "-o", str(so)] + [str(o) for o in sorted(objs[False])]
            subprocess.run(cmd, check=True)
            _write_stamp(so, stamp)
        out["host"] = so
    if cuda and objs[True]:
        so = LIB / "libr4dxb_cuda.so"
        stamp = _hash(objs[True], "cuda")
        if force or not so.exists() or _read_stamp(so) != stamp:
            cmd = [NVCC, "-shared", "-o", str(so)] + [str(o) for o in sorted(objs[True])] + [
                "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
            subprocess.run(cmd, check=True)
            _write_stamp(so, stamp)
        out["cuda"] = so
    if verbose:
        print("\n".join(logs))
    return out


# ---- resource gate: what ptxas reported for every kernel (registers, spills), kept beside the objects ----------
SPILL_LIMIT_BYTES = 128         # a handful of spilled bytes in a cold path is tolerated, a spilling inner loop is not
SPILL_ALLOW = ()                # mangled-name substrings exempt from the limit (none at present)


def resource_report() -> list:
    """[(source, kernel, registers, spill_store_bytes, spill_load_bytes)] parsed from the cached ptxas logs."""
    import re
    rows = []
    for log in sorted(OBJ.glob("*.ptxas")):
        text = log.read_text()
        for m in re.finditer(r"Function properties for (\S+)\s+\d+ bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads"
                             r"\s+ptxas info\s*: Used (\d+) registers", text):
            rows.append((log.name.split(".")[0], m.group(1), int(m.group(4)), int(m.group(2)), int(m.group(3))))
    return rows


def check_resources(limit: int = SPILL_LIMIT_BYTES) -> list:
    """Raises if a kernel spills more than ``limit`` bytes; returns the report (reference: the reference build gates
    its kernels on register and scratch use in CI, tools/check_kernel_resources.py:1-60)."""
    rows = resource_report()
    bad = [r for r in rows if max(r[3], r[4]) > limit and not any(a in r[1] for a in SPILL_ALLOW)]
    if bad:
        raise RuntimeError("kernels over the spill limit: " + "; ".join(f"{s}:{k} stores {a} loads {b}" for s, k, _, a, b in bad))
    return rows


def _read_stamp(so: Path) -> str:
    s = so.with_suffix(".stamp")
    return s.read_text() if s.exists() else ""


def _write_stamp(so: Path, stamp: str) -> None:
    so.with_suffix(".stamp").write_text(stamp)


if __name__ == "__main__":
    res = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    for k, v in res.items():
        print(k, v)
    if "--gate" in sys.argv:
        rep = check_resources()
        worst = sorted(rep, key=lambda r: -r[2])[:5]
        print(f"resource gate: {len(rep)} kernels, none over {SPILL_LIMIT_BYTES} spilled bytes; most registers: "
              + ", ".join(f"{s}:{r}" for s, _, r, _, _ in worst))
