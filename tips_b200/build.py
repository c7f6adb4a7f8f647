"""In-tree build of the native libraries.

Two shared objects are produced next to this file, under ``tips_b200/lib``:

* ``libtips_core.so``    host C++17 runtime (logging, channel, threads, serializer,
  TCP RPC, bootstrap, collective engine, parameter-server host path, C API)
* ``libtips_kernels.so`` sm_100a CUDA kernels with ``extern "C"`` launchers

The reference builds one ``libtipscore.so`` with CMake and downloads its
third-party sources (CMakeLists.txt:38-81); here the toolchain is just g++ and
nvcc, there is nothing to download, and the result stays inside the package so
it travels with a copy of the repository.

Usage: ``python -m tips_b200.build [--force] [--core-only] [--sanitize=thread|address]``
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build"

CXX = os.environ.get("TIPS_CXX") or shutil.which("g++") or "g++"
NVCC = os.environ.get("TIPS_NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"

CORE_DIRS = ["core", "runtime", "collective", "ps"]
CORE_EXTRA = ["c_api.cc", "ps_c_api.cc"]
CXXFLAGS = ["-std=c++17", "-O2", "-g1", "-fPIC", "-Wall", "-Wno-sign-compare", "-pthread", f"-I{CSRC}"]
NVCCFLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", f"-I{CSRC}", "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _sources_core():
    out = []
    for d in CORE_DIRS:
        out += sorted((CSRC / d).glob("*.cc"))
    out += [CSRC / f for f in CORE_EXTRA if (CSRC / f).exists()]
    return out


def _sources_cuda():
    return sorted((CSRC / "kernels").glob("*.cu"))


def _stamp(src: Path, flags) -> str:
    h = hashlib.sha1()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    # headers: hash every header in csrc (cheap, a few dozen files)
    for hdr in sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(cmd, src, obj, stamp_file, stamp, log_file=None):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if log_file is not None:
        Path(log_file).write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    Path(stamp_file).write_text(stamp)
    return r.stderr


def _build_lib(name, sources, compiler, flags, link_cmd_tail, force, jobs):
    OBJ.mkdir(exist_ok=True)
    LIB.mkdir(exist_ok=True)
    objs, tasks = [], []
    with cf.ThreadPoolExecutor(max_workers=jobs) as pool:
        for src in sources:
            rel = src.relative_to(CSRC)
            obj = OBJ / (name + "_" + str(rel).replace("/", "_") + ".o")
            stamp_file = obj.with_suffix(".stamp")
            stamp = _stamp(src, flags)
            objs.append(obj)
            if (not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp):
                continue
            cmd = [compiler, *flags, "-c", str(src), "-o", str(obj)]
            log = obj.with_suffix(".log") if compiler == NVCC else None
            tasks.append(pool.submit(_compile, cmd, src, obj, stamp_file, stamp, log))
        for t in tasks:
            t.result()
    out = LIB / f"lib{name}.so"
    if tasks or not out.exists() or force:
        cmd = [compiler, "-shared", "-o", str(out), *map(str, objs), *link_cmd_tail]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    return out


def build_core(force=False, sanitize=None, jobs=None):
    flags = list(CXXFLAGS)
    tail = ["-pthread", "-ldl"]
    name = "tips_core"
    if sanitize:
        flags += [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer", "-O1"]
        tail += [f"-fsanitize={sanitize}"]
        name = f"tips_core_{sanitize}"
    return _build_lib(name, _sources_core(), CXX, flags, tail, force, jobs or os.cpu_count() or 4)


def build_kernels(force=False, jobs=None):
    srcs = _sources_cuda()
    if not srcs:
        return None
    if not Path(NVCC).exists():
        raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")
    tail = ["-Xcompiler", "-fPIC", "-lcudart", "-lcuda"]
    return _build_lib("tips_kernels", srcs, NVCC, NVCCFLAGS, tail, force, jobs or os.cpu_count() or 4)


def build_all(force=False):
    return build_core(force=force), build_kernels(force=force)


def build_native_tests(sanitize=None):
    """Compile csrc/tests/*.cc into executables under build/, linked against libtips_core.so or, with
    `sanitize` ("thread" / "address"), against that sanitizer build of the library (executables get the suffix)."""
    core = build_core(sanitize=sanitize)
    OBJ.mkdir(exist_ok=True)
    outs = []
    libname = "tips_core" + (f"_{sanitize}" if sanitize else "")
    extra = [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer"] if sanitize else []
    for src in sorted((CSRC / "tests").glob("*.cc")):
        exe = OBJ / (src.stem + (f"_{sanitize}" if sanitize else ""))
        if (not exe.exists() or exe.stat().st_mtime < max(src.stat().st_mtime, core.stat().st_mtime)):
            cmd = [CXX, "-std=c++17", "-O1", "-g1", "-pthread", *extra, f"-I{CSRC}", str(src), f"-L{LIB}",
                   f"-l{libname}", f"-Wl,-rpath,{LIB}", "-o", str(exe)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stderr}")
        outs.append(exe)
    return outs


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, from the nvcc logs of the last build."""
    lines = []
    for log in sorted(OBJ.glob("tips_kernels_*.log")):
        lines.append(f"== {log.name}")
        lines.append(log.read_text())
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--core-only", action="store_true")
    ap.add_argument("--sanitize", choices=["thread", "address"])
    ap.add_argument("--ptxas", action="store_true", help="print the ptxas resource report after building")
    a = ap.parse_args(argv)
    core = build_core(force=a.force, sanitize=a.sanitize)
    print("built", core)
    if not a.core_only and not a.sanitize:
        k = build_kernels(force=a.force)
        print("built", k)
        if a.ptxas:
            print(ptxas_report())


if __name__ == "__main__":
    main(sys.argv[1:])
