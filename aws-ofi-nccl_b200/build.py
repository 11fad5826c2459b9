"""In-tree native build: nvcc for the sm_100a kernels, g++ for the host plugin libraries.

Everything lands in ``aws-ofi-nccl_b200/lib/`` so the shared objects travel with the source tree
(no JIT cache, no site-packages install).  ``python -m aws_ofi_nccl_b200.build`` rebuilds what is
stale; ``build_all(force=True)`` rebuilds everything.

Targets
  libb200ops.so            CUDA kernels (GEMM, collectives, GIN device API users, model ops)
  libnccl-net-ofi-b200.so  ncclNet / ncclTuner / GIN / RMA plugin (also installed under the
                           names NCCL searches for: libnccl-net.so, libnccl-tuner-ofi-b200.so)
  unit test executables    csrc/tests/*.cpp -> lib/tests/<name>
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = ROOT / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
# Sanitizer builds need a compiler that ships the sanitizer runtimes (the default one may not).
SAN_CXX = os.environ.get("SAN_CXX", "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else CXX)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-I", str(CSRC / "include"), "-I", str(CSRC / "kernels"),
]
CXX_FLAGS = [
    "-std=c++20", "-O2", "-g", "-fPIC", "-fno-rtti", "-Wall", "-Wextra", "-Wno-unused-parameter",
    "-pthread", "-I", str(CSRC / "include"), "-I", f"{CUDA_HOME}/include",
]


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _run(cmd: list[str]) -> None:
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} ... {cmd[-1]}")


def _headers() -> list[Path]:
    return [p for p in CSRC.rglob("*") if p.suffix in (".h", ".cuh", ".hpp")]


def _compile_many(jobs: list[tuple[list[str], Path]]) -> None:
    if not jobs:
        return
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        futs = [ex.submit(_run, cmd) for cmd, _ in jobs]
        for f in futs:
            f.result()


def build_kernels(force: bool = False, extra_flags: list[str] | None = None) -> Path:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a and link libb200ops.so."""
    LIB.mkdir(exist_ok=True)
    (OBJ / "kernels").mkdir(parents=True, exist_ok=True)
    hdrs = _headers()
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    out = LIB / "libb200ops.so"
    if not force and not extra_flags and not _stale(out, srcs + hdrs):
        return out   # the library is newer than every source: nothing to do, even without the object files
    objs, jobs = [], []
    for s in srcs:
        o = OBJ / "kernels" / (s.stem + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append(([NVCC, *NVCC_FLAGS, *(extra_flags or []), "-c", str(s), "-o", str(o)], o))
    _compile_many(jobs)
    if force or jobs or not out.exists():
        _run([NVCC, "-shared", "-o", str(out), *map(str, objs), "-cudart", "static",
              "-gencode", "arch=compute_100a,code=sm_100a"])
    return out


def _host_sources() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*.cpp") if "tests" not in p.parts and "kernels" not in p.parts)


def _embed_net_kernels(force: bool = False) -> Path:
    """csrc/device/net_kernels.cu -> sm_100a cubin -> a byte list the plugin compiles in
    (the plugin loads it with cuModuleLoadData; it links no CUDA library)."""
    gen = OBJ / "gen"
    gen.mkdir(parents=True, exist_ok=True)
    src = CSRC / "device" / "net_kernels.cu"
    cubin, inc = gen / "net_kernels.cubin", gen / "net_kernels_cubin.inc"
    if force or _stale(inc, [src, CSRC / "include" / "b200net" / "net_kernel_args.h"]):
        try:
            _run([NVCC, "-cubin", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
                  "-I", str(CSRC / "include"), str(src), "-o", str(cubin)])
            data = cubin.read_bytes()
        except OSError:
            data = b"\0"   # no nvcc: the plugin then reports the kernels as unavailable and uses the copy engine
                           # (a compile error is a build failure, not a reason to ship without the kernels)
        inc.write_text(",".join(str(b) for b in data) + "\n")
    return gen


def build_host(force: bool = False, sanitize: str | None = None) -> Path | None:
    """Compile the host plugin (C++20) and link the NCCL-loadable shared objects."""
    srcs = _host_sources()
    if not srcs:
        return None
    LIB.mkdir(exist_ok=True)
    tag = f"host-{sanitize}" if sanitize else "host"
    (OBJ / tag).mkdir(parents=True, exist_ok=True)
    hdrs = _headers()
    if not sanitize and not force:
        fresh = LIB / "libnccl-net-ofi-b200.so"
        deps = srcs + hdrs + [CSRC / "device" / "net_kernels.cu"]
        if not _stale(fresh, deps) and not _stale(LIB / "libinternal_plugin.a", deps) and all(
                (LIB / a).exists() for a in ("libnccl-net.so", "libnccl-tuner-ofi-b200.so", "libnccl-net-b200.so")):
            return fresh   # newer than every source: nothing to do, even without the object files
    gen = _embed_net_kernels(force)
    hdrs = hdrs + [gen / "net_kernels_cubin.inc"]   # the kernel image is compiled into device/net_kernels.cpp
    flags = list(CXX_FLAGS) + ["-I", str(gen)]
    if sanitize:
        flags += [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer"]
    objs, jobs = [], []
    for s in srcs:
        o = OBJ / tag / ("_".join(s.relative_to(CSRC).with_suffix("").parts) + ".o")
        objs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append(([SAN_CXX if sanitize else CXX, *flags, "-c", str(s), "-o", str(o)], o))
    _compile_many(jobs)
    # sanitizer builds stay under build/ (large, and of no use on a GPU box)
    outdir = LIB if not sanitize else OBJ / "san"
    outdir.mkdir(parents=True, exist_ok=True)
    name = "libnccl-net-ofi-b200.so" if not sanitize else f"libnccl-net-ofi-b200-{sanitize}.so"
    out = outdir / name
    if force or jobs or not out.exists():
        link = [SAN_CXX if sanitize else CXX, "-shared", "-o", str(out), *map(str, objs), "-pthread", "-ldl", "-lrt",
                "-Wl,-Bsymbolic", "-Wl,--no-undefined"]
        if sanitize:
            link = [x for x in link if x != "-Wl,--no-undefined"] + [f"-fsanitize={sanitize}"]
        _run(link)
        if not sanitize:
            for alias in ("libnccl-net.so", "libnccl-tuner-ofi-b200.so", "libnccl-net-b200.so"):
                shutil.copyfile(out, LIB / alias)
    # static archive for unit tests that reach internals
    ar = outdir / ("libinternal_plugin.a" if not sanitize else f"libinternal_plugin-{sanitize}.a")
    if force or jobs or not ar.exists():
        if ar.exists():
            ar.unlink()
        _run(["ar", "rcs", str(ar), *map(str, objs)])
    return out


def build_tests(force: bool = False, sanitize: str | None = None) -> list[Path]:
    """Each csrc/tests/<name>.cpp (or .c) is a program that reports its result through its exit status."""
    tdir = CSRC / "tests"
    if not tdir.exists():
        return []
    base = LIB if not sanitize else OBJ / "san"
    outdir = base / ("tests" if not sanitize else f"tests-{sanitize}")
    outdir.mkdir(parents=True, exist_ok=True)
    ar = base / ("libinternal_plugin.a" if not sanitize else f"libinternal_plugin-{sanitize}.a")
    hdrs = _headers()
    jobs, outs = [], []
    for s in sorted(list(tdir.glob("*.cpp")) + list(tdir.glob("*.c"))):
        o = outdir / s.stem
        outs.append(o)
        if not (force or _stale(o, [s, ar] + hdrs)):
            continue
        if s.suffix == ".c":
            jobs.append((["gcc", "-O1", "-g", "-Wall", str(s), "-o", str(o), "-ldl"], o))
        else:
            flags = list(CXX_FLAGS)
            if sanitize:
                flags += [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer"]
            jobs.append(([SAN_CXX if sanitize else CXX, *flags, str(s), str(ar), "-o", str(o), "-pthread", "-ldl", "-lrt"], o))
    _compile_many(jobs)
    return outs


def build_cuda_tests(force: bool = False) -> list[Path]:
    """csrc/tests/<name>.cu: GPU test programs that use the device API (nvcc, sm_100a)."""
    tdir = CSRC / "tests"
    outdir = LIB / "tests"
    outdir.mkdir(parents=True, exist_ok=True)
    hdrs = _headers()
    jobs, outs = [], []
    for s in sorted(tdir.glob("*.cu")):
        o = outdir / s.stem
        outs.append(o)
        if force or _stale(o, [s] + hdrs):
            jobs.append(([NVCC, *NVCC_FLAGS, "-cudart", "static", str(s), "-o", str(o), "-ldl"], o))
    _compile_many(jobs)
    return outs


def build_fake_cuda(force: bool = False, sanitize: str | None = None) -> Path:
    """The stand-in driver for CPU tests of the device-buffer paths: lib/tests/fake_cuda/libcuda.so.1
    (with `sanitize`, an instrumented copy under build/san, so that a race detector sees the
    release / acquire pairs between its "kernels" and the plugin)."""
    src = CSRC / "tests" / "fake_cuda" / "fake_libcuda.cpp"
    outdir = LIB / "tests" / "fake_cuda" if not sanitize else OBJ / "san" / f"fake_cuda-{sanitize}"
    outdir.mkdir(parents=True, exist_ok=True)
    out = outdir / "libcuda.so.1"
    if force or _stale(out, [src, CSRC / "include" / "b200net" / "net_kernel_args.h"]):
        extra = [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer"] if sanitize else []
        _run([SAN_CXX if sanitize else CXX, "-std=c++20", "-O1", "-g", "-fPIC", "-shared", *extra, "-I", f"{CUDA_HOME}/include",
              "-I", str(CSRC / "include"),
              str(src), "-o", str(out), "-pthread", "-lrt"])
    return out


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_host(force)
    build_tests(force)
    build_cuda_tests(force)
    build_fake_cuda(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", sorted(p.name for p in LIB.glob("*.so")))
