"""In-tree native build: compiles every CUDA / C++ source of the framework into shared libraries and tools under
``umdk_b200/_lib``. CUDA sources are compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``).

Usage: ``python -m umdk_b200._build [--force] [--verbose]`` or :func:`build_all` from Python.
The reference project builds with CMake/Bazel plus CANN scripts (build/cam/build.sh); here one dependency-free
driver does the same job so that the libraries sit next to the Python package that loads them.
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

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIB = Path(__file__).resolve().parent / "_lib"
OBJ = ROOT / "build" / "obj"

NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread", "-fvisibility=hidden"]


def _targets():
    """name -> dict(kind, sources, includes, libs, out)."""
    t = {}
    cam = sorted((CSRC / "cam").glob("*.cu")) + sorted((CSRC / "cam").glob("*.cpp"))
    t["umdk_cam"] = dict(kind="cuda_shared", sources=cam, includes=[CSRC / "cam", CSRC / "common"],
                         libs=["-lcudart", "-lpthread", "-ldl", "-lrt"], out=LIB / "libumdk_cam.so")
    for name, dirs, deps in [
        ("umdk_urma", ["common", "urma"], []),
        ("umdk_umq", ["umq"], ["umdk_urma"]),
        ("umdk_urpc", ["urpc"], ["umdk_umq", "umdk_urma"]),
        ("umdk_dlock", ["dlock"], ["umdk_urma"]),
        ("umdk_usock", ["usock"], ["umdk_urma"]),
    ]:
        srcs = []
        for d in dirs:
            srcs += sorted((CSRC / d).glob("*.cpp"))
        srcs = [s for s in srcs if not s.name.endswith("_preload.cpp")]
        if not srcs:
            continue
        t[name] = dict(kind="cxx_shared", sources=srcs,
                       includes=[CSRC / "common", CSRC / "urma", CSRC / "umq", CSRC / "urpc", CSRC / "dlock",
                                 CSRC / "usock"],
                       libs=["-L" + str(LIB), "-Wl,-rpath,$ORIGIN"] + ["-l" + d for d in deps] +
                            (["-lssl", "-lcrypto"] if name == "umdk_urma" else []) + ["-lpthread", "-ldl", "-lrt"],
                       deps=deps, out=LIB / f"lib{name}.so")
    cu_prov = sorted((CSRC / "urma_cuda").glob("*.cu"))
    if cu_prov and "umdk_urma" in t:
        # URMA provider plug-in for GPU memory: found by urma_init in <lib dir>/urma/liburma-*.so
        t["urma_cuda_ipc"] = dict(kind="cuda_shared", sources=cu_prov, includes=[CSRC / "urma", CSRC / "common"],
                                  libs=["-lcudart", "-L" + str(LIB), "-Xlinker", "-rpath=$ORIGIN/..", "-lumdk_urma",
                                        "-lpthread"], deps=["umdk_urma"], out=LIB / "urma" / "liburma-cuda-ipc.so")
    # operator library for torch (schemas + Meta shape functions + Autograd registration): needs torch's headers
    tx = sorted((CSRC / "torch_ext").glob("*.cpp"))
    if tx:
        try:
            import torch
            from torch.utils import cpp_extension as _ce
            tinc = [Path(p) for p in _ce.include_paths()]
            tlib = Path(torch.__file__).resolve().parent / "lib"
            t["umdk_cam_torch"] = dict(
                kind="cxx_shared", sources=tx, includes=tinc,
                cxxflags=["-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI), "-Wno-attributes"],
                libs=["-L" + str(tlib), "-Wl,-rpath," + str(tlib), "-ltorch", "-ltorch_cpu", "-lc10"],
                out=LIB / "libumdk_cam_torch.so")
        except Exception:   # no torch in this interpreter: the Python package then registers the schemas itself
            pass
    pre = CSRC / "usock" / "ums_preload.cpp"
    if pre.exists():
        t["ums_preload"] = dict(kind="cxx_shared", sources=[pre], includes=[CSRC / "usock", CSRC / "common"],
                                libs=["-L" + str(LIB), "-Wl,-rpath,$ORIGIN", "-lumdk_usock", "-ldl", "-lpthread",
                                      "-lrt"], deps=["umdk_usock"], out=LIB / "libums_preload.so")
    have = [n for n in ("umdk_urpc", "umdk_umq", "umdk_dlock", "umdk_usock", "umdk_urma") if n in t]
    for tool in sorted((CSRC / "tools").glob("*.cpp")):
        t["tool_" + tool.stem] = dict(
            kind="cxx_exe", sources=[tool],
            includes=[CSRC / "common", CSRC / "urma", CSRC / "umq", CSRC / "urpc", CSRC / "dlock", CSRC / "usock"],
            libs=["-L" + str(LIB), "-Wl,-rpath,$ORIGIN/.."] + ["-l" + n for n in have] + ["-lpthread", "-ldl", "-lrt"],
            deps=have, out=LIB / "bin" / tool.stem)
    return t


def _headers_digest(includes) -> str:
    h = hashlib.sha1()
    for inc in includes:
        for p in sorted(Path(inc).glob("*.h")) + sorted(Path(inc).glob("*.cuh")) + sorted(Path(inc).glob("*.hpp")):
            st = p.stat()
            h.update(f"{p}:{st.st_mtime_ns}:{st.st_size}".encode())
    return h.hexdigest()


def _run(cmd, verbose, log_path=None):
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path is not None:
        Path(log_path).write_text(" ".join(map(str, cmd)) + "\n" + p.stdout)
    if p.returncode != 0:
        raise RuntimeError("build command failed:\n" + " ".join(map(str, cmd)) + "\n" + p.stdout)
    if verbose and p.stdout.strip():
        print(p.stdout)
    return p.stdout


def _compile_one(src: Path, tgt: dict, force: bool, verbose: bool, hdr_digest: str) -> Path:
    obj = OBJ / (src.parent.name + "_" + src.stem + ".o")
    stamp = obj.with_suffix(".stamp")
    key = f"{src.stat().st_mtime_ns}:{src.stat().st_size}:{hdr_digest}"
    if not force and obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj
    inc = []
    for i in tgt["includes"]:
        inc += ["-I", str(i)]
    if src.suffix == ".cu":
        cmd = [NVCC, *NVCC_FLAGS, *inc, "-c", str(src), "-o", str(obj)]
    elif tgt["kind"] == "cuda_shared":
        cmd = [NVCC, "-O2", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden", *inc, "-c", str(src), "-o",
               str(obj)]
    else:
        cmd = [CXX, *CXX_FLAGS, *tgt.get("cxxflags", []), *inc, "-c", str(src), "-o", str(obj)]
    _run(cmd, verbose, log_path=obj.with_suffix(".log"))
    stamp.write_text(key)
    return obj


def build_all(force: bool = False, verbose: bool = False, only=None) -> dict:
    """Builds all targets (or those whose names are in ``only``); returns name -> output path."""
    LIB.mkdir(parents=True, exist_ok=True)
    (LIB / "bin").mkdir(parents=True, exist_ok=True)
    (LIB / "urma").mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    targets = _targets()
    order = ["umdk_cam", "umdk_urma", "urma_cuda_ipc", "umdk_umq", "umdk_usock", "umdk_dlock", "umdk_urpc",
             "ums_preload", "umdk_cam_torch"]
    order += [n for n in targets if n.startswith("tool_")]
    outs = {}
    # compile all objects of all targets in parallel first
    jobs = {}
    with cf.ThreadPoolExecutor(max_workers=max(2, (os.cpu_count() or 4))) as ex:
        for name in order:
            if name not in targets or (only and name not in only):
                continue
            tgt = targets[name]
            dig = _headers_digest(tgt["includes"])
            jobs[name] = [ex.submit(_compile_one, s, tgt, force, verbose, dig) for s in tgt["sources"]]
        objs = {name: [f.result() for f in fs] for name, fs in jobs.items()}
    for name in order:
        if name not in objs:
            continue
        tgt = targets[name]
        out = tgt["out"]
        newest = max(o.stat().st_mtime_ns for o in objs[name])
        if force or not out.exists() or out.stat().st_mtime_ns < newest:
            if tgt["kind"] == "cuda_shared":
                cmd = [NVCC, "-shared", "-o", str(out), *map(str, objs[name]), *tgt["libs"]]
            elif tgt["kind"] == "cxx_shared":
                cmd = [CXX, "-shared", "-o", str(out), *map(str, objs[name]), *tgt["libs"], *LINK_EXTRA]
            else:
                cmd = [CXX, "-o", str(out), *map(str, objs[name]), *tgt["libs"], *LINK_EXTRA]
            _run(cmd, verbose)
        outs[name] = out
    return outs


LINK_EXTRA: list = []


HOST_LIBS = ("umdk_urma", "umdk_umq", "umdk_urpc", "umdk_dlock", "umdk_usock")


def build_sanitized(kind: str = "address", only=HOST_LIBS + ("tool_umq_perftest", "tool_urpc_perftest")) -> dict:
    """Host libraries and tools compiled with -fsanitize=<kind> ('address', 'thread' or 'undefined') into
    build/lib_<kind>/ (objects in build/obj_<kind>/), leaving the normal build untouched. The counterpart of the
    reference's asan / tsan build flavours (src/urma/.bazelrc:39-50, umdk.spec:2-8). CUDA targets are not built."""
    global LIB, OBJ, CXX_FLAGS, LINK_EXTRA, CXX
    assert kind in ("address", "thread", "undefined")
    saved = (LIB, OBJ, CXX_FLAGS, LINK_EXTRA)
    saved_cxx = CXX
    # the distribution compiler carries the sanitizer runtimes; a toolchain named by $CXX may not
    CXX = os.environ.get("UMDK_SANITIZER_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else CXX)
    LIB = ROOT / "build" / f"lib_{kind}"
    OBJ = ROOT / "build" / f"obj_{kind}"
    CXX_FLAGS = [f for f in CXX_FLAGS if f != "-O2"] + ["-O1", f"-fsanitize={kind}", "-fno-omit-frame-pointer"]
    # the static runtime goes into the executables (this image ships no shared sanitizer runtimes)
    LINK_EXTRA = [f"-fsanitize={kind}", {"address": "-static-libasan", "thread": "-static-libtsan",
                                          "undefined": "-static-libubsan"}[kind]]
    try:
        names = [n for n in only if not n.startswith("umdk_cam") and n != "urma_cuda_ipc"]
        if any(n.startswith("tool_") for n in names):   # the tools link every host library
            names = list(dict.fromkeys(list(HOST_LIBS) + names))
        return build_all(only=names)
    finally:
        LIB, OBJ, CXX_FLAGS, LINK_EXTRA = saved
        CXX = saved_cxx


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of the last CUDA compile (registers, spills, shared memory)."""
    parts = []
    for log in sorted(OBJ.glob("cam_*.log")):
        parts.append(f"== {log.name}\n{log.read_text()}")
    return "\n".join(parts)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--only", nargs="*")
    ap.add_argument("--sanitize", choices=["address", "thread", "undefined"],
                    help="build the host libraries / tools named by --only with this sanitizer into build/lib_<kind>")
    a = ap.parse_args(argv)
    if a.sanitize:
        outs = build_sanitized(a.sanitize, *([tuple(a.only)] if a.only else []))
    else:
        outs = build_all(a.force, a.verbose, a.only)
    for k, v in outs.items():
        print(f"{k}: {v}")


if __name__ == "__main__":
    main(sys.argv[1:])
