"""In-tree build of the native code: the collective library, the bundled minimal MPI, the torch
extension, the benchmark binaries and the C/C++ test programs.

Everything is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``).  Objects go
to ``build/`` at the repository root, products to ``nano_nccl_b200/lib``.  Builds are incremental:
a translation unit is rebuilt when its command line, its source or any header it included changed
(compiler-written dependency files).

The reference builds with CMake (reference CMakeLists.txt, src/CMakeLists.txt); targets map as:
``nano_nccl`` + ``nano_nccl_mpi`` + ``nano_nccl_mpi_c`` -> ``libnano_nccl.so`` (+ ``libminimpi.so``
when no MPI installation exists), benchmarks -> ``lib/nano_nccl_*_bench``, tests -> ``lib/tests/*``.
"""
from __future__ import annotations

import hashlib
import os
import shlex
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = ROOT / "build" / "obj"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
CXX = os.environ.get("CXX", "g++")
CC = os.environ.get("CC", "gcc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
INCLUDES = ["-I", str(CSRC), "-I", str(CSRC / "include")]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
                           "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function", "-diag-suppress", "177"] + INCLUDES
CXX_FLAGS = ["-O2", "-g1", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-DNANO_NCCL_ENABLE_RDMA_PROXY_TIMELINE",
             "-pthread", "-I", str(CUDA_HOME / "include")] + INCLUDES

# NANO_NCCL_BUILD_DEFINES: comma-separated macro names added to every compile line (e.g. the opt-in
# NANO_NCCL_ENABLE_BENCH_PROFILING of the native benchmarks).
EXTRA_DEFINES = ["-D" + d for d in os.environ.get("NANO_NCCL_BUILD_DEFINES", "").split(",") if d.strip()]
NVCC_FLAGS += EXTRA_DEFINES
CXX_FLAGS += EXTRA_DEFINES

_print_lock = threading.Lock()


def _log(msg: str, verbose: bool) -> None:
    if verbose:
        with _print_lock:
            print(msg, file=sys.stderr, flush=True)


def _run(cmd: list[str], verbose: bool) -> None:
    _log("  $ " + " ".join(shlex.quote(c) for c in cmd), verbose)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed (%d): %s\n%s\n%s" % (
            proc.returncode, " ".join(shlex.quote(c) for c in cmd), proc.stdout[-4000:], proc.stderr[-8000:]))
    if verbose and proc.stderr.strip():
        _log(proc.stderr.strip(), verbose)


def _deps_changed(dep_file: Path, target: Path) -> bool:
    if not dep_file.exists() or not target.exists():
        return True
    t = target.stat().st_mtime
    text = dep_file.read_text().replace("\\\n", " ")
    if ":" not in text:
        return True
    for dep in text.split(":", 1)[1].split():
        p = Path(dep)
        if not p.exists() or p.stat().st_mtime > t:
            return True
    return False


def compile_one(src: Path, extra: list[str], tag: str, verbose: bool, cxx: str | None = None) -> Path:
    """Compiles one translation unit; returns the object path."""
    rel = src.relative_to(CSRC)
    obj = OBJ / tag / rel.with_suffix(rel.suffix + ".o")
    dep = obj.with_suffix(".d")
    stamp = obj.with_suffix(".cmd")
    obj.parent.mkdir(parents=True, exist_ok=True)
    if src.suffix == ".cu":
        cmd = [NVCC] + NVCC_FLAGS + extra + ["-MD", "-MF", str(dep), "-c", str(src), "-o", str(obj)]
    elif src.suffix == ".c":
        cmd = [CC, "-O2", "-std=c11", "-fPIC", "-Wall", "-I", str(CUDA_HOME / "include")] + INCLUDES + extra + [
            "-MD", "-MF", str(dep), "-c", str(src), "-o", str(obj)]
    else:
        cmd = [cxx or CXX] + CXX_FLAGS + extra + ["-MD", "-MF", str(dep), "-c", str(src), "-o", str(obj)]
    digest = hashlib.sha1(" ".join(cmd).encode()).hexdigest()
    if stamp.exists() and stamp.read_text() == digest and not _deps_changed(dep, obj):
        return obj
    _run(cmd, verbose)
    stamp.write_text(digest)
    return obj


def _compile_many(sources: list[Path], extra: list[str], tag: str, verbose: bool, jobs: int, cxx: str | None = None) -> list[Path]:
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        return list(pool.map(lambda s: compile_one(s, extra, tag, verbose, cxx), sources))


def _link(objs: list[Path], out: Path, flags: list[str], verbose: bool, shared: bool) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    if out.exists() and all(o.stat().st_mtime <= out.stat().st_mtime for o in objs):
        stamp = out.with_suffix(out.suffix + ".cmd")
        digest = hashlib.sha1(" ".join(map(str, objs + flags)).encode()).hexdigest()
        if stamp.exists() and stamp.read_text() == digest:
            return
    cmd = [NVCC] + ARCH_FLAGS + (["-shared"] if shared else []) + ["-o", str(out)] + [str(o) for o in objs] + flags
    _run(cmd, verbose)
    out.with_suffix(out.suffix + ".cmd").write_text(
        hashlib.sha1(" ".join(map(str, objs + flags)).encode()).hexdigest())


CORE_DIRS = ["core", "bootstrap", "topology", "symm", "kernels", "collective", "transport", "capi", "gemm", "ops"]


def core_sources() -> list[Path]:
    out: list[Path] = []
    for d in CORE_DIRS:
        base = CSRC / d
        if base.exists():
            out += sorted(p for p in base.rglob("*") if p.suffix in (".cc", ".cu"))
    return out


def have_system_mpi() -> bool:
    return shutil.which("mpicxx") is not None and os.environ.get("NANO_NCCL_USE_SYSTEM_MPI", "0") == "1"


def build_core(verbose: bool = False, jobs: int | None = None) -> Path:
    """libminimpi.so (unless a system MPI is selected) and libnano_nccl.so."""
    jobs = jobs or max(1, (os.cpu_count() or 4))
    mpi_inc = ["-I", str(CSRC / "minimpi")]
    objs = _compile_many(core_sources(), mpi_inc, "core", verbose, jobs)
    link_flags = ["-ldl", "-lpthread", "-lrt"]
    mini = CSRC / "minimpi"
    if mini.exists() and any(mini.glob("*.cc")):
        mobjs = _compile_many(sorted(mini.glob("*.cc")), mpi_inc, "minimpi", verbose, jobs)
        objs += mobjs
    out = LIB / "libnano_nccl.so"
    _link(objs, out, link_flags, verbose, shared=True)
    build_mpi_c_alias(out, verbose)
    return out


def build_mpi_c_alias(core: Path, verbose: bool = False) -> Path:
    """libnano_nccl_mpi_c.so: the name of the reference's shared C library (src/CMakeLists.txt:87-95,
    target nano_nccl_mpi_c).  A library without code of its own that depends on libnano_nccl.so, so a
    program that was linked against the reference's library finds the whole C ABI and the MPI C ABI when the
    loader resolves the old name.  (`install` lays down a symbolic link instead, which also serves -l.)"""
    alias = LIB / "libnano_nccl_mpi_c.so"
    if alias.exists() and alias.stat().st_mtime >= core.stat().st_mtime:
        return alias
    _run([CXX, "-shared", "-fPIC", "-o", str(alias), "-Wl,-soname,libnano_nccl_mpi_c.so", "-Wl,--no-as-needed",
          "-L", str(LIB), "-lnano_nccl", "-Wl,-rpath,$ORIGIN"], verbose)
    return alias


def install(prefix: Path, verbose: bool = False) -> dict[str, Path]:
    """Copies the public headers, the libraries and the launcher under `prefix` (include/nano_nccl, lib, bin)
    and writes lib/cmake/nano_nccl/nano_ncclConfig.cmake with the imported targets nano_nccl::nano_nccl and
    nano_nccl::nano_nccl_mpi_c, the names a CMake consumer of the reference links (reference CMakeLists.txt,
    src/CMakeLists.txt:69-95)."""
    core = build_core(verbose)
    build_programs(verbose)
    prefix = Path(prefix)
    inc, lib, bindir = prefix / "include" / "nano_nccl", prefix / "lib", prefix / "bin"
    cmake = lib / "cmake" / "nano_nccl"
    for d in (inc, lib, bindir, cmake):
        d.mkdir(parents=True, exist_ok=True)
    for h in sorted((CSRC / "include" / "nano_nccl").glob("*.h")):
        shutil.copy2(h, inc / h.name)
    if (CSRC / "minimpi" / "mpi.h").exists() and not have_system_mpi():
        (prefix / "include" / "nano_nccl" / "minimpi").mkdir(exist_ok=True)
        shutil.copy2(CSRC / "minimpi" / "mpi.h", prefix / "include" / "nano_nccl" / "minimpi" / "mpi.h")
    shutil.copy2(core, lib / core.name)
    # Under the installed tree the old name is a symbolic link: the link editor follows it at build time and
    # the loader at run time.  (The in-tree alias is a dependency-only library, which serves the loader alone.)
    alias = lib / "libnano_nccl_mpi_c.so"
    if alias.exists() or alias.is_symlink():
        alias.unlink()
    alias.symlink_to(core.name)
    for exe in ("nano_nccl_mpirun", "nano_nccl_all_reduce_bench", "nano_nccl_collective_bench"):
        if (LIB / exe).exists():
            shutil.copy2(LIB / exe, bindir / exe)
    (cmake / "nano_ncclConfig.cmake").write_text(
        "# Imported targets of the installed library: nano_nccl::nano_nccl (C++ API, C ABI, MPI C ABI) and\n"
        "# nano_nccl::nano_nccl_mpi_c (the same entry points under the reference's library name).\n"
        "get_filename_component(_nano_prefix \"${CMAKE_CURRENT_LIST_DIR}/../../..\" ABSOLUTE)\n"
        "foreach(_t nano_nccl nano_nccl_mpi_c)\n"
        "  if(NOT TARGET nano_nccl::${_t})\n"
        "    add_library(nano_nccl::${_t} SHARED IMPORTED)\n"
        "    set_target_properties(nano_nccl::${_t} PROPERTIES\n"
        "      IMPORTED_LOCATION \"${_nano_prefix}/lib/lib${_t}.so\"\n"
        "      INTERFACE_INCLUDE_DIRECTORIES \"${_nano_prefix}/include\")\n"
        "  endif()\n"
        "endforeach()\n"
        "set(nano_nccl_FOUND TRUE)\n")
    return {"include": inc, "lib": lib, "bin": bindir, "cmake": cmake}


def build_programs(verbose: bool = False, jobs: int | None = None) -> list[Path]:
    """Benchmarks and native test programs; each source file with a main() is one executable."""
    jobs = jobs or max(1, (os.cpu_count() or 4))
    lib = build_core(verbose, jobs)
    outs: list[Path] = []
    groups = [("bench", LIB), ("tests", LIB / "tests"), ("examples", LIB / "examples")]
    mpi_inc = ["-I", str(CSRC / "minimpi")]
    for sub, dest in groups:
        base = CSRC / sub
        if not base.exists():
            continue
        sources = sorted(p for p in base.iterdir() if p.suffix in (".cc", ".cu", ".c"))
        objs = _compile_many(sources, mpi_inc, sub, verbose, jobs)
        for src, obj in zip(sources, objs):
            name = src.stem if sub != "bench" else "nano_nccl_" + src.stem
            exe = dest / name
            _link([obj], exe, ["-L", str(LIB), "-lnano_nccl", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN" if sub == "bench" else "$ORIGIN/..",
                               "-ldl", "-lpthread", "-lrt"], verbose, shared=False)
            outs.append(exe)
    return outs


SANITIZER_FLAGS = {"address": ["-fsanitize=address,undefined"], "thread": ["-fsanitize=thread"]}
# Host-only translation units (no kernels) and the native tests that need nothing else: the proxies, the bootstraps,
# the verbs providers, shared-memory regions, the CPU ring.
SANITIZED_DIRS = ["core", "bootstrap", "transport/socket", "transport/rdma", "transport/shm"]
SANITIZED_EXTRA = ["collective/host_ring.cc", "collective/signature.cc", "collective/tuner.cc"]
SANITIZED_TESTS = ["socket_protocol_test", "bootstrap_test", "rdma_proxy_test", "host_ring_test", "rdma_ibv_contract_test"]


def sanitizer_compiler(kind: str) -> str | None:
    """A C++ compiler that can link with the sanitizer's run-time library: $CXX if it can, else the system g++ / clang++;
    None when none of them can."""
    import tempfile

    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "probe.cc"
        src.write_text("int main() { return 0; }\n")
        for cxx in dict.fromkeys([CXX, "/usr/bin/g++", "g++", "clang++"]):
            if shutil.which(cxx) is None:
                continue
            if subprocess.run([cxx] + SANITIZER_FLAGS[kind] + [str(src), "-o", str(Path(tmp) / "probe")],
                              capture_output=True).returncode == 0:
                return cxx
    return None


def build_sanitized(kind: str, verbose: bool = False, jobs: int | None = None) -> list[Path]:
    """The host-side native tests rebuilt with AddressSanitizer + UndefinedBehaviorSanitizer (kind "address") or
    ThreadSanitizer (kind "thread"): sources compiled straight into the test programs, no shared library, no device
    code.  The stand-in for a GPU memory checker on the host side of the library (proxy threads, bootstraps, the
    verbs providers, the CPU ring); the reference has no sanitizer targets (its CMake files define none)."""
    jobs = jobs or max(1, (os.cpu_count() or 4))
    cxx = sanitizer_compiler(kind)
    if cxx is None:
        raise RuntimeError(f"no C++ compiler on this machine links with -fsanitize={kind}")
    flags = SANITIZER_FLAGS[kind] + ["-O1", "-fno-omit-frame-pointer", "-I", str(CSRC / "minimpi")]
    sources: list[Path] = []
    for d in SANITIZED_DIRS:
        sources += sorted((CSRC / d).glob("*.cc"))
    sources += [CSRC / rel for rel in SANITIZED_EXTRA]
    tag = "san_" + kind
    objs = _compile_many(sources, flags, tag, verbose, jobs, cxx=cxx)
    tests = [CSRC / "tests" / (name + ".cc") for name in SANITIZED_TESTS]
    test_objs = _compile_many(tests, flags, tag, verbose, jobs, cxx=cxx)
    outs = []
    for src, obj in zip(tests, test_objs):
        exe = LIB / "tests" / "san" / f"{src.stem}_{kind}"
        exe.parent.mkdir(parents=True, exist_ok=True)
        cmd = [cxx] + SANITIZER_FLAGS[kind] + ["-o", str(exe), str(obj)] + [str(o) for o in objs] + [
            "-L", str(CUDA_HOME / "lib64"), "-lcudart", "-ldl", "-lpthread", "-lrt", "-Wl,-rpath," + str(CUDA_HOME / "lib64")]
        if not exe.exists() or any(o.stat().st_mtime > exe.stat().st_mtime for o in objs + [obj]):
            _run(cmd, verbose)
        outs.append(exe)
    return outs


def torch_flags() -> tuple[list[str], list[str]]:
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = inc + ["-DTORCH_API_INCLUDE_EXTENSION_H", "-DTORCH_EXTENSION_NAME=_nano_torch",
                    f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DUSE_C10D_NCCL", "-Wno-deprecated-declarations"]
    torch_lib = str(Path(torch.__file__).parent / "lib")
    lflags = ["-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
              "-Xlinker", "-rpath", "-Xlinker", torch_lib]
    return cflags, lflags


def build_torch_extension(verbose: bool = False, jobs: int | None = None) -> Path | None:
    """_nano_torch.so: c10d backend + torch ops, linked against libnano_nccl.so."""
    base = CSRC / "torch"
    if not base.exists() or not any(base.glob("*.c*")):
        return None
    jobs = jobs or max(1, (os.cpu_count() or 4))
    lib = build_core(verbose, jobs)
    cflags, lflags = torch_flags()
    sources = sorted(p for p in base.iterdir() if p.suffix in (".cc", ".cu"))
    objs = _compile_many(sources, cflags, "torch", verbose, jobs)
    out = LIB / "_nano_torch.so"
    _link(objs, out, ["-L", str(LIB), "-lnano_nccl", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"] + lflags,
          verbose, shared=True)
    return out


def build_all(verbose: bool = False, with_torch: bool = True) -> dict[str, object]:
    out: dict[str, object] = {"core": build_core(verbose)}
    out["programs"] = build_programs(verbose)
    if with_torch:
        out["torch"] = build_torch_extension(verbose)
    return out


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        for exe in build_sanitized(sys.argv[sys.argv.index("--sanitize") + 1], verbose="-q" not in sys.argv):
            print("built", exe)
        sys.exit(0)
    if "--install" in sys.argv:
        where = install(Path(sys.argv[sys.argv.index("--install") + 1]), verbose="-q" not in sys.argv)
        for k, v in where.items():
            print("installed", k, "->", v)
        sys.exit(0)
    res = build_all(verbose="-q" not in sys.argv, with_torch="--no-torch" not in sys.argv)
    for k, v in res.items():
        print(k, "->", v)
