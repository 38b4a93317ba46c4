"""Compile the CUDA kernels and the C++ control library in-tree, on demand.

Each ``.cu`` file under ``csrc/kernels`` becomes one shared library, compiled
with ``nvcc -gencode arch=compute_100a,code=sm_100a`` the first time one of its
launchers is called (nvcc cross-compiles, so this works on a machine without a
GPU), and the pybind11 module of ``csrc/control`` is compiled with ``g++``.  The
file name of a built library carries a hash of its sources and flags, so an
edited source is rebuilt and an unchanged one is loaded as it is.  Libraries go
to ``einf_b200/_build`` when that is writable, else to a per-user folder under
the system's temporary directory.

The reference builds its 33 sources with ``torch.utils.cpp_extension.load``
(``src/einf/executors/torch/ops/loader.py:37-123``); here nothing includes
torch headers, which keeps a cold build to seconds.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent.parent
KERNEL_DIR = PACKAGE_DIR / "csrc" / "kernels"
CONTROL_DIR = PACKAGE_DIR / "csrc" / "control"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden"]


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[einf_b200 build] {message}", file=sys.stderr, flush=True)


def build_dir() -> Path:
    override = os.environ.get("EINF_B200_BUILD_DIR")
    candidates = [Path(override)] if override else []
    candidates.append(PACKAGE_DIR / "_build")
    candidates.append(Path(tempfile.gettempdir()) / f"einf_b200_build_{os.getuid()}")
    for candidate in candidates:
        try:
            candidate.mkdir(parents=True, exist_ok=True)
            probe = candidate / f".probe_{os.getpid()}_{threading.get_ident()}"
            probe.write_text("")
            probe.unlink()
            return candidate
        except OSError:
            continue
    raise BuildError("no writable folder for built libraries; set EINF_B200_BUILD_DIR")


def _find_nvcc() -> str:
    for candidate in (
        os.environ.get("NVCC"),
        shutil.which("nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if candidate and Path(candidate).is_file():
            return candidate
    raise BuildError("nvcc not found: the CUDA kernels cannot be compiled (set NVCC)")


def _digest(sources: list[Path], flags: list[str]) -> str:
    """Sources, headers and flags; not the include folders, which say where the checkout lies and
    would give a library built in one place another name in a copy of the tree."""
    h = hashlib.sha256()
    for part in flags:
        if part.startswith("-I"):
            continue
        h.update(part.encode())
    for source in sources:
        h.update(source.name.encode())
        h.update(source.read_bytes())
    return h.hexdigest()[:16]


def _run(cmd: list[str], what: str) -> None:
    started = time.time()
    process = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    # Say something now and then while a long compile runs.
    done = threading.Event()

    def ticker() -> None:
        while not done.wait(15.0):
            _say(f"still compiling {what} ({time.time() - started:.0f} s)")

    thread = threading.Thread(target=ticker, daemon=True)
    thread.start()
    try:
        output, _ = process.communicate()
    finally:
        done.set()
    if process.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n{' '.join(cmd)}\n{output}")


def _build_one(name: str, sources: list[Path], deps: list[Path], cmd_prefix: list[str],
               flags: list[str], suffix: str) -> Path:
    out_dir = build_dir()
    digest = _digest(sources + deps, flags)
    target = out_dir / f"{name}.{digest}{suffix}"
    if target.is_file():
        return target
    lock_path = out_dir / f".{name}.lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if target.is_file():
                return target
            _say(f"compiling {name} ...")
            started = time.time()
            partial = out_dir / f"{name}.{digest}.{os.getpid()}.tmp{suffix}"
            _run(cmd_prefix + flags + ["-o", str(partial)] + [str(s) for s in sources], name)
            os.replace(partial, target)
            for stale in out_dir.glob(f"{name}.*{suffix}"):
                if stale != target and ".tmp" not in stale.name:
                    try:
                        stale.unlink()
                    except OSError:
                        pass
            _say(f"compiled {name} in {time.time() - started:.1f} s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return target


def kernel_sources() -> dict[str, Path]:
    return {path.stem: path for path in sorted(KERNEL_DIR.glob("*.cu"))}


def kernel_include_dirs() -> list[str]:
    return [str(KERNEL_DIR)]


#: sources that are compiled once per value of a macro, and the values build_all() compiles
SPECIALISED = {"attention_bf16": ("HEAD_SIZE", (64, 128)), "attention_tcgen05": ("HEAD_SIZE", (64, 128))}


def split_variant(name: str) -> tuple[str, dict[str, str]]:
    """``attention_bf16:HEAD_SIZE=64`` -> (``attention_bf16``, {``HEAD_SIZE``: ``64``})."""
    source, _, rest = name.partition(":")
    defines = {}
    for item in filter(None, rest.split(",")):
        key, _, value = item.partition("=")
        defines[key] = value
    return source, defines


def build_kernel_library(name: str) -> Path:
    """Compile one kernel library; ``name`` is a source stem, optionally followed by
    ``:MACRO=value`` for a source that is specialised at compile time."""
    source, defines = split_variant(name)
    sources = kernel_sources()
    if source not in sources:
        raise BuildError(f"no kernel source {source}.cu in {KERNEL_DIR}")
    if source in SPECIALISED and SPECIALISED[source][0] not in defines:
        raise BuildError(f"{source} is compiled per {SPECIALISED[source][0]}; ask for {source}:{SPECIALISED[source][0]}=<n>")
    headers = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    flags = NVCC_FLAGS + [f"-I{d}" for d in kernel_include_dirs()] + [f"-D{k}={v}" for k, v in sorted(defines.items())]
    out_name = source + "".join(f"_{k.lower()}{v}" for k, v in sorted(defines.items()))
    return _build_one(out_name, [sources[source]], headers, [_find_nvcc()], flags, ".so")


def build_kernel_libraries(names: list[str] | None = None) -> dict[str, Path]:
    """Compile several kernel libraries side by side."""
    if names is None:
        names = []
        for source in kernel_sources():
            if source in SPECIALISED:
                macro, values = SPECIALISED[source]
                names.extend(f"{source}:{macro}={value}" for value in values)
            else:
                names.append(source)
    names = list(names)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(names)))) as pool:
        paths = list(pool.map(build_kernel_library, names))
    return dict(zip(names, paths))


def build_control_module() -> Path:
    import pybind11

    sources = sorted(CONTROL_DIR.glob("*.cpp"))
    headers = sorted(CONTROL_DIR.glob("*.h"))
    if not sources:
        raise BuildError(f"no C++ sources in {CONTROL_DIR}")
    flags = CXX_FLAGS + [
        f"-I{pybind11.get_include()}",
        f"-I{sysconfig.get_paths()['include']}",
        f"-I{CONTROL_DIR}",
    ]
    compiler = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not compiler:
        raise BuildError("no C++ compiler found for the control library (set CXX)")
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return _build_one("_control", sources, headers, [compiler], flags, suffix)


def build_all() -> dict[str, Path]:
    built = build_kernel_libraries()
    built["_control"] = build_control_module()
    return built
