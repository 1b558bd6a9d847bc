"""Compiles the CUDA sources of this folder for sm_100a and loads them through ctypes.

Each source file becomes one shared object (one per set of ``-D`` defines, so that a
kernel specialised on a size is compiled only for the sizes a model needs).  Objects are
kept in ``gguf2bin_b200/_build`` when that folder can be written, else in a per-user
folder under the system's temporary directory; the file name carries a hash of the
source, its headers and the flags, so a changed source is recompiled and a stale object
is never loaded.  While nvcc runs, a line is printed every few seconds.

There is no fallback: when neither a built object nor nvcc is there, ``KernelBuildError``
says so.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Iterable, Sequence

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    """The CUDA extension could not be built or loaded."""


class KernelError(RuntimeError):
    """A kernel launcher refused its arguments or the launch failed."""


def _log(msg: str) -> None:
    print(f"[gguf2bin_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    return None


_build_dir_cache: Path | None = None
_build_dir_lock = threading.Lock()


def build_dir() -> Path:
    with _build_dir_lock:
        return _build_dir_locked()


def _build_dir_locked() -> Path:
    global _build_dir_cache
    if _build_dir_cache is not None:
        return _build_dir_cache
    env = os.environ.get("GGUF2BIN_B200_BUILD_DIR")
    candidates = [Path(env)] if env else []
    candidates += [CSRC.parent / "_build",
                   Path(tempfile.gettempdir()) / f"gguf2bin_b200_build_{os.getuid()}"]
    for d in candidates:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe_{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            _build_dir_cache = d
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for built kernels; set GGUF2BIN_B200_BUILD_DIR")


_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _with_includes(source: Path, seen: dict) -> None:
    """``source`` and every file of this folder that it includes with quotes, recursively."""
    if source.name in seen or not source.is_file():
        return
    text = source.read_text()
    seen[source.name] = text
    for name in _INCLUDE.findall(text):
        _with_includes(CSRC / name, seen)


def _digest(source: Path, defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    files: dict = {}
    _with_includes(source, files)
    for name in sorted(files):
        h.update(name.encode())
        h.update(files[name].encode())
    h.update(" ".join(list(defines) + ARCH_FLAGS + BASE_FLAGS).encode())
    return h.hexdigest()[:16]


def object_path(source_name: str, defines: Sequence[str] = ()) -> Path:
    src = CSRC / source_name
    tag = "".join("_" + d.replace("=", "") for d in defines)
    return build_dir() / f"{src.stem}{tag}-{_digest(src, defines)}.so"


def _find_prebuilt(source_name: str, defines: Sequence[str]) -> Path | None:
    """A built object with the right hash in any known folder (the in-tree folder may be
    read-only yet hold objects built earlier)."""
    src = CSRC / source_name
    tag = "".join("_" + d.replace("=", "") for d in defines)
    name = f"{src.stem}{tag}-{_digest(src, defines)}.so"
    for d in (CSRC.parent / "_build", build_dir()):
        if (d / name).is_file():
            return d / name
    return None


def compile_unit(source_name: str, defines: Sequence[str] = (), verbose: bool = False) -> Path:
    """Builds one source with the given ``-D`` defines if it is not built yet."""
    src = CSRC / source_name
    if not src.is_file():
        raise KernelBuildError(f"{src}: no such kernel source")
    found = _find_prebuilt(source_name, defines)
    if found is not None:
        return found
    nvcc = find_nvcc()
    if nvcc is None:
        raise KernelBuildError(
            f"{source_name} is not built and nvcc was not found (PATH, $NVCC, /usr/local/cuda); "
            "the CUDA kernels are required, there is no fallback")
    out = object_path(source_name, defines)
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *(f"-D{d}" for d in defines), f"-I{CSRC}",
           "-o", str(tmp), str(src)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    what = source_name + (" [" + " ".join(defines) + "]" if defines else "")
    _log(f"compiling {what} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _log(f"  still compiling {what} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=heartbeat, daemon=True)
    th.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {what}:\n{output}")
    if verbose and output:
        print(output, file=sys.stderr)
    os.replace(tmp, out)
    prefix = out.name.rsplit("-", 1)[0] + "-"
    for old in out.parent.glob(prefix + "*.so"):        # objects of older versions of this source
        if old != out and old.name.rsplit("-", 1)[0] + "-" == prefix:
            try:
                old.unlink()
            except OSError:
                pass
    _log(f"  built {out.name} in {time.time() - t0:.1f} s")
    return out


def compile_many(units: Iterable[tuple[str, Sequence[str]]], jobs: int | None = None) -> list[Path]:
    """Builds several units in parallel threads (each runs its own nvcc)."""
    units = list(units)
    out: list = [None] * len(units)
    errors: list = []
    sem = threading.Semaphore(jobs or min(8, os.cpu_count() or 2))

    def work(i, name, defines):
        with sem:
            try:
                out[i] = compile_unit(name, defines)
            except Exception as e:          # noqa: BLE001 - re-raised below
                errors.append(e)

    threads = [threading.Thread(target=work, args=(i, n, d)) for i, (n, d) in enumerate(units)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return out


_loaded: dict[tuple, ctypes.CDLL] = {}


def load_unit(source_name: str, defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = (source_name, tuple(defines))
    lib = _loaded.get(key)
    if lib is None:
        path = compile_unit(source_name, defines)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from None
        lib.g2b_last_error.restype = ctypes.c_char_p
        lib.g2b_last_error.argtypes = []
        lib.g2b_set_pdl.argtypes = [ctypes.c_int]
        lib.g2b_set_pdl.restype = None
        lib.g2b_set_pdl(1 if _pdl else 0)
        _loaded[key] = lib
    return lib


# Programmatic dependent launch (kernels start while their predecessor drains, and wait
# on the device before touching its results).  On unless GGUF2BIN_B200_PDL=0.
_pdl = os.environ.get("GGUF2BIN_B200_PDL", "1") != "0"


def set_pdl(on: bool) -> None:
    global _pdl
    _pdl = bool(on)
    for lib in _loaded.values():
        lib.g2b_set_pdl(1 if _pdl else 0)
