"""Build and load the CUDA libraries of ``edgerag_b200/csrc``.

Each source file becomes one shared library per element type (``float`` for the 32-bit path,
``bfloat16`` for serving), built with nvcc for sm_100a the first time it is needed and loaded with
``ctypes``.  A run therefore compiles what its model and dtype need, and nothing else.  Libraries
are kept in ``edgerag_b200/_ext`` (inside the package, so that they travel with the tree); if that
folder cannot be written, a per-user folder under the system's temporary directory is used.

There is no fallback: if a library is missing and cannot be built, loading raises
``NativeBuildError`` and nothing runs.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
PACKAGE_EXT = Path(__file__).resolve().parent.parent / "_ext"

#: library -> (source file, extra link flags, built per element type)
LIBRARIES: dict[str, tuple[str, tuple[str, ...], bool]] = {
    "elementwise": ("elementwise.cu", (), True),
    "attention": ("attention.cu", (), True),
    "attention_tc": ("attention_tc.cu", ("-lcuda",), False),
    "attention_prefill": ("attention_prefill.cu", ("-lcuda",), False),
    "gemm": ("gemm.cu", ("-lcublasLt",), True),
    "linear_tc": ("linear_tc.cu", ("-lcuda",), False),
    "sampling": ("sampling.cu", (), False),
}

NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-shared",
    "-Xcompiler", "-fPIC", "-diag-suppress", "177",
)

ELEM_CODES = {"float32": 0, "bfloat16": 1}


class NativeBuildError(RuntimeError):
    """A CUDA library of the engine is missing and could not be built."""


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise NativeBuildError("nvcc not found (looked at $NVCC, PATH and /usr/local/cuda/bin)")


def _ext_dir() -> Path:
    override = os.environ.get("EDGERAG_B200_EXT_DIR")
    candidates = [Path(override)] if override else []
    candidates += [PACKAGE_EXT, Path(tempfile.gettempdir()) / f"edgerag_b200_ext_{os.getuid()}"]
    for cand in candidates:
        try:
            cand.mkdir(parents=True, exist_ok=True)
            probe = cand / f".write_probe_{os.getpid()}_{threading.get_ident()}"
            probe.write_text("")
            probe.unlink()
            return cand
        except OSError:
            continue
    raise NativeBuildError("no writable folder for the compiled libraries")


def _lib_names(library: str, elem: str | None) -> tuple[str, list[str]]:
    source, link, per_elem = LIBRARIES[library]
    if per_elem:
        if elem not in ELEM_CODES:
            raise ValueError(f"library {library} is built per element type; got {elem!r}")
        return f"lib{library}_{elem}.so", [f"-DERB_ELEM={ELEM_CODES[elem]}"]
    return f"lib{library}.so", ["-DERB_ELEM=0"]


def _fingerprint(library: str, defines: list[str]) -> str:
    source, link, _ = LIBRARIES[library]
    h = hashlib.sha256()
    for path in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [CSRC / source]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join((*NVCC_FLAGS, *defines, *link)).encode())
    return h.hexdigest()


def _say(msg: str) -> None:
    print(f"[edgerag_b200] {msg}", file=sys.stderr, flush=True)


def _find_prebuilt(name: str, stamp: str) -> Path | None:
    """A library built earlier, in the package folder or the fallback folder, for these sources."""
    folders = [PACKAGE_EXT, Path(tempfile.gettempdir()) / f"edgerag_b200_ext_{os.getuid()}"]
    if os.environ.get("EDGERAG_B200_EXT_DIR"):
        folders.insert(0, Path(os.environ["EDGERAG_B200_EXT_DIR"]))
    for folder in folders:
        lib, mark = folder / name, folder / (name + ".stamp")
        try:
            if lib.is_file() and mark.is_file() and mark.read_text().strip() == stamp:
                return lib
        except OSError:
            continue
    return None


def build(library: str, elem: str | None = None, verbose: bool = True) -> Path:
    """Compile one library if its sources changed since the last build; return its path."""
    name, defines = _lib_names(library, elem)
    stamp = _fingerprint(library, defines)
    ready = _find_prebuilt(name, stamp)
    if ready is not None:
        return ready
    folder = _ext_dir()
    lib, mark = folder / name, folder / (name + ".stamp")
    source, link, _ = LIBRARIES[library]
    with open(folder / (name + ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if lib.is_file() and mark.is_file() and mark.read_text().strip() == stamp:
                return lib  # another process built it while we waited
            tmp = folder / f".{name}.{os.getpid()}.tmp.so"
            cmd = [_nvcc(), *NVCC_FLAGS, *defines, "-o", str(tmp), str(CSRC / source), *link]
            if verbose:
                _say(f"compiling {name} for sm_100a (first use) ...")
            env = dict(os.environ)
            env.setdefault("TMPDIR", tempfile.gettempdir())
            t0 = time.time()
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
            done = threading.Event()

            def _heartbeat() -> None:
                while not done.wait(10.0):
                    if verbose:
                        _say(f"  still compiling {name} ({time.time() - t0:.0f} s)")

            beat = threading.Thread(target=_heartbeat, daemon=True)
            beat.start()
            out, _ = proc.communicate()
            done.set()
            if proc.returncode != 0:
                tmp.unlink(missing_ok=True)
                raise NativeBuildError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{out}")
            os.replace(tmp, lib)
            mark.write_text(stamp)
            if verbose:
                _say(f"built {name} in {time.time() - t0:.1f} s")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_loaded: dict[tuple[str, str | None], ctypes.CDLL] = {}


def load(library: str, elem: str | None = None) -> ctypes.CDLL:
    """The loaded library (built first if need be).  Raises ``NativeBuildError`` on any failure."""
    key = (library, elem if LIBRARIES[library][2] else None)
    if key in _loaded:
        return _loaded[key]
    path = build(library, key[1])
    if library == "gemm":
        import torch  # noqa: F401  (its CUDA libraries provide libcublasLt.so.12 at run time)
    try:
        lib = ctypes.CDLL(str(path))
    except OSError as exc:
        raise NativeBuildError(f"cannot load {path}: {exc}") from exc
    lib.erb_last_error.restype = ctypes.c_char_p
    _loaded[key] = lib
    return lib


def build_all(verbose: bool = True, jobs: int | None = None) -> list[Path]:
    """Compile every library for both element types (the "does it build" check)."""
    from concurrent.futures import ThreadPoolExecutor

    work = []
    for library, (source, _, per_elem) in LIBRARIES.items():
        if not (CSRC / source).is_file():
            continue
        for elem in (ELEM_CODES if per_elem else (None,)):
            work.append((library, elem))
    with ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 2)) as pool:
        return list(pool.map(lambda w: build(w[0], w[1], verbose), work))
