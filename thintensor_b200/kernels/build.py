"""Compiling the CUDA sources for sm_100a and loading them.

Each ``.cu`` file under ``csrc/`` becomes one shared library, built with nvcc the first
time something in it is called and loaded with ctypes; a model therefore compiles only
the sources its dtype and parts use.  Libraries are kept in ``thintensor_b200/_build``
(or, when the package folder is read-only, in a per-user folder under the system's
temporary directory) under a name that carries a hash of the source, the shared header
and the flags, so an edited source is rebuilt and a current one is reused.  There is
no fallback: without nvcc, or if compilation fails, the call raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import stat
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr"]

# source stem -> extra nvcc flags
SOURCES: dict[str, list[str]] = {
    "elementwise": [],
    "attention": [],
    "gemm_simt": [],
    "sampling": [],
    "attention_static_scratch": [],
    "gemm_tcgen05": [],
    "attention_mma": [],
    "attention_tcgen05": [],
}


class KernelBuildError(RuntimeError):
    pass


_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _log(message: str) -> None:
    print(f"[thintensor_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for candidate in candidates:
        if candidate.is_file():
            return str(candidate)
    found = shutil.which("nvcc")
    if found:
        return found
    raise KernelBuildError(
        "nvcc was not found (looked in $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
        "the CUDA kernels of thintensor_b200 cannot be built and there is no other path"
    )


_build_dir: Path | None = None
_build_dir_lock = threading.Lock()


def build_dir() -> Path:
    """Where libraries live: in the package if it can be written, else per user under
    the temporary directory."""
    global _build_dir
    with _build_dir_lock:
        if _build_dir is None:
            _build_dir = _choose_build_dir()
        return _build_dir


def _temp_folder() -> Path:
    return Path(tempfile.gettempdir()) / f"thintensor_b200-build-{os.getuid()}"


def _is_private(folder: Path) -> bool:
    """Whether libraries found in ``folder`` can be trusted: a real directory (no symbolic link)
    that this user owns and that neither its group nor others may write to.  The system's temporary
    directory is writable by everyone, so another user could have made a folder of the expected
    name there first and put a library of the expected file name in it."""
    try:
        info = os.lstat(folder)
    except OSError:
        return False
    return stat.S_ISDIR(info.st_mode) and info.st_uid == os.getuid() and not info.st_mode & (stat.S_IWGRP | stat.S_IWOTH)


def _private_temp_folder() -> Path:
    """The per-user folder under the temporary directory, made with mode 0700; if a folder of that
    name exists that is not this user's alone, a fresh one that is (its libraries are then built
    anew by every process)."""
    folder = _temp_folder()
    try:
        os.mkdir(folder, 0o700)
    except FileExistsError:
        pass
    if _is_private(folder):
        return folder
    return Path(tempfile.mkdtemp(prefix="thintensor_b200-build-"))     # mode 0700, owned by this user


def _choose_build_dir() -> Path:
    override = os.environ.get("THINTENSOR_B200_BUILD_DIR")
    candidates = [lambda: Path(override)] if override else []
    candidates.append(lambda: CSRC.parent / "_build")
    candidates.append(_private_temp_folder)
    tried = []
    for make in candidates:
        try:
            folder = make()
            tried.append(str(folder))
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".write-{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise KernelBuildError(f"no writable folder for compiled kernels among {tried}")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update((CSRC / f"{name}.cu").read_bytes())
    for header in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(header.read_bytes())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS + SOURCES[name]).encode())
    return h.hexdigest()[:16]


def library_path(name: str, folder: Path | None = None) -> Path:
    return (folder or build_dir()) / f"tt_{name}-{_digest(name)}.so"


def _find_built(name: str) -> Path | None:
    """A current library for ``name`` in the folder this process builds into, or in the package's
    own folder (a library built there earlier serves a later user who may only read it).  The
    folder under the temporary directory is searched only as the chosen build folder, which
    :func:`_private_temp_folder` has checked to be this user's alone."""
    file = f"tt_{name}-{_digest(name)}.so"
    for folder in (build_dir(), CSRC.parent / "_build"):
        if (folder / file).is_file():
            return folder / file
    return None


def compile_source(name: str, verbose: bool = True) -> Path:
    """Build ``csrc/<name>.cu`` if its library is missing; return the library's path."""
    if name not in SOURCES:
        raise KernelBuildError(f"no CUDA source named {name!r}; known: {', '.join(SOURCES)}")
    existing = _find_built(name)
    if existing is not None:
        return existing
    nvcc = find_nvcc()
    folder = build_dir()
    target = library_path(name, folder)
    scratch = target.with_suffix(f".{os.getpid()}.tmp")
    command = [nvcc, *ARCH_FLAGS, *COMMON_FLAGS, *SOURCES[name], "-I", str(CSRC), "-o", str(scratch), str(CSRC / f"{name}.cu")]
    if verbose:
        _log(f"compiling {name}.cu for sm_100a ...")
    started = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    output: list[str] = []
    reader = threading.Thread(target=lambda: output.append(process.stdout.read()), daemon=True)
    reader.start()
    next_note = 10.0
    while process.poll() is None:
        time.sleep(0.2)
        if verbose and time.time() - started > next_note:
            _log(f"still compiling {name}.cu ({int(time.time() - started)} s)")
            next_note += 10.0
    reader.join()
    if process.returncode != 0:
        scratch.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed on {name}.cu (exit {process.returncode}):\n{''.join(output)}\ncommand: {' '.join(command)}")
    os.replace(scratch, target)
    for stale in folder.glob(f"tt_{name}-*.so"):
        if stale != target:
            stale.unlink(missing_ok=True)
    if verbose:
        _log(f"compiled {name}.cu in {time.time() - started:.1f} s -> {target}")
    return target


def load(name: str) -> ctypes.CDLL:
    """The loaded library of ``csrc/<name>.cu``, compiling it first if needed."""
    with _lock:
        if name not in _loaded:
            _loaded[name] = ctypes.CDLL(str(compile_source(name)))
        return _loaded[name]


def build_all(names: list[str] | None = None, verbose: bool = True) -> dict[str, Path]:
    """Compile every source (in parallel); used by the build check and before tests."""
    names = list(names or SOURCES)
    results: dict[str, Path] = {}
    errors: list[BaseException] = []

    def work(n: str) -> None:
        try:
            results[n] = compile_source(n, verbose)
        except BaseException as exc:  # noqa: BLE001 - reported below
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return results
