"""Compiles the CUDA sources of ``csrc/`` for sm_100a on first use and loads them with ctypes.

Every library is one ``.cu`` file with ``extern "C"`` entry points, built by one ``nvcc``
call into ``csrc/_build/<name>-<hash>.so`` (the hash covers the source, the shared headers,
the flags and the ``-D`` definitions, so an edited kernel or another head size is another
file and an unchanged one is reused).  A model asks only for the libraries and
specialisations it needs, so a first run compiles what that model uses and nothing else;
while ``nvcc`` runs a line is printed every few seconds.  If the source tree cannot be
written the build goes to a per-user folder under the system's temporary directory.

There is no fallback: without ``nvcc`` or with a failed build this raises.
"""

from __future__ import annotations

import ctypes
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
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
COMMON_FLAGS = (
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-shared",
)

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class NativeBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise NativeBuildError(
            "nvcc was not found (PATH and /usr/local/cuda/bin); the CUDA kernels of this "
            "framework cannot be built and there is no other path"
        )
    return found


def _build_dir() -> Path:
    preferred = CSRC / "_build"
    try:
        preferred.mkdir(parents=True, exist_ok=True)
        probe = preferred / f".write-test-{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"cie_b200_build_{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def library_path(source: str, defines: dict[str, object] | None = None) -> tuple[Path, list[str]]:
    src = CSRC / source
    if not src.is_file():
        raise NativeBuildError(f"CUDA source {src} is missing")
    defines = dict(defines or {})
    define_flags = [f"-D{key}={value}" for key, value in sorted(defines.items())]
    digest = hashlib.sha256()
    for path in [src, *_headers()]:
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join([*ARCH_FLAGS, *COMMON_FLAGS, *define_flags]).encode())
    suffix = "".join(f"-{key.lower()}{value}" for key, value in sorted(defines.items()))
    name = f"{src.stem}{suffix}-{digest.hexdigest()[:12]}.so"
    return _build_dir() / name, define_flags


def _compile(source: str, target: Path, define_flags: list[str], extra: tuple[str, ...]) -> None:
    scratch = target.with_suffix(f".tmp{os.getpid()}.so")
    command = [
        _nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, *define_flags, *extra,
        "-I", str(CSRC), "-o", str(scratch), str(CSRC / source),
    ]
    label = f"{source} {' '.join(define_flags)}".strip()
    print(f"[cie-b200] compiling {label} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    output: list[bytes] = []
    reader = threading.Thread(target=lambda: output.append(process.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            process.wait(timeout=5.0)
            break
        except subprocess.TimeoutExpired:
            print(
                f"[cie-b200] still compiling {label} ({time.time() - started:.0f} s)",
                file=sys.stderr, flush=True,
            )
    reader.join()
    text = b"".join(output).decode(errors="replace")
    if process.returncode != 0:
        scratch.unlink(missing_ok=True)
        raise NativeBuildError(f"nvcc failed for {label}:\n{' '.join(command)}\n{text}")
    os.replace(scratch, target)
    print(f"[cie-b200] built {target.name} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)


def load_library(
    source: str, defines: dict[str, object] | None = None, extra_flags: tuple[str, ...] = ()
) -> ctypes.CDLL:
    """Builds (if needed) and loads ``csrc/<source>``; one handle per (source, defines)."""
    target, define_flags = library_path(source, defines)
    key = str(target)
    with _lock:
        if key in _loaded:
            return _loaded[key]
        if not target.exists():
            _compile(source, target, define_flags, extra_flags)
        try:
            handle = ctypes.CDLL(str(target))
        except OSError as exc:
            raise NativeBuildError(f"cannot load {target}: {exc}") from exc
        _loaded[key] = handle
        return handle


def build_only(source: str, defines: dict[str, object] | None = None,
               extra_flags: tuple[str, ...] = ()) -> Path:
    """Compiles without loading (a machine without a GPU can still check that it builds)."""
    target, define_flags = library_path(source, defines)
    with _lock:
        if not target.exists():
            _compile(source, target, define_flags, extra_flags)
    return target
