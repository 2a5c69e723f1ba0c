"""Builds the framework's one native library, `libnanospec_b200.so`, for sm_100a.

Every `.cu` file of this folder is compiled by nvcc into an object file and the objects
are linked into one shared library under `csrc/_build/` (or, when the package folder is
not writable, under a per-user folder in the system's temporary directory).  The sources
include no framework headers, so a cold build takes about a minute; a stamp of the
sources' contents decides whether a rebuild is needed.  While compiling, a line is printed
to stderr for every file so that a first call does not look hung.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path

SRC_DIR = Path(__file__).resolve().parent
LIB_NAME = "libnanospec_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[nanospec_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NANOSPEC_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NANOSPEC_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built and there is no other execution path")


def sources() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cuh")) + sorted(SRC_DIR.glob("*.h"))


def source_stamp() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    override = os.environ.get("NANOSPEC_BUILD_DIR")
    if override:
        d = Path(override)
        d.mkdir(parents=True, exist_ok=True)
        return d
    in_tree = SRC_DIR / "_build"
    if _writable(in_tree):
        return in_tree
    d = Path(tempfile.gettempdir()) / f"nanospec_b200_build_{os.getuid()}"
    d.mkdir(parents=True, exist_ok=True)
    return d


def _is_current(d: Path, stamp: str) -> bool:
    lib, meta = d / LIB_NAME, d / "stamp.json"
    if not (lib.is_file() and meta.is_file()):
        return False
    try:
        return json.loads(meta.read_text()).get("stamp") == stamp
    except (OSError, ValueError):
        return False


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> tuple[Path, float, str]:
    t0 = time.time()
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return src, time.time() - t0, proc.stderr


def ensure_built(force: bool = False, verbose: bool = False) -> Path:
    """Path of an up-to-date library, compiling whatever is stale first."""
    stamp = source_stamp()
    in_tree = SRC_DIR / "_build"
    if not force and _is_current(in_tree, stamp):
        return in_tree / LIB_NAME
    d = build_dir()
    if not force and _is_current(d, stamp):
        return d / LIB_NAME

    nvcc = find_nvcc()
    srcs = sources()
    _say(f"building {LIB_NAME} for sm_100a in {d} ({len(srcs)} files, this happens once)")
    # per-file object reuse: an object is kept when its own source and the headers are unchanged
    hdr = hashlib.sha256(b"".join(p.read_bytes() for p in _headers())).hexdigest()
    flags = " ".join(ARCH_FLAGS + NVCC_FLAGS)
    objs, todo = [], []
    for s in srcs:
        key = hashlib.sha256(s.read_bytes() + hdr.encode() + flags.encode()).hexdigest()[:16]
        obj = d / f"{s.stem}.{key}.o"
        objs.append(obj)
        if force or not obj.is_file():
            todo.append((s, obj))
    for old in d.glob("*.o"):
        if old not in objs:
            old.unlink(missing_ok=True)
    t0 = time.time()
    done = 0
    with ThreadPoolExecutor(max_workers=min(8, max(1, os.cpu_count() or 1))) as pool:
        futs = [pool.submit(_compile_one, nvcc, s, o.with_suffix(".tmp.o"), verbose) for s, o in todo]
        for fut in as_completed(futs):
            src, dt, log = fut.result()
            done += 1
            _say(f"compiled {src.name} in {dt:.0f} s ({done}/{len(todo)})")
            if verbose and log:
                print(log, file=sys.stderr)
    for s, o in todo:
        o.with_suffix(".tmp.o").replace(o)
    tmp_lib = d / f"{LIB_NAME}.{os.getpid()}.tmp"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *[str(o) for o in objs]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    tmp_lib.replace(d / LIB_NAME)
    (d / "stamp.json").write_text(json.dumps({"stamp": stamp, "built": time.time()}))
    _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return d / LIB_NAME


if __name__ == "__main__":
    print(ensure_built(force="--force" in sys.argv, verbose="-v" in sys.argv))
