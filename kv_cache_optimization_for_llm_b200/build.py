"""Compiles the native parts of the package, each source into a library of its own.

Two kinds of library are built, both for this machine only:

* kernel modules: one ``csrc/kernels/<name>.cu`` -> ``_lib/<name>.so`` with nvcc for
  ``sm_100a``, loaded through ctypes by :mod:`..ops`;
* the host runtime: ``csrc/host/*.cpp`` -> ``_lib/_kvb_host<ext>.so`` with g++ and
  pybind11.

A library is rebuilt when the hash of its sources and flags changes.  Building is
lazy: a model compiles what it uses at its first call and prints a line now and
then meanwhile.  Libraries go beside the package (``_lib/``) when that folder can
be written, so that they travel with the tree; otherwise to a per-user folder
under the system's temporary directory.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import subprocess
import sys
import sysconfig
import tempfile
import time
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
KERNEL_DIR = CSRC / "kernels"
HOST_DIR = CSRC / "host"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--shared", "-cudart", "static", "--expt-relaxed-constexpr",
]
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-Wall"]


def _log(msg: str) -> None:
    print(f"[kvb200 build] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("KVB200_NVCC"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    from shutil import which
    found = which("nvcc")
    if not found:
        raise RuntimeError("nvcc was not found: the CUDA kernels of this package cannot be built "
                           "(set KVB200_NVCC to its path)")
    return found


_lib_dir_cache: Path | None = None


def lib_dir() -> Path:
    """Folder that holds the built libraries (created if needed)."""
    global _lib_dir_cache
    if _lib_dir_cache is not None:
        return _lib_dir_cache
    env = os.environ.get("KVB200_LIB_DIR")
    cands = [Path(env)] if env else []
    cands.append(PKG_DIR / "_lib")
    cands.append(Path(tempfile.gettempdir()) / f"kvb200-lib-{os.getuid()}")
    for c in cands:
        try:
            c.mkdir(parents=True, exist_ok=True)
            probe = c / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            _lib_dir_cache = c
            return c
        except OSError:
            continue
    raise RuntimeError(f"no writable folder for built libraries among {cands}")


def _hash(paths, flags) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _kernel_sources(name: str):
    src = KERNEL_DIR / f"{name}.cu"
    if not src.exists():
        raise FileNotFoundError(f"no kernel module {name!r} ({src})")
    deps = [src] + sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    return src, deps


def kernel_lib_path(name: str) -> Path:
    return lib_dir() / f"{name}.so"


def _host_lib_path() -> Path:
    return lib_dir() / ("_kvb_host" + sysconfig.get_config_var("EXT_SUFFIX"))


def _up_to_date(out: Path, digest: str) -> bool:
    stamp = out.with_suffix(out.suffix + ".hash")
    return out.exists() and stamp.exists() and stamp.read_text() == digest


def _jobs_for(names):
    jobs = []
    for name in names:
        if name == "_host":
            srcs = sorted(HOST_DIR.glob("*.cpp"))
            deps = srcs + sorted(HOST_DIR.glob("*.h"))
            import pybind11
            inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
            out = _host_lib_path()
            cmd = ["g++"] + HOST_FLAGS + inc + [str(s) for s in srcs]
            digest = _hash(deps, HOST_FLAGS + [sys.version])
        else:
            src, deps = _kernel_sources(name)
            out = kernel_lib_path(name)
            cmd = [_nvcc()] + NVCC_FLAGS + ["-I", str(KERNEL_DIR), str(src)]
            digest = _hash(deps, NVCC_FLAGS)
        jobs.append((name, out, cmd, digest))
    return jobs


def ensure_built(names, verbose: bool | None = None) -> None:
    """Builds every named module that is missing or stale, all at once.

    ``names`` are kernel module names (``csrc/kernels/<name>.cu``) or ``"_host"``.
    """
    jobs = [j for j in _jobs_for(list(dict.fromkeys(names))) if not _up_to_date(j[1], j[3])]
    if not jobs:
        return
    lock_path = lib_dir() / ".build.lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            jobs = [j for j in jobs if not _up_to_date(j[1], j[3])]  # another process may have built
            if not jobs:
                return
            _log("compiling " + ", ".join(j[0] for j in jobs) + f" into {lib_dir()} (first use only)")
            t0 = time.time()
            procs = []
            for name, out, cmd, digest in jobs:
                tmp = out.with_name(out.name + f".tmp{os.getpid()}")
                logf = tempfile.TemporaryFile(mode="w+")
                p = subprocess.Popen(cmd + ["-o", str(tmp)], stdout=logf, stderr=subprocess.STDOUT)
                procs.append((name, out, tmp, digest, p, logf))
            last = t0
            pending = list(procs)
            while pending:
                time.sleep(0.2)
                still = []
                for item in pending:
                    name, out, tmp, digest, p, logf = item
                    rc = p.poll()
                    if rc is None:
                        still.append(item)
                        continue
                    logf.seek(0)
                    text = logf.read()
                    logf.close()
                    if rc != 0:
                        for other in pending:
                            if other[4].poll() is None:
                                other[4].kill()
                        raise RuntimeError(f"building {name} failed (exit {rc}):\n{text[-6000:]}")
                    os.replace(tmp, out)
                    out.with_suffix(out.suffix + ".hash").write_text(digest)
                    _log(f"built {name} in {time.time() - t0:.0f}s")
                pending = still
                if pending and time.time() - last > 10:
                    last = time.time()
                    _log(f"still compiling {', '.join(i[0] for i in pending)} ... {last - t0:.0f}s")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def all_kernel_modules():
    return sorted(p.stem for p in KERNEL_DIR.glob("*.cu"))


def build_all() -> None:
    """Everything: every kernel module and the host runtime."""
    ensure_built(all_kernel_modules() + ["_host"])


def load_host():
    """Imports the host runtime module, building it first if needed."""
    ensure_built(["_host"])
    import importlib.util
    path = _host_lib_path()
    spec = importlib.util.spec_from_file_location("_kvb_host", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    build_all()
    _log("all libraries are up to date")
