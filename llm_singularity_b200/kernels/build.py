"""Compiling the CUDA libraries for sm_100a, at first use, into a folder of their own.

Each ``csrc/<name>.cu`` becomes one shared library with plain C entry points
(no Python or torch headers, so a file compiles in seconds).  A library is
rebuilt when its source, a shared header or the flags change: the file name
carries a hash of all three.  Builds go to ``csrc/_build`` inside the package if
that can be written, else to a per-user folder under the system's temporary
directory, so a read-only checkout and an empty HOME both work.  Several
libraries compile in parallel and a line is printed every few seconds meanwhile.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from typing import Dict, Iterable, List, Optional

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]
# No --use_fast_math: expf, sincosf and division must stay exact.

SOURCES: Dict[str, object] = {          # library -> its source file (or files)
    "embedding": "embedding.cu",
    "norm": "norm.cu",
    "activation": "activation.cu",
    "cache_table": "cache_table.cu",
    "rope_cache": "rope_cache.cu",
    "attention": "attention.cu",
    "attention_tc": "attention_tc.cu",
    "attention_tc5": "attention_tc5.cu",
    "gemm": "gemm.cu",
    "gemm_tc": "gemm_tc.cu",
    "gemm_small": "gemm_small.cu",
    "gemm_stream": "gemm_stream.cu",
    "sampling": "sampling.cu",
    "random_init": "random_init.cu",
    # host code only: pools, block tables, prefix tree; scheduler
    "host_runtime": ("host_memory.cpp", "host_scheduler.cpp", "host_step.cpp"),
}
HEADERS = ["common.cuh", "attention_tc_noalloc.h", "stream_warm.cuh"]     # of the CUDA libraries
HOST_HEADERS = ["host_memory.h"]                          # of the host runtime


def _files(name: str) -> List[str]:
    src = SOURCES[name]
    return [src] if isinstance(src, str) else list(src)


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $NVCC, $CUDA_HOME/bin, /usr/local/cuda/bin, PATH); "
                     "the engine has no path without its CUDA libraries")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = tempfile.NamedTemporaryFile(dir=path, delete=True)
        probe.close()
        return True
    except OSError:
        return False


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    if _build_dir is None:
        cands = [os.environ.get("LLM_SINGULARITY_B200_BUILD_DIR"), os.path.join(CSRC, "_build"),
                 os.path.join(tempfile.gettempdir(), f"llm_singularity_b200_build_{os.getuid()}")]
        for c in cands:
            if c and _writable_dir(c):
                _build_dir = c
                break
        else:
            raise BuildError(f"no writable folder for compiled kernels (tried {cands[1:]})")
    return _build_dir


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for fn in _files(name) + (HOST_HEADERS if name == "host_runtime" else HEADERS):
        with open(os.path.join(CSRC, fn), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def library_path(name: str) -> str:
    if name not in SOURCES:
        raise BuildError(f"no kernel library named '{name}' (known: {', '.join(sorted(SOURCES))})")
    return os.path.join(build_dir(), f"lsb_{name}.{_digest(name)}.so")


def _prune(name: str, keep: str) -> None:
    """Drop builds of ``name`` made from older sources (the hash in the file name differs)."""
    d = os.path.dirname(keep)
    for f in os.listdir(d):
        if f.startswith(f"lsb_{name}.") and f.endswith(".so") and os.path.join(d, f) != keep:
            try:
                os.unlink(os.path.join(d, f))
            except OSError:
                pass


def ensure_built(names: Iterable[str], verbose: bool = False) -> Dict[str, str]:
    """Compile the named libraries if their current build is absent; returns name -> path."""
    names = list(dict.fromkeys(names))
    paths = {n: library_path(n) for n in names}
    todo = [n for n in names if not os.path.isfile(paths[n])]
    if not todo:
        return paths
    nvcc = find_nvcc()
    out = sys.stderr
    what = "host librar" if all(n == "host_runtime" for n in todo) else "CUDA librar"
    print(f"[llm_singularity_b200] compiling {len(todo)} {what}{'y' if len(todo) == 1 else 'ies'} "
          f"{'' if what.startswith('host') else 'for sm_100a '}({', '.join(todo)}) into {build_dir()}",
          file=out, flush=True)
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    procs: List = []
    t0 = time.time()
    for n in todo:
        tmp = f"{paths[n]}.{os.getpid()}.tmp"
        cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp] + [os.path.join(CSRC, f) for f in _files(n)]
        procs.append((n, tmp, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                               env=env, text=True)))
    pending = list(procs)
    last = t0
    errors = []
    while pending:
        still = []
        for n, tmp, p in pending:
            if p.poll() is None:
                still.append((n, tmp, p))
                continue
            log = p.stdout.read()
            if p.returncode != 0:
                errors.append(f"--- {', '.join(_files(n))} (exit {p.returncode}) ---\n{log}")
                if os.path.exists(tmp):
                    os.unlink(tmp)
            else:
                os.replace(tmp, paths[n])          # atomic: a concurrent process sees all or nothing
                _prune(n, paths[n])
                if verbose:
                    print(f"[llm_singularity_b200]   {n} done after {time.time() - t0:.0f} s",
                          file=out, flush=True)
        pending = still
        if pending:
            time.sleep(0.2)
            if time.time() - last >= 5.0:
                last = time.time()
                print(f"[llm_singularity_b200]   still compiling {', '.join(n for n, _, _ in pending)} "
                      f"({last - t0:.0f} s)", file=out, flush=True)
    if errors:
        raise BuildError("nvcc failed:\n" + "\n".join(errors))
    print(f"[llm_singularity_b200] compiled in {time.time() - t0:.0f} s", file=out, flush=True)
    return paths


def build_all(verbose: bool = True) -> Dict[str, str]:
    return ensure_built(SOURCES.keys(), verbose=verbose)
