"""Compiling the CUDA sources of this folder for sm_100a, on first use.

Each ``.cu`` file is one kernel family and becomes one shared library with
``extern "C"`` entry points, loaded through ``ctypes``.  A family is compiled the
first time something asks for it (or all at once by ``build_all``); a model asks
only for the families its parts use.  Libraries are kept beside the sources in
``_build/`` under a name that carries a hash of the source, the headers of this folder and
the compiler flags, so an edited source is recompiled and an old library is never
picked up.  If that folder cannot be written, a per-user folder under the system's
temporary directory is used instead.

There is no fallback: without ``nvcc`` or with a failed compile the import of a
kernel raises, and nothing on the product path runs without its kernels.
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
from typing import Dict, Iterable, List

_HERE = os.path.dirname(os.path.abspath(__file__))

# family name -> source file
SOURCES: Dict[str, str] = {
    "embed": "embed.cu",
    "norm": "norm.cu",
    "rope": "rope.cu",
    "act": "act.cu",
    "attention": "attention.cu",
    "attention_decode": "attention_decode.cu",
    "attention_decode_tc": "attention_decode_tc.cu",
    "attention_prefill": "attention_prefill.cu",
    "attention_prefill_tc": "attention_prefill_tc.cu",
    "linear": "linear.cu",
    "linear_mma": "linear_mma.cu",
    "linear_tc": "linear_tc.cu",
    "gemm_tc": "gemm_tc.cu",
    "sampling": "sampling.cu",
    "argmax_noalloc": "argmax_noalloc.cu",
}

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]
# No --use_fast_math: softmax, norms and rotation angles need exact expf and sincosf.
# Further flags for builds of one's own (-DBN_TRACE: timestamp probes; -DBN_NO_PDL: no programmatic
# dependent launch).  Set before anything is loaded; they enter the libraries' names.
EXTRA_FLAGS: List[str] = []

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for cand in (os.environ.get("BN_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $BN_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                           "the CUDA kernels of this library cannot be built and there is no fallback")


def _writable_dir(path: str) -> bool:
    try:
        os.makedirs(path, exist_ok=True)
        probe = os.path.join(path, f".probe-{os.getpid()}-{threading.get_ident()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def build_dir() -> str:
    local = os.path.join(_HERE, "_build")
    if _writable_dir(local):
        return local
    alt = os.path.join(tempfile.gettempdir(), f"bitnet_c_b200_build_{os.getuid()}")
    if _writable_dir(alt):
        return alt
    raise KernelBuildError(f"neither '{local}' nor '{alt}' can be written; nowhere to put the compiled kernels")


def _digest(family: str) -> str:
    h = hashlib.sha256()
    headers = sorted(fn for fn in os.listdir(_HERE) if fn.endswith((".cuh", ".h")))
    for fn in [SOURCES[family]] + headers:
        with open(os.path.join(_HERE, fn), "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS).encode())
    return h.hexdigest()[:12]


def library_path(family: str) -> str:
    """Where the compiled library of ``family`` lies, or would lie, for the current sources."""
    name = f"libbn_{family}-{_digest(family)}.so"
    local = os.path.join(_HERE, "_build", name)
    if os.path.isfile(local):
        return local
    return os.path.join(build_dir(), name)


def _compile(family: str, out: str, log: List[str]) -> None:
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + EXTRA_FLAGS + ["-I", _HERE, "-o", tmp, os.path.join(_HERE, SOURCES[family])]
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if p.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {SOURCES[family]}:\n{' '.join(cmd)}\n{p.stdout}")
    os.replace(tmp, out)
    # libraries of older versions of this source are of no use any more
    folder, keep = os.path.dirname(out), os.path.basename(out)
    for fn in os.listdir(folder):
        if fn.startswith(f"libbn_{family}-") and fn.endswith(".so") and fn != keep:
            try:
                os.remove(os.path.join(folder, fn))
            except OSError:
                pass
    if p.stdout.strip():
        log.append(p.stdout)


def ensure_built(families: Iterable[str], quiet: bool = False) -> None:
    """Compile whatever of ``families`` is not built yet, in parallel, printing progress lines."""
    todo = []
    for fam in dict.fromkeys(families):
        if fam not in SOURCES:
            raise KernelBuildError(f"unknown kernel family '{fam}'; known: {', '.join(sorted(SOURCES))}")
        if fam not in _loaded and not os.path.isfile(library_path(fam)):
            todo.append(fam)
    if not todo:
        return

    def say(msg: str) -> None:
        if not quiet:
            print(f"[bitnet.c_b200] {msg}", file=sys.stderr, flush=True)

    say(f"compiling {len(todo)} CUDA kernel famil{'y' if len(todo) == 1 else 'ies'} for sm_100a: {', '.join(todo)}")
    errors: List[BaseException] = []
    done: List[str] = []
    logs: List[str] = []

    def work(fam: str) -> None:
        try:
            _compile(fam, library_path(fam), logs)
            done.append(fam)
        except BaseException as e:  # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(f,), daemon=True) for f in todo]
    t0 = time.time()
    for t in threads:
        t.start()
    last = 0
    while any(t.is_alive() for t in threads):
        time.sleep(0.5)
        if time.time() - t0 - last >= 5:
            last = time.time() - t0
            say(f"  still compiling ({len(done)}/{len(todo)} done, {last:.0f} s)")
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    say(f"compiled {len(todo)} in {time.time() - t0:.1f} s")


def library(family: str) -> ctypes.CDLL:
    """The loaded library of ``family``; compiled first if need be."""
    lib = _loaded.get(family)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(family)
        if lib is None:
            ensure_built([family])
            path = library_path(family)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load '{path}': {e}") from None
            _loaded[family] = lib
    return lib


def build_all(quiet: bool = False) -> List[str]:
    ensure_built(SOURCES, quiet=quiet)
    return [library_path(f) for f in SOURCES]
