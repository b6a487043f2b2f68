"""The C interface of the library (``bn_api.h``): a shared object that C programs link, in the
shape of the reference's public headers, over the library's one engine.

``build()`` compiles ``libbitnet_b200.so`` beside the sources (``capi/_build/``) with the system's C
compiler against this interpreter's headers and returns its path.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

_HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(_HERE, "bn_api.h")


def build(force: bool = False) -> str:
    out_dir = os.path.join(_HERE, "_build")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "libbitnet_b200.so")
    src = os.path.join(_HERE, "bn_api.c")
    if not force and os.path.isfile(out) and os.path.getmtime(out) >= max(os.path.getmtime(src), os.path.getmtime(HEADER)):
        return out
    inc = sysconfig.get_paths()["include"]
    libdir = sysconfig.get_config_var("LIBDIR") or ""
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    cmd = [os.environ.get("CC", "gcc"), "-O2", "-shared", "-fPIC", f'-DBN_PYTHON_EXECUTABLE="{sys.executable}"',
           "-I", inc, "-I", _HERE, src, "-o", out,
           f"-L{libdir}", f"-Wl,-rpath,{libdir}", f"-lpython{ver}", "-ldl"]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"building the C interface failed:\n{' '.join(cmd)}\n{p.stdout}")
    return out


def link_flags() -> list:
    """What a C program adds to its compiler line to use the interface."""
    out = build()
    d = os.path.dirname(out)
    return ["-I", _HERE, f"-L{d}", f"-Wl,-rpath,{d}", "-lbitnet_b200"]
