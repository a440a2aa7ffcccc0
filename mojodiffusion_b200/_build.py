"""In-tree build of the native library.

Every ``csrc/*.cu`` file is compiled by nvcc for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``)
into ``build/obj`` and linked, together with the torch binding (``csrc/bindings.cpp``, built by g++ against
the torch headers), into ``mojodiffusion_b200/_C.so``. Objects are cached by a hash of the source, the
headers it can include and the flags, so a rebuild after a one-file edit takes seconds. The library stays
inside the package directory on purpose: it is loaded from there with ``torch.ops.load_library`` and never
installed into site-packages.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG.parent / "build" / "obj"
LIB = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _hash(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _flags_for(src: Path):
    """A source whose first line is ``// build: precise-math`` is compiled without fast-math and without
    multiply-add contraction (bit-stable fp32 arithmetic for the image filters)."""
    first = src.read_text().split("\n", 1)[0]
    if "build: precise-math" in first:
        return [f for f in NVCC_FLAGS if f != "--use_fast_math"] + ["-fmad=false"]
    return NVCC_FLAGS


def _compile_cu(src: Path, headers, verbose: bool) -> Path:
    NVCC_FLAGS = _flags_for(src)
    tag = _hash([src, *headers], " ".join(NVCC_FLAGS))
    out = OBJ / f"{src.stem}.{tag}.o"
    if out.exists():
        return out
    for old in OBJ.glob(f"{src.stem}.*.o"):
        old.unlink()
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(out)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return out


def _compile_cpp(src: Path, headers) -> Path:
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    flags = ["-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             "-DTORCH_EXTENSION_NAME=_C", "-I", "/usr/local/cuda/include", "-I", str(CSRC)]
    tag = _hash([src, *headers], " ".join(flags) + torch.__version__)
    out = OBJ / f"{src.stem}.{tag}.o"
    if out.exists():
        return out
    for old in OBJ.glob(f"{src.stem}.*.o"):
        old.unlink()
    cmd = ["g++", *flags, *inc, "-c", str(src), "-o", str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return out


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile (if needed) and link ``_C.so``; returns its path."""
    import torch
    from torch.utils import cpp_extension as ce

    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))
    cus = sorted(CSRC.glob("*.cu"))
    cpps = sorted(CSRC.glob("*.cpp"))
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        futs = [ex.submit(_compile_cu, s, headers, verbose) for s in cus]
        futs += [ex.submit(_compile_cpp, s, headers) for s in cpps]
        objs = [f.result() for f in futs]
    stamp = OBJ / "link.stamp"
    key = " ".join(o.name for o in objs)
    if LIB.exists() and stamp.exists() and stamp.read_text() == key and not force:
        return LIB
    libdirs = ce.library_paths()
    cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-Xcompiler", "-fPIC"]
    for d in libdirs:
        cmd += ["-L", d, "-Xlinker", f"-rpath={d}"]
    cmd += ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(key)
    return LIB


SERVE = PKG / "serve"


def build_control_plane(force: bool = False):
    """Compile the serving control plane (``serve/control_plane/*.cpp``, C++17, no dependencies beyond libc/pthread)
    into ``serve/bin/mdb-server`` and ``serve/bin/mdb-lower``. Returns the two paths."""
    src = SERVE / "control_plane"
    out_dir = SERVE / "bin"
    out_dir.mkdir(parents=True, exist_ok=True)
    headers = sorted(src.glob("*.hpp"))
    outs = []
    for name, main in (("mdb-server", "server.cpp"), ("mdb-lower", "lower_main.cpp")):
        out = out_dir / name
        tag = _hash([src / main, *headers], "c++17 O2")
        stamp = out_dir / f".{name}.stamp"
        if not (out.exists() and stamp.exists() and stamp.read_text() == tag and not force):
            cmd = ["g++", "-std=c++17", "-O2", "-pthread", "-o", str(out), str(src / main)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"g++ failed for {main}:\n{r.stdout}\n{r.stderr}")
            stamp.write_text(tag)
        outs.append(out)
    return outs


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
    print(*build_control_plane(force="-f" in sys.argv))
