"""In-tree build of the native libraries.

``build_all()`` compiles every ``.cu`` under ``csrc/cuda`` for sm_100a into
``torchrec_b200/_C_cuda.so`` and every ``.cpp`` under ``csrc/cpu`` into
``torchrec_b200/_C_cpu.so``.  Objects are cached under ``csrc/_obj`` keyed by a hash of the
source, the headers next to it and the flags, so an unchanged file is never recompiled.
nvcc cross-compiles without a GPU, which makes this usable as a build check on a CPU box.

Usage: ``python -m torchrec_b200.csrc.build [--verbose] [--force]``
"""
from __future__ import annotations

import glob
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OBJ = os.path.join(HERE, "_obj")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _torch_paths() -> Tuple[List[str], str]:
    import torch
    from torch.utils import cpp_extension as ce

    return ce.include_paths("cuda"), os.path.join(os.path.dirname(torch.__file__), "lib")


def _cuda_home() -> str:
    for c in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if c and os.path.exists(os.path.join(c, "bin", "nvcc")):
            return c
    nv = shutil.which("nvcc")
    if nv:
        return os.path.dirname(os.path.dirname(nv))
    raise RuntimeError("nvcc not found")


def _hash(paths: List[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:24]


def _run(cmd: List[str], verbose: bool) -> str:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed ({r.returncode}): {' '.join(cmd)}\n{r.stdout}")
    return r.stdout


def _compile_objects(sources: List[str], headers: List[str], make_cmd, flags_key: str, verbose: bool, force: bool) -> List[str]:
    os.makedirs(OBJ, exist_ok=True)
    jobs = []
    objs = []
    for src in sources:
        base = os.path.splitext(os.path.basename(src))[0]
        tag = _hash([src] + headers, flags_key)
        obj = os.path.join(OBJ, f"{base}.{tag}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            for old in glob.glob(os.path.join(OBJ, f"{base}.*.o")):
                os.remove(old)
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            outs = list(ex.map(lambda so: _run(make_cmd(so[0], so[1]), verbose), jobs))
        if verbose:
            for o in outs:
                if o.strip():
                    print(o)
    return objs


def build_cuda(verbose: bool = False, force: bool = False, ptxas_verbose: bool = False) -> str:
    inc, torch_lib = _torch_paths()
    cuda = _cuda_home()
    nvcc = os.path.join(cuda, "bin", "nvcc")
    srcs = sorted(glob.glob(os.path.join(HERE, "cuda", "*.cu")))
    hdrs = sorted(glob.glob(os.path.join(HERE, "cuda", "*.cuh")) + glob.glob(os.path.join(HERE, "cuda", "*.h")))
    flags = (
        NVCC_ARCH
        + ["-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda", "--use_fast_math",
           "-Xcompiler", "-fPIC", "-DTORCH_API_INCLUDE_EXTENSION_H", "-D_GLIBCXX_USE_CXX11_ABI=1",
           "-diag-suppress", "177,550,186"]
        + (["-Xptxas", "-v"] if ptxas_verbose else [])
        + [f"-I{p}" for p in inc]
    )

    def cmd(src: str, obj: str) -> List[str]:
        return [nvcc] + flags + ["-c", src, "-o", obj]

    objs = _compile_objects(srcs, hdrs, cmd, " ".join(flags), verbose or ptxas_verbose, force)
    out = os.path.join(PKG, "_C_cuda.so")
    link_tag = _hash(objs, "link-cuda")
    stamp = os.path.join(OBJ, "cuda.link")
    if force or not os.path.exists(out) or not os.path.exists(stamp) or open(stamp).read() != link_tag:
        _run(
            ["g++", "-shared", "-o", out] + objs
            + [f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda",
               f"-L{os.path.join(cuda, 'lib64')}", "-lcudart", f"-Wl,-rpath,{torch_lib}"],
            verbose,
        )
        with open(stamp, "w") as f:
            f.write(link_tag)
    return out


def build_cpu(verbose: bool = False, force: bool = False) -> str:
    inc, torch_lib = _torch_paths()
    srcs = sorted(glob.glob(os.path.join(HERE, "cpu", "*.cpp")))
    out = os.path.join(PKG, "_C_cpu.so")
    if not srcs:
        return out
    hdrs = sorted(glob.glob(os.path.join(HERE, "cpu", "*.h")))
    flags = ["-O2", "-std=c++17", "-fPIC", "-D_GLIBCXX_USE_CXX11_ABI=1", "-pthread", "-Wno-unused-result"] + [
        f"-I{p}" for p in inc if "cuda" not in os.path.basename(p.rstrip("/"))
    ]

    def cmd(src: str, obj: str) -> List[str]:
        return ["g++"] + flags + ["-c", src, "-o", obj]

    objs = _compile_objects(srcs, hdrs, cmd, " ".join(flags), verbose, force)
    link_tag = _hash(objs, "link-cpu")
    stamp = os.path.join(OBJ, "cpu.link")
    if force or not os.path.exists(out) or not os.path.exists(stamp) or open(stamp).read() != link_tag:
        _run(
            ["g++", "-shared", "-o", out] + objs
            + [f"-L{torch_lib}", "-lc10", "-ltorch_cpu", "-ltorch", "-ldl", "-pthread", f"-Wl,-rpath,{torch_lib}"],
            verbose,
        )
        with open(stamp, "w") as f:
            f.write(link_tag)
    return out


def build_plugins(verbose: bool = False, force: bool = False) -> List[str]:
    """Run-time plugins of the dynamic-embedding library (``cpu/plugins/<name>.cpp`` -> ``torchrec_b200/_tde_<name>.so``); they
    depend on the plugin ABI header only, not on the tensor library."""
    outs = []
    hdrs = sorted(glob.glob(os.path.join(HERE, "cpu", "*.h")))
    for src in sorted(glob.glob(os.path.join(HERE, "cpu", "plugins", "*.cpp"))):
        name = os.path.splitext(os.path.basename(src))[0]
        out = os.path.join(PKG, f"_tde_{name}.so")
        tag = _hash([src] + hdrs, "plugin")
        stamp = os.path.join(OBJ, f"plugin_{name}.stamp")
        os.makedirs(OBJ, exist_ok=True)
        if force or not os.path.exists(out) or not os.path.exists(stamp) or open(stamp).read() != tag:
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-o", out, src], verbose)
            with open(stamp, "w") as f:
                f.write(tag)
        outs.append(out)
    return outs


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_cuda(verbose=verbose, force=force)
    build_cpu(verbose=verbose, force=force)
    build_plugins(verbose=verbose, force=force)


if __name__ == "__main__":
    v = "--verbose" in sys.argv
    if "--ptxas" in sys.argv:
        build_cuda(verbose=True, force=True, ptxas_verbose=True)
    else:
        build_all(verbose=v, force="--force" in sys.argv)
    print("built:", os.path.join(PKG, "_C_cuda.so"), os.path.join(PKG, "_C_cpu.so"))
