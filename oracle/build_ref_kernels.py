"""Builds the reference's OWN CUDA kernels for the hot path, outside the Ruby extension
(TEST / BENCH INFRASTRUCTURE, not product).

`python -m oracle.build_ref_kernels [reference checkout]` expands the reference's kernel
templates for sfloat, dfloat, int32, int64 and bit (oracle/ref_templates.py: the generator restated
without Ruby), writes the expanded units under oracle/_ref/src/, compiles them with nvcc against
the reference's own headers (`ext/cumo/include`) for plain sm_100 -- the way the extension's own
build would on this GPU, no fast-math (ext/cumo/extconf.rb:29-35) -- and links
oracle/_ref/libcumo_ref_kernels.so together with the three host callbacks of oracle/ref_callbacks.cu.
Everything it writes stays under oracle/_ref/, which is not tracked: no reference source enters
the repository.  The library is the baseline that bench.py times beside libcumo_b200 on the same
GPU and the second oracle of tests/test_gpu_ref_kernels.py (bit-for-bit where both run the same
CUDA math library).  It is never linked into, loaded by or shipped with libcumo_b200.

The reference checkout is only needed to BUILD; where it is absent (the GPU box) the prebuilt
library is used as it is, and where that is absent too the users skip.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
LIB = OUT / "libcumo_ref_kernels.so"
# where the reference checkout is looked for: CUMO_REFERENCE_ROOT, else a `reference` directory beside this repository
DEFAULT_REF = Path(os.environ.get("CUMO_REFERENCE_ROOT") or HERE.parent.parent / "reference")

# templates (by erb_base) expanded per element type: the hot path and the rows next to it
VALUE_TEMPLATES = {"binary", "binary_s", "unary", "unary_s", "unary2", "cond_binary", "cond_unary", "pow", "ewcomp",
                   "store_from", "accum", "accum_index", "accum_arg", "accum_binary", "bincount", "cum",
                   "clip", "fill", "seq", "binary2", "unary_ret2", "frexp", "store_bit", "poly", "eye"}
BIT_TEMPLATES = {"bit_count", "where", "mask", "binary", "unary", "bit_reduce", "store_from", "store_bit", "fill"}
TYPES = ("sfloat", "dfloat", "int32", "int64", "bit")

NVCC_FLAGS = ["-gencode", "arch=compute_100,code=sm_100", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-DHAVE_STDINT_H", "-DHAVE_STDBOOL_H", "-DHAVE_TYPE_BOOL", "-DHAVE_SYS_TYPES_H",
              # what the extension's own configure step finds on Linux/glibc (ext/cumo/extconf.rb:140 have_func("exp10")):
              # with it m_exp10 is exp10(x), without it pow(10, x) (types/float_macro_kernel.h:96-100)
              "-DHAVE_EXP10", "-w"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def up_to_date() -> bool:
    if not LIB.exists():
        return False
    t = LIB.stat().st_mtime
    return all(p.stat().st_mtime <= t for p in (Path(__file__), HERE / "ref_templates.py", HERE / "ref_callbacks.cu"))


def build(ref_root: Path = DEFAULT_REF, force: bool = False) -> Path | None:
    """Returns the library's path, or None when there is neither a reference checkout nor a prebuilt library."""
    ref_root = Path(ref_root)
    if not (ref_root / "ext/cumo/narray/gen/spec.rb").exists():
        return LIB if LIB.exists() else None
    if not force and up_to_date():
        return LIB
    from oracle import ref_templates as rt

    src_dir = OUT / "src"
    src_dir.mkdir(parents=True, exist_ok=True)
    units = []
    for t in TYPES:
        gen = rt.Generator(ref_root, t)
        text = gen.kernel_unit(BIT_TEMPLATES if t == "bit" else VALUE_TEMPLATES)
        p = src_dir / f"{t}_kernel.cu"
        p.write_text(text)
        units.append(p)
    units.append(HERE / "ref_callbacks.cu")

    def compile_one(src: Path) -> Path:
        obj = OUT / (src.stem + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(ref_root / "ext/cumo/include"), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=max(1, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(compile_one, units))
    # -Bsymbolic: the library's calls to the three callbacks bind to its own definitions even when libcumo_b200
    # (which carries weak ones of the same names) is already loaded with global visibility in the same process
    cmd = [_nvcc(), "-shared", "-cudart", "static", "-Xlinker", "-Bsymbolic", "-o", str(LIB), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link of libcumo_ref_kernels.so failed")
    return LIB


if __name__ == "__main__":
    paths = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(Path(paths[0]) if paths else DEFAULT_REF, force="--force" in sys.argv))
