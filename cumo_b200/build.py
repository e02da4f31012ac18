"""In-tree build of libcumo_b200.so (sm_100a only).

`python -m cumo_b200.build` compiles every translation unit under `csrc/` with
nvcc for `arch=compute_100a,code=sm_100a` (objects in `cumo_b200/_build/`, several
nvcc processes in parallel) and links `cumo_b200/libcumo_b200.so`.  Nothing is
rebuilt when the library is newer than every source; an object is rebuilt when
its source or a header nvcc recorded for it (`-MD`) is newer than it.  nvcc cross-compiles, so no
GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "_build"
LIB = PKG / "libcumo_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xcudafe", "--diag_suppress=550",
]
# CB200_NVTX=1 in the environment of the build puts an NVTX range (the launch function's full name, template arguments
# included) around every host-side launch function; without it the ranges compile to nothing.  (A change of this
# variable needs `--force`: objects are not keyed by it.)
if os.environ.get("CB200_NVTX", "0") not in ("", "0"):
    NVCC_FLAGS.append("-DCB200_NVTX")


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libcumo_b200 cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(CSRC.rglob("*.cu")) + sorted(CSRC.rglob("*.cpp"))


def _deps() -> list[Path]:
    return sources() + sorted(CSRC.rglob("*.cuh")) + sorted(CSRC.rglob("*.h")) + sorted((PKG.parent / "include").glob("*.h")) + [Path(__file__)]


def up_to_date() -> bool:
    if not LIB.exists():
        return False
    t = LIB.stat().st_mtime
    return all(p.stat().st_mtime <= t for p in _deps())


def _recorded_deps(depfile: Path) -> list[Path] | None:
    """The headers nvcc listed for one object (make-style .d file); None when there is no usable record."""
    if not depfile.exists():
        return None
    text = depfile.read_text().replace("\\\n", " ")
    parts = text.split(":", 1)
    if len(parts) != 2:
        return None
    deps = [Path(p) for p in parts[1].split() if p.startswith(str(PKG.parent))]
    return deps if all(p.exists() for p in deps) else None


def _compile(src: Path, verbose: bool, extra: list[str]) -> Path:
    obj = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
    depfile = obj.with_suffix(".d")
    deps = _recorded_deps(depfile)
    if deps is None:                       # no record yet: any header of the project counts
        deps = [p for p in _deps() if p.suffix in (".cuh", ".h") or p == src]
    newest = max([p.stat().st_mtime for p in deps] + [src.stat().st_mtime, Path(__file__).stat().st_mtime])
    if obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, *extra, "-MD", "-MF", str(depfile), "-I", str(PKG.parent / "include"), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if src.suffix == ".cpp":
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}")
    return obj


def build(force: bool = False, verbose: bool = False, jobs: int | None = None, extra: list[str] | None = None) -> Path:
    if not force and up_to_date():
        return LIB
    OBJ.mkdir(exist_ok=True)
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    jobs = jobs or max(1, (os.cpu_count() or 2))
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, extra or []), sources()))
    cmd = [nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link of libcumo_b200.so failed")
    return LIB


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="pass -Xptxas -v (registers, spills, shared memory)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose or a.ptxas_info, extra=["-Xptxas", "-v"] if a.ptxas_info else None))
