"""Failures injected on the host: an allocator callback that answers NULL, and a launch check that records.

The three callbacks of the kernel layer (`cumo_cuda_runtime_malloc/free/check_kernel_launch`) belong to the host
program; libcumo_b200 carries weak defaults.  Here a small stub library with strong definitions is loaded first with
global visibility, the way the Ruby extension's own definitions take precedence inside cumo.so, and the library is
driven from a child process.  Nothing here needs a GPU (no kernel ever runs: the descriptors point nowhere), and
nothing faults one.
"""
import subprocess
import sys
import textwrap
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

STUB = r"""
#include <stddef.h>
static int mallocs, frees, checks;
char* cumo_cuda_runtime_malloc(size_t n) { (void)n; ++mallocs; return NULL; }     /* the pool is exhausted */
void  cumo_cuda_runtime_free(char* p) { (void)p; ++frees; }
void  cumo_cuda_runtime_check_kernel_launch(void) { ++checks; }
int stub_mallocs(void) { return mallocs; }
int stub_frees(void) { return frees; }
int stub_checks(void) { return checks; }
"""

CHILD = r"""
import ctypes, os, sys
from ctypes import byref
sys.path.insert(0, {root!r})
stub = ctypes.CDLL({stub!r}, mode=os.RTLD_NOW | os.RTLD_GLOBAL)          # strong definitions first, globally visible
from cumo_b200 import _lib
L = _lib.load()
fake = 0x10000000                                                        # never dereferenced: no kernel runs

def reduction(shape_in, steps_in, shape_out, steps_out):
    arg = _lib.NaReductionArg()
    arg.in_.ptr, arg.out.ptr = fake, fake
    arg.in_indexer.ndim, arg.out_indexer.ndim = len(shape_in), len(shape_out)
    total = 1
    for d, (n, s) in enumerate(zip(shape_in, steps_in)):
        arg.in_indexer.shape[d] = n; arg.in_.step[d] = s; total *= n
    arg.in_indexer.total_size = total
    total = 1
    for d, (n, s) in enumerate(zip(shape_out, steps_out)):
        arg.out_indexer.shape[d] = n; arg.out.step[d] = s; total *= n
    arg.out_indexer.total_size = total
    return arg

before = L.cb200_launch_count()
for sym, arg in (("cumo_sfloat_sum_kernel_launch", reduction((1 << 24,), (4,), (), ())),                       # long row, split
                 ("cumo_sfloat_max_index_int64_kernel_launch", reduction((1 << 24,), (4,), (), ())),
                 ("cumo_dfloat_sum_kernel_launch", reduction((4096, 65536), (8, 8 * 4096), (4096,), (8,))),    # column plan, split
                 ("cumo_int32_sum_kernel_launch", reduction((64, 1 << 16, 3), (4 * 3 * (1 << 16), 4 * 3 + 4, 4), (64,), (8,)))):   # generic plan, split
    f = getattr(L, sym); f.restype = None; f.argtypes = None
    n0 = stub.stub_mallocs()
    f(byref(arg))
    assert stub.stub_mallocs() == n0 + 1, sym + ": scratch was not asked for"
f = L.cumo_sfloat_mulsum_reduce_kernel_launch; f.restype = None
f(ctypes.c_void_p(fake), ctypes.c_void_p(fake), ctypes.c_void_p(fake), ctypes.c_ssize_t(4), ctypes.c_ssize_t(4), ctypes.c_uint64(1 << 24))
assert stub.stub_mallocs() == 5
# with no scratch nothing may be launched (a first pass would write its partials through the null pointer)
assert L.cb200_launch_count() == before, "kernels were launched without scratch"
assert stub.stub_frees() == 0 and stub.stub_checks() == 0
# the launch check belongs to the host program too: it is called once per entry point that launches
ix = _lib.NaIndexer(); ix.ndim = 1; ix.total_size = 64; ix.shape[0] = 64
a = _lib.NaIArray(); a.ptr = fake; a.step[0] = 4
g = L.cumo_iter_sfloat_add_kernel_launch; g.restype = None; g.argtypes = None
g(byref(a), byref(a), byref(a), byref(ix), None)
assert stub.stub_checks() == 1
print("ok")
"""


def test_null_scratch_launches_nothing_and_the_strong_callbacks_win(tmp_path):
    src = tmp_path / "stub.c"
    src.write_text(STUB)
    lib = tmp_path / "libstub_callbacks.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(lib), str(src)], check=True)
    child = tmp_path / "child.py"
    child.write_text(textwrap.dedent(CHILD.format(root=str(ROOT), stub=str(lib))))
    res = subprocess.run([sys.executable, str(child)], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "ok" in res.stdout, res.stdout + res.stderr
