"""The C-ABI library loads without a GPU and exports every function that include/*.h declares."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADERS = sorted((ROOT / "include").glob("*.h"))


def declared_functions(header: Path) -> list[str]:
    text = subprocess.run(["gcc", "-E", "-P", "-x", "c", str(header)], check=True, capture_output=True, text=True).stdout
    # prototypes only: `type name(args);` at file scope after preprocessing
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}()]*(?:\([^)]*\)[^;{}()]*)*\)\s*;", text)
    return sorted({n for n in names if n.startswith(("cumo_", "cb200_"))})


def test_headers_declare_the_expected_families():
    names = declared_functions(ROOT / "include" / "cumo_b200.h")
    for must in ("cumo_iter_sfloat_add_kernel_launch", "cumo_iter_sfloat_add_s_kernel_launch",
                 "cumo_iter_sfloat_math_s_exp_kernel_launch", "cumo_iter_int32_mod_kernel_launch",
                 "cumo_iter_int32_gt_s_kernel_launch", "cumo_sfloat_sum_kernel_launch", "cumo_dfloat_mean_kernel_launch",
                 "cumo_sfloat_max_index_int32_kernel_launch", "cumo_dfloat_argmin_nan_int64_kernel_launch",
                 "cumo_iter_bit_count_true_stride_kernel_launch", "cumo_int64_mulsum_reduce_kernel_launch",
                 "cumo_cuda_runtime_malloc"):
        assert must in names, must
    assert len(names) > 400


@pytest.mark.parametrize("header", HEADERS, ids=lambda p: p.name)
def test_library_exports_every_declared_symbol(header):
    from cumo_b200 import _lib

    lib = _lib.load()
    missing = []
    for name in declared_functions(header):
        try:
            getattr(lib, name)
        except AttributeError:
            missing.append(name)
    assert not missing, f"{len(missing)} declared but not exported, e.g. {missing[:5]}"


def test_descriptor_layouts_match_the_reference_abi():
    """sizeof/offsets that a C caller compiled against the reference's indexer.h would use."""
    from cumo_b200 import _lib

    assert ctypes.sizeof(_lib.NaIArray) == 8 + 12 * 8
    assert ctypes.sizeof(_lib.NaIndexer) == 8 + 8 + 12 * 8 + 12 * 8 + 8
    assert _lib.NaIndexer.total_size.offset == 8
    assert _lib.NaIndexer.shape.offset == 16
    assert ctypes.sizeof(_lib.NaBitIArray) == 8 + 8 + 12 * 8
    assert ctypes.sizeof(_lib.NaReductionArg) == 2 * ctypes.sizeof(_lib.NaIArray) + 2 * ctypes.sizeof(_lib.NaIndexer)
    src = r'''
    #include <stdio.h>
    #include "cumo_b200.h"
    int main(void) { printf("%zu %zu %zu %zu %zu %zu\n", sizeof(cumo_na_iarray_t), sizeof(cumo_na_indexer_t),
        sizeof(cumo_na_bit_iarray_t), sizeof(cumo_na_reduction_arg_t), offsetof(cumo_na_indexer_t, shape),
        offsetof(cumo_na_reduction_arg_t, in_indexer)); return 0; }
    '''
    import tempfile
    with tempfile.TemporaryDirectory() as d:
        c = Path(d) / "t.c"
        c.write_text(src)
        subprocess.run(["gcc", "-I", str(ROOT / "include"), str(c), "-o", str(Path(d) / "t")], check=True)
        got = subprocess.run([str(Path(d) / "t")], check=True, capture_output=True, text=True).stdout.split()
    assert [int(v) for v in got] == [ctypes.sizeof(_lib.NaIArray), ctypes.sizeof(_lib.NaIndexer), ctypes.sizeof(_lib.NaBitIArray),
                                     ctypes.sizeof(_lib.NaReductionArg), _lib.NaIndexer.shape.offset, _lib.NaReductionArg.in_indexer.offset]
