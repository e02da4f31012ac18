"""libcumo_b200 against the reference-derived list of launch functions (tests/golden/abi_manifest.txt).

The list holds every function that the reference's generated kernel units define for the templates the
drop-in overlay blanks (made by tests/golden/make_abi_manifest.py from the reference, not from this
project's header).  With the overlay in place those definitions are gone from cumo.so, so each of them
must be exported by the library, and declared in include/cumo_b200.h with the same return type and
argument types -- otherwise `require 'cumo/narray'` fails at load, or calls go through a mismatched
prototype.  Needs no GPU and no reference checkout.
"""
import re
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
MANIFEST = ROOT / "tests" / "golden" / "abi_manifest.txt"
ALIASES = {"CUMO_BIT_DIGIT": "unsigned int", "cb200_cuda_status_t": "cudaError_t", "u_int64_t": "uint64_t", "u_int32_t": "uint32_t"}


def norm_type(t: str) -> str:
    t = re.sub(r"\s*\*\s*", "*", t.strip())
    t = re.sub(r"\s+", " ", t)
    for a, b in ALIASES.items():
        t = re.sub(rf"\b{a}\b", b, t)
    return t


def manifest():
    out = {}
    for line in MANIFEST.read_text().splitlines():
        if not line or line.startswith("#"):
            continue
        m = re.fullmatch(r"(.+?) (\w+)\((.*)\)", line)
        args = [norm_type(a) for a in m.group(3).split(",") if a.strip()]
        out[m.group(2)] = (norm_type(m.group(1)), args)
    return out


def header_prototypes():
    text = subprocess.run(["gcc", "-E", "-P", "-x", "c", str(ROOT / "include" / "cumo_b200.h")], check=True, capture_output=True, text=True).stdout
    out = {}
    for m in re.finditer(r"([A-Za-z_][\w \t]*?[\w*])\s*\b((?:cumo|cb200)_\w+)\s*\(([^;{}()]*)\)\s*;", text):
        ret, name, args = m.group(1), m.group(2), m.group(3)
        ret = ret.split(";")[-1].replace("extern", "").strip()
        types = []
        for a in args.split(","):
            a = a.strip()
            if not a or a == "void":
                continue
            a = re.sub(r"\bconst\b", "", a)
            a = re.sub(r"\b\w+$", "", a).strip() if re.search(r"[\w*]\s*\b\w+$", a) and not re.fullmatch(r"(unsigned |signed )?\w+\**", a) else a
            types.append(norm_type(a))
        out[name] = (norm_type(ret), types)
    return out


def test_manifest_is_not_trivial():
    m = manifest()
    assert len(m) > 430
    for name in ("cumo_iter_sfloat_store_uint8_kernel_launch", "cumo_iter_int64_store_int64_stridx_kernel_launch",
                 "cumo_dfloat_kahan_sum_nan_kernel_launch", "cumo_iter_int32_pow_int32_s_left_kernel_launch",
                 "cumo_iter_bit_count_false_index_stride_kernel_launch", "cumo_bit_mask_kernel_launch"):
        assert name in m, name


def test_library_exports_every_function_the_overlay_removes():
    from cumo_b200 import _lib

    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], check=True, capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if l.split()[-2:-1] and l.split()[-2] in ("T", "W")}
    missing = sorted(set(manifest()) - exported)
    assert not missing, f"{len(missing)} reference launch functions are not exported, e.g. {missing[:8]}"


def test_header_declares_them_with_the_reference_argument_lists():
    want, got = manifest(), header_prototypes()
    undeclared = sorted(set(want) - set(got))
    assert not undeclared, f"{len(undeclared)} not declared in include/cumo_b200.h, e.g. {undeclared[:8]}"
    wrong = [(n, want[n], got[n]) for n in sorted(want) if want[n] != got[n]]
    assert not wrong, f"{len(wrong)} prototypes differ from the reference's, e.g. {wrong[:3]}"
