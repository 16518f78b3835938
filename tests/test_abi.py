"""CPU tests of the drop-in boundary: the shared library loads without a GPU and exports every symbol that
include/nt_b200.h declares, plus the reference's mangled C++ launcher names (src/cuda/kernels.h:10-74)."""
import re
import subprocess
from pathlib import Path

from ntransformer_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "nt_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(nt_b200_\w+|nt_cuda_\w+)\s*\(", text))


def test_library_loads_and_exports_every_declared_symbol():
    lib = _lib.lib()
    decl = declared_symbols()
    assert len(decl) >= 30
    for name in sorted(decl):
        assert hasattr(lib, name), f"{name} declared in include/nt_b200.h but not exported"
    assert decl == set(_lib.SIGNATURES), "python binding table and header disagree"
    assert lib.nt_b200_version().startswith(b"ntransformer_b200")
    assert lib.nt_b200_xq_bytes(8192) == 3 * 8192 + 8192 // 32 * 4 + 8192 // 16 * 4


def test_reference_cxx_launcher_names_are_exported():
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", str(_lib.LIB_PATH)], capture_output=True, text=True, check=True).stdout
    for fn in _lib.CXX_LAUNCHERS:
        assert re.search(rf"\bnt::cuda::{fn}\(", out), f"nt::cuda::{fn} missing"
    # the exact signature the reference host code calls (kernels.h:34-36)
    assert "nt::cuda::launch_gemv(float*, void const*, float const*, int, int, nt::DType, void*)" in out


def test_emulator_hooks_stay_out_of_the_product():
    """tests/cusim compiles some product sources with -DNT_CUSIM; the product build never defines it and carries no emulator code."""
    from ntransformer_b200 import build as nb

    assert not any("NT_CUSIM" in f for f in nb.COMMON + nb.ARCH)
    syms = subprocess.run(["nm", "-D", "-C", str(_lib.LIB_PATH)], capture_output=True, text=True, check=True).stdout
    assert "cusim" not in syms
    pkg = ROOT / "ntransformer_b200"
    for f in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cpp")) + list(pkg.rglob("*.h")) + list(pkg.rglob("*.cuh")):
        if "_build" in f.parts:
            continue
        text = f.read_text(errors="replace")
        if re.search(r'cusim::|#include "cusim', text):               # code (not a comment pointing at tests/cusim)
            assert "#ifdef NT_CUSIM" in text, f


def test_product_never_touches_the_oracle():
    """The oracle is test infrastructure: nothing under ntransformer_b200/ may import, link or execute it."""
    pkg = ROOT / "ntransformer_b200"
    for f in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cpp")) + list(pkg.rglob("*.h")) + list(pkg.rglob("*.cuh")):
        if "_build" in f.parts:
            continue
        text = f.read_text(errors="replace")
        assert "nt_oracle" not in text and "import oracle" not in text and "from oracle" not in text, f
    out = subprocess.run(["ldd", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout
    assert "oracle" not in out
