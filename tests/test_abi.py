"""CPU: the shared library loads and exports every symbol the header declares."""
import os
import re

from ternainfer_b200.lib import EXPORTED_SYMBOLS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ternaspmm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\(", text)) - {"defined"})


def test_header_symbols_are_exported(lib):
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ternaspmm.h but not exported"
    assert set(EXPORTED_SYMBOLS) == set(names)


def test_reference_entry_points_present(lib):
    # the eight extern "C" symbols of the reference's kernels/TernaSpMM.cu
    for n in ("checkLastCudaError", "bitlinear_TernaSpMM", "bitlinear_TernaSpMM_decode",
              "bitlinear_TernaSpMM_prefill", "bitlinear_TernaSpMM_benchmark", "reorder_WT_h",
              "convert_reorderd", "gpu_sleep"):
        assert hasattr(lib, n)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "ternainfer_b200")
    for dp, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dp, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"
