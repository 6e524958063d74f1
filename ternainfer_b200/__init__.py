"""TernaSpMM for NVIDIA B200: compressed ternary weights x int8 activations
-> bf16, behind the C ABI of the reference's ``libternaspmm.so``.

``ternainfer_b200.lib``      ctypes binding of the in-tree shared library
``ternainfer_b200.linear``   ``TernaInfer_linear`` / ``SpBitLinear`` call site
``ternainfer_b200.convert``  weight packer (B200 tile order) and converter
"""
from .lib import load_library, library_path  # noqa: F401

__all__ = ["load_library", "library_path"]
