"""The shared library loads without a GPU and exports every function include/bpdq.h declares."""
import ctypes
import os
import re

from bpd_substrate_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "bpdq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?(?:void|int|float|size_t)\s*\*?\s*(\w+)\s*\(", text, flags=re.M)
    return sorted(set(names))


def test_header_declares_the_reference_surface():
    names = declared_functions()
    for must in ("bpd_dequant_q4k_gpu", "bpd_qmatmul_q4k_q8k_cuda", "qgpu_alloc", "qgpu_h2d", "qgpu_d2h", "qgpu_sync",
                 "run_bpd", "run_llamacpp", "dequant_v1_32", "dequant_multi8", "sgpu_alloc", "galloc", "gpu_alloc",
                 "gpu_copy_h2d", "gpu_sync", "gpu_vecmat_q4k", "gpu_matmul_q4k"):
        assert must in names, must
    assert len(names) >= 60


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(capi.lib_path()) if os.path.exists(capi.lib_path()) else capi.load()
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_table_matches_header():
    assert sorted(capi.SIGNATURES) == declared_functions()
    capi.load()   # binds every entry; raises AttributeError on a missing symbol
