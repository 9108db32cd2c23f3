"""The reference's own launcher source (src/gpu_ops.cpp) and module loader (src/kernel_loader.cpp), compiled UNCHANGED
against the hip/ shim headers into oracle/_ref/libref_gpu_ops.so (oracle/Makefile, target ref_programs), driving this
library's kernels by name: INFERENCE_KERNEL_DIR points at a directory holding a module image as gpu_ops.co, and the
reference's gpu_add_rmsnorm / gpu_swiglu then give the results of this library's native launchers of the same name on
the same inputs (identical up to the summation order inside a row reduction: compared at 1e-6 of the row maximum;
integer outputs exactly). The image is built here from the library's named kernels plus empty kernels under the
twenty names of other model families that the reference's init insists on finding (tests/ref_init_image.cu)."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

from rocm_hip_b200 import _lib
from util import max_rel_rows

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libref_gpu_ops.so")
NAMES = ["gpu_add_rmsnorm", "gpu_swiglu"]


@pytest.fixture(scope="module")
def both(ops, tmp_path_factory):
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libref_gpu_ops.so was not built (the reference's source tree was absent at build time)")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is needed to build the module image for the reference's loader")
    d = tmp_path_factory.mktemp("kernels")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                    "-I", os.path.join(ROOT, "rocm_hip_b200", "csrc"), "-fatbin", "-o", str(d / "gpu_ops.co"),
                    os.path.join(ROOT, "tests", "ref_init_image.cu")], check=True)
    os.environ["INFERENCE_KERNEL_DIR"] = str(d)
    ref = C.CDLL(REF_LIB)
    ref.gpu_ops_init.restype, ref.gpu_ops_init.argtypes = C.c_int, [C.c_char_p]
    for n in NAMES:
        getattr(ref, n).restype, getattr(ref, n).argtypes = _lib.SIGNATURES[n]
    assert ref.gpu_ops_init(b"gpu_ops.co") == 0, "the reference's gpu_ops_init did not find its kernels in the module image"
    yield ref, _lib.load()
    ref.gpu_ops_free()
    del os.environ["INFERENCE_KERNEL_DIR"]


P = lambda t: None if t is None else C.c_void_p(t.data_ptr())
R = lambda *s: torch.randn(*s, device="cuda")
Z = lambda *s: torch.zeros(*s, device="cuda")
ST = C.c_void_p(0)


def run_both(both, name, make_args, outputs, exact=False):
    """Calls launcher `name` of the reference build and of this library with fresh argument lists from make_args()
    (which returns (args, output tensors)) and compares the outputs."""
    ref, mine = both
    res = []
    for lib in (ref, mine):
        torch.manual_seed(1234)
        args, outs = make_args()
        code = getattr(lib, name)(*args)
        torch.cuda.synchronize()
        assert code == 0, (name, code)
        res.append([o.clone() for o in outs])
    for a, b in zip(*res):
        if exact or a.dtype != torch.float32:
            assert torch.equal(a, b), name
        else:
            an, bn = a.cpu().numpy(), b.cpu().numpy()
            assert max_rel_rows(an.reshape(an.shape[0], -1), bn.reshape(bn.shape[0], -1)) <= 1e-6, name


def q8_struct(K, keep):
    bufs = dict(q0=torch.zeros(K, dtype=torch.int8, device="cuda"), d0=Z(K // 32), qK=torch.zeros(K, dtype=torch.int8, device="cuda"),
                dK=Z(K // 256), bsK=torch.zeros(K // 16, dtype=torch.int32, device="cuda"),
                s0=torch.zeros(K // 32, dtype=torch.int32, device="cuda"), xh=torch.zeros(K, dtype=torch.int16, device="cuda"))
    keep.append(bufs)
    g = lambda k: bufs[k].data_ptr()
    return _lib.qmatvec_q8(g("q0"), g("d0"), g("qK"), g("dK"), g("bsK"), g("s0"), K, g("xh"), 1), bufs


def test_add_rmsnorm_and_swiglu_through_the_reference_launchers(both):
    keep = []
    T, n = 9, 1024

    def rms(add, q8):
        def mk():
            x, a, w = R(T, n), R(T, n), 1 + 0.1 * R(n)
            xo, y = Z(T, n), Z(T, n)
            s, bufs = q8_struct(T * n, keep) if q8 else (None, {})
            keep.extend([x, a, w])
            return [P(x), P(a) if add else None, P(xo), P(w), P(y), n, T, 1e-6, C.byref(s) if q8 else None, ST], \
                [y, xo] + [bufs[k] for k in ("q0", "qK", "xh")] if q8 else [y, xo]
        return mk
    for add in (False, True):
        for q8 in (False, True):
            run_both(both, "gpu_add_rmsnorm", rms(add, q8), None)

    def swiglu():
        g, u, o = R(T * n), R(T * n), Z(T * n)
        s, bufs = q8_struct(T * n, keep)
        keep.extend([g, u])
        return [P(g), P(u), P(o), T * n, C.byref(s), ST], [o.view(T, n), bufs["q0"], bufs["xh"]]
    run_both(both, "gpu_swiglu", swiglu, None)
