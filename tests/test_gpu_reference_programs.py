"""The reference's own component test programs that need no model file, tests/layernorm_verify.cpp and
tests/rope_verify.cpp, compiled UNCHANGED from the reference's tree (oracle/Makefile, target ref_programs; the binaries
live in oracle/_ref/ and travel with the repository) against the hip/ shim headers, and run here against this
library's kernels: each loads "layernorm.co" / "rope_embedding.co" from its working directory with hipModuleLoadData,
asks for "rmsnorm" / "rope_rotate_half" by name, launches with its own grid and argument list on pinned host memory,
and applies its own pass rule. The module image it gets is rocm_hip_b200/gpu_ops.fatbin."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FATBIN = os.path.join(ROOT, "rocm_hip_b200", "gpu_ops.fatbin")


@pytest.mark.parametrize("prog,module,args,verdict", [
    ("layernorm_verify", "layernorm.co", ["--sweep"], "LAYERNORM VERIFICATION PASSED (5 shapes)"),
    ("layernorm_verify", "layernorm.co", ["--tokens", "300", "--embd", "5120", "--eps", "1e-6"], "LAYERNORM VERIFICATION PASSED (1 shape)"),
    ("rope_verify", "rope_embedding.co", ["--sweep"], "PASSED"),
    ("rope_verify", "rope_embedding.co", ["--rows", "200", "--dim", "256"], "PASSED"),
])
def test_reference_program_passes_on_this_library(tmp_path, prog, module, args, verdict):
    exe = os.path.join(ROOT, "oracle", "_ref", prog)
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/%s was not built (the reference's source tree was absent at build time)" % prog)
    shutil.copy(FATBIN, tmp_path / module)
    r = subprocess.run([exe] + args, cwd=tmp_path, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert verdict in r.stdout and "MISMATCH" not in r.stdout and "failures=0" in r.stdout, r.stdout[-2000:]
