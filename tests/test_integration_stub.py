"""CPU: the drop-in replacement for the reference's src/matmul_kernel.cu really compiles against the reference's
own headers and defines exactly the symbols its binding layer declares for this path.

Needs the reference checkout (skipped where it is absent); set AAKAAR_REFERENCE to its root."""
import os
import re
import subprocess
import sysconfig

import pytest

from util import ROOT

REF = os.environ.get("AAKAAR_REFERENCE", "/root/reference")
STUB = os.path.join(ROOT, "oracle", "integration", "matmul_kernel_stub.cpp")

DECLARED = [   # src/bindings.cpp:13-16, 142-143, 187-188, 260-261
    "set_tf32_enabled(bool)", "get_tf32_enabled()", "set_cudnn_tf32_enabled(bool)", "get_cudnn_tf32_enabled()",
    "cuda_synchronize()",
    "run_cublas_matmul(std::shared_ptr<Tensor>, std::shared_ptr<Tensor>)",
    "run_cublas_matmul_a_bt(std::shared_ptr<Tensor>, std::shared_ptr<Tensor>)",
    "run_cublas_matmul_at_b(std::shared_ptr<Tensor>, std::shared_ptr<Tensor>)",
    "run_cuda_matmul_f64(std::shared_ptr<Tensor>, std::shared_ptr<Tensor>)",
    "run_cuda_matmul_int_typed(std::shared_ptr<Tensor>, std::shared_ptr<Tensor>)",
]


def test_integration_section_is_the_compiled_file():
    stub = open(STUB).read()
    snip = stub[stub.index("// BEGIN INTEGRATION SNIPPET\n") + len("// BEGIN INTEGRATION SNIPPET\n"):
                stub.index("// END INTEGRATION SNIPPET")]
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    assert snip in doc, "INTEGRATION.md section 2 and oracle/integration/matmul_kernel_stub.cpp differ"


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src")), reason="reference checkout not present")
def test_stub_compiles_against_the_reference_headers(tmp_path):
    import pybind11
    obj = tmp_path / "stub.o"
    cmd = ["g++", "-std=c++17", "-c", "-fPIC", "-w", f"-I{os.path.join(REF, 'src')}", f"-I{os.path.join(ROOT, 'include')}",
           f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", "-I/usr/local/cuda/include",
           STUB, "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-3000:]
    syms = subprocess.run(["nm", "-C", "--defined-only", str(obj)], capture_output=True, text=True).stdout
    defined = {re.sub(r"^\S+\s+T\s+", "", line).strip() for line in syms.splitlines() if " T " in line}
    for want in DECLARED:
        assert want in defined, (want, sorted(defined))
    # and the declarations this list restates are the ones in the reference's binding layer
    text = open(os.path.join(REF, "src", "bindings.cpp")).read()
    for want in DECLARED:
        name = want.split("(")[0]
        assert re.search(r"^[\w:<> ]+\b" + name + r"\(", text, re.M), name
