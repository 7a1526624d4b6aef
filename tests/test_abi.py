"""CPU-side checks of the drop-in boundary: the shared library loads without a GPU, exports
every symbol include/h3b200.h declares plus every h3_gpu_* symbol of the reference's device
API (so a full libh3 links), and fails loudly - not silently - when no device is present."""
import ctypes as C
import re
import subprocess
import os
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "h3.c_b200" / "libh3b200.so"
REFERENCE_HEADER = Path(os.environ.get("H3_REFERENCE_DIR", ROOT.parent / "reference")) / "h3_gpu.h"


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as entry
    if not LIB.exists():
        entry.build()
    return entry.load_package()


def exported_symbols():
    out = subprocess.run(["nm", "-D", "--defined-only", str(LIB)], capture_output=True, text=True,
                         check=True).stdout
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


def test_header_symbols_are_exported(pkg):
    declared = pkg.declared_functions()
    assert len(declared) >= 70
    missing = sorted(set(declared) - exported_symbols())
    assert not missing, missing


@pytest.mark.skipif(not REFERENCE_HEADER.exists(), reason="reference tree not present")
def test_every_reference_entry_point_is_exported(pkg):
    names = set(re.findall(r"\b(h3_gpu_[a-z0-9_]+)\s*\(", REFERENCE_HEADER.read_text()))
    names.add("h3_cuda_probe")        # h3_cuda.h:9, called by the pipeline (h3.c:465)
    assert len(names) > 100
    missing = sorted(names - exported_symbols())
    assert not missing, missing


def test_prototypes_parse_to_the_expected_ctypes(pkg):
    d = pkg.declared_functions()
    assert d["h3_gpu_create"] == (C.c_void_p, [C.c_char_p, C.c_char_p, C.c_size_t])
    assert d["h3_gpu_linear_bf16"][1] == [C.c_void_p] * 5 + [C.c_uint32] * 3
    assert d["h3_gpu_euler_bf16"][1] == [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p,
                                         C.c_uint32, C.c_float, C.c_float]
    assert d["h3_gpu_sdpa_bf16"][1] == [C.c_void_p] * 5 + [C.c_uint32] * 3 + [C.c_float]


def test_no_device_fails_loudly(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(pkg.H3Error):
        pkg.Gpu(0)


def test_product_does_not_reference_the_oracle():
    """The shipped package must not import, link or call anything under oracle/."""
    for path in (ROOT / "h3.c_b200").rglob("*"):
        if path.suffix in {".py", ".cu", ".cuh", ".h"}:
            text = path.read_text()
            assert "h3_oracle" not in text and "oracle/" not in text, path
    needed = subprocess.run(["ldd", str(LIB)], capture_output=True, text=True).stdout
    assert "oracle" not in needed


def test_prototypes_agree_with_the_reference_header(tmp_path):
    """Both headers in one C11 translation unit: the compiler rejects any prototype of
    include/h3b200.h whose argument or return types differ from the reference's declaration."""
    if not REFERENCE_HEADER.exists():
        pytest.skip("the reference tree is not present")
    import subprocess
    src = tmp_path / "both.c"
    src.write_text('#include "h3_gpu.h"\n#include "h3_cuda.h"\n#include "h3b200.h"\n#include "h3b200_offpath.h"\n'
                   'int main(void) { return 0; }\n')
    res = subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-I", str(REFERENCE_HEADER.parent),
                          "-I", str(ROOT / "include"), "-c", str(src), "-o", str(tmp_path / "both.o")],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-2000:]


def test_a_c_host_links_and_fails_loudly_without_a_device(tmp_path):
    """A plain C11 host built against include/h3b200.h and linked with libh3b200.so: on a machine
    without a GPU h3_gpu_create returns NULL with a message (no CPU fallback)."""
    import subprocess
    import torch
    src = tmp_path / "host.c"
    src.write_text('''
#include <stdio.h>
#include "h3b200.h"
int main(void) {
    char error[256] = {0};
    h3_gpu *gpu = h3_gpu_create(NULL, error, sizeof(error));
    if (!gpu) { printf("create failed: %s\\n", error); return 3; }
    h3_gpu_tensor *t = h3_gpu_tensor_new_bf16(gpu, 64);
    int ok = t && h3_gpu_begin(gpu) && h3_gpu_add_bf16(gpu, t, t, t, 64) && h3_gpu_submit(gpu);
    h3_gpu_tensor_free(t);
    h3_gpu_free(gpu);
    printf("ran: %d\\n", ok);
    return ok ? 0 : 4;
}
''')
    exe = tmp_path / "host"
    res = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(ROOT / "include"), str(src), "-o", str(exe),
                          "-L", str(LIB.parent), "-lh3b200", f"-Wl,-rpath,{LIB.parent}"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    if torch.cuda.is_available():
        assert run.returncode == 0 and "ran: 1" in run.stdout, run.stdout + run.stderr
    else:
        assert run.returncode == 3 and "create failed:" in run.stdout and len(run.stdout.strip()) > 16
