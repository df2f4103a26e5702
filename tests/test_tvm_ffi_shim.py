"""The TVM-FFI binding of the C ABI (ako4x_b200/ffi/tvm_ffi_shim.cc, the reference's
`language = "cuda"` route) compiles with the host compiler against the installed apache-tvm-ffi and
this library, loads, and exports the typed functions. No GPU is needed: nothing is called."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_shim_compiles_loads_and_exports(built_lib, tmp_path):
    tvm_ffi = pytest.importorskip("tvm_ffi")
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no host C++ compiler")
    pkg = Path(tvm_ffi.__file__).resolve().parent
    lib_dir = ROOT / "ako4x_b200" / "lib"
    out = tmp_path / "ako4x_tvm_ffi_shim.so"
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-I", str(pkg / "include"), "-I", str(ROOT / "include"),
           str(ROOT / "ako4x_b200" / "ffi" / "tvm_ffi_shim.cc"), "-o", str(out), "-L", str(lib_dir), "-lako4x_b200",
           "-L", str(pkg / "lib"), "-ltvm_ffi", f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{pkg / 'lib'}"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr[-3000:]
    mod = tvm_ffi.load_module(str(out))
    for name in ("rmsnorm_h128", "gqa_paged_decode"):
        assert mod.get_function(name) is not None
