"""The C-ABI library loads and exports every symbol the public header declares.
No compute entry point is called here (no GPU needed)."""
import ctypes
import os
import re

from kan_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(chebykan_\w+)\s*\(", text))
    return names


def test_header_symbols_exported(built_lib):
    lib = ctypes.CDLL(built_lib)
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"


def test_binding_table_covers_header(built_lib):
    assert set(_lib.SIGNATURES) == declared_symbols()


def test_pure_host_entry_points(built_lib):
    lib = _lib.load()
    assert lib.chebykan_abi_version() == 7
    assert _lib.strerror(0) == "ok"
    assert "aligned" in _lib.strerror(-2)
    # packed sizes: fp32 [K_pad][N_pad] with blocks of 8 inputs, outputs padded to 64
    assert lib.chebykan_packed_bytes(1024, 1024, 8, _lib.MODE_FP32) == 1024 * 9 * 1024 * 4
    assert lib.chebykan_packed_bytes(1, 1, 8, _lib.MODE_FP32) == 8 * 9 * 64 * 4
    # bf16 [N_pad][K_pad]: inputs padded to 64, outputs to 128
    # tensor-core modes: degrees 1..deg in the matrix plus one K block whose first slot is the bias (degree 0), and the
    # bias again as a vector of N_pad floats behind the matrices
    assert lib.chebykan_packed_bytes(1024, 1024, 8, _lib.MODE_BF16) == (1024 * 8 + 64) * 1024 * 2 + 1024 * 4
    assert lib.chebykan_packed_bytes(784, 64, 4, _lib.MODE_BF16) == (832 * 4 + 64) * 128 * 2 + 128 * 4
    assert lib.chebykan_packed_bytes(784, 64, 0, _lib.MODE_BF16) == 64 * 128 * 2 + 128 * 4    # degree 0: the bias alone
    # TF32, narrow layer (<= 128 outputs, in % 4 == 0): the tf32 matrix, then a 256-byte header and an fp16 plane in the BF16 layout
    assert lib.chebykan_packed_bytes(784, 64, 4, _lib.MODE_TF32) == (800 * 4 + 32) * 128 * 4 + 256 + (832 * 4 + 64) * 128 * 2 + 128 * 4
    assert lib.chebykan_packed_bytes(1024, 1024, 8, _lib.MODE_TF32) == (1024 * 8 + 32) * 1024 * 4 + 1024 * 4
    assert lib.chebykan_packed_bytes(783, 64, 4, _lib.MODE_TF32) == (800 * 4 + 32) * 128 * 4 + 128 * 4
    # invalid arguments come back as error codes, never exceptions or crashes
    assert lib.chebykan_packed_bytes(0, 4, 4, 0) == -1
    assert lib.chebykan_packed_bytes(4, 4, 200, 0) == -1
    assert lib.chebykan_packed_bytes(4, 4, 4, 7) == -1
    assert lib.chebykan_workspace_bytes(_lib.OP_FWD, 128, 8, 8, 4, 0) == 0
    assert lib.chebykan_workspace_bytes(99, 128, 8, 8, 4, 0) == -1
    ws = lib.chebykan_workspace_bytes(_lib.OP_BWD_DCOEFF, 1 << 20, 64, 64, 32, 0)
    assert ws > 0 and ws % (64 * 64 * 33 * 4) == 0
    # dx workspace: the repacked tf32 coefficients (degrees 0..deg counted, 32-output pitch); in bf16 mode from 512
    # outputs on a header, fp16 coefficients (degrees 1..deg, 64-output pitch), the fp16 copy of dY and a scale per row
    assert lib.chebykan_workspace_bytes(_lib.OP_BWD_DX, 4096, 64, 64, 32, _lib.MODE_TF32) == 64 * 33 * 64 * 4
    assert lib.chebykan_workspace_bytes(_lib.OP_BWD_DX, 4096, 64, 64, 32, _lib.MODE_BF16) == 64 * 33 * 64 * 4
    assert lib.chebykan_workspace_bytes(_lib.OP_BWD_DX, 4096, 128, 1000, 8, _lib.MODE_TF32) == 128 * 9 * 1024 * 4
    assert (lib.chebykan_workspace_bytes(_lib.OP_BWD_DX, 4096, 128, 1000, 8, _lib.MODE_BF16)
            == 256 + 128 * 8 * 1024 * 2 + 4096 * 1024 * 2 + 4096 * 4)
    assert lib.chebykan_workspace_bytes(_lib.OP_BWD_DX, 4096, 128, 1000, 8, _lib.MODE_FP32) == 0
    assert lib.chebykan_fwd_host_scratch_bytes(100, 4, 4, 3, 0) > 100 * 4 * 4 * 2
