"""CPU checks of the C-ABI boundary: the library loads without a GPU and exports exactly the
entry points that include/nvfp4_b200.h declares; argument validation returns error codes with
text (no compute is launched)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "nvfp4_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp4_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    from sageattention_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built: run `python -m sageattention_b200.build`")
    handle = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert "nvfp4_pack" in names and "nvfp4_fwd" in names and "nvfp4_decode" in names
    for n in names:
        assert hasattr(handle, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"
    assert _lib.lib().nvfp4_abi_version() >= 1


def test_argument_validation_returns_error_text():
    from sageattention_b200 import _lib
    if not os.path.exists(_lib.LIB_PATH):
        pytest.skip("library not built")
    L = _lib.lib()
    rc = L.nvfp4_pack(None, 0, 1, 1, 24, 24, 0, 0, 1, None, 0, 0, None, 0, 0, None)
    assert rc < 0 and b"multiple of 16" in L.nvfp4_last_error()
    ns, sk, wb = ctypes.c_int(), ctypes.c_int64(), ctypes.c_size_t()
    # fixed splits: few units, long cache
    assert L.nvfp4_decode_plan(131072, 4, 128, 148, ctypes.byref(ns), ctypes.byref(sk), ctypes.byref(wb)) == 0
    assert ns.value >= 1 and sk.value % 128 == 0 and ns.value * sk.value >= 131072
    assert wb.value == 4 * ns.value * (16 * 128 + 32) * 4
    # many units: the balanced decomposition (nsplit = 0), two partial slots per CTA
    assert L.nvfp4_decode_plan(32768, 128, 128, 148, ctypes.byref(ns), ctypes.byref(sk), ctypes.byref(wb)) == 0
    assert ns.value == 0 and sk.value == 0 and wb.value == 148 * 2 * (16 * 128 + 32) * 4
    assert L.nvfp4_decode_plan(0, 1, 128, 148, None, None, None) < 0
    assert L.nvfp4_decode_plan(10, 1, 64, 148, None, None, None) < 0


def test_product_path_rejects_cpu_tensors_and_has_no_oracle_import():
    import torch
    import sageattention_b200.nvfp4 as nv
    with pytest.raises(RuntimeError, match="no CPU path"):
        nv._quant_nvfp4(torch.zeros(1, 1, 16, dtype=torch.bfloat16))
    pkg = os.path.join(ROOT, "sageattention_b200")
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(root, f)).read()
                assert "oracle" not in src.replace("oracle B", "").replace("the oracle", "") or f == "never", f


def test_host_policy_tables():
    from sageattention_b200.nvfp4 import flash
    r = flash._resolve_backward_grad_dots
    assert r(None, 1000, False, 4) == "bf16" and r(None, 4096, False, 4) == "fp4_rownorm"
    assert r("bf16", 100, True, 4) == "fp4_rownorm" and r("bf16", 100, False, 16) == "fp4_rownorm"
    assert r("fp8_rownorm", 100, False, 1) == "fp8_rownorm"
    with pytest.raises(ValueError):
        r("int8", 100, False, 1)
    assert flash._next_mult(129, 128) == 256
    assert flash._resolve_fwd_tiles(128, 64, 128, 8, 3) == (128, 128, 8, 2)
    assert flash._resolve_fwd_tiles(128, 32, 64, 4, 2) == (32, 64, 4, 2)
    cu = torch_cu = None
    import torch
    cu = torch.tensor([0, 3, 3, 10], dtype=torch.int32)
    sid, st, en = flash._varlen_seq_arrays(cu, 10, "cpu")
    assert sid.tolist() == [0, 0, 0, 2, 2, 2, 2, 2, 2, 2] and st.tolist()[3] == 3 and en.tolist()[0] == 3
    with pytest.raises(AssertionError, match=r"cu_seqlens\[-1\]"):
        flash._varlen_seq_arrays(torch.tensor([0, 4], dtype=torch.int32), 10, "cpu")
