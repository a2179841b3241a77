"""The C-ABI library loads without a GPU and exports every symbol that
include/dice_b200.h declares; host-side argument checks answer without a
device."""
import ctypes
import os
import re

from dice_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "dice_b200.h")).read()
    return sorted(set(re.findall(r"DICE_API[^;(]*?\b(dice_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    names = _declared()
    assert len(names) >= 14
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.library_path())
    for name in _declared():
        assert hasattr(lib, name), f"{name} is declared in dice_b200.h but not exported"


def test_version_and_messages():
    lib = _lib.load()
    assert lib.dice_abi_version() == 2
    assert lib.dice_strerror(0) == b"ok"
    assert b"shape" in lib.dice_strerror(-2)
    assert lib.dice_status_message(0) == b"ok"
    assert b"timed out" in lib.dice_status_message(1)
    assert lib.dice_w13_rows(4608) == 9216 and lib.dice_w13_rows(64) == 256
    assert lib.dice_permute_scratch_bytes(32768, 8) == 128 * 8 * 4


def test_argument_errors_are_reported_on_the_host():
    lib = _lib.load()
    # bad expert count / dtype / null pointers: rejected before any CUDA call
    assert lib.dice_router_top2(None, None, 4, 64, 1, 0, 0, None, None, None, None, None, None, None) == -2
    assert lib.dice_router_top2(None, None, 4, 64, 8, 7, 0, None, None, None, None, None, None, None) == -3
    assert lib.dice_permute_rows(None, None, 4, 3, 64, 0, None, None) == -2
    assert lib.dice_grouped_gemm(None, 4, 60, None, 1, 32, None, None, 1, 0, None, 32, 32, 0, None, None) == -2
    assert lib.dice_grouped_gemm(None, 4, 64, None, 1, 32, None, None, 300, 0, None, 32, 32, 0, None, None) == -7
    assert lib.dice_grouped_ffn(None, 4, 64, 64, 5, None, None, 1, None, None, 1, None, None, None, 0, 0, None, None, None, None, 0, None,
                                None, None, None) == -1


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.DiceLibraryError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_cpu_tensors_are_refused():
    import pytest
    import torch

    from dice_b200 import ops
    from dice_b200.moe_block import ParaMode, SparseMoeBlock

    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.router_top2(torch.zeros(4, 64), torch.zeros(8, 64))
    blk = SparseMoeBlock(32, 4, 8, 2, 1, 0, 1, ParaMode()).eval()
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        blk(torch.zeros(1, 4, 32))
