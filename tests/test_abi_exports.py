"""The C-ABI library loads without a GPU and exports every function that
include/inkling_b200.h declares (no compute calls here)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_functions() -> list[str]:
    text = (ROOT / "include" / "inkling_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ink_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_functions()
    for expected in ("ink_router_forward", "ink_router_plan_forward", "ink_expert_plan", "ink_routed_decode",
                     "ink_moe_decode", "ink_last_error"):
        assert expected in names


def test_library_exports_every_declared_symbol():
    import inkling_b200
    from inkling_b200.kernels import _abi

    handle = _abi.lib()
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert sorted(_abi.exported_symbols()) == declared_functions()
    assert handle.ink_abi_version() == _abi.ABI_VERSION
    assert handle.ink_router_workspace_bytes(1, 258) >= 258 * 4
    assert handle.ink_last_error() == b""


def test_argument_errors_are_reported_without_a_gpu():
    from inkling_b200.kernels import _abi

    handle = _abi.lib()
    # null pointers are rejected on the host before any launch
    rc = handle.ink_routed_decode(None, None, None, None, None, None, 1, 6, 4096, 2048, 255, 1, None, None)
    assert rc < 0 and b"null" in handle.ink_last_error()
    rc = handle.ink_add_rmsnorm(None, None, None, ctypes.c_float(1e-6), None, 1, 4096, None)
    assert rc < 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from inkling_b200.kernels import _abi
    import pytest

    monkeypatch.setattr(_abi, "_lib", None)
    monkeypatch.setattr(_abi, "LIBRARY", tmp_path / "libinkling_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _abi.lib()


def test_bank_names_and_launch_syntax():
    import inkling_b200

    k = inkling_b200.kernels
    assert k.expert_bank_names(True) == ["gate_up_proj", "gate_up_proj_scale", "gate_up_proj_scale2",
                                         "down_proj", "down_proj_scale", "down_proj_scale2"]
    assert k.expert_bank_names(False) == ["gate_up_proj", "down_proj"]
    assert callable(k.expert_plan[(1,)]) and callable(k.expert_copy[(128, 0)])


def test_encode_banks_rejects_bad_arguments():
    """ink_moe_stack_encode_banks validates on the host before it touches the driver: no GPU needed."""
    import ctypes

    from inkling_b200.kernels import _abi

    lib = _abi.lib()
    out = (ctypes.c_char * 512)()
    # null output
    assert lib.ink_moe_stack_encode_banks(None, 256, 1 << 20, 256, 1 << 17, 256, 1 << 20, 256, 1 << 17, 4, 1024, 512) != 0
    # shapes that do not tile by 128 rows x 256 columns
    assert lib.ink_moe_stack_encode_banks(out, 256, 1 << 20, 256, 1 << 17, 256, 1 << 20, 256, 1 << 17, 4, 1000, 512) != 0
    assert b"tile" in lib.ink_last_error()


def test_even_spacing_of_the_banks_is_detected():
    """The tensor-core variant needs the banks of one kind evenly spaced in memory; the host logic
    that decides it works on addresses only."""
    from inkling_b200.layer import ResidentExperts

    spaced = ResidentExperts._even_spacing([[4096, 4096 + 1024, 4096 + 2048], [64, 64 + 256, 64 + 512]], [1024, 128])
    assert spaced == [(4096, 1024), (64, 256)]                      # a gap between experts is fine, overlap is not
    assert ResidentExperts._even_spacing([[4096, 4096 + 512]], [1024]) is None          # overlapping
    assert ResidentExperts._even_spacing([[4096, 8192, 8192 + 1024]], [1024]) is None   # uneven
    assert ResidentExperts._even_spacing([[4100, 4100 + 1024]], [1024]) is None         # misaligned
    assert ResidentExperts._even_spacing([[4096]], [1024]) == [(4096, 1024)]            # a single expert
