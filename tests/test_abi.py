"""The C-ABI library loads and exports every symbol that include/pyre_b200.h declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "pyre_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_boundary():
    syms = declared_symbols()
    for must in ("pb_ctx_create", "pb_qmat_upload", "pb_qmat_dequant", "pb_gemv", "pb_model_create", "pb_forward",
                 "pb_step_greedy", "pb_verify", "pb_keep", "pb_state_snapshot", "pb_state_restore", "pb_moe_forward",
                 "pb_deltanet_step", "pb_attn_step"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    import pyre_b200.build as b
    lib_path = b.build()          # nvcc cross-compiles here; no GPU required
    lib = ctypes.CDLL(str(lib_path))
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in include/pyre_b200.h but not exported: {missing}"


def test_no_cpu_fallback_without_gpu():
    """Without a CUDA device the product fails loudly instead of computing on the host."""
    import torch
    import pyre_b200 as pb
    if torch.cuda.is_available():
        pytest.skip("a GPU is visible")
    with pytest.raises(pb.PyreError):
        pb.Ctx(0)


def test_product_does_not_import_the_oracle():
    for p in (ROOT / "pyre_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".h") and "oracle" in p.read_text(errors="ignore"):
            lines = [l for l in p.read_text(errors="ignore").splitlines() if "oracle" in l and "import" in l]
            assert not lines, f"{p} imports the oracle: {lines}"
