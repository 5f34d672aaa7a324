"""The C-ABI library loads and exports every symbol include/lumen_moe.h declares
(no compute call here: that needs a GPU)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "lumen_moe.h").read_text()
    return sorted(set(re.findall(r"\b(lumen_(?:moe|lbc)_[a-z0-9_]+)\s*\(", text)))


def test_header_and_loader_agree():
    from lumen_b200 import _lib
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_library_exports_every_declared_symbol(cuda_lib):
    for name in declared_symbols():
        assert hasattr(cuda_lib, name), name
    assert b"sm_100a" in cuda_lib.lumen_moe_version()


def test_create_fails_loudly_without_gpu(cuda_lib):
    import torch
    if torch.cuda.is_available():
        return
    from lumen_b200 import _lib
    cfg = _lib.MoeConfig(2048, 768, 128, 8, 16, 0, 0, 0)
    h = ctypes.c_void_p()
    rc = cuda_lib.lumen_moe_create(ctypes.byref(cfg), ctypes.byref(h))
    assert rc == _lib.CUDA_ERROR and b"no CPU path" in cuda_lib.lumen_moe_last_error()


def test_synthetic_layout_matches_converter_layout():
    # [router f32 [E,H]] [e0: gate | up | down] ... (crates/lumen-convert/src/arch/qwen35_moe.rs:257-260)
    from lumen_b200.synth import LayerLayout
    lay = LayerLayout(2048, 768, 128, 1)
    m = lay.meta()
    assert lay.gate_bytes == 884736 and lay.down_bytes == 884736 and lay.expert_bytes == 2654208
    assert lay.router_bytes == 1048576
    assert int(m.expert_gate_offs[0]) == 1048576
    assert int(m.expert_up_offs[0]) == 1048576 + 884736
    assert int(m.expert_down_offs[127]) + 884736 == lay.blob_bytes
    assert LayerLayout(2048, 768, 128, 0).expert_bytes == 5013504
    assert LayerLayout(2048, 768, 128, 2).expert_bytes == 9437184


def test_build_moe_meta_returns_none_for_dense_layers():
    from lumen_b200.moe import build_moe_meta
    assert build_moe_meta(None, [{"gate": (0, 1), "up": (0, 1), "down": (0, 1)}]) is None
    assert build_moe_meta(0, []) is None


def test_integration_binding_matches_the_header():
    """Every function of the Rust extern block shown in INTEGRATION.md is declared in the
    header with the same number of parameters."""
    header = (ROOT / "include" / "lumen_moe.h").read_text()
    doc = (ROOT / "INTEGRATION.md").read_text()
    block = doc[doc.index('extern "C" {'):]
    block = block[:block.index("```")]
    rust = re.findall(r"pub fn (lumen_\w+)\s*\(([^)]*)\)", block, flags=re.S)
    assert len(rust) >= 10
    for name, params in rust:
        m = re.search(r"\b" + name + r"\s*\(([^;]*?)\)\s*;", header, flags=re.S)
        assert m, name
        c_params = [p for p in m.group(1).split(",") if p.strip() and p.strip() != "void"]
        r_params = [p for p in params.split(",") if p.strip()]
        assert len(c_params) == len(r_params), (name, len(c_params), len(r_params))
