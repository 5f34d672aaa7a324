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


def test_rust_binding_matches_the_header():
    """rust/lumen_moe_sys.rs (the extern block a lumen-runtime maintainer adds; it cannot be
    compiled in this image) declares exactly the functions of the header, each with the same
    number of parameters."""
    header = (ROOT / "include" / "lumen_moe.h").read_text()
    src = (ROOT / "rust" / "lumen_moe_sys.rs").read_text()
    block = src[src.index('extern "C" {'):]
    block = re.sub(r"/\*.*?\*/", "", block[:block.index("\n}\n")], flags=re.S)
    block = re.sub(r"//[^\n]*", "", block)
    rust = dict(re.findall(r"pub fn (lumen_\w+)\s*\(([^)]*)\)", block, flags=re.S))
    c_decls = dict(re.findall(r"LUMEN_MOE_API\s+[\w\s\*]+?\b(lumen_\w+)\s*\(([^;]*?)\)\s*;", header, flags=re.S))
    assert set(rust) == set(c_decls), set(rust) ^ set(c_decls)
    for name, params in rust.items():
        c_params = [q for q in c_decls[name].split(",") if q.strip() and q.strip() != "void"]
        r_params = [q for q in params.split(",") if q.strip()]
        assert len(c_params) == len(r_params), (name, len(c_params), len(r_params))


def test_header_is_plain_c_and_a_c_program_reads_an_lbc_index(cuda_lib, tmp_path):
    """include/lumen_moe.h compiles as C99 (-pedantic) and a C consumer linked against the
    library gets the offsets of an LBC layer (the path a non-Python host takes)."""
    import subprocess
    from lumen_b200 import _lib
    from oracle import lbc_writer as W
    exe = tmp_path / "lbc_c_consumer"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", str(ROOT / "include"),
                    str(ROOT / "tests" / "native" / "lbc_c_consumer.c"), "-o", str(exe),
                    str(_lib.LIB_PATH), f"-Wl,-rpath,{_lib.LIB_PATH.parent}"], check=True)
    m = W.Model(num_layers=1, hidden_dim=64, intermediate_dim=32, num_experts=3, num_active_experts=2)
    gb, db = 32 * 2 * 18, 64 * 1 * 18
    experts = [((1000 + e * (2 * gb + db), gb, W.Q4_0), (1000 + e * (2 * gb + db) + gb, gb, W.Q4_0),
                (1000 + e * (2 * gb + db) + 2 * gb, db, W.Q4_0)) for e in range(3)]
    L = W.Layer(router_weight=(232, 3 * 64 * 4, W.F32), experts=experts)
    path = tmp_path / "m.lbc"
    path.write_bytes(W.write_lbc(m, [L], [bytes(1000 + 3 * (2 * gb + db))]))
    r = subprocess.run([str(exe), str(path), "0"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = r.stdout.splitlines()
    assert lines[0] == "version 4 layers 1 hidden 64 experts 3 top_k 2"
    assert lines[1] == f"is_moe 1 num_experts 3 quant {_lib.Q4_0} router_off 232"
    assert lines[2] == f"expert0 1000 {1000 + gb} {1000 + 2 * gb} last_down {1000 + 2 * (2 * gb + db) + 2 * gb}"
