"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol the header
declares, agrees with the ctypes layout, and refuses to run without a GPU instead of falling back."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "decode_attn.h"
PKG = ROOT / "tensorrt-llm_b200"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(dx_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for s in ["dx_attn_create", "dx_attn_destroy", "dx_attn_workspace_size", "dx_attn_enqueue_generation",
              "dx_attn_enqueue_generation_host", "dx_attn_validate", "dx_strerror"]:
        assert s in syms


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load_library()
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} declared in include/decode_attn.h but not exported"
    assert set(declared_symbols()) == set(pkg.plugin.EXPORTED_SYMBOLS)
    assert lib.dx_abi_version() == 1
    assert lib.dx_strerror(0) == b"ok"
    assert lib.dx_strerror(3) == b"workspace too small"


def test_struct_layout_matches_ctypes_and_cpp_mirror_links(pkg, tmp_path):
    exe = tmp_path / "host_mirror_check"
    lib = pkg.library_path()
    subprocess.run(["g++", "-std=c++17", "-O1", str(Path(__file__).parent / "host_mirror_check.cpp"),
                    "-I", str(PKG / "csrc"), "-o", str(exe),
                    str(lib), f"-Wl,-rpath,{lib.parent}"], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    m = re.search(r"abi=(\d+) config=(\d+) params=(\d+)", out)
    assert m and int(m.group(1)) == 1
    assert int(m.group(2)) == ctypes.sizeof(pkg.plugin._Config)
    assert int(m.group(3)) == ctypes.sizeof(pkg.plugin._GenParams)
    assert "bad argument" in out


def test_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "decode_attn.h"\nint main(void){dx_attn_config c; c.struct_size=sizeof c; return DX_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{ROOT / 'include'}", str(src), "-o",
                    str(tmp_path / "t")], check=True)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_gpu_means_an_error_not_a_fallback(pkg):
    with pytest.raises(pkg.DecodeAttnError) as e:
        pkg.GPTAttentionPlugin(num_heads=8, num_kv_heads=2, head_size=128, kv_cache_quant_mode=pkg.QuantMode.FP8_KV_CACHE,
                               type_id=torch.bfloat16)
    assert e.value.status == pkg.plugin.DX_ERR_CUDA


def test_argument_checks_happen_before_any_cuda_call(pkg):
    lib = pkg.load_library()
    P = pkg.plugin
    h = ctypes.c_void_p()
    bad = [dict(head_size=72), dict(head_size=104, kv_cache_quant_mode=1 << 6), dict(num_heads=7, num_kv_heads=2), dict(tokens_per_block=48), dict(type_id=5),
           dict(tokens_per_block=8), dict(q_scaling=0.0), dict(kv_cache_quant_mode=(1 << 6) | (1 << 7)),
           dict(paged_kv_cache=0)]
    for kw in bad:
        base = dict(layer_idx=0, num_heads=8, num_kv_heads=2, head_size=128, q_scaling=1.0, tp_size=1, tp_rank=0,
                    multi_block_mode=1, enable_xqa=1, kv_cache_quant_mode=0, paged_kv_cache=1, tokens_per_block=64,
                    type_id=1, device=0)
        base.update(kw)
        cfg = P._Config(ctypes.sizeof(P._Config), **base)
        st = lib.dx_attn_create(ctypes.byref(cfg), ctypes.byref(h))
        assert st in (P.DX_ERR_BAD_ARG, P.DX_ERR_UNSUPPORTED), kw
        assert not h.value
    cfg = P._Config(3)  # wrong struct_size
    assert lib.dx_attn_create(ctypes.byref(cfg), ctypes.byref(h)) == P.DX_ERR_BAD_ARG
    assert lib.dx_attn_create(None, ctypes.byref(h)) == P.DX_ERR_BAD_ARG
    assert lib.dx_attn_enqueue_generation(None, None, None) == P.DX_ERR_BAD_ARG
    assert lib.dx_attn_workspace_size(None, 4, 100) == 0
