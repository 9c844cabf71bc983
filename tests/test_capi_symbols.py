"""The C-ABI library builds, loads without a GPU, and exports every symbol include/muse_proj.h
declares (no compute call is made here)."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "muse_proj.h").read_text()


def declared_symbols() -> list[str]:
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(muse_[a-z0-9_]+)\s*\(", body)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("muse_gemv1", "muse_skinny_tc", "muse_tmap_encode_2d", "muse_query", "muse_abi_version"):
        assert must in names


def test_library_builds_loads_and_exports_every_declared_symbol():
    from llm_inference_engine_b200 import _capi, build

    path = build.build()
    assert path.exists()
    raw = ctypes.CDLL(str(path))
    for name in declared_symbols():
        assert hasattr(raw, name), f"{name} declared in muse_proj.h but not exported"
    lib = _capi.load()
    assert set(_capi.SIGNATURES) == set(declared_symbols()), "ctypes table and header disagree"
    assert lib.muse_abi_version() == int(re.search(r"MUSE_PROJ_ABI_VERSION\s+(\d+)", HEADER).group(1))
    # constants mirrored by hand in the binding and the planner
    from llm_inference_engine_b200 import plan

    assert _capi.MAX_WORLD == int(re.search(r"MUSE_MAX_WORLD\s+(\d+)", HEADER).group(1))
    assert _capi.LL_TOKENS == plan.LL_TOKENS == int(re.search(r"MUSE_LL_TOKENS\s+(\d+)", HEADER).group(1))
    assert _capi.RP_TOKENS == int(re.search(r"MUSE_RP_TOKENS\s+(\d+)", HEADER).group(1))
    assert ctypes.sizeof(_capi.PeerSync) == 16 + 3 * 8 * _capi.MAX_WORLD
    assert ctypes.sizeof(_capi.Boundary) == 8 * 8 and ctypes.sizeof(_capi.FfnBoundary) == 7 * 8


def test_pure_host_entry_points_without_a_gpu():
    from llm_inference_engine_b200 import _capi, plan

    lib = _capi.load()
    assert lib.muse_skinny_tiles(32, 12288, 32) == 96
    assert lib.muse_skinny_tiles(300, 200, 256) == 4
    assert lib.muse_skinny_ws_floats(32, 12288, 32) == 96 * 128 * 32
    assert lib.muse_skinny_tiles(0, 1, 16) < 0
    for m, k, warps in ((2, 4096, 16), (8, 1024, 32), (9, 4096, 32), (16, 2048, 16)):
        assert lib.muse_fewtok_smem_bytes(m, k, warps) == plan.fewtok_smem_bytes(m, k, warps)
    for ntok, pair, stages, cluster, m, wgs, rows, atoms in ((16, 0, 1, 1, 5, 1, 128, 1), (64, 1, 3, 4, 64, 4, 128, 1), (256, 1, 3, 2, 256, 4, 128, 1),
                                                             (112, 0, 4, 9, 100, 2, 128, 1), (256, 0, 4, 16, 1000, 4, 128, 1),
                                                             (160, 1, 8, 3, 300, 3, 128, 1), (32, 0, 12, 1, 32, 4, 88, 1), (16, 0, 10, 1, 9, 2, 8, 1),
                                                             (64, 0, 8, 2, 64, 4, 56, 1), (32, 0, 3, 1, 32, 4, 88, 4), (128, 0, 3, 4, 128, 4, 128, 2)):
        assert (lib.muse_gemm_tc_smem_bytes(ntok, pair, stages, cluster, m, wgs, rows, atoms)
                == plan.gemm_smem_bytes(ntok, bool(pair), stages, cluster, m, wgs, rows, atoms))
    for m, n, ntok, pair, split, rows in ((256, 12288, 256, 1, 3, 128), (100, 1000, 112, 1, 3, 128), (256, 1024, 256, 0, 16, 128),
                                          (40, 700, 48, 0, 20, 128), (64, 512, 64, 0, 1, 128), (1000, 4096, 256, 1, 2, 128),
                                          (48, 2304, 48, 0, 2, 40)):
        assert lib.muse_gemm_tc_ws_floats(m, n, ntok, pair, split, rows) == plan.gemm_ws_floats(m, n, ntok, bool(pair), split, rows)
    for ntok in plan.NTOK_CHOICES:
        for hilo in (False, True):
            assert lib.muse_skinny_stage_bytes(ntok, int(hilo)) == plan.stage_bytes(ntok, hilo)
            for stages, cluster, m in ((1, 1, 1), (4, 3, 32), (12, 8, 5), (3, 16, 300)):
                assert (lib.muse_skinny_smem_bytes(ntok, int(hilo), stages, cluster, m)
                        == plan.smem_bytes(ntok, hilo, stages, cluster, m))


def test_status_bits_match_between_header_and_kernels():
    common = (ROOT / "llm_inference_engine_b200" / "csrc" / "common.cuh").read_text()
    for name, value in re.findall(r"#define MUSE_(ST_[A-Z_]+)\s+(\d+)", HEADER):
        assert re.search(rf"{name}\s*=\s*{value}\b", common), f"{name} differs between header and common.cuh"


def test_product_package_never_imports_the_oracle():
    for py in (ROOT / "llm_inference_engine_b200").rglob("*.py"):
        text = py.read_text()
        assert "oracle" not in re.sub(r'""".*?"""', "", text, flags=re.S), f"{py.name} refers to the oracle"


def test_no_cpu_fallback_when_given_cpu_tensors():
    import torch

    from llm_inference_engine_b200 import muse_bf16_proj

    with pytest.raises(RuntimeError, match="CUDA device only"):
        muse_bf16_proj.prepare({"o": torch.zeros((128, 64), dtype=torch.bfloat16)})
