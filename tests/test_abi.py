"""The C-ABI library: builds, loads without a GPU, exports every symbol the headers declare, and reports errors the
reference's way (0 / -1 / NULL + ne_last_error). No compute calls here."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from ijah_b200 import engine as E
from ijah_b200 import packgen

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = []
    for h in sorted((ROOT / "include").glob("*.h")):
        names += re.findall(r"NE_API\s+[^;(]*?\b(ne_\w+)\s*\(", h.read_text())
    return names


@pytest.fixture(scope="module")
def eng():
    return E.Engine()


def test_every_declared_symbol_is_exported_and_bound(eng):
    decl = declared_symbols()
    assert len(decl) >= 40
    for n in decl:
        assert hasattr(eng.lib, n), n
        assert n in E.SIGNATURES, f"{n} declared in include/ but not bound in ijah_b200/engine.py"
    assert eng.lib.ne_abi_version() == 1


def test_dtype_table_matches_reference_codes(eng):
    want = {0: ("F32", 4), 1: ("F16", 2), 2: ("BF16", 2), 3: ("U8", 1), 4: ("U16", 2), 5: ("U32", 4), 6: ("I32", 4),
            7: ("I64", 8), 8: ("I8", 1), 9: ("I16", 2), 10: ("U64", 8), 11: ("F64", 8), 12: ("BOOL", 1)}
    for code, (name, size) in want.items():
        assert eng.lib.ne_dtype_name(code).decode() == name and eng.lib.ne_dtype_size(code) == size
    assert eng.lib.ne_dtype_name(99) == b"?" and eng.lib.ne_dtype_size(99) == 0


def test_pack_reader_reads_the_reference_layout(eng, tmp_path):
    rng = np.random.default_rng(5)
    t = packgen.moe_layer(rng, hidden=256, inter=128, experts=4)
    packgen.write_pack(tmp_path / "p", t, {"num_experts_per_tok": 2}, shards=3, misalign=2)
    p = eng.pack_open(tmp_path / "p")
    assert p.config()["expert_quant"]["window"] == 15
    assert p.names() == sorted(t)
    for name, (dt, arr) in t.items():
        d = p.info(name)
        assert d.dtype == dt and d.shape == arr.shape and d.nbytes == arr.nbytes
        assert np.array_equal(d.host().view(np.uint16), np.ascontiguousarray(arr).view(np.uint16))
        assert Path(d.file).exists() and d.file_offset > 8
    with pytest.raises(KeyError):
        p.info("nope")
    assert "no tensor named nope" in eng.last_error()
    p.close()


def test_errors_are_reported_not_raised_across_the_abi(eng, tmp_path):
    assert eng.lib.ne_pack_open(str(tmp_path / "missing").encode()) is None
    assert "missing" in eng.last_error()
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "model-00001-of-00001.safetensors").write_bytes(b"\xff" * 4)
    assert eng.lib.ne_pack_open(str(bad).encode()) is None
    assert "too short" in eng.last_error()
    (bad / "model-00001-of-00001.safetensors").write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    assert eng.lib.ne_pack_open(str(bad).encode()) is None
    assert "header length" in eng.last_error()
    assert eng.lib.ne_fn_set_ref_rounding(1) == -1
    assert eng.lib.ne_fn_layer_step(None, None, None, None) == -1
    assert eng.lib.ne_run_kernel(b"fn_moe_gateup_k5_r1", None, 0, None, 0, None, None, 0, 1, None, None) == -1
    assert eng.lib.ne_kernel_exists(b"stream_gemm_kernel") == 1 and eng.lib.ne_kernel_exists(b"t6_simd") == 0
    w = E.Exl3WeightC(None, None, None, 256, 128, 5)
    assert eng.lib.ne_exl3_linear(ctypes.byref(w), None, 1, None, None) == -1
    assert "null" in eng.last_error()


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(E.EngineError):
        E.Engine(tmp_path / "libnope.so")


def test_launch_plans_fit_shared_memory_for_every_row_count(eng):
    # host arithmetic only: every row count 1..64 at every K plans to a layout that fits an SM (one or two CTAs), with at
    # least two ring stages and three A slots; the MoE block of the benchmark dims likewise
    info = (ctypes.c_int * 8)()
    scratch = ctypes.c_uint64(0)
    for n_in, n_out in ((2048, 4096), (2048, 512), (4096, 2048), (768, 2048), (96, 160), (320, 48)):
        for K in (4, 5, 6, 7, 8):
            for rows in range(1, 65):
                assert eng.lib.ne_exl3_linear_plan(n_in, n_out, K, rows, info, ctypes.byref(scratch)) == 0, (n_in, n_out, K, rows, eng.last_error())
                S, kc, stages, aslots, grid, mt, smem, stage_bytes = list(info)
                assert stages >= 2 and aslots >= (3 if rows <= 40 else 2) and smem <= 226 * 1024 and kc % 16 == 0 and S * kc >= n_in // 16 and rows <= 8 * mt
                assert grid <= 2 * 148 and (smem <= 113 * 1024 or grid <= 148), "a layout beyond half an SM runs one CTA per SM"
                assert scratch.value >= rows * (4 * S * n_out + 2 * n_in)
    for rows in range(1, 65):
        assert eng.lib.ne_moe_plan(2048, 768, 512, 10, 5, 6, rows, info) == 0, eng.last_error()
        assert info[4] >= 2 and info[5] >= 2 and info[7] <= 113 * 1024 and info[0] <= 16 and info[2] <= 16
    assert eng.lib.ne_exl3_linear_plan(100, 128, 5, 1, info, None) == -1 and "multiples of 16" in eng.last_error()
