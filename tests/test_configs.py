"""param_map.json -> table generator and the run-time lookup."""

import ctypes
import json

import pytest

from tuna_b200 import _lib, make_configs

BASELINE_SHAPES = [
    (6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336),
    (10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672),
    (229376, 4096), (32768, 14336),
]
SHARD_SHAPES = [(768, 4096), (3584, 4096), (7168, 8192), (1280, 8192), (28672, 4096), (4096, 1792), (8192, 3584), (8192, 1024)]


def test_bucket_rule():
    assert [make_configs.token_bucket(n) for n in (1, 8, 9, 16, 17, 64, 65, 1024, 1025, 100000)] == \
        [8, 8, 16, 16, 32, 64, 128, 1024, 2048, 2048]


def test_committed_param_map_is_valid_and_rendered():
    pm = make_configs.load()
    make_configs.validate(pm)
    text = make_configs.render(pm)
    assert make_configs.TABLE_INC.read_text() == text, "run python -m tuna_b200.make_configs"
    assert text.count("\n") == len(pm) + 1


def test_render_rejects_bad_entries():
    with pytest.raises(ValueError):
        make_configs.render({"4096_16_4097": {}})
    with pytest.raises(ValueError):
        make_configs.render({"4096_17_4096": {}})
    with pytest.raises(ValueError):
        make_configs.render({"4096_16_4096": {"path": "wgmma"}})
    with pytest.raises(ValueError):
        make_configs.render({"4096_16_4096": {"tile_m": 128}})


def test_render_field_order():
    text = make_configs.render({"4096_16_4096": {"path": "stream", "tile_tok": 16, "rows_per_warp": 2,
                                                 "warps_m": 4, "warps_k": 4, "k_steps": 8, "us": 4.2}})
    assert "{4096, 16, 4096, {1, 16, 2, 4, 4, 8, 0, 0, 0, 0, 0, 0, 0, {0, 0, 0}}}," in text


@pytest.mark.parametrize("n", [1, 8, 16])
@pytest.mark.parametrize("m,k", BASELINE_SHAPES + SHARD_SHAPES)
def test_lookup_always_yields_a_runnable_config(tuna_lib, m, k, n):
    cfg = _lib.TunaConfig()
    assert tuna_lib.tuna_lookup_config(m, n, k, ctypes.byref(cfg)) == 0
    assert cfg.path in (_lib.PATH_STREAM, _lib.PATH_UMMA, _lib.PATH_TSTREAM)
    if cfg.path == _lib.PATH_TSTREAM:
        assert cfg.tile_tok in (16, 32, 64) and cfg.row_blocks in (1, 2, 4) and cfg.k_steps in (4, 8)
        assert cfg.row_blocks * cfg.tile_tok <= 64
    if cfg.path == _lib.PATH_STREAM:
        assert cfg.tile_tok in (8, 16, 32) and cfg.rows_per_warp in (1, 2)
        assert 1 <= cfg.warps_m * cfg.warps_k <= 16 and cfg.k_steps in (4, 8, 16, 32, 64)
    ws = tuna_lib.tuna_matmul_workspace_bytes(m, n, k)
    assert ws < (1 << 31)


def test_table_size_matches_param_map(tuna_lib):
    assert tuna_lib.tuna_config_table_size() == len(json.loads(make_configs.PARAM_MAP.read_text()))
