"""Host logic of the tuner: genome handling and configuration validity, no GPU needed."""

import random

from tuna_b200 import _lib, tuner


def test_genomes_stay_inside_the_search_space():
    rng = random.Random(0)
    for path in ("stream", "tstream", "umma"):
        space = tuner.space_for(path)
        g = tuner.random_genome(rng, path)
        for _ in range(50):
            g = tuner.mutate(rng, tuner.crossover(rng, g, tuner.random_genome(rng, path)), path)
            assert set(g) == set(space)
            assert all(g[k] in space[k] for k in g)


def test_validity_filter_matches_the_launcher(tuna_lib):
    ok = tuner.to_config("stream", 16, dict(rows_per_warp=1, warps_m=16, warps_k=1, k_steps=8))
    assert tuner.is_valid(tuna_lib, 4096, 16, 4096, ok)
    too_many_warps = tuner.to_config("stream", 16, dict(rows_per_warp=1, warps_m=16, warps_k=2, k_steps=8))
    assert not tuner.is_valid(tuna_lib, 4096, 16, 4096, too_many_warps)
    bad_steps = tuner.to_config("stream", 16, dict(rows_per_warp=1, warps_m=16, warps_k=1, k_steps=4))
    assert not tuner.is_valid(tuna_lib, 4096, 16, 4096, bad_steps)
    umma = tuner.to_config("umma", 256, dict(row_blocks=1, stages_w=4, stages_x=4, stages_a=4, dequant_warps=16, k_accs=1))
    assert tuner.is_valid(tuna_lib, 4096, 2048, 4096, umma)
    umma_bad = tuner.to_config("umma", 256, dict(row_blocks=2, stages_w=4, stages_x=4, stages_a=4, dequant_warps=16, k_accs=1))
    assert not tuner.is_valid(tuna_lib, 4096, 2048, 4096, umma_bad)
    # combinations no GPU test exercises are refused by the launcher
    for bad in (dict(dequant_warps=12), dict(k_accs=2), dict(stages_w=2), dict(row_blocks=3)):
        g = dict(row_blocks=1, stages_w=4, stages_x=4, dequant_warps=16, k_accs=1)
        g.update(bad)
        assert not tuner.is_valid(tuna_lib, 4096, 2048, 4096, tuner.to_config("umma", 64, g))


def test_config_fields_round_trip():
    cfg = tuner.to_config("umma", 64, dict(row_blocks=2, stages_w=6, stages_x=4, stages_a=8, dequant_warps=8, k_accs=1))
    d = cfg.as_dict()
    assert d["path"] == _lib.PATH_UMMA and d["tile_tok"] == 64 and d["row_blocks"] == 2 and d["k_accs"] == 1
    assert all(v == (0,) for v in tuner.UMMA_SPACE.values())  # the TMA-staged kernel: defaults only


def test_path_is_part_of_the_search():
    assert tuner.candidate_paths(16) == ("tstream", "stream")
    assert "umma" in tuner.candidate_paths(64) and "tstream" in tuner.candidate_paths(64)
    assert tuner.candidate_paths(2048) == ("tstream", "umma")
    assert tuner.tile_tok_for("tstream", 9) == 16 and tuner.tile_tok_for("tstream", 40) == 64
    assert tuner.tile_tok_for("tstream", 65) == 128 and tuner.tile_tok_for("tstream", 2048) == 128
    assert tuner.tile_tok_for("stream", 8) == 8 and tuner.tile_tok_for("umma", 2048) == 256


def test_tstream_validity(tuna_lib):
    ok = tuner.to_config("tstream", 16, dict(row_blocks=2, k_steps=8))
    assert tuner.is_valid(tuna_lib, 4096, 16, 4096, ok)
    too_wide = tuner.to_config("tstream", 64, dict(row_blocks=2, k_steps=8))  # 2 x 64 accumulator columns > 64
    assert not tuner.is_valid(tuna_lib, 4096, 64, 4096, too_wide)
    bad_steps = tuner.to_config("tstream", 16, dict(row_blocks=1, k_steps=16))
    assert not tuner.is_valid(tuna_lib, 4096, 16, 4096, bad_steps)
    # 128-token tiles: one row block and 128-column slots only
    assert tuner.is_valid(tuna_lib, 4096, 300, 4096, tuner.to_config("tstream", 128, dict(row_blocks=1, k_steps=4)))
    assert not tuner.is_valid(tuna_lib, 4096, 300, 4096, tuner.to_config("tstream", 128, dict(row_blocks=2, k_steps=4)))
    assert not tuner.is_valid(tuna_lib, 4096, 300, 4096, tuner.to_config("tstream", 128, dict(row_blocks=1, k_steps=8)))
