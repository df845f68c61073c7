"""How the persistent tile kernels cut the tiles of their last wave along K, walked on the host.

The kernels' unit decoding and the summing kernel's piece enumeration are ``__host__ __device__`` functions; the
library exports a host-only walk of both (``wush_debug_unit_cover``), so that the index arithmetic is checked
here for many more shapes than the GPU parity tests visit.  No GPU work.
"""
import ctypes

import numpy as np
import pytest

from wush_int4_kernel_b200 import capi


def walk(tiles, k_steps, gran, workers, mode, step_us=0.8, piece_us=0.13):
    lib = capi.load()
    cover = np.full(tiles * k_steps, -1, dtype=np.int32)
    plan = np.zeros(7, dtype=np.int32)
    ip = ctypes.POINTER(ctypes.c_int)
    status = lib.wush_debug_unit_cover(tiles, k_steps, gran, workers, mode, step_us, piece_us,
                                       cover.ctypes.data_as(ip), 2 * workers, plan.ctypes.data_as(ip))
    return status, cover, dict(zip("n_tiles k_steps full_tiles mode split ctas gran".split(), plan.tolist()))


@pytest.mark.parametrize("workers", [148, 132, 74, 8, 3])
@pytest.mark.parametrize("mode", [1, 2, -1])
def test_every_stage_of_every_tile_is_covered_once(workers, mode, monkeypatch):
    monkeypatch.delenv("WUSH_TAIL_SPLIT", raising=False)
    rng = np.random.default_rng(workers * 10 + mode + 1)
    shapes = [(workers + 1, 128, 1), (2 * workers - 1, 128, 4), (workers // 2 + 1, 64, 4), (1, 32, 1), (workers, 16, 1),
              (3 * workers + workers // 2, 16, 4), (workers + 3, 4, 4), (workers + 3, 5, 1), (workers + 1, 7, 4)]
    for _ in range(60):
        shapes.append((int(rng.integers(1, 4 * workers)), int(rng.integers(1, 40)) * int(rng.choice([1, 4])),
                       int(rng.choice([1, 4]))))
    cut = 0
    for tiles, k_steps, gran in shapes:
        status, cover, plan = walk(tiles, k_steps, gran, workers, mode)
        assert status == 0, (tiles, k_steps, gran, plan, status)
        assert (cover == 1).all(), (tiles, k_steps, gran, plan)
        assert plan["full_tiles"] % workers == 0 or plan["mode"] == 0
        assert plan["mode"] in ((0, mode) if mode > 0 else (0, 1, 2))
        if plan["mode"] == 1:
            assert (tiles - plan["full_tiles"]) * plan["split"] <= workers       # all ranges in one round
            assert k_steps % plan["split"] == 0 and (k_steps // plan["split"]) % gran == 0
        cut += plan["mode"] != 0
    assert mode < 0 or cut > 3          # the forced modes were really exercised


def test_bench_shapes_get_the_documented_split(monkeypatch):
    monkeypatch.delenv("WUSH_TAIL_SPLIT", raising=False)
    # M = 4096, N = 57344, K = 8192 with 256 x 256 tiles of fp16: 3584 tiles, 128 stages of 64
    status, cover, plan = walk(3584, 128, 1, 148, -1, 0.8)
    assert status == 0 and (cover == 1).all()
    assert plan["full_tiles"] == 3552 and plan["mode"] in (1, 2)
    # a launch of whole waves is never cut
    status, cover, plan = walk(296, 128, 1, 148, -1, 0.8)
    assert status == 0 and plan["mode"] == 0 and (cover == 1).all()


def test_switch_disables_the_split(monkeypatch):
    monkeypatch.setenv("WUSH_TAIL_SPLIT", "0")
    status, cover, plan = walk(3584, 128, 1, 148, -1, 0.8)
    assert status == 0 and plan["mode"] == 0 and (cover == 1).all()


def test_bad_arguments_are_refused():
    lib = capi.load()
    assert lib.wush_debug_unit_cover(0, 8, 1, 148, -1, 0.8, 0.13, None, 296, None) == capi.WUSH_ERR_INVALID_ARGUMENT


def test_streaming_kernel_tile_choice():
    """Up to 32 rows the smallest tile that holds them; beyond, never more padded rows than with 32-row blocks and
    no more blocks than with 8-row ones -- 40 and 48 rows are two blocks of 24, 64 rows two of 32."""
    lib = capi.load()
    tiles = lib.wush_debug_stream_tiles
    assert [tiles(m) for m in (1, 8, 9, 16, 17, 24, 25, 32)] == [1, 1, 2, 2, 3, 3, 4, 4]
    assert tiles(40) == 3 and tiles(48) == 3 and tiles(64) == 4 and tiles(72) == 3 and tiles(128) == 4
    assert tiles(0) == 0
    for m in range(1, 600):
        t = tiles(m)
        assert 1 <= t <= 4
        blocks = -(-m // (8 * t))
        assert blocks * 8 * t - m < 32 and blocks <= -(-m // 8)
        assert blocks * 8 * t <= -(-m // 32) * 32            # never more rows of work than 32-row blocks would do
