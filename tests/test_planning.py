"""The host-side choices of shapes: how many key slices a decode step's attention takes, how many
slices and which tile widths the products take, how many query tiles a step has.  Pure
arithmetic, no device."""
import numpy as np
import pytest

from crane_b200.kernels import Kernels
from crane_b200.parts.base import query_tiles

SMS = 148


@pytest.mark.parametrize("nkv", [1, 2, 4, 8, 32])
def test_decode_splits_fill_the_device_and_fit_the_scratch(nkv):
    for entries in range(1, 300):
        s = Kernels.decode_splits(entries, nkv, SMS)
        assert 1 <= s <= 64
        if s > 1:
            # never more CTAs than two per SM, or at most 4 slices (more CTAs than fit at once are cut
            # finer so that the last round over the SMs is fuller): what the slices' scratch is sized for
            assert entries * nkv * s <= 2 * SMS or s <= 4
        assert not 8 < s <= 11 and not 32 < s <= 40      # ranges that measured slower than 8 / 32
        # clusters of 3, 5, 6 or 7 slices only where they leave places free (they must fit into a GPC each)
        assert s >= 8 or s in (1, 2, 4) or entries * nkv * s <= 0.85 * 2 * SMS
    assert Kernels.decode_splits(8, 4, SMS) == 8           # the headline shape: one cluster per (request, kv head)
    assert Kernels.decode_splits(1, 4, SMS) == 64
    assert Kernels.decode_splits(64, 4, SMS) == 1
    # more CTAs than the 296 places: slices where the last round over the SMs would be nearly empty
    assert [Kernels.decode_splits(b, 4, SMS) for b in (72, 80, 96, 112, 128, 160, 192, 256)] == [1, 4, 2, 1, 1, 2, 1, 1]
    assert Kernels.decode_splits(1, 4, SMS, cap=16) == 16
    # few keys: at most the 8 slices that merge in their cluster
    assert Kernels.decode_splits(1, 4, SMS, max_keys=1024) == 8 and Kernels.decode_splits(1, 4, SMS, max_keys=4096) == 64
    assert Kernels.decode_splits(4, 4, SMS, max_keys=2048) == 8 and Kernels.decode_splits(16, 4, SMS, max_keys=100) == 4


def test_slices_for_fills_the_last_wave():
    for tiles in (1, 3, 16, 24, 96, 148, 200, 944):
        for k in (64, 256, 2048, 6144):
            s = Kernels.slices_for(tiles, k, SMS)
            assert 1 <= s <= max(1, (k + 63) // 64)
            assert tiles * s <= max(tiles, 3 * SMS)
    assert Kernels.slices_for(944, 2048, SMS) == 1         # the head: tiles enough without slices
    assert Kernels.slices_for(16, 6144, SMS) == 9          # 144 CTAs for 148 SMs
    assert Kernels.split_plan(2048, 6) == (5, 6)
    assert Kernels.split_plan(64, 6) == (1, 1)


def test_tile_widths():
    for m in (65, 128, 300, 2048, 8192):
        for n in (256, 2048, 3072, 12288):
            assert Kernels.tile_width_for(m, n, SMS) in Kernels.WIDE_TILES
            p = Kernels.pair_width_for(m, n, 2048, SMS)
            assert p == 0 or p in Kernels.PAIR_TILES
    assert Kernels.pair_width_for(255, 12288, 2048, SMS) == 0          # fewer than 256 rows
    assert Kernels.pair_width_for(2048, 2048, 2048, SMS) == 0          # a small product
    assert Kernels.pair_width_for(2048, 12288, 2048, SMS) > 0
    assert Kernels.tile_width_for(2048, 3072, SMS) == 192              # 256 tiles: two rounds, the narrowest that does it


def test_tile_rows():
    """Which products take the tiles of twice the rows (the rules are fitted to
    measurements; these are the measured cases)."""
    for m in (200, 256, 300, 2048, 5000, 32768):
        for n in (2048, 3072, 6144, 28672):
            for k in (2048, 4096, 14336):
                for silu in (False, True):
                    bn, rows = Kernels.pair_plan(m, n, k, SMS, silu)
                    assert (bn, rows) == (0, 0) or rows == 256 and bn in Kernels.PAIR_TILES or \
                        rows == 512 and bn in Kernels.TALL_PAIR_TILES
                    assert (bn == 0) == (Kernels.pair_width_for(m, n, k, SMS) == 0)
            t = Kernels.tall_width_for(m, n, SMS)
            assert t == 0 or t in Kernels.TALL_TILES
    assert Kernels.pair_plan(2048, 12288, 2048, SMS, True) == (224, 256)   # gate/up, 2,048 tokens: epilogue in the way
    assert Kernels.pair_plan(2048, 3072, 8192, SMS) == (192, 512)          # a long inner dimension
    assert Kernels.pair_plan(8192, 8192, 8192, SMS) == (256, 512)
    assert Kernels.pair_plan(8192, 3072, 2048, SMS) == (256, 256)          # a short one
    assert Kernels.pair_plan(2048, 2048, 6144, SMS) == (256, 256)          # 512-row tiles would be too few
    assert Kernels.tall_width_for(2048, 3072, SMS) == 192                  # one round of 128 tiles instead of two
    assert Kernels.tall_width_for(2048, 2048, SMS) == 0                    # 128 x 256 tiles already take one round
    assert Kernels.tall_width_for(128, 3072, SMS) == 0


class _Ctx:
    pass


def test_query_tiles_exact_and_bound():
    c = _Ctx()
    c.n_entries, c.n_tokens, c.graph_key = 3, 300, None
    c.h_cu_q = np.array([0, 1, 130, 300], dtype=np.int32)
    assert query_tiles(c, 128) == 1 + 2 + 2
    assert query_tiles(c, 64) == 1 + 3 + 3
    # a step that replays a graph: the most tiles any step of its shape can have
    c.graph_key = ("rows", 320, 4, 4)
    c.n_entries, c.n_tokens = 4, 320
    assert query_tiles(c, 128) == 4 + 2
    for lens in ([320, 0, 0, 0], [1, 1, 1, 317], [127, 129, 63, 1], [80, 80, 80, 80]):
        exact = sum(-(-q // 128) for q in lens)
        assert exact <= query_tiles(c, 128)
