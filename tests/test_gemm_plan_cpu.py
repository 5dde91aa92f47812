"""The GEMM's work schedule, computed on the host by the kernel's own iterator (no GPU): every (tile, K block) is
covered exactly once, a tile is shared by at most two units, the unit that leaves a partial is the next one after the
unit that adds it, runs first on the tile's first K blocks, and all units carry the same number of K blocks within one."""
import pytest

from fp4_all_reduce_b200.ops import gemm as G

SHAPES = [(1024, 8192), (2048, 8192), (4096, 8192), (16384, 8192), (1024, 4096), (4096, 4096), (1024, 2048),
          (4096, 2048), (16384, 2048), (1000, 4096), (2300, 8192), (77, 4096), (8192, 64)]


@pytest.mark.parametrize("M,K", SHAPES)
@pytest.mark.parametrize("sms", [148, 132, 16])
def test_schedule_covers_every_k_block_once(M, K, sms):
    Nn = 6144
    pl = G.gemm_plan(M, Nn, K, sms)
    kblocks = K // 64
    rows_per_tile = 256 if pl["pair"] else 128
    assert pl["tiles"] == (Nn // pl["tile_n"]) * ((M + rows_per_tile - 1) // rows_per_tile)
    assert 1 <= pl["units"] <= (sms // 2 if pl["pair"] else sms)
    cover = {}
    work = []
    plans = [G.gemm_plan(M, Nn, K, sms, unit=u)["segments"] for u in range(pl["units"])]
    for u, segs in enumerate(plans):
        work.append(sum(c for _, _, c, _ in segs))
        seen_fix = False
        for i, (tile, lo, count, kind) in enumerate(segs):
            assert 0 <= tile < pl["tiles"] and count >= 1 and 0 <= lo and lo + count <= kblocks
            cover.setdefault(tile, []).append((lo, lo + count, u, kind))
            if kind == 0:
                assert lo == 0 and count == kblocks
            elif kind == 1:                      # leaves a partial: first thing the unit does, the tile's first K blocks
                assert pl["stream_k"] and i == 0 and lo == 0 and count < kblocks and u > 0
                prev = plans[u - 1]
                fix = [s for s in prev if s[3] == 2]
                assert len(fix) == 1 and fix[0][0] == tile and fix[0][1] == count and fix[0][2] == kblocks - count
            else:                                # adds the next unit's partial: after it only whole tiles
                assert kind == 2 and pl["stream_k"] and not seen_fix and lo + count == kblocks and u + 1 < pl["units"]
                seen_fix = True
                assert all(s[3] == 0 for s in segs[i + 1:])
                assert plans[u + 1][0][3] == 1 and plans[u + 1][0][0] == tile
    for tile in range(pl["tiles"]):
        parts = sorted(cover[tile])
        assert len(parts) <= 2 and parts[0][0] == 0 and parts[-1][1] == kblocks
        if len(parts) == 2:
            assert parts[0][1] == parts[1][0] and parts[0][3] == 1 and parts[1][3] == 2
    if pl["stream_k"]:
        assert max(work) - min(work) <= kblocks          # the cut region is balanced to one K block; whole tiles follow
        whole_waves = (pl["tiles"] - (pl["units"] + pl["tiles"] % pl["units"])) // pl["units"]
        cut = [w - whole_waves * kblocks for w in work]
        assert max(cut) - min(cut) <= 1


def test_shape_choice_for_the_bench_shapes():
    assert G.gemm_plan(4096, 6144, 8192)["pair"] == 1 and G.gemm_plan(4096, 6144, 8192)["stream_k"] == 1
    assert G.gemm_plan(16384, 6144, 8192)["stream_k"] == 0            # 1536 pair tiles on 74 pairs: 20.8 waves
    small = G.gemm_plan(1024, 6144, 2048)
    assert small["pair"] == 0 and small["tile_n"] == 192 and small["stream_k"] == 0
    with pytest.raises(ValueError):
        G.gemm_plan(128, 100, 64)
