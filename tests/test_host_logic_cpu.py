"""Host-side logic that needs no GPU: the band schedule of the host-operand pipeline -- the library's own C code,
reached through qgemm_host_band_schedule -- and the order in which the bands are uploaded."""
import pytest

from qgemm_b200.host_api import band_schedule


@pytest.mark.parametrize("extent", [1, 200, 256, 257, 1000, 4096, 8192, 32768, 100000])
@pytest.mark.parametrize("bands", [1, 3, 8, 16])
def test_bands_tile_the_extent(extent, bands):
    for shrink in (True, False):
        edges = band_schedule(extent, bands, shrink)
        assert edges[0][0] == 0 and edges[-1][1] == extent
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
        assert all(hi > lo for lo, hi in edges)
        # every band but the last is made of whole 256-wide tiles
        assert all((hi - lo) % 256 == 0 for lo, hi in edges[:-1])
    shr = band_schedule(extent, bands, True)
    assert shr[-1][1] - shr[-1][0] <= 256  # the last band of a shrinking schedule is at most one tile wide


def test_upload_order_covers_every_block_once_and_ends_with_row_strips():
    """Replays the order rule of qgemm_gemm_host (B first, then alternately, B complete before the thin last row
    bands): every (row band, column band) block of C is produced exactly once, by the later of its two bands, and the
    strips after the last column band are whole rows."""
    M, N = 8192, 8192
    mb, nb = band_schedule(M, 8, True), band_schedule(N, 8, False)
    rows_up = cols_up = 0
    ia = ib = 0
    covered = {}
    order = []
    while ia < len(mb) or ib < len(nb):
        take_a = ib >= len(nb) or (ia < len(mb) and rows_up * N < cols_up * M)
        if take_a:
            lo, hi = mb[ia]
            ia += 1
            rows_up = hi
            order.append("A")
            strips = [(i, j) for i in [ia - 1] for j in range(ib)]
        else:
            lo, hi = nb[ib]
            ib += 1
            cols_up = hi
            order.append("B")
            strips = [(i, j) for j in [ib - 1] for i in range(ia)]
        for blk in strips:
            assert blk not in covered
            covered[blk] = order[-1]
    assert len(covered) == len(mb) * len(nb)
    assert order[0] == "B" and order[-3:] == ["A", "A", "A"]
    assert "".join(order).startswith("BABABA")
