"""Host-side checks of index arithmetic that the device code shares with the host (no GPU needed: the functions are compiled for both)."""
import pytest

from supergrok15_b200 import _build
from supergrok15_b200.ops import sg2

C = _build.load()
pytestmark = pytest.mark.skipif(C is None, reason="native extension not built")


@pytest.mark.parametrize("nm", [1, 2, 15, 16, 17, 31, 32, 33, 64, 100])
@pytest.mark.parametrize("nn_", [1, 2, 3, 32, 33])
def test_gemm_tile_order_visits_every_tile_once(nm, nn_):
    """The grouped tile order of the plain tcgen05 GEMM (groups of 16 tile rows, m fastest inside a group) is a permutation of the
    tile grid, and inside a full group consecutive work items walk down the tile rows first."""
    order = C.gemm_tile_order(nm, nn_)
    assert len(order) == nm * nn_ and set(order) == {(m, n) for m in range(nm) for n in range(nn_)}
    if nm >= 16:
        assert [m for m, _ in order[:16]] == list(range(16)) and all(n == 0 for _, n in order[:16])


def test_embedding_table_splits_are_bounded():
    """Token-range splits of the shared-memory embedding gradient: none for tables that do not fit, otherwise between 1 and 64 with
    at least 64 positions per split (except for tiny inputs)."""
    assert C.embedding_bwd_table_splits(32768, 512, 115) == 64
    assert C.embedding_bwd_table_splits(32, 32, 99) == 1
    assert C.embedding_bwd_table_splits(4096, 512, 300) == 0 and C.embedding_bwd_table_splits(0, 512, 100) == 0
    for tokens in (1, 63, 64, 65, 1000, 4096, 10 ** 6):
        for D in (8, 256, 264, 4096):
            s = C.embedding_bwd_table_splits(tokens, D, 208)
            assert 1 <= s <= 64 and (s == 1 or tokens / s >= 32)


def test_scan_chunks_fill_whole_waves():
    """Chunk length of the v2 scan: a multiple of 16, at least 512, and the items (two directions) never exceed the resident wave(s)."""
    wave = sg2._wave_items()
    assert wave % (148 * 8) == 0
    for numels in ([1], [100, 200_000], [1_048_576] * 12 + [786_432] * 6 + [512] * 40, [2_359_296], [50_000_000]):
        L = sg2._pick_chunk_len(numels)
        items = 2 * sum(max(1, -(-n // L)) for n in numels)
        waves = 1 if 2 * sum(numels) <= wave * 2048 else 2
        assert L % 16 == 0 and L >= 512 and items <= wave * waves - 8
