"""Index arithmetic of the peer-gathered GEMM, restated on the CPU: every row of every peer's shard is produced exactly
once, tiles of the own shard come first (or alternate with remote ones), and the ready word a tile waits for is the
one its copy piece publishes."""
import pytest


def tile_to_rows(m_blk, a_peers, a_rows, a_first, interleave):
    """Mirror of the kernel's mapping (gemm_sm100.cu): m tile -> (peer, first local row, tile index in the shard)."""
    a_tiles = (a_rows + 127) // 128
    slot = m_blk % a_peers if interleave else m_blk // a_tiles
    lm = m_blk // a_peers if interleave else m_blk % a_tiles
    return (slot + a_first) % a_peers, lm * 128, lm


@pytest.mark.parametrize("a_peers,a_rows,rank,interleave", [(2, 328, 0, True), (2, 328, 1, False), (4, 17408, 2, True),
                                                              (8, 130, 5, False), (3, 128, 1, True)])
def test_every_row_once_and_own_shard_first(a_peers, a_rows, rank, interleave):
    a_tiles = (a_rows + 127) // 128
    seen = set()
    for m_blk in range(a_tiles * a_peers):
        peer, r0, lm = tile_to_rows(m_blk, a_peers, a_rows, rank, interleave)
        for r in range(r0, min(r0 + 128, a_rows)):
            key = peer * a_rows + r                     # the output row number the epilogue uses
            assert key not in seen
            seen.add(key)
    assert seen == set(range(a_peers * a_rows))
    assert tile_to_rows(0, a_peers, a_rows, rank, interleave)[0] == rank
    if not interleave:
        assert all(tile_to_rows(i, a_peers, a_rows, rank, False)[0] == rank for i in range(a_tiles))


@pytest.mark.parametrize("rows", [128, 328, 640, 17408, 69632])
def test_ready_word_of_a_tile_matches_its_copy_piece(rows):
    tiles = (rows + 127) // 128
    chunks = max(1, min(4, tiles))                      # ops/tp_fused.py
    chunk_tiles = (tiles + chunks - 1) // chunks        # same formula in gemm_host.cu
    chunk_rows = chunk_tiles * 128
    for lm in range(tiles):
        word = min(lm // chunk_tiles, chunks - 1)       # kernel: which ready word the tile polls
        # stream_ops.cpp: piece c covers rows [c * chunk_rows, (c + 1) * chunk_rows), the last one to the end
        c0 = word * chunk_rows
        c1 = rows if word == chunks - 1 else min(c0 + chunk_rows, rows)
        assert c0 <= lm * 128 and min(lm * 128 + 128, rows) <= c1
