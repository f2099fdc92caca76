"""Addressing of the tensor-parallel norm's 16-byte scale pieces, restated on the CPU: the scale
bytes of the four rows q, q + 32, q + 64, q + 96 of a 128-row tile, for the four 16-wide groups of
one 64-wide slice of K, are exactly the 16 consecutive bytes at piece q of that slice's 512-byte
atom (crates/velox-core/src/format.rs:345-354), in the order the kernel assembles them (row index
times four plus group)."""
import numpy as np

from velox_inferer_b200 import nvfp4_scale_offset


def test_four_rows_of_a_tile_fill_one_16_byte_piece_per_atom():
    k = 5120
    k_tiles = k // 64
    for row0 in (0, 256, 1792):                  # first row of a rank's block (a multiple of 128)
        for block in (0, 5, 31, 32, 63):         # the kernel's block index within the rank's rows
            quad_first = (block // 32) * 128 + block % 32
            for atom in (0, 1, k_tiles - 1):
                piece_off = (((row0 + quad_first) // 128) * k_tiles + atom) * 512 + (quad_first % 32) * 16
                got = {}
                for ri in range(4):
                    row = row0 + quad_first + 32 * ri
                    for g4 in range(4):
                        g = atom * 4 + g4
                        got[ri * 4 + g4] = nvfp4_scale_offset(row, g, k)
                assert [got[i] for i in range(16)] == list(range(piece_off, piece_off + 16))


def test_pieces_of_all_blocks_tile_the_scale_plane_of_the_ranks_rows():
    k, rows, row0 = 512, 256, 128
    k_tiles = k // 64
    seen = np.zeros((row0 + rows) // 128 * k_tiles * 512, dtype=np.int32)
    for block in range(rows // 4):
        quad_first = (block // 32) * 128 + block % 32
        for atom in range(k_tiles):
            off = (((row0 + quad_first) // 128) * k_tiles + atom) * 512 + (quad_first % 32) * 16
            seen[off:off + 16] += 1
    first = row0 // 128 * k_tiles * 512
    assert not seen[:first].any() and np.all(seen[first:] == 1)
