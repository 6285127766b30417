"""CPU decoder of the packed structured half (test infrastructure; product code never imports it).

The packed form is this library's own (the reference's A1 formats, csrc/SpMM_API.cu:1127-1553, serve
its Ampere kernel), so there is no reference output to pin it against: parity unpinned for the
format itself.  What is pinned is the meaning: `unpack_a1(pack(A1)) == A1`, and the GPU product of
the packed form against the fp64 product of A1.  The 4-bit selector code of a group of four is the
reference's (index of the first kept element | index of the second << 2, csrc/SpMM_API.cu:1404-1416).
"""
import numpy as np

ROWS = 128      # rows of a block
COLS = 128      # logical k extent of a block
VALUE_BYTES = ROWS * COLS       # 128 rows x 64 kept halves x 2 bytes
META_WORDS = ROWS * 4           # 128 entries x four 32-bit words


def unpack_a1(values, meta, M, K):
    """values: uint8[blocks * 16384], meta: uint32[blocks * 512] -> dense A1 as uint16[M][K]."""
    values = np.asarray(values, dtype=np.uint8)
    meta = np.asarray(meta, dtype=np.uint32)
    blocks_m, blocks_k = M // ROWS, K // COLS
    assert values.size == blocks_m * blocks_k * VALUE_BYTES and meta.size == blocks_m * blocks_k * META_WORDS
    A1 = np.zeros((M, K), np.uint16)
    halves = values.view(np.uint16).reshape(blocks_m * blocks_k, ROWS * 64)
    words = meta.reshape(blocks_m * blocks_k, ROWS, 4)
    r = np.arange(ROWS)[:, None]            # row in block
    g = np.arange(COLS // 4)[None, :]       # group of four along k
    step, half, pos = g // 8, (g % 8) // 4, g % 4
    entry = (r % 8) + 8 * half + 16 * (r // 16)
    shift = 16 * ((r % 16) // 8) + 4 * pos
    for b in range(blocks_m * blocks_k):
        rb, kb = divmod(b, blocks_k)
        code = (words[b][entry, step] >> shift.astype(np.uint32)) & 0xF
        block = np.zeros((ROWS, COLS), np.uint16)
        for e, idx in ((0, code & 3), (1, code >> 2)):
            c = 2 * g + e                                               # column in the 128 x 64 value tile
            offset = r * 64 + (((c >> 3) ^ (r & 7)) << 3) + (c & 7)     # in halves: 128-byte swizzle
            np.put_along_axis(block.reshape(ROWS, COLS // 4, 4), idx[..., None].astype(np.int64),
                              halves[b][offset][..., None], axis=2)
        A1[rb * ROWS:(rb + 1) * ROWS, kb * COLS:(kb + 1) * COLS] = block
    return A1
