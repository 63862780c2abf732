"""The lane / row / group arithmetic of the five-bit decode kernel (csrc/tsp_gemv_k5.cu), replayed on the CPU for shapes the GPU
tests do not reach (group counts that are not powers of two: the reference model's 2560 channels and 640 hidden units): every
(row, group) pair of a block's rows is visited by exactly one lane, the lanes that share a row form one aligned run whose
width the shuffle reduction covers, and the staged activation index stays inside the shared-memory extent the host sizes."""
import pytest

BLOCK_ROWS, WARPS = 64, 8


def lanes_per_row(groups):
    lpr = 1
    while lpr * 2 <= groups and lpr < 32:
        lpr *= 2
    return lpr


@pytest.mark.parametrize("rows,cols", [(640, 2560), (2560, 640), (512, 2048), (2048, 512), (16, 64), (96, 96), (8, 32), (72, 160), (24, 2048)])
@pytest.mark.parametrize("count", [1, 8])
def test_every_row_group_pair_is_visited_once(rows, cols, count):
    groups = cols // 32
    lpr = lanes_per_row(groups)
    rpw = 32 // lpr
    assert lpr & (lpr - 1) == 0 and 1 <= lpr <= 32 and lpr <= max(groups, 1)
    smem_float4 = count * groups * 9                      # what launch_gemv_k5 sizes for `count` token rows
    for block in range((rows + BLOCK_ROWS - 1) // BLOCK_ROWS):
        row0 = block * BLOCK_ROWS
        seen = {}
        for warp in range(WARPS):
            rb = row0 + warp * rpw
            while rb < row0 + BLOCK_ROWS and rb < rows:   # the kernel's loop bound: uniform over the warp
                for lane in range(32):
                    sub, lig = lane // lpr, lane & (lpr - 1)
                    r = rb + sub
                    live = r < rows and r < row0 + BLOCK_ROWS
                    # lanes of one row: an aligned run of lpr lanes (what the xor shuffles with offsets < lpr add up)
                    assert (lane ^ lig) // lpr * lpr == lane - lig
                    grp = lig
                    while grp < groups:
                        for j in range(count):
                            for i4 in (0, 7):
                                assert (j * groups + grp) * 9 + i4 < smem_float4
                        if live:
                            seen[(r, grp)] = seen.get((r, grp), 0) + 1
                        grp += lpr
                rb += WARPS * rpw
        want_rows = range(row0, min(row0 + BLOCK_ROWS, rows))
        assert set(seen) == {(r, g) for r in want_rows for g in range(groups)}
        assert all(v == 1 for v in seen.values())


def test_staging_covers_each_activation_piece_once():
    """The staging loop writes piece (token j, group, i4) from float4 index `rem` of the token's row."""
    for groups, count in ((80, 3), (20, 8), (2, 1)):
        written = {}
        total = count * groups * 8
        for i in range(total):
            j, rem = divmod(i, groups * 8)
            written[(j * groups + (rem >> 3)) * 9 + (rem & 7)] = (j, rem)
        assert len(written) == total                                   # no two pieces share a slot
        assert all((slot % 9) < 8 for slot in written)                 # the ninth float4 of every group is padding
        assert {v for v in written.values()} == {(j, r) for j in range(count) for r in range(groups * 8)}


def test_q8_span_boxes_of_the_grouped_kernel_are_aligned_and_inside_the_row():
    """csrc/tsp_grouped_mma.cu, Q8_0 GGUF blocks: a quant stage is a 144-byte box per row starting at 136 * span for even spans and
    8 bytes earlier for odd ones. A tensor copy must start on a 16-byte boundary and here never leaves the row; the chunk a
    dequantise thread reads (68 bytes = 17 words) lies inside the five 16-byte pieces it loads."""
    for cols in range(256, 8192 + 1, 256):
        row_bytes = cols // 32 * 34
        spans = cols // 128
        assert row_bytes % 16 == 0 and spans % 2 == 0
        for sb in range(spans):
            x = sb * 136 - (8 if sb & 1 else 0)
            assert x % 16 == 0 and x >= 0 and x + 144 <= row_bytes
            for half in (0, 1):
                start = (8 if sb & 1 else 0) + 68 * half          # byte of the chunk inside the 144-byte line
                piece0 = half * 4                                  # first 16-byte piece loaded
                ws = half + 2 * (sb & 1)                           # first word of the chunk among the 20 loaded
                assert start == piece0 * 16 + ws * 4
                assert piece0 * 16 <= start and start + 68 <= (piece0 + 5) * 16 <= 144
                # the blocks of the chunk inside the row: 2 * half and 2 * half + 1 of the span's four
                assert x + start == sb * 136 + 68 * half == (sb * 4 + 2 * half) * 34
