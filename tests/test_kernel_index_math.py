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


def _funnelshift_r(lo, hi, n):
    return (((hi << 32) | lo) >> n) & 0xFFFFFFFF


def _byte_perm(a, b, sel):
    src = [(a >> (8 * i)) & 255 for i in range(4)] + [(b >> (8 * i)) & 255 for i in range(4)]
    return sum(src[(sel >> (4 * i)) & 7] << (8 * i) for i in range(4))


def test_q8_chunk_words_give_the_blocks_codes_in_tile_order():
    """q8_chunk_row of csrc/tsp_grouped_mma.cu replayed with integers: from the five 16-byte pieces a dequantise thread loads, the
    scale half-words and the realigned code words of the chunk's two blocks, and the 0x6400 | (byte ^ 0x80) operand (1152 + q as
    binary16 bits) in the order the tiles use inside every run of eight (0, 2, 1, 3, 4, 6, 5, 7)."""
    import numpy as np
    rng = np.random.default_rng(7)
    for parity in (0, 1):
        blocks = rng.integers(0, 256, size=(4, 34), dtype=np.uint8)          # one span: four Q8_0 blocks
        line = np.zeros(144, dtype=np.uint8)
        line[:] = rng.integers(0, 256, size=144, dtype=np.uint8)              # neighbouring bytes are arbitrary
        off = 8 if parity else 0
        line[off:off + 136] = blocks.reshape(-1)
        words = line.view("<u4").astype(np.uint64)
        for half in (0, 1):
            L = [int(w) for w in words[half * 4 * 4: half * 4 * 4 + 20]]
            ws = half + 2 * parity
            s0, s1 = L[ws] & 0xFFFF, L[ws + 8] >> 16
            b0, b1 = blocks[2 * half], blocks[2 * half + 1]
            assert s0 == int(b0[0]) | (int(b0[1]) << 8) and s1 == int(b1[0]) | (int(b1[1]) << 8)
            for u in range(8):
                if u < 4:
                    a = _funnelshift_r(L[ws + 2 * u], L[ws + 2 * u + 1], 16)
                    b = _funnelshift_r(L[ws + 2 * u + 1], L[ws + 2 * u + 2], 16)
                else:
                    a, b = L[ws + 9 + 2 * (u - 4)], L[ws + 10 + 2 * (u - 4)]
                a ^= 0x80808080
                b ^= 0x80808080
                w = [_byte_perm(a, 0x64646464, 0x4240), _byte_perm(a, 0x64646464, 0x4341), _byte_perm(b, 0x64646464, 0x4240), _byte_perm(b, 0x64646464, 0x4341)]
                halves = [h for x in w for h in (x & 0xFFFF, x >> 16)]       # eight binary16 bit patterns in staged order
                codes = (b0 if u < 4 else b1)[2 + 8 * (u % 4): 2 + 8 * (u % 4) + 8].astype(np.int8)
                for pos, k in enumerate((0, 2, 1, 3, 4, 6, 5, 7)):
                    assert halves[pos] == 0x6400 | ((int(codes[k]) + 128) & 255)       # 1024 + (q + 128) = 1152 + q
                    assert np.array([halves[pos]], dtype=np.uint16).view(np.float16)[0] == 1152 + int(codes[k])


def test_five_bit_code_assembly():
    """Group5 of csrc/tsp_gemv_k5.cu replayed with integers: Q5_1 spreads four fifth bits to bit 4 of four bytes with one multiply,
    Q5_K takes bit g of the fifth-bit bytes; byte k of the result converts through the 0x4B000000 magic number."""
    import numpy as np
    for hb in range(16):
        spread = ((hb * 0x00204081) & 0x01010101) << 4
        assert spread == sum(((hb >> k) & 1) << (8 * k + 4) for k in range(4))
    rng = np.random.default_rng(11)
    for _ in range(200):
        qs, qh, g = int(rng.integers(0, 1 << 32)), int(rng.integers(0, 1 << 32)), int(rng.integers(0, 8))
        q = ((qs >> (4 * (g & 1))) & 0x0F0F0F0F) | (((qh >> g) & 0x01010101) << 4)
        for k in range(4):
            want = (((qs >> (8 * k)) & 255) >> (4 * (g & 1)) & 15) | ((((qh >> (8 * k)) & 255) >> g & 1) << 4)
            assert (q >> (8 * k)) & 255 == want
            bits = _byte_perm(q, 0x4B000000, 0x7440 + k)
            assert np.array([bits], dtype=np.uint32).view(np.float32)[0] - np.float32(8388608.0) == want
