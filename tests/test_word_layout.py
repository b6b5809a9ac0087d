"""Index arithmetic of the {payload, epoch} word format the GPUs exchange, modelled in numpy.

The publisher turns every 16-byte word of q [B][Hq][128] (16-bit) into four 8-byte words
{two 16-bit values, epoch}; a consumer lane (g = lane / 4 its head within the group,
t = lane % 4) reads fixed word indices of its head's row.  The partial rows go back as
{fp32, epoch} words, lane l owning dims 4l..4l+3.  These tests restate both sides'
formulas (peerkv_b200/csrc/ptx.cuh `st_ll_q16`, `st_ll_row`, `ld_ll_row4`; the q loads of
peerkv_b200/csrc/decode_kernel.cuh) and check that what is read is what was written.
"""
import numpy as np

D = 128


def publish_q(q_u16: np.ndarray, epoch: int) -> np.ndarray:
    """q_u16 [B, Hq, 128] uint16 -> inbox [B * Hq * 64] uint64 words, written 16 bytes at a time."""
    flat32 = q_u16.reshape(-1).view(np.uint32)              # 32-bit pairs, as the kernel sees them
    n16 = flat32.size // 4
    inbox = np.zeros(n16 * 4, dtype=np.uint64)
    tag = np.uint64(epoch & 0xFFFFFFFF) << np.uint64(32)
    for i in range(n16):                                     # one lane's st_ll_q16
        x, y, z, w = (np.uint64(v) for v in flat32[4 * i:4 * i + 4])
        inbox[4 * i + 0] = x | tag
        inbox[4 * i + 1] = y | tag
        inbox[4 * i + 2] = z | tag
        inbox[4 * i + 3] = w | tag
    return inbox


def test_q_words_16bit_pools():
    rng = np.random.default_rng(0)
    B, Hq, G = 2, 8, 4
    q = rng.integers(0, 65536, size=(B, Hq, D), dtype=np.uint16)
    epoch = 0x1_0000_0007                                    # only the low half travels
    inbox = publish_q(q, epoch)
    for s in range(B):
        for kvh in range(Hq // G):
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                if g >= G:
                    continue
                row = (s * Hq + kvh * G + g) * (D // 2)     # q_ll_row
                for ks in range(8):
                    for half, word in ((0, ks * 8 + t), (1, ks * 8 + 4 + t)):
                        w = int(inbox[row + word])
                        assert w >> 32 == epoch & 0xFFFFFFFF
                        d = 16 * ks + 8 * half + 2 * t       # the pair the MMA B-fragment register holds
                        lo, hi = w & 0xFFFF, (w >> 16) & 0xFFFF
                        assert (lo, hi) == (int(q[s, kvh * G + g, d]), int(q[s, kvh * G + g, d + 1]))


def test_q_words_1byte_pools():
    rng = np.random.default_rng(1)
    B, Hq, G = 1, 8, 8
    q = rng.integers(0, 65536, size=(B, Hq, D), dtype=np.uint16)
    inbox = publish_q(q, 5)
    for lane in range(32):
        g, t = lane >> 2, lane & 3
        row = g * (D // 2)
        for i in range(8):
            d0 = 32 * (i >> 1) + 16 * (i & 1) + 4 * t       # four consecutive values, two words
            assert d0 % 4 == 0 and (d0 // 2) % 2 == 0       # a 16-byte aligned pair of words
            w0, w1 = int(inbox[row + d0 // 2]), int(inbox[row + d0 // 2 + 1])
            assert w0 >> 32 == 5 and w1 >> 32 == 5
            got = [w0 & 0xFFFF, (w0 >> 16) & 0xFFFF, w1 & 0xFFFF, (w1 >> 16) & 0xFFFF]
            assert got == [int(v) for v in q[0, g, d0:d0 + 4]]


def test_partial_row_words_round_trip_and_stale_detection():
    rng = np.random.default_rng(2)
    rows = 6
    o = rng.standard_normal((rows, D)).astype(np.float32)
    lse = rng.standard_normal(rows).astype(np.float32)
    o_ll = np.zeros(rows * D, dtype=np.uint64)
    lse_ll = np.zeros(rows, dtype=np.uint64)

    def store(epoch, which):
        tag = np.uint64(epoch) << np.uint64(32)
        for r in which:
            for lane in range(32):                           # st_ll_row
                for k in range(4):
                    o_ll[r * D + lane * 4 + k] = np.uint64(o[r, lane * 4 + k].view(np.uint32)) | tag
            lse_ll[r] = np.uint64(lse[r].view(np.uint32)) | tag

    def load(epoch, r):
        """(fresh, O row, lse) as ld_ll_row4 of 32 lanes plus the lse word see it."""
        words = o_ll[r * D:(r + 1) * D]
        fresh = bool(np.all(words >> np.uint64(32) == np.uint64(epoch))) and int(lse_ll[r]) >> 32 == epoch
        vals = (words & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32)
        return fresh, vals, np.uint32(int(lse_ll[r]) & 0xFFFFFFFF).view(np.float32)

    store(3, range(rows))
    for r in range(rows):
        fresh, vals, l = load(3, r)
        assert fresh and np.array_equal(vals, o[r]) and l == lse[r]
    # the next step has only reached some rows: the others still carry epoch 3 and are refused
    store(4, [0, 2])
    assert [load(4, r)[0] for r in range(rows)] == [True, False, True, False, False, False]
    # a row that is half written (some lanes' words of the new step, the rest old) is refused too
    tag5 = np.uint64(5) << np.uint64(32)
    o_ll[1 * D:1 * D + 64] = (o_ll[1 * D:1 * D + 64] & np.uint64(0xFFFFFFFF)) | tag5
    assert not load(5, 1)[0]


def test_exchange_sizes():
    """Bytes of one GPU's mailbox slab as pkv_exchange_create lays it out (256-byte aligned
    regions: q inbox, O slots, lse slots, probe flag)."""
    def align(v, a=256):
        return (v + a - 1) // a * a
    B, Hq, world = 16, 32, 8
    q_inbox = align(B * Hq * (D // 2) * 8)
    o_slots = align(world * B * Hq * D * 8)
    lse_slots = align(world * align(B * Hq, 64) * 8)
    assert q_inbox == 262144 and o_slots == 4194304 and lse_slots == 32768
    assert q_inbox + o_slots + lse_slots + 256 == 4489472    # the 4.5 MB of the bench workload on 8 GPUs
