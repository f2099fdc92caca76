"""CPU restatement of what the Q4_K tensor-core decode kernel computes, against the oracle's exact
decoder: the 6-bit scale decode four bytes at a time, the 16 + q operand encoding with its
correction term, and the assignment of a lane's bytes to MMA K slots (a permutation of K that the
activations follow). Host-side arithmetic only; the kernel itself is held to the oracle by the GPU
parity tests."""
import numpy as np

from oracle import oracle as O

Q4 = O.FMT_Q4K


def _scale_words(block: np.ndarray):
    """sc[0..8), mn[0..8) of one 144-byte block, decoded as the kernel does (ggml.rs:159-169)."""
    w0, w1, w2 = (int.from_bytes(block[4 + 4 * i:8 + 4 * i].tobytes(), "little") for i in range(3))
    sc03 = w0 & 0x3F3F3F3F
    mn03 = w1 & 0x3F3F3F3F
    sc47 = (w2 & 0x0F0F0F0F) | ((w0 >> 2) & 0x30303030)
    mn47 = ((w2 >> 4) & 0x0F0F0F0F) | ((w1 >> 2) & 0x30303030)
    byte = lambda w, i: (w >> (8 * i)) & 0xFF
    sc = [byte(sc03, i) for i in range(4)] + [byte(sc47, i) for i in range(4)]
    mn = [byte(mn03, i) for i in range(4)] + [byte(mn47, i) for i in range(4)]
    return sc, mn


def _bf16_bits_to_f32(bits: int) -> float:
    return float(np.array([bits << 16], dtype=np.uint32).view(np.float32)[0])


def test_nibble_encoding_is_sixteen_plus_q():
    for q in range(16):
        assert _bf16_bits_to_f32(0x4100 | 0x80 | (q << 3)) == 16.0 + q


def test_group_sums_with_offset_reproduce_the_decoded_row():
    r = O.Rng(5)
    n, k = 3, 512
    payload = r.random_weight(Q4, n, k)
    w = O.decode_rows(Q4, payload, n, k, 0, n).reshape(n, k).astype(np.float64)
    x = r.vec(k, 1.0).astype(np.float64)
    want = w @ x
    blocks = np.frombuffer(payload.tobytes(), dtype=np.uint8)[: n * (k // 256) * 144].reshape(n, k // 256, 144)
    got = np.zeros(n)
    for row in range(n):
        for b in range(k // 256):
            blk = blocks[row, b]
            d = float(np.frombuffer(blk[0:2].tobytes(), dtype=np.float16)[0])
            dmin = float(np.frombuffer(blk[2:4].tobytes(), dtype=np.float16)[0])
            sc, mn = _scale_words(blk)
            qs = blk[16:144]
            for c in range(4):                      # 64-weight chunk: 32 bytes, low then high nibbles
                chunk = qs[32 * c:32 * c + 32]
                for half in range(2):
                    s = 2 * c + half
                    k0 = b * 256 + s * 32
                    cfr, sx = 0.0, 0.0
                    # lane t holds bytes 8t..8t+7; its first four feed the first MMA, the rest the second:
                    # a permutation of the group's 32 values, applied to x alike
                    for mma in range(2):
                        for t in range(4):
                            for i in range(4):
                                e = 8 * t + 4 * mma + i
                                q = int(chunk[e] >> 4) if half else int(chunk[e] & 15)
                                cfr += (16.0 + q) * x[k0 + e]
                                sx += x[k0 + e]
                    ds = d * sc[s]
                    got[row] += ds * cfr - (16.0 * ds + dmin * mn[s]) * sx
    assert np.allclose(got, want, rtol=1e-9, atol=1e-9)
