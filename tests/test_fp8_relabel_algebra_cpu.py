"""The arithmetic behind the FP8-row kernels that use bf16 tensor-core operands, restated in numpy
and held to the oracle's E4M3 decoder (crates/velox-core/src/format.rs:320-332): an E4M3 byte
placed in a bf16 as s.0000eeee.mmm0000 is the value times 2^-120 for every finite code, the word-wise
form the kernels use (two masks and a shift per two bytes, then a byte permute) keeps the bytes in
order, and the powers of two the decode kernel moves around (2^64 on the activations, 2^56 in the
epilogue) cancel exactly."""
import numpy as np

from oracle import oracle as O


def _bf16_bits_to_f32(u16):
    return (np.asarray(u16, dtype=np.uint32) << 16).view(np.float32)


def _e4m3_values():
    # decode all 256 codes with the oracle: an FP8-row payload of one row with unit scale
    k = 256
    codes = np.arange(256, dtype=np.uint8)
    payload = np.zeros(256 + 2, dtype=np.uint8)
    payload[:k] = codes
    payload[256:258] = np.frombuffer(np.uint16(0x3F80).tobytes(), dtype=np.uint8)   # bf16 1.0
    return O.decode_rows(O.FMT_FP8, payload, 1, k, 0, 1).reshape(-1)


def test_relabelled_byte_is_the_value_times_two_to_minus_120():
    vals = _e4m3_values()
    b = np.arange(256, dtype=np.uint32)
    relabelled = _bf16_bits_to_f32(((b & 0x80) << 8) | ((b & 0x7F) << 4)).astype(np.float64)
    finite = (b & 0x7F) != 0x7F
    assert np.array_equal((relabelled * 2.0 ** 120)[finite], vals.astype(np.float64)[finite])
    # the conversion inside the GEMM multiplies by 2^120 in bf16: every finite E4M3 value is a bf16 number
    back = (relabelled * 2.0 ** 120).astype(np.float32)
    assert np.array_equal((back.view(np.uint32) & 0xFFFF)[finite], np.zeros(256, dtype=np.uint32)[finite])


def _word_form(w):
    """even = (byte0, byte2), odd = (byte1, byte3) as bf16 pairs, the kernels' three operations each."""
    w = np.asarray(w, dtype=np.uint64)
    odd = ((w >> 4) & 0x07F007F0) | (w & 0x80008000)
    v = (w << 8) & 0xFFFFFFFF
    even = ((v >> 4) & 0x07F007F0) | (v & 0x80008000)
    return even.astype(np.uint32), odd.astype(np.uint32)


def test_word_form_and_byte_permutes_keep_the_bytes_in_order():
    rng = np.random.default_rng(5)
    words = rng.integers(0, 2 ** 32, size=4096, dtype=np.uint64)
    even, odd = _word_form(words)
    by = [(words >> (8 * i)) & 0xFF for i in range(4)]
    want = [(((x & 0x80) << 8) | ((x & 0x7F) << 4)).astype(np.uint32) for x in by]
    assert np.array_equal(even & 0xFFFF, want[0]) and np.array_equal(even >> 16, want[2])
    assert np.array_equal(odd & 0xFFFF, want[1]) and np.array_equal(odd >> 16, want[3])
    # __byte_perm(even, odd, 0x5410) = (byte0, byte1); 0x7632 = (byte2, byte3): the GEMM's operand order
    lo = (even & 0xFFFF) | ((odd & 0xFFFF) << 16)
    hi = (even >> 16) | ((odd >> 16) << 16)
    assert np.array_equal(lo & 0xFFFF, want[0]) and np.array_equal(lo >> 16, want[1])
    assert np.array_equal(hi & 0xFFFF, want[2]) and np.array_equal(hi >> 16, want[3])


def test_the_powers_of_two_of_the_decode_kernel_cancel_exactly():
    vals = _e4m3_values()
    finite = (np.arange(256) & 0x7F) != 0x7F
    w = vals[finite].astype(np.float64)
    rng = np.random.default_rng(6)
    x = (rng.standard_normal(w.size) * 10.0 ** rng.uniform(-8, 8, w.size)).astype(np.float32)
    xb = (((x.view(np.uint32).astype(np.uint64) + 0x7FFF + ((x.view(np.uint32) >> 16) & 1)) & 0xFFFF0000)
          .astype(np.uint32).view(np.float32))                      # bf16 activations
    x_up = (xb.astype(np.float64) * 2.0 ** 64).astype(np.float32)    # HMUL2.BF16 by 2^64
    assert np.array_equal(x_up.view(np.uint32) & 0xFFFF, np.zeros(w.size, dtype=np.uint32))   # still bf16: exact
    prod = ((w * 2.0 ** -120) * x_up.astype(np.float64)).astype(np.float32)                    # one product in f32
    assert np.array_equal(prod.astype(np.float64) * 2.0 ** 56, w * xb.astype(np.float64))     # 12 significant bits: exact
