"""The CPU oracle against the reference project's own known answers (tests/golden)."""
import json
import math
import os

import numpy as np

from oracle import oracle as O

KATS = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))
L = O.lib()


def test_e4m3fn_reference_values():
    for code, want in KATS["e4m3fn_decode"]["cases"]:
        assert L.vo_e4m3fn_to_f32(code) == want
    for code in KATS["e4m3fn_decode"]["nan_codes"]:
        assert math.isnan(L.vo_e4m3fn_to_f32(code))


def test_e2m1_and_bf16():
    k = KATS["e2m1_bf16"]
    for code, want in k["e2m1"]:
        assert L.vo_e2m1_to_f32(code) == want
    for bits, want in k["bf16_to_f32"]:
        assert L.vo_bf16_to_f32(bits) == want
    for v, bits in k["f32_to_bf16"]:
        assert L.vo_f32_to_bf16(v) == bits
    for v in k["bf16_roundtrip_fixed"]:
        assert L.vo_bf16_to_f32(L.vo_f32_to_bf16(v)) == v


def test_payload_sizes_match_layout_contract():
    fmt = {"fp8": O.FMT_FP8, "nvfp4": O.FMT_NVFP4, "bf16": O.FMT_BF16}
    for c in KATS["payload_sizes"]["cases"]:
        assert O.payload_bytes(fmt[c["fmt"]], c["n"], c["k"]) == c["bytes"]
    q = KATS["q4k_block_bits"]
    assert O.payload_bytes(O.FMT_Q4K, 1, q["block_values"]) == q["block_bytes"]
    assert q["block_bytes"] * 8 == 4 * 256 + 128


def test_nvfp4_encoding_round_trips_its_grid():
    n, k = KATS["nvfp4_roundtrip"]["n"], KATS["nvfp4_roundtrip"]["k"]
    x = np.array([np.float32(np.float32((i * 37 % 101) - 50.0) * np.float32(0.013))
                  for i in range(n * k)], dtype=np.float32)
    x[5] = 0.0
    p = O.encode_nvfp4_ref(x.reshape(n, k))
    assert p.size == O.payload_bytes(O.FMT_NVFP4, n, k)
    y = O.decode_rows(O.FMT_NVFP4, p, n, k, 0, n)
    again = O.encode_nvfp4_ref(y)
    assert np.array_equal(O.decode_rows(O.FMT_NVFP4, again, n, k, 0, n), y)
    xs, ys = x.reshape(-1, 16), y.reshape(-1, 16)
    amax = np.abs(xs).max(axis=1, keepdims=True)
    assert (np.abs(xs - ys) <= amax / 6.0 * 1.07 + 1e-6).all()
    for v, code in KATS["e4m3_lower_encoder"]["cases"]:
        assert L.vo_f32_to_e4m3fn_lower(v) == code
    assert L.vo_e4m3fn_to_f32(L.vo_f32_to_e4m3fn_lower(1.0)) == 1.0


def test_nvfp4_scale_swizzle_is_a_permutation():
    n, k = KATS["swizzle_permutation"]["n"], KATS["swizzle_permutation"]["k"]
    seen = set()
    for r in range(n):
        for g in range(k // 16):
            o = O.nvfp4_scale_offset(r, g, k)
            assert o not in seen and o < n * k // 16
            seen.add(o)
    assert len(seen) == n * k // 16


def test_e4m3_round_trips_every_finite_code():
    for b in range(256):
        if b & 0x7F == 0x7F:
            continue
        v = L.vo_e4m3fn_to_f32(b)
        back = L.vo_f32_to_e4m3fn(v)
        if v == 0.0:
            assert back & 0x7F == 0
        else:
            assert back == b


def test_e4m3_rounds_to_nearest_even_and_saturates():
    for v, code in KATS["e4m3_rne"]["cases"]:
        assert L.vo_f32_to_e4m3fn(v) == code, v


def test_e2m1_round_trips_and_ties_to_even():
    for c in range(16):
        v = L.vo_e2m1_to_f32(c)
        if v != 0.0:
            assert L.vo_f32_to_e2m1(v) == c
    for x, want in KATS["e2m1_rne"]["decoded_after_rounding"]:
        assert L.vo_e2m1_to_f32(L.vo_f32_to_e2m1(x)) == want, x


def test_nvfp4_activation_error_is_bounded_by_the_block_scale():
    k = KATS["nvfp4_act_bound"]
    x = np.array([np.float32(np.float32((i * 37 % 29) - 14.0) * np.float32(0.37))
                  for i in range(64)], dtype=np.float32)
    q = O.quantize_activations(x, 64, O.ACT_NVFP4, k["divisor"])
    for g, o in zip(q.reshape(-1, 16), x.reshape(-1, 16)):
        amax = np.abs(o).max()
        assert (np.abs(g - o) <= amax / 6.0 * 1.07 + 1e-6).all()


def test_q4k_decoder_matches_gguf_py_known_answer():
    k = KATS["q4k_known_answer"]
    data = O.kat_q4k_blocks(k["seed"])
    v = O.decode_rows(O.FMT_Q4K, data, 1, 512, 0, 1).reshape(-1)
    v64 = v.astype(np.float64)
    close = lambda got, want: abs(got - want) <= 1e-9 * (1.0 + abs(want))
    # sequential f64 sums, as the reference test accumulates them
    s = a = w = 0.0
    for i, x in enumerate(v64):
        s += x
        a += abs(x)
        w += x * (i + 1)
    assert close(s, k["stats"][0]) and close(a, k["stats"][1]) and close(w, k["stats"][2])
    for i, want in zip(k["picks"], k["values"]):
        assert v[i] == np.float32(want), i


def test_matmul_small_and_linear_bf16():
    k = KATS["matmul_small"]
    y = O.matmul(np.array(k["x"]).reshape(k["m"], k["k"]), np.array(k["w"]).reshape(k["n"], k["k"]))
    assert y.reshape(-1).tolist() == k["y"]
    k = KATS["linear_bf16_matches_matmul"]
    payload = np.array(k["words"], dtype=np.uint16).view(np.uint8)
    y = O.linear(np.array(k["x"], dtype=np.float32), payload, O.FMT_BF16, 2, 2, 0, 2, 1)
    assert y.reshape(-1).tolist() == k["y"]


def test_f16_converter_round_trips():
    # Every finite f16 is a fixed point of f16 -> f32 -> f16; midpoints go to the even neighbour
    # (the property quant.rs:227-243 checks for its own f16 rounding).
    for h in range(0, 0x7C00, 7):
        v = L.vo_f16_to_f32(h)
        assert L.vo_f32_to_f16(v) == h
        nxt = L.vo_f16_to_f32(h + 1)
        mid = float(np.float32((np.float32(v) + np.float32(nxt)) / np.float32(2.0)))
        want = h if h % 2 == 0 else h + 1
        if h + 1 < 0x7C00:
            assert L.vo_f32_to_f16(mid) == want, hex(h)
    assert L.vo_f32_to_f16(1e6) == 0x7C00


def test_encoders_round_trip_within_format_error():
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((128, 256)) * 0.02).astype(np.float32)
    for enc, fmt, bound in ((O.encode_nvfp4_rne, O.FMT_NVFP4, 0.2), (O.encode_fp8_row, O.FMT_FP8, 0.07),
                            (O.encode_q4k, O.FMT_Q4K, 0.2)):
        p = enc(w)
        assert p.size == O.payload_bytes(fmt, 128, 256)
        d = O.decode_rows(fmt, p, 128, 256, 0, 128)
        rel = np.abs(d - w).max() / np.abs(w).max()
        assert rel < bound, (fmt, rel)
    # the RNE encoder's output is a fixed point of decode -> encode (codes on the grid stay put)
    p = O.encode_nvfp4_rne(w)
    d = O.decode_rows(O.FMT_NVFP4, p, 128, 256, 0, 128)
    # stored divisor is 448*6/amax (format.rs:392)
    div = p[-4:].view(np.float32)[0]
    assert div == np.float32(np.float32(448.0 * 6.0) / np.abs(w).max())


def test_linear_shape_errors_follow_check_linear():
    # check.rs:100-131: m != 0, rows inside the parent, payload and x / y long enough
    n, k = 128, 64
    pb = O.payload_bytes(O.FMT_NVFP4, n, k)
    assert O.linear_rc(k, pb, O.FMT_NVFP4, n, k, 0, n, 1, n) == 0
    assert O.linear_rc(k, pb, O.FMT_NVFP4, n, k, 0, n, 0, n) == -2
    assert O.linear_rc(k, pb, O.FMT_NVFP4, n, k, 100, 29, 1, 29) == -2
    assert O.linear_rc(k, pb, O.FMT_NVFP4, n, k, 0, 0, 1, 1) == -2
    assert O.linear_rc(k, pb - 8, O.FMT_NVFP4, n, k, 0, n, 1, n) == -2
    assert O.linear_rc(k - 1, pb, O.FMT_NVFP4, n, k, 0, n, 1, n) == -2
    assert O.linear_rc(k, pb, O.FMT_NVFP4, n, k, 0, n, 1, n - 1) == -2
    assert O.linear_rc(k, pb, O.FMT_NVFP4, 100, k, 0, 100, 1, 100) == -2  # N % 128
    assert O.linear_rc(200, O.payload_bytes(O.FMT_Q4K, 4, 200), O.FMT_Q4K, 4, 200, 0, 4, 1, 4) == -2


def test_linear_threads_do_not_change_results():
    r = O.Rng(7)
    p = r.random_weight(O.FMT_NVFP4, 256, 320)
    x = r.vec(33 * 320, 1.0)
    a = O.linear(x, p, O.FMT_NVFP4, 256, 320, 0, 256, 33, threads=1)
    b = O.linear(x, p, O.FMT_NVFP4, 256, 320, 0, 256, 33, threads=4)
    assert np.array_equal(a, b)
    w = O.decode_rows(O.FMT_NVFP4, p, 256, 320, 0, 256)
    want = (x.reshape(33, 320).astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)
    assert O.max_err(a, want) < 1e-6
