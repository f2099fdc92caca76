"""Why the bf16-kind GEMM feeds Q4_K values as three bf16 terms and sums K in chunks.

A CPU model of a tensor-core sum: products of one MMA instruction (16 values of K) are added
exactly, the running f32 sum is rounded toward zero after every instruction. On the reference's
random Q4_K blocks at K = 2560 (values up to 30, sums that cancel) this model reproduces what the
GPU showed: two bf16 terms per value miss the 2e-4 conformance bound even with exact summation,
three terms with one long truncating sum miss it too, three terms with sums of 16 instructions
added in ordinary f32 arithmetic (what the kernel's epilogue does with its two accumulators) meet
it with room to spare. The shape and the data recipe are those of
crates/velox-conformance/src/lib.rs:4153-4176."""
import numpy as np

from oracle import oracle as O

N, K, M = 96, 2560, 70
TOL = 2e-4   # crates/velox-conformance/src/lib.rs:356


def _bf16(a):
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)


def _toward_zero(a, bits=24):
    m, e = np.frexp(a)
    return np.ldexp(np.trunc(m * 2.0 ** bits) / 2.0 ** bits, e)


def _data():
    r = O.Rng(0x51a7)
    payload = r.random_weight(O.FMT_Q4K, N, K)
    x = _bf16(r.vec(M * K, 1.0)).reshape(M, K).astype(np.float64)
    w = O.decode_rows(O.FMT_Q4K, payload, N, K, 0, N).astype(np.float32)
    return x, w, x @ w.astype(np.float64).T


def _metric(got, want):
    return float(np.max(np.abs(got - want) / (1.0 + np.abs(want))))


def _terms(w):
    hi = _bf16(w)
    mid = _bf16(w - hi)
    lo = _bf16(w - hi - mid)
    return hi, mid, lo


def test_three_bf16_terms_hold_a_q4k_value_exactly_and_two_do_not_meet_the_bound():
    x, w, want = _data()
    hi, mid, lo = _terms(w)
    assert np.array_equal(hi.astype(np.float64) + mid.astype(np.float64) + lo.astype(np.float64), w.astype(np.float64))
    two = x @ (hi.astype(np.float64) + mid.astype(np.float64)).T
    assert _metric(two, want) > TOL           # 2^-17 per weight is not enough on sums that cancel
    assert _metric(x @ hi.astype(np.float64).T, want) > 100 * TOL


def _summed(x, terms, chunk):
    total = np.zeros((M, N), dtype=np.float32)
    acc = np.zeros((M, N))
    steps = 0
    for t in terms:
        t = t.astype(np.float64)
        for s in range(0, K, 16):
            acc = _toward_zero(acc + x[:, s:s + 16] @ t[:, s:s + 16].T)
            steps += 1
            if chunk and steps % chunk == 0:
                total = (total + acc.astype(np.float32)).astype(np.float32)
                acc = np.zeros((M, N))
    return (total + acc.astype(np.float32)).astype(np.float64)


def test_one_long_truncating_sum_misses_the_bound_and_chunked_sums_meet_it():
    x, w, want = _data()
    terms = _terms(w)
    assert _metric(_summed(x, terms, None), want) > TOL
    assert _metric(_summed(x, terms, 16), want) < TOL / 3     # four k-blocks of four MMAs each: the kernel's chunk
