"""The persistent decode kernel forms the Q8_0 block scale amax / 127 as a product with RN(1/127) plus one
fused correction step instead of calling the generic division routine.  The identity was checked
exhaustively (every finite non-negative float32) when it was introduced; this is the sampled regression
guard: the same three operations, emulated in float64 where each step is exact before its single
rounding to float32, against numpy's IEEE division."""
import numpy as np

F32 = np.float32


def fma32(a, b, c):
    """float32 fused multiply-add for operands whose exact product fits float64 (24 x 24 bit significands)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(F32)


def test_div_by_127_via_fma_correction():
    rng = np.random.default_rng(5)
    bits = np.concatenate([
        rng.integers(0, 0x7F800000, size=2_000_000, dtype=np.uint32),       # any finite non-negative float
        np.arange(0, 70000, dtype=np.uint32),                               # zero and the smallest subnormals
        np.uint32(0x00800000) + np.arange(-5000, 5000).astype(np.uint32),   # around the smallest normal
        np.uint32(0x7F7FFFFF) - np.arange(0, 5000, dtype=np.uint32),        # the largest finite values
        (np.arange(1, 250, dtype=np.uint32) << 23),                         # powers of two
    ])
    a = bits.view(F32)
    r = F32(1.0) / F32(127.0)
    q0 = (a * r).astype(F32)
    rem = fma32(-q0, np.full_like(a, 127.0), a)
    q = fma32(rem, np.full_like(a, r), q0)
    ref = (a / F32(127.0)).astype(F32)
    assert np.array_equal(q.view(np.uint32), ref.view(np.uint32))
