"""Host-side checks of arithmetic identities that the kernels rely on (no GPU)."""
import numpy as np


def test_float_division_as_double_product_with_the_reciprocal():
    """The stream kernel's penalty loop computes x / rep as float(double(x) * (1.0 / double(rep))), which keeps the
    division's out-of-line slow path out of the loop (sampler_stream.cu, penalise_rcp). The oracle divides in
    float. The two agree for every pair of floats: a quotient of two 24-bit numbers is at least 2^-49 of itself
    away from every midpoint of two floats, the product's error is below 2^-52."""
    rng = np.random.default_rng(20240607)
    n = 4_000_000
    x = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32).view(np.float32)
    y = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32).view(np.float32)
    # half of the divisors where penalties live: [1, 2)
    y[::2] = (y[::2].view(np.uint32) & np.uint32(0x007FFFFF) | np.uint32(0x3F800000)).view(np.float32)
    # a quarter of the dividends in the range of logits
    x[1::4] = (rng.standard_normal(x[1::4].size) * 8.0).astype(np.float32)
    keep = (x > 0) & np.isfinite(x) & ~np.isnan(y)
    x, y = x[keep], y[keep]
    with np.errstate(all="ignore"):
        q_float = x / y
        q_prod = (x.astype(np.float64) * (1.0 / y.astype(np.float64))).astype(np.float32)
    same = (q_float.view(np.uint32) == q_prod.view(np.uint32)) | (np.isnan(q_float) & np.isnan(q_prod))
    assert same.all(), (x[~same][:4], y[~same][:4])
    # the corners: denormal, huge, zero and infinite divisors
    xs = np.array([1.0, 3.0, 1e-38, 1e38, 1.17549435e-38, 5e-45, 7.0], np.float32)
    ys = np.array([3.0, 1e-45, 1e38, 1e-38, 3.0, 7.0, 0.0, np.inf, -2.5, 1.0000001], np.float32)
    for a in xs:
        with np.errstate(all="ignore"):
            qf = a / ys
            qp = (np.float64(a) * (1.0 / ys.astype(np.float64))).astype(np.float32)
        assert np.array_equal(qf.view(np.uint32), qp.view(np.uint32)), (a, qf, qp)
