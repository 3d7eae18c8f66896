"""NumPy twin of the random-weights generator (quench6k_b200/csrc/fill_normal.h), written out
operation by operation so that it gives the same bits as the host and the device: two splitmix64
outputs per element, a logarithm and a cosine made of IEEE double additions, multiplications,
divisions and one square root, Box-Muller, then float arithmetic for the scale and the mean."""
import numpy as np

_M = np.uint64(0xFFFFFFFFFFFFFFFF)


def _u64(x):
    return np.uint64(x & 0xFFFFFFFFFFFFFFFF)


def fnv1a(name):
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def stream_key(seed, name):
    return (seed * 0x9E3779B97F4A7C15 + fnv1a(name)) & 0xFFFFFFFFFFFFFFFF


def _mix(z):
    with np.errstate(over="ignore"):
        z = (z ^ (z >> np.uint64(30))) * _u64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * _u64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _log_of_uniform(n):
    bits = n.astype(np.float64).view(np.uint64)
    e = ((bits >> np.uint64(52)) & np.uint64(0x7FF)).astype(np.int64) - 1023
    m = ((bits & np.uint64(0x000FFFFFFFFFFFFF)) | np.uint64(0x3FF0000000000000)).view(np.float64)
    big = m > 1.4142135623730951
    m = np.where(big, m * 0.5, m)
    e = e + big
    s = (m + -1.0) / (m + 1.0)
    s2 = s * s
    p = np.float64(1.0) / 23.0
    for d in (21.0, 19.0, 17.0, 15.0, 13.0, 11.0, 9.0, 7.0, 5.0, 3.0):
        p = p * s2 + np.float64(1.0) / d
    p = p * s2 + 1.0
    return (e - 53).astype(np.float64) * 0.6931471805599453 + (2.0 * s) * p


def _cos_of_uniform(n):
    octant = (n >> np.uint64(50)).astype(np.int64)
    f = n & np.uint64((1 << 50) - 1)
    f = np.where(octant & 1, np.uint64(1 << 50) - f, f)
    x = (f.astype(np.float64) * 8.8817841970012523e-16) * 0.78539816339744831
    x2 = x * x
    ps = np.float64(1.0) / 355687428096000.0
    for c in (-1.0 / 1307674368000.0, 1.0 / 6227020800.0, -1.0 / 39916800.0, 1.0 / 362880.0, -1.0 / 5040.0, 1.0 / 120.0, -1.0 / 6.0):
        ps = ps * x2 + c
    ps = ps * x2 + 1.0
    sin = x * ps
    pc = np.float64(1.0) / 20922789888000.0
    for c in (-1.0 / 87178291200.0, 1.0 / 479001600.0, -1.0 / 3628800.0, 1.0 / 40320.0, -1.0 / 720.0, 1.0 / 24.0, -1.0 / 2.0):
        pc = pc * x2 + c
    cos = pc * x2 + 1.0
    v = np.where(np.isin(octant, (1, 2, 5, 6)), sin, cos)
    return np.where((octant >= 2) & (octant <= 5), -v, v)


def standard_normal(seed, name, start, count):
    """float32 [count]: elements start.. of the N(0, 1) stream of (seed, name)."""
    key = _u64(stream_key(seed, name))
    with np.errstate(over="ignore"):
        j = np.arange(start, start + count, dtype=np.uint64)
        a, b = _mix(j * np.uint64(2) + key), _mix(j * np.uint64(2) + np.uint64(1) + key)
    r = np.sqrt(-2.0 * _log_of_uniform((a >> np.uint64(11)) + np.uint64(1)))
    return (r * _cos_of_uniform(b >> np.uint64(11))).astype(np.float32)


def element_values(seed, name, start, count, std, mean):
    """float32 [count]: z * std + mean in float arithmetic (what is then cast to the tensor's dtype)."""
    return standard_normal(seed, name, start, count) * np.float32(std) + np.float32(mean)
