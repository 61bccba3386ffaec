"""Seeded synthetic problems with the shapes and value laws of the benchmark configurations."""
import numpy as np


def w8a8_dense(m, n, k, seed, lo=-127, hi=127):
    """A int8 [m,k] row-major, B logical [k,n]; scales uniform in [1e-3, 1e-2]."""
    rng = np.random.default_rng(seed)
    a = rng.integers(lo, hi + 1, size=(m, k), dtype=np.int8)
    b = rng.integers(lo, hi + 1, size=(k, n), dtype=np.int8)
    scale = rng.uniform(1e-3, 1e-2, size=n).astype(np.float32)
    per_token = rng.uniform(1e-3, 1e-2, size=m).astype(np.float32)
    return a, b, scale, per_token


def b_storage(b_kn, layout_col_major):
    """Flat storage of logical B[k,n]: column-major = n columns of k contiguous bytes."""
    return np.ascontiguousarray(b_kn.T) if layout_col_major else np.ascontiguousarray(b_kn)


def zipf_group_sizes(total_rows, groups, seed, s=1.1):
    """Rows per expert: multinomial over p_e ~ (e+1)^-s (Zipf law over expert rank)."""
    rng = np.random.default_rng(seed)
    p = (np.arange(1, groups + 1, dtype=np.float64)) ** (-s)
    p /= p.sum()
    return rng.multinomial(total_rows, p).astype(np.int64)


def w8a8_grouped(group_sizes, n, k, seed, m_capacity=None, lo=-127, hi=127):
    """A [m,k], B logical [G,k,n], scale [G,n], per_token [m], group_list = prefix sums (int64)."""
    rng = np.random.default_rng(seed)
    group_sizes = np.asarray(group_sizes, dtype=np.int64)
    g = len(group_sizes)
    rows = int(group_sizes.sum())
    m = rows if m_capacity is None else m_capacity
    a = rng.integers(lo, hi + 1, size=(m, k), dtype=np.int8)
    b = rng.integers(lo, hi + 1, size=(g, k, n), dtype=np.int8)
    scale = rng.uniform(1e-3, 1e-2, size=(g, n)).astype(np.float32)
    per_token = rng.uniform(1e-3, 1e-2, size=m).astype(np.float32)
    group_list = np.cumsum(group_sizes).astype(np.int64)
    return a, b, scale, per_token, group_list


def zn_storage(b_kn):
    """Logical int8 B[k,n] -> the reference's zN fractal storage (layout::zN::MakeLayout<int8_t>(k, n)):
    fractals of 16 rows x 32 bytes, rows contiguous inside a fractal, fractals running down a 32-column panel
    first; k padded to 16 and n to 32 with zeros.  offset(r, c) = (c/32)*(k16*32) + r*32 + c%32."""
    k, n = b_kn.shape
    k16, n32 = (k + 15) // 16 * 16, (n + 31) // 32 * 32
    padded = np.zeros((k16, n32), np.int8)
    padded[:k, :n] = b_kn
    # [k16, n32] -> [n32/32 panels, k16, 32]
    return np.ascontiguousarray(padded.reshape(k16, n32 // 32, 32).transpose(1, 0, 2))


def zn_offset(rows, cols, r, c):
    """Offset of element (r, c) in the int8 zN layout of a rows x cols matrix (the layout class's GetOffset)."""
    rows16 = (rows + 15) // 16 * 16
    return (r // 16) * 512 + (c // 32) * (rows16 * 32) + (r % 16) * 32 + (c % 32)
