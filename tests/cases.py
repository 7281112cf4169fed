"""Seeded input generators shared by the parity tests and the golden-vector
script. Shapes and seed formulas follow the reference's own tests
(tests/test_attention.py:48-79 for the contiguous cases,
tests/test_attention_paged.py:40-59 for the paged ones); the five benchmark
configurations are reduced to oracle-sized versions of the same shapes."""

import numpy as np

PAGE = 16

# (batch, q heads, kv heads, cache rows, dim, with_lens) - the reference's
# SHAPES matrix, tests/test_attention.py:58-68
SHAPES = [
    (1, 8, 2, 1, 64, False),
    (1, 32, 8, 517, 128, False),
    (1, 32, 32, 100, 64, False),
    (3, 12, 4, 64, 32, True),
    (2, 6, 3, 33, 8, True),
    (1, 4, 1, 16, 4, True),
    (1, 8, 8, 0, 64, False),
    (2, 4, 4, 0, 32, True),
    (1, 2, 2, 4096, 256, False),
]


def shape_seed(b, hq, hkv, t, d):
    """tests/test_attention.py:73"""
    return b * 1000 + hq * 31 + hkv * 7 + t + d


def make_case(rng, b, hq, hkv, t, d, with_lens):
    """tests/test_attention.py:48-55"""
    q = rng.standard_normal((b, hq, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, t, d)).astype(np.float32)
    lens = None
    if with_lens:
        lens = rng.integers(0, t + 1, size=b).astype(np.int32)
    return q, k, v, lens


def make_paged_case(rng, b, hq, hkv, d, nb, lens, page=PAGE):
    """Pools, a random (non-monotonic, possibly repeating) block table and the
    contiguous cache the table materialises to.
    tests/test_attention_paged.py:40-59"""
    nseq = len(lens)
    width = max((l + page - 1) // page for l in lens) if nseq else 1
    width = max(width, 1)
    k_pool = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
    v_pool = rng.standard_normal((nb, hkv, page, d)).astype(np.float32)
    table = rng.integers(0, nb, (b, width)).astype(np.int32)
    t_rows = width * page
    k_cache = np.zeros((b, hkv, t_rows, d), dtype=np.float32)
    v_cache = np.zeros((b, hkv, t_rows, d), dtype=np.float32)
    for bi in range(b):
        for s in range(width):
            k_cache[bi, :, s * page:(s + 1) * page] = k_pool[table[bi, s]]
            v_cache[bi, :, s * page:(s + 1) * page] = v_pool[table[bi, s]]
    q = rng.standard_normal((b, hq, d)).astype(np.float32)
    return q, k_pool, v_pool, table, k_cache, v_cache, np.asarray(lens, np.int32)


# name -> (seed, b, hq, hkv, d, nb, lens): the reference's paged pins
PAGED_CASES = {
    "paged_41": (41, 3, 8, 2, 64, 20, [37, 16, 48]),
    "paged_42": (42, 3, 4, 4, 32, 8, [37, 16, 0]),
    "paged_43": (43, 2, 2, 2, 128, 4, [1, PAGE]),
    "paged_47": (47, 3, 8, 2, 64, 20, [511, 100, 1024]),
    "paged_49": (49, 2, 8, 2, 64, 12, [100, 512]),
}


# (batch, q heads, kv heads, seq, dim) - the reference's PREFILL_SHAPES,
# tests/test_attention.py:176-184
PREFILL_SHAPES = [
    (1, 4, 2, 1, 32),
    (1, 8, 8, 5, 64),
    (2, 6, 3, 17, 16),
    (1, 32, 8, 40, 128),
    (1, 4, 1, 33, 8),
    (1, 8, 2, 64, 256),
    (1, 4, 2, 9, 512),
]


def make_prefill_case(b, hq, hkv, s, d, causal):
    """Seed and generators of tests/test_attention.py:191-196."""
    rng = np.random.default_rng(b * 100 + hq * 17 + s * 3 + d + int(causal))
    q = rng.standard_normal((b, hq, s, d)).astype(np.float32)
    k = rng.standard_normal((b, hkv, s, d)).astype(np.float32)
    v = rng.standard_normal((b, hkv, s, d)).astype(np.float32)
    return q, k, v


def round_to(x, dtype):
    """Round float32 values to bf16 / fp16 storage and widen back to float32:
    the 'half-rounded inputs' the oracle is fed for half-precision cases."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    return t.to(dtype).to(torch.float32).numpy()


# ---- the five benchmark configurations, reduced to oracle size -------------
# Each keeps the head layout, dim, dtype, value distribution and (for the
# ragged ones) the length distribution of the full configuration; batch and
# length are cut so the CPU oracle finishes in seconds.

def config1():
    """B=1, 8 q = 8 kv heads, D=64, T=512, fp32, seed 0, q then k then v."""
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 8, 64)).astype(np.float32)
    k = rng.standard_normal((1, 8, 512, 64)).astype(np.float32)
    v = rng.standard_normal((1, 8, 512, 64)).astype(np.float32)
    return q, k, v


def config2(batch=2, t=4096):
    """Llama-3-8B shape: 32 q / 8 kv heads, D=128, K and V scaled by 0.5."""
    rng = np.random.default_rng(0)
    q = rng.standard_normal((batch, 32, 128)).astype(np.float32)
    k = (rng.standard_normal((batch, 8, t, 128)) * 0.5).astype(np.float32)
    v = (rng.standard_normal((batch, 8, t, 128)) * 0.5).astype(np.float32)
    return q, k, v


def config3_lens(batch=64):
    """Ragged lengths uniform in [128, 8192] (first draw of seed 0)."""
    return np.random.default_rng(0).integers(128, 8193, batch).astype(np.int32)


def config5_lens(batch=256):
    """Ragged lengths log-uniform in [1024, 32768] (first draw of seed 0)."""
    u = np.random.default_rng(0).uniform(np.log(1024), np.log(32768), batch)
    return np.floor(np.exp(u)).astype(np.int32)


def paged_layout(lens, page=PAGE, slack=1.1, seed=1):
    """Block table = random permutation of a pool sized to the sum of pages
    plus slack, dealt row by row; unused slots 0."""
    pages = (np.asarray(lens, np.int64) + page - 1) // page
    total = int(pages.sum())
    nb = max(1, int(np.ceil(slack * total)))
    width = max(1, int(pages.max()) if len(pages) else 1)
    perm = np.random.default_rng(seed).permutation(nb).astype(np.int32)
    table = np.zeros((len(lens), width), np.int32)
    pos = 0
    for i, n in enumerate(pages):
        table[i, :n] = perm[pos:pos + n]
        pos += int(n)
    return table, nb, width
