"""Property tests (hypothesis) of the oracle's integer stages: the invariants the
GPU tests rely on when they check large inputs without a golden answer."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from oracle import cenc, ptv3_oracle as O

ORDERS = ["z", "z-trans", "hilbert", "hilbert-trans"]


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 16), st.integers(0, 2 ** 31 - 1), st.sampled_from(ORDERS))
def test_encode_is_hierarchical_and_bounded(depth, seed, order):
    rng = np.random.default_rng(seed)
    g = rng.integers(0, 1 << depth, size=(200, 3)).astype(np.int32)
    b = rng.integers(0, 4, size=200)
    c = cenc.encode(g, b, depth, order)
    assert (c >= 0).all() and (c >> (3 * depth) == b).all()
    if depth > 1:
        parent = cenc.encode(g >> 1, b, depth - 1, order)
        assert (((c & ((1 << 3 * depth) - 1)) >> 3) == (parent & ((1 << 3 * (depth - 1)) - 1))).all()


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 16), st.integers(0, 2 ** 31 - 1))
def test_decode_inverts_encode(depth, seed):
    rng = np.random.default_rng(seed)
    g = rng.integers(0, 1 << depth, size=(100, 3)).astype(np.int64)
    for order in ("z", "hilbert"):
        grid, batch = cenc.decode(cenc.encode(g, None, depth, order), depth, order)
        assert (grid == g).all() and (batch == 0).all()


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(1, 700), min_size=1, max_size=5), st.integers(1, 300))
def test_pad_plan_invariants(counts, K):
    """model.py:382-438: every rank appears in `pad`, owns exactly one padded row, scenes
    longer than K are padded to a multiple of K by rows of the same scene."""
    offset = torch.cumsum(torch.tensor(counts), 0)
    pad, unpad, cu = O.pad_plan(offset, K)
    n = sum(counts)
    assert unpad.shape[0] == n and torch.equal(pad[unpad], torch.arange(n))
    assert int(cu[-1]) == pad.shape[0] and bool((cu[1:] > cu[:-1]).all())
    starts = [0] + offset.tolist()
    pos = 0
    for s, c in enumerate(counts):
        cp = c if c <= K else (c + K - 1) // K * K
        seg = pad[pos:pos + cp]
        assert bool((seg >= starts[s]).all()) and bool((seg < starts[s + 1]).all())
        assert torch.equal(seg[:c], torch.arange(starts[s], starts[s + 1]))
        pos += cp
    assert pos == pad.shape[0]


@settings(max_examples=25, deadline=None)
@given(st.integers(0, 2 ** 31 - 1), st.integers(50, 400))
def test_pooled_orders_equal_argsort_of_pooled_codes(seed, n):
    """Children of a parent cell are contiguous in every order, so the pooled order of a
    row is its fine order with repeated cluster ids removed (what the CUDA plan does)."""
    rng = np.random.default_rng(seed)
    g = np.unique(rng.integers(0, 40, size=(n, 3)), axis=0).astype(np.int32)
    batch = torch.zeros(g.shape[0], dtype=torch.int64)
    code, order, inverse, depth = O.serialization(torch.from_numpy(g), batch, ORDERS)
    plan = O.pooling_plan(code, depth, 2)
    cluster = plan["cluster"]
    for r in range(4):
        seq = cluster[order[r]]
        keep = torch.ones_like(seq, dtype=torch.bool)
        keep[1:] = seq[1:] != seq[:-1]
        assert torch.equal(seq[keep], plan["order"][r])


@settings(max_examples=20, deadline=None)
@given(st.integers(0, 2 ** 31 - 1), st.sampled_from([3, 5]))
def test_kernel_map_is_symmetric(seed, k):
    rng = np.random.default_rng(seed)
    g = np.unique(rng.integers(0, 12, size=(150, 3)), axis=0)
    ind = torch.from_numpy(np.concatenate([np.zeros((g.shape[0], 1), np.int64), g], 1)).int()
    nbr = O.kernel_map(ind, k)
    kv = k ** 3
    ar = torch.arange(ind.shape[0])
    for o in range(kv):
        j = nbr[:, o]
        m = j >= 0
        assert torch.equal(nbr[j[m], kv - 1 - o], ar[m])
