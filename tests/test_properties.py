"""Property tests (hypothesis) of the host-side logic that decides where sequences go: the batch cuts, the
token-balanced partition the library and the one-process-per-GPU driver share, packing, and pair truncation.
No GPU: the partitioner and the cost model are host functions of the C ABI."""
import numpy as np
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from infinity_b200 import batching as bt
from infinity_b200 import configs as cf
from infinity_b200 import packing as pk
from infinity_b200 import sharding as sh
from infinity_b200.engine import partition
from oracle import batching as ob

lengths_st = st.lists(st.integers(min_value=1, max_value=600), min_size=0, max_size=200)
SETTINGS = dict(max_examples=150, deadline=None)


@settings(**SETTINGS)
@given(lengths_st, st.integers(min_value=1, max_value=5000), st.one_of(st.none(), st.integers(min_value=1, max_value=64)),
       st.sampled_from([0.0, 0.001, 0.01]))
def test_token_budget_batches_cut_the_sorted_list_once(lengths, budget, max_seqs, qw):
    batches = bt.token_budget_batches(lengths, budget, max_seqs, qw)
    flat = [i for b in batches for i in b]
    assert sorted(flat) == list(range(len(lengths)))                      # every item exactly once
    assert flat == sorted(range(len(lengths)), key=lambda i: lengths[i])   # in stable length order
    assert all(b for b in batches)
    cost = lambda i: lengths[i] + qw * lengths[i] * lengths[i]
    for b in batches:
        assert max_seqs is None or len(b) <= max_seqs
        # over budget only when a single item is
        assert sum(cost(i) for i in b) <= budget + 1e-9 or len(b) == 1
    # greedy: a batch could not have taken the first item of the next one
    for b, nxt in zip(batches, batches[1:]):
        full_by_count = max_seqs is not None and len(b) >= max_seqs
        assert full_by_count or sum(cost(i) for i in b) + cost(nxt[0]) > budget


@settings(**SETTINGS)
@given(lengths_st, st.integers(min_value=1, max_value=64))
def test_count_batches_is_the_reference_cut(lengths, size):
    """Same cut as the restated reference queue (oracle/batching.py, pinned to the reference's own orders)."""
    got = bt.count_batches(lengths, size)
    flat = [i for b in got for i in b]
    assert sorted(flat) == list(range(len(lengths)))
    assert all(len(b) == size for b in got[:-1]) and (not got or 1 <= len(got[-1]) <= size)
    if len(lengths) > size:
        assert flat == sorted(range(len(lengths)), key=lambda i: lengths[i])
    else:
        assert flat == list(range(len(lengths)))
    # one pop that takes everything = the restated reference queue with a large max_n_batches
    assert got == ob.pop_all_batches(list(lengths), size, max_n_batches=len(lengths) + 1)


@settings(**SETTINGS)
@given(st.lists(st.integers(min_value=1, max_value=2048), min_size=0, max_size=300), st.integers(min_value=1, max_value=8),
       st.sampled_from([(1.0, 0.0), (1.0, 0.01), (24000.0, 64.0)]))
def test_partition_is_a_balanced_assignment(lengths, n_shards, coef):
    a, b = coef
    owner = partition(lengths, n_shards, a, b)
    assert owner.shape == (len(lengths),) and ((owner >= 0) & (owner < n_shards)).all()
    assert np.array_equal(owner, partition(lengths, n_shards, a, b))       # deterministic
    cost = np.array([a * L + b * L * L for L in lengths], dtype=np.float64)
    loads = np.array([cost[owner == s].sum() for s in range(n_shards)])
    if len(lengths):
        # longest-processing-time bound: no shard exceeds the mean by more than one item
        assert loads.max() <= cost.sum() / n_shards + cost.max() + 1e-6
        # nobody idles while another shard holds two or more items it could have given away
        if len(lengths) >= n_shards:
            assert (np.bincount(owner, minlength=n_shards) > 0).all()


@settings(max_examples=40, deadline=None)
@given(st.lists(st.integers(min_value=1, max_value=512), min_size=1, max_size=120), st.integers(min_value=1, max_value=8),
       st.sampled_from(["bert", "moe", "decoder"]))
def test_shards_keep_batch_order_and_scatter_restores_it(lengths, n_shards, arch):
    spec = cf.tiny_spec(arch)
    shards = sh.shard_indices(lengths, n_shards, spec)
    assert len(shards) == n_shards
    allidx = np.concatenate(shards) if shards else np.zeros(0, int)
    assert sorted(allidx.tolist()) == list(range(len(lengths)))
    out = np.full((len(lengths), 3), -1.0)
    for idx in shards:
        assert (np.diff(idx) > 0).all()                                    # ascending inside a shard
        sh.scatter_rows(out, np.stack([idx, idx * 2, idx * 3], axis=1).astype(float), idx)
    assert np.array_equal(out[:, 0], np.arange(len(lengths)))


@settings(**SETTINGS)
@given(st.lists(st.lists(st.integers(min_value=0, max_value=30000), min_size=1, max_size=40), min_size=0, max_size=30))
def test_packing_round_trip(seqs):
    f = pk.pack_sequences(seqs)
    assert f.cu_seqlens[0] == 0 and (np.diff(f.cu_seqlens) == [len(s) for s in seqs]).all()
    assert f.input_ids.dtype == np.int32 and f.cu_seqlens.dtype == np.int32
    for i, s in enumerate(seqs):
        assert f.input_ids[f.cu_seqlens[i]:f.cu_seqlens[i + 1]].tolist() == s


def test_packing_rejects_empty_sequences():
    with pytest.raises(ValueError):
        pk.pack_sequences([[1, 2], []])


@settings(**SETTINGS)
@given(st.lists(st.integers(0, 9), max_size=60), st.lists(st.integers(0, 9), max_size=60), st.integers(min_value=0, max_value=100))
def test_pair_truncation_longest_first(q, d, budget):
    q2, d2 = pk.truncate_pair_longest_first(q, d, budget)
    assert q2 == q[:len(q2)] and d2 == d[:len(d2)]                         # only tails are removed
    assert len(q2) + len(d2) == min(budget, len(q) + len(d))
    if len(q) + len(d) > budget and q2 and d2:
        assert abs(len(q2) - len(d2)) <= max(1, abs(len(q) - len(d)))      # the longer side gave first
