"""Host-side choices of launch shapes: pure functions of the step's sizes, checked without a GPU."""

from gtar_kimik3_public_b200.ops.functional import SCRATCH_SPLITS_FROM, decode_splits, split_k_for


def test_decode_splits_stay_within_what_the_kernels_take():
    for n_seqs in (1, 2, 3, 4, 8, 12, 16, 20, 24, 32, 40, 48, 64, 200):
        for n_kv in (1, 2, 8):
            for length in (1, 63, 64, 65, 600, 2304, 8192, 40000):
                pages = -(-length // 64)
                s = decode_splits(n_seqs, n_kv, length, 64, 148)
                assert 1 <= s <= max(1, min(pages, 64)), (n_seqs, n_kv, length, s)
                # more than eight splits (scratch and a second kernel) only for long contexts and few sequences
                assert s in (1, 2, 4, 8) or (s >= SCRATCH_SPLITS_FROM and length >= 8192), (n_seqs, n_kv, length, s)


def test_decode_splits_at_measured_points():
    """The choices that measured step times (batch 1 to 64, 2,048-token contexts, 8 kv heads, 148 SMs) favour."""
    want = {1: 8, 2: 8, 8: 4, 12: 2, 16: 2, 24: 1, 32: 1, 40: 2, 48: 2, 64: 1}
    assert {b: decode_splits(b, 8, 2304, 64, 148) for b in want} == want


def test_decode_splits_count_waves_with_the_clusters_that_fit():
    """Clusters are placed inside a GPC: a B200 holds 296 single blocks of the decode attention kernel at once but only
    71 clusters of four and 33 of eight.  Nine sequences of eight kv heads are 72 clusters of four (a second wave for
    one cluster) and are cut in two instead; four sequences take four splits, not eight (measured: 0.82 against 0.89 ms
    a step)."""
    places = (296, 148, 71, 33)
    got = {b: decode_splits(b, 8, 2304, 64, 148, places) for b in (1, 2, 4, 8, 9, 11, 12)}
    assert got == {1: 8, 2: 8, 4: 4, 8: 4, 9: 2, 11: 2, 12: 2}
    assert decode_splits(9, 8, 2304, 64, 148) == 4  # what two blocks an SM, whatever the cluster, would suggest


def test_split_k_for_seventeen_to_twenty_row_tiles():
    assert split_k_for(8, 2560, 9728) == 8 and split_k_for(64, 4096, 12288) == 4 and split_k_for(8, 19456, 2560) == 1


def test_decode_splits_one_page_one_block():
    assert decode_splits(1, 8, 40, 64, 148) == 1
    assert decode_splits(64, 8, 64, 64, 148) == 1


def test_split_k_is_a_cluster_size():
    for m in (1, 8, 17, 64):
        for n, k in ((4096, 1024), (6144, 1024), (1024, 2048), (1024, 3072), (151936, 1024), (128, 64)):
            assert split_k_for(m, n, k) in (1, 2, 4, 8)


def test_length_bounds_of_captured_decode_steps():
    """1, 1.5, 2, 3, 4, ... times the least bound, never beyond the cache; launch shapes are chosen for the middle of
    the lengths a bound covers."""
    from types import SimpleNamespace

    from gtar_kimik3_public_b200.engine.graphs import StepGraphs

    graphs = SimpleNamespace(cache=SimpleNamespace(max_seq_len=40960), MIN_LENGTH_BOUND=StepGraphs.MIN_LENGTH_BOUND)
    got = {}
    for length in (1, 1024, 1025, 1536, 1537, 2049, 3072, 3073, 4097, 40000):
        step = SimpleNamespace(all_single=True, max_kv_len=length)
        got[length] = StepGraphs.length_bounds(graphs, step)
        bound, typical = got[length]
        assert length <= bound <= 40960 and typical <= bound
    assert got[1] == got[1024] == (1024, 512)
    assert got[1025] == got[1536] == (1536, 1280)
    assert got[1537] == (2048, 1792) and got[2049] == got[3072] == (3072, 2560) and got[3073] == (4096, 3584)
    assert got[4097] == (6144, 5120) and got[40000] == (40960, 36864)
    assert StepGraphs.length_bounds(graphs, SimpleNamespace(all_single=False, max_kv_len=77)) == (40960, 0)


def test_twenty_four_sequences_are_not_cut():
    """192 (sequence, kv head) pairs of some 2,500 tokens each fit the device at once uncut; cut in four they are 192
    clusters where 71 run at once (measured: 48 us an attention kernel cut in four, which a bound of 4,096 tokens
    taken for the length had chosen; 31 us is what its pages take)."""
    places = (296, 148, 71, 33)
    assert decode_splits(24, 8, 2560, 64, 148, places) == 1
    assert decode_splits(24, 8, 3584, 64, 148, places) == 1


def test_three_sequences_take_eight_splits_and_short_contexts_no_scratch():
    """Measured, ms a step: three sequences of 2,048 tokens 0.70 cut in four and 0.65 in eight (of 1,024: 0.62 / 0.60), four
    sequences 0.73 / 0.76; one and two sequences of 8,192 tokens 0.83 and 0.91 as clusters of eight against 0.85 and 0.98
    with 37 and 18 splits through scratch, but of 16,384 tokens 1.18 and 1.45 against 1.03 and 1.32."""
    places = (296, 148, 71, 33)
    assert decode_splits(3, 8, 2560, 64, 148, places) == 8 and decode_splits(3, 8, 1280, 64, 148, places) == 8
    assert decode_splits(4, 8, 2560, 64, 148, places) == 4 and decode_splits(4, 8, 1280, 64, 148, places) == 4
    assert decode_splits(1, 8, 10240, 64, 148, places) == 8 and decode_splits(2, 8, 10240, 64, 148, places) == 8
    assert decode_splits(1, 8, 14336, 64, 148, places) == 37 and decode_splits(2, 8, 14336, 64, 148, places) == 18


def test_the_even_deal_where_the_equal_cut_fits_badly():
    """Measured (28 layers of the 0.6B sizes, ms a step, equal cut / dealt evenly): contexts of 2,048: 40 sequences 2.86 /
    2.57, 44: 2.88 / 2.78, 48: 2.89 / 2.91, but 8: 0.82 / 1.1, 16: 1.25 / 1.5, 20: 1.66 / 1.70, 24: 1.71 / 1.83, 32: 1.98 / 2.2,
    56: 3.13 / 3.21, 64: 3.26 / 3.5; contexts of 8,192: 20: 4.06 / 3.70, but 6: 1.50 / 1.74, 12: 2.33 / 2.48."""
    from gtar_kimik3_public_b200.ops.functional import decode_flat_wins

    places = (296, 148, 71, 33)
    evenly = {b: decode_flat_wins(b, 8, 2560, 64, 148, places, 296) for b in (1, 8, 16, 20, 24, 32, 40, 48, 56, 64)}
    assert evenly == {1: False, 8: False, 16: False, 20: False, 24: False, 32: False, 40: True, 48: True, 56: False, 64: False}
    assert decode_flat_wins(20, 8, 7168, 64, 148, places, 296) and decode_flat_wins(20, 8, 3584, 64, 148, places, 296)
    assert not decode_flat_wins(6, 8, 7168, 64, 148, places, 296) and not decode_flat_wins(12, 8, 7168, 64, 148, places, 296)
    # few pages a block: the parts, tickets and merges of the even deal cost more than it saves
    assert not decode_flat_wins(20, 8, 512, 64, 148, places, 296)
    # more than eight splits go through scratch and a second kernel: not this kernel's case
    assert not decode_flat_wins(1, 8, 40000, 64, 148, places, 296)


def test_the_even_deal_for_a_few_long_sequences():
    """Clusters of eight that share SMs stream long contexts badly (ms a step, equal cut / dealt evenly: 32,768 tokens,
    3 sequences 2.66 / 2.42, 4: 3.17 / 2.92; 16,384 tokens, 4: 2.09 / 2.05), but one and two sequences (all their blocks
    have an SM each), shorter contexts and sequences cut in four stay with the equal cut (8,192 tokens, 3: 0.96 / 1.24,
    4: 1.19 / 1.45; 16,384 tokens, 3: 1.34 / 1.64, 6: 2.37 / 2.63).  The lengths below are the middles of the bounds that
    captured steps of those contexts get."""
    from gtar_kimik3_public_b200.ops.functional import decode_flat_wins

    places = (296, 148, 71, 33)
    assert decode_flat_wins(4, 8, 14336, 64, 148, places, 296) and not decode_flat_wins(6, 8, 14336, 64, 148, places, 296)
    assert decode_flat_wins(3, 8, 28672, 64, 148, places, 296) and decode_flat_wins(4, 8, 28672, 64, 148, places, 296)
    assert not decode_flat_wins(3, 8, 7168, 64, 148, places, 296) and not decode_flat_wins(3, 8, 14336, 64, 148, places, 296)
    assert not decode_flat_wins(4, 8, 7168, 64, 148, places, 296) and not decode_flat_wins(4, 8, 5120, 64, 148, places, 296)
    for length in (10240, 20480, 36864):
        assert not decode_flat_wins(1, 8, length, 64, 148, places, 296) and not decode_flat_wins(2, 8, length, 64, 148, places, 296)
