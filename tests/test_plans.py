"""The launch plans of the device operations are plain arithmetic on the host: which
arrangement and split a product takes, how many CTAs share a decode step's pages and whether
clusters serve the pairs.  Checked here without a GPU; what the device would answer (how many
clusters run at once) is given by the test."""
import pytest

from wpc_engine_b200 import ops

# what one B200 answered: clusters of 2..16 CTAs of the cluster decode kernel that run at once
CAPACITY = {(128, False): [148, 93, 71, 56, 45, 37, 33, 30, 26, 21, 21, 17, 14, 14, 14],
            (128, True): [74, 45, 33, 26, 22, 15, 15, 15, 11, 7, 7, 7, 7, 7, 7],
            (64, False): [222, 142, 104, 82, 71, 56, 48, 45, 41, 31, 31, 28, 24, 24, 21],
            (64, True): [74, 45, 33, 26, 22, 15, 15, 15, 11, 7, 7, 7, 7, 7, 7]}


@pytest.fixture
def capacity(monkeypatch):
    monkeypatch.setattr(ops, "decode_cluster_capacity", lambda hd, c, alone: CAPACITY[(hd, bool(alone))][c - 2])


def test_decode_ctas_fit_the_device():
    for seqs, heads, ctx in [(1, 4, 4096), (8, 4, 4096), (64, 4, 4096), (3, 2, 70), (200, 1, 33000), (1, 1, 1)]:
        n = ops.plan_decode_ctas(seqs, heads, ctx, None)
        assert 1 <= n <= 1024
        blocks = (ctx + 63) // 64
        assert n <= max(seqs * heads * blocks, 1) or n <= 2 * 148
    # a window bounds the pages that a query sees
    assert ops.plan_decode_ctas(8, 4, 100000, 128) == ops.plan_decode_ctas(8, 4, 192, 128)
    # about two pairs to an SM: a CTA to a pair, no combining
    assert ops.plan_decode_ctas(64, 4, 4096, None) == 256


def test_decode_clusters_only_where_all_run_at_once(capacity):
    # 32 pairs of 64 pages: clusters of 8 would need 32 of the 33 that fit; 7 leave room
    assert ops.plan_decode_cluster(8, 4, 28, 128, 4096, None) == (7, 1)
    # one sequence: 4 pairs, as many ranks as a cluster can have
    assert ops.plan_decode_cluster(1, 4, 28, 128, 4096, None) == (16, 1)
    # one long sequence: several clusters to a pair, on all SMs
    c, g = ops.plan_decode_cluster(1, 4, 28, 128, 32768, None)
    assert g > 1 and 148 < 4 * c * g <= 296
    # too many pairs, too wide a group, or switched off: the fixed grid
    assert ops.plan_decode_cluster(64, 4, 28, 128, 4096, None) == (0, 1)
    assert ops.plan_decode_cluster(8, 1, 16, 128, 4096, None) == (0, 1)
    for seqs in range(1, 40):
        for ctx in (1, 64, 65, 1000, 4096, 20000, 100000):
            c, g = ops.plan_decode_cluster(seqs, 4, 28, 128, ctx, None)
            if c:
                pairs, alone = seqs * 4, seqs * 4 * c * g <= 148
                assert 2 <= c <= 16 and 1 <= g and c * g <= (ctx + 63) // 64 and pairs * c * g <= 296
                assert pairs * g * 1.1 <= CAPACITY[(128, alone)][c - 2]


def test_decode_clusters_can_be_switched_off(capacity, monkeypatch):
    monkeypatch.setattr(ops, "CLUSTER_DECODE", False)
    assert ops.plan_decode_cluster(8, 4, 28, 128, 4096, None) == (0, 1)
