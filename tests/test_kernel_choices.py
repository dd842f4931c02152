"""Host-side choices of the kernel wrappers that need no GPU: into how many key ranges decode
attention cuts a request."""

from __future__ import annotations

import pytest

from tinyserve_b200.kernels import ops


@pytest.mark.parametrize("slots", [148, 444, 592])
def test_key_ranges_fit_the_machine_and_leave_room_for_clusters(slots) -> None:
    for ctas in range(1, slots + 50):
        for most in (1, 2, 5, 16, 64):
            plain = ops.choose_splits(ctas, slots, most)
            inside = ops.choose_splits(ctas, slots, most, cluster=True)
            for s in (plain, inside):
                assert 1 <= s <= max(1, most)
                assert s == 1 or s * ctas <= slots
            assert plain <= 12
            assert inside <= ops.CLUSTER_MAX
            if inside > 1:
                assert inside * ctas <= slots - ops.CLUSTER_ROOM * inside
            if inside > 2:
                assert inside * ctas <= ops.CLUSTER_FILL * slots
            if 2 * ctas > slots:
                assert plain == inside == 1


def test_key_ranges_at_the_measured_batches() -> None:
    # 8 kv heads, three CTAs of the TMA kernel per SM: batch -> ranges that measured best
    for batch, want in [(1, 8), (4, 8), (7, 6), (8, 5), (9, 4), (11, 4), (12, 3), (15, 3), (16, 2), (24, 2), (32, 1), (64, 1)]:
        assert ops.choose_splits(batch * 8, 444, 64, cluster=True) == want
    assert ops.choose_splits(8, 444, 3, cluster=True) == 3          # a short context is cut less


def test_without_cluster_merge_the_old_rule_holds(monkeypatch) -> None:
    monkeypatch.setattr(ops, "CLUSTER_MERGE", False)
    assert ops.choose_splits(64, 444, 64, cluster=True) == ops.choose_splits(64, 444, 64) == 6
