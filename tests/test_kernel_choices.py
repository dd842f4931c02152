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


def test_which_tiles_the_tcgen05_product_takes() -> None:
    """Pairs of CTAs (256-row tiles) where those fill at least 85 % of the rounds they take on 74 pairs,
    single CTAs (128-row tiles) where only those do on 148 SMs, else the vendor library."""
    # 2,048 rows: qkv of the 0.6B sizes (8 x 16 pair tiles: two rounds, 86 %) and of the 8B sizes
    assert ops.tcgen05_tiles(2048, 4096, 256) == "pairs"
    assert ops.tcgen05_tiles(2048, 6144, 256) == "pairs"
    # gate/up with the activation in the epilogue: tiles of 128 output columns
    assert ops.tcgen05_tiles(2048, 3072, 128) == "pairs"
    # narrow outputs (o and down of the 0.6B sizes: 32 pair tiles) and 320 tiles of 2.2 rounds: the library
    assert ops.tcgen05_tiles(2048, 1024, 256) == ""
    assert ops.tcgen05_tiles(2048, 5120, 256) == ""
    # nine 128-row tiles x sixteen fill 148 SMs (97 %), five 256-row tiles x sixteen do not fill 74 pairs twice
    assert ops.tcgen05_tiles(1152, 2048, 128) == "single"
    assert ops.tcgen05_tiles(2304, 2048, 128) == "pairs"
    for m in (128, 512, 2048, 8192):
        for n in (1024, 4096, 24576, 151936):
            kind = ops.tcgen05_tiles(m, n, 256)
            if kind == "pairs":
                assert ops.tcgen05_pairs_fill_the_machine(m, n, 256)
            elif kind == "single":
                assert ops.tcgen05_fills_the_machine(m, n, 256) and not ops.tcgen05_pairs_fill_the_machine(m, n, 256)
            else:
                assert not ops.tcgen05_fills_the_machine(m, n, 256)


def test_pairs_can_be_switched_off(monkeypatch) -> None:
    monkeypatch.setattr(ops, "TCGEN05_PAIR", False)
    assert ops.tcgen05_tiles(2048, 4096, 256) == "single"


def test_parts_of_the_sums_of_squares_that_the_stream_product_leaves() -> None:
    """``ts_gemm_skinny_to_stream`` cuts narrow outputs into tiles of 8 columns (N / 8 parts of the rows'
    sums of squares) where that spreads the weights better over the SMs and all of K fits a CTA's loads in
    flight, else into tiles of 16; the rule is a host function of the library, so it runs without a GPU.
    The product that folds the norm in adds up at most 128 parts a row."""
    from tinyserve_b200.kernels.build import KernelBuildError, library

    try:
        parts = library().ts_gemm_skinny_to_stream_parts
    except (KernelBuildError, OSError) as e:      # no nvcc or no CUDA runtime on this host
        pytest.skip(f"the kernel library cannot be built or loaded here: {e}")
    assert parts(1, 1024, 2048) == parts(8, 1024, 3072) == parts(16, 1024, 2048) == 128      # o and down of the 0.6B sizes
    assert parts(8, 1024, 4096) == 64                  # K too long for one CTA's loads in flight
    assert parts(8, 2048, 1024) == 128                 # 128 tiles of 16 columns: halves spread no better
    assert parts(8, 4096, 4096) == 256
    for n in range(16, 2049, 16):
        for m in (1, 8, 9, 16):
            p = parts(m, n, 1024)
            assert p in (n // 16, n // 8)
            assert p == n // 16 or p <= 128
