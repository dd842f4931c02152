"""How close the engine's logits must be to the plain implementation's (shared by the GPU tests
and by the smoke test of ``__graft_entry__``)."""

from __future__ import annotations

import torch

FP32_TOL = {"atol": 3e-5, "rtol": 3e-5}    # sums in another order than the CPU's


def close_enough(rows: torch.Tensor, want32: torch.Tensor, want16: torch.Tensor | None, dtype: torch.dtype) -> None:
    """float32: equal to the plain implementation up to summation order. bfloat16: the error
    against the 32-bit oracle is measured against the error that the plain implementation
    itself makes when it runs in bfloat16 with upstream's rounding points; the engine may not
    be worse than that by more than a quarter in the root mean square, nor by more than twice
    at the worst logit."""
    if dtype == torch.float32:
        torch.testing.assert_close(rows, want32, **FP32_TOL)
        return
    err = (rows - want32).abs()
    ref = (want16 - want32).abs()
    rms, ref_rms = float(err.pow(2).mean().sqrt()), float(ref.pow(2).mean().sqrt())
    assert rms <= 1.25 * ref_rms + 1e-3, f"rms error {rms:.4f} against {ref_rms:.4f} of plain bfloat16"
    assert float(err.max()) <= 2.0 * float(ref.max()) + 1e-2, \
        f"worst error {float(err.max()):.4f} against {float(ref.max()):.4f} of plain bfloat16"


def engine_logits_close_to_plain(engine, ids, prompts, plain_forward32, plain_forward16, dtype: torch.dtype) -> int:
    """Every logits row that ``engine`` (made with ``record_logits=True``) sampled from, held
    against the plain implementation on the request's final token sequence. ``plain_forward*``
    map a token list to ``[T, vocab]`` logits. Returns how many rows were compared."""
    rows_of: dict[int, dict[int, torch.Tensor]] = {}
    for rid, pos, row in engine.logits_log:
        rows_of.setdefault(rid, {})[pos] = row
    compared = 0
    for rid, prompt in zip(ids, prompts):
        seq = list(prompt) + engine.requests[rid].output
        places = list(range(len(prompt) - 1, len(seq) - 1))
        assert set(places) <= set(rows_of[rid]), "a position the request sampled from was not recorded"
        got = torch.stack([rows_of[rid][p] for p in places]).float().cpu()
        assert not got.isnan().any()
        want32 = plain_forward32(seq)[places]
        want16 = plain_forward16(seq)[places] if dtype == torch.bfloat16 else None
        close_enough(got, want32, want16, dtype)
        compared += len(places)
    return compared
