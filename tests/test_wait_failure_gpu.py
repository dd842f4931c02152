"""A bounded wait that runs out ends as an error on the host, never as a hang or as wrong tokens.

Every kernel family that waits on mbarriers is launched once with its copies switched off (the test
switch of ``csrc/bounded_wait.cuh``: the copy-issuing thread skips its copies and the expect-tx that
arms the barrier, as if the copies had been lost) and with a wait bound of 20,000 cycles, so that the
wait runs out after some ten microseconds on a healthy GPU. The kernel must then leave its code in
the error word, free what it holds and return: the same launch, with the switch off again, gives the
right result on the same context straight afterwards. Nothing here waits long, traps or faults.
Upstream's analogue is a hard error on the host (src/tinyserve/engine.py:173-175)."""

from __future__ import annotations

import pytest
import torch

import kernel_refs as ref
from test_kernels_gpu import _attention_case, rnd, tol
from tiny_configs import TINIES, random_prompt, write_tiny
from tinyserve_b200.kernels import ops

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


class lost_copies:
    """While open: waits of 20,000 cycles and no copies. Closing restores the defaults and clears
    the error word."""

    def __enter__(self) -> "lost_copies":
        torch.cuda.synchronize()
        ops.set_wait_control(cycles=20_000, unarmed=True)
        return self

    def __exit__(self, *exc) -> None:
        torch.cuda.synchronize()
        ops.set_wait_control()
        for w in ops._error_words.values():
            w.zero_()


def error_code() -> int:
    torch.cuda.synchronize()
    return int(ops._error_word(torch.device("cuda", torch.cuda.current_device())).item())


def gemm_case(swiglu: bool, pairs: bool):
    # single CTAs: nine row tiles x sixteen column tiles fill the machine; pairs: nine 256-row tiles x sixteen
    rows = 2304 if pairs else 1152
    x, w = rnd(rows, 256, dtype=BF16, seed=1), rnd(4096, 256, dtype=BF16, seed=2, scale=0.05)
    if swiglu:
        assert ops.tcgen05_tiles(rows, 2048, 128) == ("pairs" if pairs else "single")
        out = torch.zeros(rows, 2048, device="cuda", dtype=BF16)
        run = lambda: ops.gemm_swiglu(x, w, out, None)
        want = torch.empty_like(out)
        ref.gemm_swiglu(x, w, want, None)
    else:
        out = torch.zeros(rows, 4096, device="cuda", dtype=BF16)
        run = lambda: ops.gemm_tcgen05(x, w, out, ops.TCGEN05_PAIR_TILE if pairs else 256)
        want = torch.empty_like(out)
        ref.gemm(x, w, want)
    return run, out, want


@pytest.mark.parametrize("pairs", [False, True])
@pytest.mark.parametrize("swiglu", [False, True])
def test_gemm_tcgen05_gives_up_and_recovers(swiglu, pairs) -> None:
    run, out, want = gemm_case(swiglu, pairs)
    with lost_copies():
        run()
        assert error_code() == 1
        with pytest.raises(ops.KernelError, match="gemm_tcgen05"):
            ops.check_device_errors()
        assert error_code() == 0           # raising clears the word
    run()                                  # tensor memory was freed and the context is usable
    ops.check_device_errors()
    torch.testing.assert_close(out.float(), want.float(), **tol(BF16))


@pytest.mark.parametrize("kernel,lens,d,page,code", [
    ("tcgen05", [(300, 300), (700, 130)], 128, 16, 2),        # tcgen05 prefill attention
    ("mma", [(300, 300), (700, 130)], 64, 8, 3),              # mma.sync prefill attention with TMA tiles
    ("tcgen05", [(300, 1), (40, 1)], 128, 16, 4),             # TMA decode attention, unsplit
    ("tcgen05", [(2048, 1), (777, 1)], 64, 16, 4),            # the same with key ranges merged in a cluster
    ("tcgen05", [(300, 1), (40, 1)], 32, 4, 5),               # bulk-copy decode attention (other head sizes)
])
def test_attention_gives_up_and_recovers(kernel, lens, d, page, code, monkeypatch) -> None:
    monkeypatch.setattr(ops, "PREFILL_ATTENTION", kernel)
    with lost_copies():
        _attention_case(BF16, 8, 2, d, page, lens, 0, seed=3)
        assert error_code() == code
        with pytest.raises(ops.KernelError, match=ops.WAIT_FAILURES[code]):
            ops.check_device_errors()
    out, want = _attention_case(BF16, 8, 2, d, page, lens, 0, seed=3)
    ops.check_device_errors()
    torch.testing.assert_close(out.float(), want.float(), **tol(BF16))


def test_engine_and_replay_raise_instead_of_returning_tokens(tmp_path) -> None:
    """Through the entry points: the status word comes back with the sampled tokens (one copy, no
    extra synchronisation) and ``Engine.step`` raises; trace replay raises too; and a fresh engine
    on the same context generates normally afterwards."""
    from tinyserve_b200 import LLM
    from tinyserve_b200.engine.replay import Replayer
    from tinyserve_b200.model import DecoderModel

    cfg, page, _ = TINIES["B"]
    folder = write_tiny(tmp_path, "B", BF16)
    prompts = [random_prompt(n, cfg["vocab_size"], 5 + n) for n in (9, 24)]

    def llm() -> "LLM":
        return LLM.from_folder(folder, dtype="bfloat16", page_size=page, num_pages=64, max_num_seqs=4,
                               max_batch_tokens=128, decode_graphs=True)

    good = llm().generate(prompts, 6)
    with lost_copies():
        with pytest.raises(ops.KernelError, match="gave up waiting"):
            llm().generate(prompts, 6)
        rep = Replayer(DecoderModel.from_folder(folder, BF16, "cuda"), 128, page)
        rep.run_step([("a", prompts[0], [0])])                   # a prompt portion: simt kernels, no waits
        with pytest.raises(ops.KernelError, match="decode_attention_mma"):
            rep.run_step([("a", [1], [0])])
    assert llm().generate(prompts, 6) == good
