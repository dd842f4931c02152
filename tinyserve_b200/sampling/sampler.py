"""Batched next-token selection for one step: one kernel launch for the whole batch, one
device-to-host copy of the chosen tokens (the step's only synchronisation).

Every request draws from its own noise stream: a Philox key made of its seed (its own, or one
derived from the engine's seed and the request's id) and a counter made of how many tokens it
has drawn so far. So the noise a request draws does not depend on its batch-mates, on how its
prompt was cut into portions, or on being recomputed after a preemption (upstream keeps a
``torch.Generator`` per seeded request for the same end, src/tinyserve/engine.py:126-147). The
logits it is applied to are the model's: in float32 they do not depend on the batch either; in
bfloat16 they do within rounding (decode steps of up to 16 rows fold the RMSNorm into the products
around it, with other rounding points than the norm kernel that larger steps run), so a bfloat16
request may draw another token at a near-tie when it runs in a batch of another size.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from ..kernels import ops
from .params import SamplingParams

_MASK = (1 << 64) - 1


def derive_seed(engine_seed: int, request_id: int) -> int:
    """A well-mixed 63-bit seed for a request that brought none (splitmix64 finaliser)."""
    z = (engine_seed * 0x9E3779B97F4A7C15 + (request_id + 1) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return (z ^ (z >> 31)) & 0x7FFF_FFFF_FFFF_FFFF


@dataclass(frozen=True)
class TokenLogprobs:
    logprob: float
    top: list[tuple[int, float]]


class SampleTicket:
    """Tokens on their way to the host: ``device_tokens`` (int32, on the device, valid until the
    sampler's next launch has run) can feed the next step at once; ``wait()`` returns the host
    list once the copy has arrived."""

    __slots__ = ("device_tokens", "_host", "_event", "_rows", "_tokens")

    def __init__(self, device_tokens: torch.Tensor, host: torch.Tensor, event: "torch.cuda.Event | None", rows: int) -> None:
        self.device_tokens, self._host, self._event, self._rows = device_tokens, host, event, rows
        self._tokens: list[int] | None = None

    def wait(self) -> list[int]:
        """The tokens; raises ``KernelError`` if a kernel of the step gave up on a bounded wait (the
        device's error word arrives in the same copy, in front of the tokens)."""
        if self._tokens is None:
            if self._event is not None:
                self._event.synchronize()
            got = self._host[: self._rows + 1].tolist()
            self._tokens = got[1:]
            if got[0] != 0:
                ops.raise_for_status(got[0], self.device_tokens.device)
        return self._tokens


class _Staging:
    """Pinned host buffers of one launch (parameters out, tokens back) and the event that says
    the tokens have arrived."""

    def __init__(self, max_rows: int, pin: bool) -> None:
        self.f_host = torch.empty(2 * max_rows, dtype=torch.float32, pin_memory=pin)
        self.i_host = torch.empty(2 * max_rows, dtype=torch.int64, pin_memory=pin)
        self.out_host = torch.zeros(max_rows + 1, dtype=torch.int32, pin_memory=pin)    # status, then the tokens
        self.event = torch.cuda.Event() if pin else None
        self.ticket: SampleTicket | None = None


class Sampler:
    def __init__(self, device: torch.device | str, max_rows: int = 1024) -> None:
        self.device = torch.device(device)
        pin = self.device.type == "cuda"
        self._cap = max_rows
        # two launches may be under way at a time (the engine runs one step ahead): their host
        # buffers alternate
        self._staging = [_Staging(max_rows, pin), _Staging(max_rows, pin)]
        self._turn = 0
        self._f_dev = torch.empty(2 * max_rows, dtype=torch.float32, device=self.device)
        self._i_dev = torch.empty(2 * max_rows, dtype=torch.int64, device=self.device)
        self._out = torch.zeros(max_rows + 1, dtype=torch.int32, device=self.device)    # status, then the tokens

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draws: Sequence[int]) -> SampleTicket:
        """``logits`` ``[R, V]`` float32 on the device; row r belongs to a request with
        ``params[r]``, noise seed ``seeds[r]`` that has drawn ``draws[r]`` tokens so far. Launches
        the kernel and the copy of the tokens to the host and returns without waiting."""
        r = logits.shape[0]
        if not (len(params) == len(seeds) == len(draws) == r):
            raise ValueError(f"{r} rows, {len(params)} params, {len(seeds)} seeds, {len(draws)} draws")
        if r > self._cap:
            raise ValueError(f"{r} rows exceed the sampler's capacity {self._cap}")
        st = self._staging[self._turn]
        self._turn ^= 1
        if st.ticket is not None:
            st.ticket.wait()               # the launch that used these buffers last has been read
        out, status = self._out[1: r + 1], self._out[:1]
        if all(p.greedy for p in params):
            ops.sample(logits, out, status_out=status)
        else:
            f, i = st.f_host, st.i_host
            f[:r] = torch.tensor([p.temperature for p in params], dtype=torch.float32)
            f[r: 2 * r] = torch.tensor([p.top_p for p in params], dtype=torch.float32)
            i[:r] = torch.tensor(list(seeds), dtype=torch.int64)
            i[r: 2 * r] = torch.tensor(list(draws), dtype=torch.int64)
            self._f_dev[: 2 * r].copy_(f[: 2 * r], non_blocking=True)
            self._i_dev[: 2 * r].copy_(i[: 2 * r], non_blocking=True)
            top_p = self._f_dev[r: 2 * r] if any(p.top_p < 1 for p in params) else None
            ops.sample(logits, out, self._f_dev[:r], top_p, self._i_dev[:r], self._i_dev[r: 2 * r], status_out=status)
        st.out_host[: r + 1].copy_(self._out[: r + 1], non_blocking=True)
        if st.event is not None:
            st.event.record()
        st.ticket = SampleTicket(out, st.out_host, st.event, r)
        return st.ticket

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               draws: Sequence[int]) -> list[int]:
        """:meth:`launch` and wait: the chosen tokens as a host list."""
        return self.launch(logits, params, seeds, draws).wait()


def token_logprobs(logits: torch.Tensor, tokens: Sequence[int], ks: Sequence[int]) -> list[TokenLogprobs]:
    """log_softmax of the raw logits at each drawn token, and the ``ks[r]`` most likely tokens
    (upstream src/tinyserve/sampling.py:113-128). A reporting aid, off the hot path."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    idx = torch.tensor(list(tokens), device=logits.device, dtype=torch.long)
    chosen = lp.gather(-1, idx[:, None])[:, 0].tolist()
    top_v, top_i = lp.topk(max(ks, default=0), dim=-1)
    vals, ids = top_v.tolist(), top_i.tolist()
    return [TokenLogprobs(chosen[b], list(zip(ids[b][:k], vals[b][:k]))) for b, k in enumerate(ks)]
