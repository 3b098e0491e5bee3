"""Chooses next tokens from logits on the device with the sampling kernel.

Greedy where temperature is 0, else softmax(logits / temperature) restricted to the top-p set
(pico_vllm/sampler.py:3-37), one kernel launch for rows with different parameters (the
reference groups rows by equal parameters and runs torch ops per group, sampler.py:56-86).
Randomness is one uniform number per (seed, request, number of tokens generated so far) from a
counter-based hash, so a request's tokens do not depend on what else is in the batch.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    # splitmix64 finaliser
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform_for(seed: int, request_id: int, step: int) -> float:
    """A number in [0, 1) that depends only on (seed, request, step); 24 bits, exact in float32."""
    h = _mix(_mix(_mix(seed & _MASK) ^ (request_id & _MASK)) ^ (step & _MASK))
    return (h >> 40) / float(1 << 24)


class PendingTokens:
    """Tokens a sampling kernel is writing: ``result()`` waits for the copy to the host."""

    def __init__(self, host: torch.Tensor, event, n: int):
        self.host, self.event, self.n = host, event, n

    def result(self) -> List[int]:
        if self.event is not None:
            self.event.synchronize()
        return self.host[:self.n].tolist()


class Sampler:
    def __init__(self, device, seed: int = 0):
        self.device = torch.device(device)
        self.seed = seed
        self._host = [None, None]       # two pinned buffers, used in turn
        self._turn = 0

    def sample_async(self, logits: torch.Tensor, temperatures: Sequence[float], top_ps: Sequence[float],
                     uniforms: Optional[Sequence[float]], out: torch.Tensor) -> PendingTokens:
        """Like :meth:`sample`, but the tokens go to ``out`` (int32 on the device, at least R long)
        and to the host without waiting: the returned object's ``result()`` waits."""
        R = logits.shape[0]
        cuda = self.device.type == "cuda"
        if self._host[self._turn] is None or self._host[self._turn].numel() < max(R, 1):
            self._host[self._turn] = torch.empty(max(64, R), dtype=torch.int32, pin_memory=cuda)
        host = self._host[self._turn]
        self._turn ^= 1
        if R == 0:
            return PendingTokens(host, None, 0)
        dst = out[:R]
        if all(t <= 0 for t in temperatures):
            ops.sample(logits, None, None, None, dst)
        else:
            params = torch.tensor([list(temperatures), list(top_ps), list(uniforms)], dtype=torch.float32)
            dev = params.to(self.device, non_blocking=True)
            ops.sample(logits, dev[0], dev[1], dev[2], dst)
        host[:R].copy_(dst, non_blocking=True)
        event = None
        if cuda:
            event = torch.cuda.Event()
            event.record()
        return PendingTokens(host, event, R)

    def tokens_from(self, tokens: torch.Tensor, n: int) -> PendingTokens:
        """The first ``n`` tokens of an int32 device tensor that a kernel has been launched to fill, on their way
        to the host without waiting (``result()`` waits)."""
        cuda = self.device.type == "cuda"
        if self._host[self._turn] is None or self._host[self._turn].numel() < max(n, 1):
            self._host[self._turn] = torch.empty(max(64, n), dtype=torch.int32, pin_memory=cuda)
        host = self._host[self._turn]
        self._turn ^= 1
        if n == 0:
            return PendingTokens(host, None, 0)
        host[:n].copy_(tokens[:n], non_blocking=True)
        event = None
        if cuda:
            event = torch.cuda.Event()
            event.record()
        return PendingTokens(host, event, n)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], top_ps: Sequence[float],
               uniforms: Optional[Sequence[float]] = None) -> List[int]:
        """logits float32 [R, V] on the device -> R token ids (host ints; one device-to-host read)."""
        R = logits.shape[0]
        if R == 0:
            return []
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        if all(t <= 0 for t in temperatures):
            ops.sample(logits, None, None, None, out)
        else:
            if uniforms is None:
                raise ValueError("sampling with temperature > 0 needs uniform numbers")
            host = torch.tensor([list(temperatures), list(top_ps), list(uniforms)], dtype=torch.float32)
            dev = host.to(self.device, non_blocking=True)
            ops.sample(logits, dev[0], dev[1], dev[2], out)
        return out.cpu().tolist()
