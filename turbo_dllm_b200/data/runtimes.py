"""Data runtimes: where token batches come from.

`DataRuntime` is the contract (next batch, resumable state). `RandomTokenDataRuntime` draws
uniform token ids on the device while avoiding the mask id; `HostStagedRandomRuntime` draws them
on the host into pinned memory and copies them over a transfer stream one step ahead (the
end-to-end path of benchmarks and of any real-data runtime). Packed / indexed / blended artifact
runtimes live in `data.artifact_runtimes`.

Counterparts: DataBatch / DataRuntime ABC / RandomTokenDataRuntime
(dllm_parallel/core/data.py:38-81, :155-245) and the pinned double-buffered prefetch of
PackedTokenDataRuntime (:248-607).
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any

import torch


@dataclass
class DataBatch:
    input_ids: torch.Tensor                      # [B, L] int64 on the training device
    supervision_mask: torch.Tensor | None = None
    supervision_count: int | None = None
    sample_ids: torch.Tensor | None = None
    h2d_bytes: int = 0
    # trajectory step units: weight of this turn inside its trajectory and its supervised-token counts
    # (plain, and without position 0 for objectives with shifted labels)
    turn_weight: float | None = None
    supervision_count_shifted: int | None = None
    # padding: True on the real tokens (one contiguous prefix per example); None = no padding
    valid_mask: torch.Tensor | None = None


class DataRuntime(ABC):
    @abstractmethod
    def next_batch(self) -> DataBatch: ...

    def next_optimizer_step_batches(self, micro_batches: int) -> list[DataBatch]:
        return [self.next_batch() for _ in range(micro_batches)]

    @abstractmethod
    def state_dict(self) -> dict[str, Any]: ...

    @abstractmethod
    def load_state_dict(self, state: dict[str, Any]) -> None: ...

    def close(self) -> None:
        pass


class RandomTokenDataRuntime(DataRuntime):
    """Uniform random ids in [0, vocab) \\ {mask_token_id}, generated on the training device."""

    def __init__(self, *, batch_size: int, seq_len: int, vocab_size: int, mask_token_id: int | None,
                 seed: int, device="cpu", vocab_sample_size: int | None = None):
        self.batch_size, self.seq_len = batch_size, seq_len
        self.vocab = min(vocab_size, vocab_sample_size) if vocab_sample_size else vocab_size
        self.mask_token_id = mask_token_id
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device)
        self.gen.manual_seed(int(seed))
        self.batches = 0

    def _draw(self, gen, device):
        hi = self.vocab - 1 if (self.mask_token_id is not None and self.mask_token_id < self.vocab) else self.vocab
        ids = torch.randint(0, hi, (self.batch_size, self.seq_len), generator=gen, device=device)
        if hi != self.vocab:
            ids = ids + (ids >= self.mask_token_id).long()  # skip the mask id
        return ids

    def next_batch(self) -> DataBatch:
        self.batches += 1
        return DataBatch(self._draw(self.gen, self.device))

    def state_dict(self):
        return {"kind": "random", "batches": self.batches, "generator_state": self.gen.get_state().cpu()}

    def load_state_dict(self, state):
        self.batches = int(state["batches"])
        self.gen.set_state(state["generator_state"].cpu())


class HostStagedRandomRuntime(RandomTokenDataRuntime):
    """Same distribution, produced on the host: every batch is written into pinned memory and
    copied host→device on a transfer stream while the previous step computes."""

    def __init__(self, *, device, **kw):
        super().__init__(device="cpu", **kw)
        self.target = torch.device(device)
        self.use_cuda = self.target.type == "cuda"
        shape = (self.batch_size, self.seq_len)
        self.pinned = [torch.empty(shape, dtype=torch.int64, pin_memory=self.use_cuda) for _ in range(2)]
        self.dev = [torch.empty(shape, dtype=torch.int64, device=self.target) for _ in range(2)]
        self.stream = torch.cuda.Stream(device=self.target) if self.use_cuda else None
        self.events = [None, None]
        self.slot = 0
        self._stage(0)

    def _stage(self, slot: int) -> None:
        self.pinned[slot].copy_(self._draw(self.gen, "cpu"))
        if self.use_cuda:
            self.stream.wait_stream(torch.cuda.current_stream(self.target))  # consumer of this slot is done
            with torch.cuda.stream(self.stream):
                self.dev[slot].copy_(self.pinned[slot], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.stream)
            self.events[slot] = ev
        else:
            self.dev[slot].copy_(self.pinned[slot])

    def next_batch(self) -> DataBatch:
        slot = self.slot
        if self.use_cuda:
            torch.cuda.current_stream(self.target).wait_event(self.events[slot])
        batch = DataBatch(self.dev[slot], h2d_bytes=self.pinned[slot].numel() * 8)
        self.slot ^= 1
        self._stage(self.slot)  # prefetch the next one
        self.batches += 1
        return batch
