"""Corruption runtimes of the block-diffusion objectives.

Randomness is counter-based (Philox, `objectives/philox.py` and `csrc/noising.cu`): batch k of a
runtime with seed s uses offsets 2k (block times) and 2k+1 (token uniforms), so CPU and GPU runs
corrupt identically and the resumable state is just the batch counter.

standard_block_diffusion: one diffusion time t per (sample, block), antithetic-stratified by
default (one uniform draw, strata rotated by it), scaled to [eps_min, eps_max]; a token is
masked iff rand <= t; labels are the clean token on masked positions and -100 elsewhere; the
per-block loss weight is 1/t (or 1).
diffusiongemma_native_sft: same block times, uniform random-token replacement, labels on every scored
position, unit weights, a per-sample self-conditioning draw (see DiffusionGemmaNativeRuntime).
fast_dllm_v2: t ~ U(0,1) per (sample, block), move chance (1-eps)·t + eps, two complementary
views (mask, ~mask) share the clean copy, labels are shifted left by one, weights are 1 and the
denominator is batch·(L-1).

Semantics follow dllm_parallel/core/objectives/runtime.py:112-212 and
dllm_parallel/core/objectives/fast_dllm_v2.py:66-179; generator state is part of the
checkpoint (`state_dict`, cf. runtime.py:214-282).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch

LABEL_IGNORE_INDEX = -100
STATE_VERSION = 3


@dataclass
class CorruptedBatch:
    clean_input_ids: torch.Tensor   # [B, L]
    noisy_input_ids: torch.Tensor   # [B, V, L]  (V noisy views per sample)
    labels: torch.Tensor            # [B, V, L]  clean token or -100
    diffusion_times: torch.Tensor   # [B, nblocks]
    noise_levels: torch.Tensor      # [B, nblocks]
    loss_weights: torch.Tensor      # [B, V, nblocks]
    active_tokens: torch.Tensor     # scalar int64 tensor: supervised positions
    valid_tokens: int
    loss_denominator: float

    @property
    def views(self) -> int:
        return int(self.noisy_input_ids.shape[1])

    # Response-suffix packing (diffusiongemma_native_sft): when set, the noisy / label / weight tensors cover only
    # the decoder rows, offset o standing for position response_start + o (clamped to the last valid position for
    # the padding rows that fill the last block), with blocks counted from the response start.
    response_start = None      # int: first scored position, shared by the batch
    valid_length = None        # int: tokens before the padding, shared by the batch


@dataclass(frozen=True)
class TokenAccountingPolicy:
    """Which token counts feed throughput numbers."""

    count_clean_copy: bool = False

    def input_tokens(self, batch: CorruptedBatch) -> int:
        b, l = batch.clean_input_ids.shape
        return b * l


class _ObjectiveRuntime:
    name = "base"
    views = 1
    exclude_mask_token = True

    def __init__(self, *, block_size: int, mask_token_id: int, max_seq_len: int, seed: int,
                 device="cpu"):
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.block_size = int(block_size)
        self.mask_token_id = int(mask_token_id)
        self.max_seq_len = int(max_seq_len)
        self.device = torch.device(device)
        self.generator = torch.Generator(device=self.device)
        self.generator.manual_seed(int(seed))
        self.seed = int(seed)
        self.batches_corrupted = 0
        self.loss_tokens_seen = 0
        self.valid_tokens_seen = 0

    # -- helpers
    def _check(self, x0: torch.Tensor, min_len: int = 1) -> tuple[int, int, int]:
        if x0.ndim != 2:
            raise ValueError(f"expected rank-2 input_ids, got {tuple(x0.shape)}")
        b, l = map(int, x0.shape)
        if not min_len <= l <= self.max_seq_len:
            raise ValueError(f"sequence length {l} outside [{min_len}, {self.max_seq_len}]")
        if l % self.block_size:
            raise ValueError("input sequence length must divide evenly by block_size")
        return b, l, l // self.block_size

    def _rand(self, shape) -> torch.Tensor:
        return torch.rand(shape, dtype=torch.float32, device=self.device, generator=self.generator)

    def _block_uniforms(self, n: int) -> torch.Tensor:
        """Counter-based uniforms for the per-block diffusion times of the current batch (identical on
        every device type; the token-level stream uses the next offset)."""
        from .philox import uniform01

        return torch.from_numpy(uniform01(self.seed, 2 * self.batches_corrupted, n)).to(self.device)

    def _tokens(self, x0, move_chance, eligible, shift: bool):
        return fused_corrupt(x0, move_chance, eligible, block_size=self.block_size, views=self.views, shift=shift,
                             mask_id=self.mask_token_id, seed=self.seed, offset=2 * self.batches_corrupted + 1)

    def skip(self, steps: int, batch_shape: tuple[int, int]) -> None:
        """Advances the generator as `steps` calls of corrupt() on this shape would."""
        x = torch.zeros(batch_shape, dtype=torch.long, device=self.device)
        for _ in range(int(steps)):
            self.corrupt(x)

    def state_dict(self) -> dict[str, Any]:
        return {"version": STATE_VERSION, "name": self.name, "seed": self.seed,
                "generator_state": self.generator.get_state().cpu(),
                "batches_corrupted": self.batches_corrupted,
                "loss_tokens_seen": int(self.loss_tokens_seen),
                "valid_tokens_seen": int(self.valid_tokens_seen)}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        if state.get("version") != STATE_VERSION or state.get("name") != self.name:
            raise ValueError(f"objective state mismatch: have {self.name} v{STATE_VERSION}, "
                             f"checkpoint has {state.get('name')} v{state.get('version')}")
        self.generator.set_state(state["generator_state"].to("cpu"))
        self.batches_corrupted = int(state["batches_corrupted"])
        self.loss_tokens_seen = int(state["loss_tokens_seen"])
        self.valid_tokens_seen = int(state["valid_tokens_seen"])


class StandardBlockDiffusionRuntime(_ObjectiveRuntime):
    name = "standard_block_diffusion"
    views = 1
    exclude_mask_token = True

    def __init__(self, *, loss_weighting="inverse_move_chance", noise_schedule_epsilon=1e-3,
                 sampling_epsilon_min=1e-3, sampling_epsilon_max=1.0, antithetic_sampling=True, **kw):
        super().__init__(**kw)
        if loss_weighting not in ("inverse_move_chance", "unit"):
            raise ValueError(f"unknown loss_weighting {loss_weighting!r}")
        self.loss_weighting = loss_weighting
        self.noise_schedule_epsilon = float(noise_schedule_epsilon)
        self.eps_min, self.eps_max = float(sampling_epsilon_min), float(sampling_epsilon_max)
        self.antithetic = bool(antithetic_sampling)

    def sample_times(self, b: int, nblk: int) -> torch.Tensor:
        if self.antithetic:
            n = b * nblk
            u = self._block_uniforms(1)
            strata = torch.arange(n, dtype=torch.float32, device=self.device).view(b, nblk) / float(n)
            t = (u + strata).remainder(1.0)
        else:
            t = self._block_uniforms(b * nblk).view(b, nblk)
        return t * (self.eps_max - self.eps_min) + self.eps_min

    def corrupt(self, x0, *, supervision_mask=None, supervision_count=None) -> CorruptedBatch:
        b, l, nblk = self._check(x0)
        x0 = x0.to(self.device)
        if supervision_mask is None:
            if supervision_count is not None:
                raise ValueError("supervision_count requires an explicit supervision_mask")
            eligible, valid = None, b * l
        else:
            if supervision_mask.shape != x0.shape:
                raise ValueError("supervision_mask must match input_ids")
            eligible = supervision_mask.to(self.device, torch.bool)
            valid = int(eligible.sum()) if supervision_count is None else int(supervision_count)
        if valid <= 0:
            raise ValueError("each training batch must contain supervised tokens")
        t = self.sample_times(b, nblk)
        weights = torch.ones_like(t) if self.loss_weighting == "unit" else t.reciprocal()
        noise = (-torch.log1p(-t)).clamp(max=-math.log(self.noise_schedule_epsilon))
        xt, labels = self._tokens(x0, t, eligible, shift=False)
        active = (labels != LABEL_IGNORE_INDEX).sum(dtype=torch.int64)
        self.batches_corrupted += 1
        self.valid_tokens_seen += valid
        return CorruptedBatch(x0, xt, labels, t, noise, weights[:, None], active, valid, float(valid))


class FastDLLMv2Runtime(_ObjectiveRuntime):
    name = "fast_dllm_v2"
    views = 2
    exclude_mask_token = False

    def __init__(self, *, noise_schedule_epsilon=1e-3, **kw):
        super().__init__(**kw)
        self.noise_schedule_epsilon = float(noise_schedule_epsilon)

    def corrupt(self, x0, *, supervision_mask=None, supervision_count=None) -> CorruptedBatch:
        b, l, nblk = self._check(x0, min_len=2)
        x0 = x0.to(self.device)
        if supervision_mask is None:
            if supervision_count is not None:
                raise ValueError("supervision_count requires an explicit supervision_mask")
            eligible = torch.ones_like(x0, dtype=torch.bool)
            valid = b * (l - 1)  # position 0 has no preceding query under the shifted loss
        else:
            if supervision_mask.shape != x0.shape:
                raise ValueError("supervision_mask must match input_ids")
            eligible = supervision_mask.to(self.device, torch.bool)
            valid = (int(eligible[:, 1:].sum()) if supervision_count is None
                     else int(supervision_count) - int(eligible[:, 0].sum()))
        if valid <= 0:
            raise ValueError("each training batch must contain shifted supervised tokens")
        t = self._block_uniforms(b * nblk).view(b, nblk)
        move = (1.0 - self.noise_schedule_epsilon) * t + self.noise_schedule_epsilon
        noisy, labels = self._tokens(x0, move, None if supervision_mask is None else eligible, shift=True)
        active = (labels != LABEL_IGNORE_INDEX).sum(dtype=torch.int64)
        self.batches_corrupted += 1
        self.valid_tokens_seen += valid
        return CorruptedBatch(x0, noisy, labels, t, move, torch.ones(b, 2, nblk, device=self.device),
                              active, valid, float(valid))


class DiffusionGemmaNativeRuntime(StandardBlockDiffusionRuntime):
    """diffusiongemma_native_sft: uniform-replacement corruption with unit loss weights.

    Per (sample, block) a time t in [eps_min, eps_max] (antithetic-stratified by default); a scored
    token is REPLACED by a uniformly random vocabulary token with probability t (no mask token); the
    label is the clean token on EVERY scored position (replaced or not), all weights are 1 and the
    denominator is the scored-token count. With probability `self_conditioning_probability` a sample
    is marked for self-conditioning (`CorruptedBatch.self_conditioning_mask`): the training step then
    runs a detached first pass and feeds its soft predictions back (`ops/soft_embedding.py`).
    The Bernoulli draws use the counter-based generator shared with the other objectives; the random
    replacement tokens and the self-conditioning draw come from a torch generator re-seeded from
    (seed, batch counter), so the resumable state is still just the counter.

    Semantics follow dllm_parallel/core/objectives/diffusiongemma.py:66-460 (all-block corruption over
    the scored region). The separate encoder next-token term is added by the training session
    (`training/session.py::forward_backward`), which also makes the clean rows attend causally for it.
    """
    name = "diffusiongemma_native_sft"
    views = 1
    exclude_mask_token = False

    def __init__(self, *, vocab_size: int, self_conditioning_probability: float = 0.5,
                 pack_response_suffix: bool = True, minimum_decoder_blocks: int = 1, **kw):
        kw.setdefault("loss_weighting", "unit")
        super().__init__(**kw)
        self.pack_response_suffix = bool(pack_response_suffix)
        self.minimum_decoder_blocks = max(int(minimum_decoder_blocks), 1)
        if vocab_size <= 1:
            raise ValueError("vocab_size must be greater than one")
        if not 0.0 <= self_conditioning_probability <= 1.0:
            raise ValueError("self_conditioning_probability must be in [0, 1]")
        if self.loss_weighting != "unit":
            raise ValueError("diffusiongemma_native_sft requires loss_weighting=unit")
        self.vocab_size = int(vocab_size)
        self.self_conditioning_probability = float(self_conditioning_probability)

    def response_suffix(self, supervision_mask, valid_mask=None):
        """(response_start, valid_length) when every row's scored positions are one contiguous suffix of its valid
        prefix and the batch shares both numbers; None otherwise (the masked full-length form then applies).
        Conditions of dllm_parallel/core/objectives/diffusiongemma.py:151-224."""
        if supervision_mask is None:
            return None
        sm = supervision_mask.to(torch.bool)
        b, l = sm.shape
        pos = torch.arange(l, device=sm.device)
        if valid_mask is None:
            lengths = torch.full((b,), l, dtype=torch.long, device=sm.device)
            valid = torch.ones_like(sm)
        else:
            valid = valid_mask.to(sm.device, torch.bool)
            lengths = valid.sum(1)
            if bool((lengths <= 0).any()) or not torch.equal(valid, pos[None, :] < lengths[:, None]):
                raise ValueError("valid_mask must be one contiguous non-empty prefix per example")
            if bool((sm & ~valid).any()):
                raise ValueError("supervision_mask cannot score padding")
        if bool((sm.sum(1) <= 0).any()):
            return None
        starts = sm.to(torch.int64).argmax(1)
        if not torch.equal(sm, (pos[None, :] >= starts[:, None]) & valid):
            return None
        if not bool(starts.eq(starts[0]).all()) or not bool(lengths.eq(lengths[0]).all()):
            return None
        return int(starts[0]), int(lengths[0])

    def _corrupt_packed(self, x0, start: int, length: int) -> CorruptedBatch:
        """Decoder rows for the response [start, length) only: blocks counted from `start`, the last block filled
        with padding rows (clamped positions, never scored), at least `minimum_decoder_blocks` blocks."""
        b = x0.shape[0]
        bs = self.block_size
        resp = length - start
        logical = (resp + bs - 1) // bs * bs
        dec_len = max(logical, self.minimum_decoder_blocks * bs)
        off = torch.arange(dec_len, device=self.device)
        real = off < resp
        dpos = (off + start).clamp(max=length - 1)
        dec_clean = x0.index_select(1, dpos)
        eligible = real[None, :].expand(b, -1)
        nblk = dec_len // bs
        t = self.sample_times(b, nblk)
        noise = (-torch.log1p(-t.clamp(max=1.0 - 1e-7))).clamp(max=-math.log(self.noise_schedule_epsilon))
        _, moved_labels = self._tokens(dec_clean, t, eligible, shift=False)
        moved = moved_labels[:, 0] != LABEL_IGNORE_INDEX
        g = torch.Generator(device=self.device)
        g.manual_seed((self.seed * 1_000_003 + 2 * self.batches_corrupted + 1) % (2 ** 63 - 1))
        random_tokens = torch.randint(0, self.vocab_size, dec_clean.shape, dtype=x0.dtype, device=self.device, generator=g)
        noisy = torch.where(moved, random_tokens, dec_clean)
        labels = torch.where(eligible, dec_clean, torch.full_like(dec_clean, LABEL_IGNORE_INDEX))
        sc_mask = torch.rand(b, device=self.device, generator=g) < self.self_conditioning_probability
        valid = b * resp
        self.batches_corrupted += 1
        self.valid_tokens_seen += valid
        out = CorruptedBatch(x0, noisy[:, None], labels[:, None], t, noise, torch.ones(b, 1, nblk, device=self.device),
                             eligible.sum(dtype=torch.int64), valid, float(valid))
        out.self_conditioning_mask = sc_mask
        out.replaced_tokens = moved.sum(dtype=torch.int64)
        out.response_start, out.valid_length = start, length
        return out

    def corrupt(self, x0, *, supervision_mask=None, supervision_count=None, valid_mask=None) -> CorruptedBatch:
        b, l, nblk = self._check(x0)
        x0 = x0.to(self.device)
        if self.pack_response_suffix:
            suffix = self.response_suffix(supervision_mask, valid_mask)
            if suffix is not None and (suffix[0] > 0 or suffix[1] < l):
                if supervision_count is not None and int(supervision_count) != b * (suffix[1] - suffix[0]):
                    raise ValueError("supervision_count must equal the explicit supervision_mask count")
                return self._corrupt_packed(x0, *suffix)
        if supervision_mask is None:
            if supervision_count is not None:
                raise ValueError("supervision_count requires an explicit supervision_mask")
            eligible, valid = None, b * l
        else:
            if supervision_mask.shape != x0.shape:
                raise ValueError("supervision_mask must match input_ids")
            eligible = supervision_mask.to(self.device, torch.bool)
            valid = int(eligible.sum()) if supervision_count is None else int(supervision_count)
        if valid <= 0:
            raise ValueError("each training batch must contain supervised tokens")
        t = self.sample_times(b, nblk)
        noise = (-torch.log1p(-t.clamp(max=1.0 - 1e-7))).clamp(max=-math.log(self.noise_schedule_epsilon))
        # which scored tokens move: the shared counter-based Bernoulli draw (positions that got the mask id)
        _, moved_labels = self._tokens(x0, t, eligible, shift=False)
        moved = moved_labels[:, 0] != LABEL_IGNORE_INDEX
        g = torch.Generator(device=self.device)
        g.manual_seed((self.seed * 1_000_003 + 2 * self.batches_corrupted + 1) % (2 ** 63 - 1))
        random_tokens = torch.randint(0, self.vocab_size, x0.shape, dtype=x0.dtype, device=self.device, generator=g)
        noisy = torch.where(moved, random_tokens, x0)
        scored = torch.ones_like(x0, dtype=torch.bool) if eligible is None else eligible
        labels = torch.where(scored, x0, torch.full_like(x0, LABEL_IGNORE_INDEX))
        sc_mask = torch.rand(b, device=self.device, generator=g) < self.self_conditioning_probability
        active = scored.sum(dtype=torch.int64)
        self.batches_corrupted += 1
        self.valid_tokens_seen += valid
        out = CorruptedBatch(x0, noisy[:, None], labels[:, None], t, noise, torch.ones(b, 1, nblk, device=self.device),
                             active, valid, float(valid))
        out.self_conditioning_mask = sc_mask
        out.replaced_tokens = moved.sum(dtype=torch.int64)
        return out


def fused_corrupt(x0: torch.Tensor, t: torch.Tensor, eligible, *, block_size: int, views: int, shift: bool,
                  mask_id: int, seed: int, offset: int):
    """Noisy ids and labels [B, V, L] from per-block move chances `t` with the counter-based
    generator: one sm_100a kernel on CUDA tensors, the bit-identical host twin elsewhere."""
    b, l = x0.shape
    if x0.is_cuda:
        from ..kernels import native
        from ..ops._util import ptr, stream

        native.register_signatures({"tdllm_corrupt": (native.c_int, [native.c_void_p] * 5 + [native.c_int] * 5
                                                      + [native.c_ll, native.c_ull, native.c_ull, native.c_void_p])})
        xt = torch.empty(b, views, l, dtype=torch.int64, device=x0.device)
        labels = torch.empty_like(xt)
        el = None if eligible is None else eligible.to(torch.uint8).contiguous()
        native.check(native.lib().tdllm_corrupt(ptr(x0.contiguous()), ptr(t.float().contiguous()), ptr(el), ptr(xt),
                                                ptr(labels), b, l, block_size, views, int(shift), mask_id, seed,
                                                offset, stream()), "corrupt")
        return xt, labels
    from .philox import corrupt_reference

    return corrupt_reference(x0, t, eligible, block_size, views, shift, mask_id, seed, offset)


def build_objective_runtime(spec, *, mask_token_id: int, seed: int, device="cpu", vocab_size: int | None = None):
    """spec: RunSpec. Returns the corruption runtime of `objective.name`."""
    o = spec.objective
    common = dict(block_size=o.block_size, mask_token_id=mask_token_id, max_seq_len=spec.model.seq_len,
                  seed=seed, device=device)
    if o.name == "standard_block_diffusion":
        return StandardBlockDiffusionRuntime(
            loss_weighting=o.loss_weighting, noise_schedule_epsilon=o.noise_schedule_epsilon,
            sampling_epsilon_min=o.sampling_epsilon_min, sampling_epsilon_max=o.sampling_epsilon_max,
            antithetic_sampling=o.antithetic_sampling, **common)
    if o.name == "fast_dllm_v2":
        return FastDLLMv2Runtime(noise_schedule_epsilon=o.noise_schedule_epsilon, **common)
    if o.name == "diffusiongemma_native_sft":
        if vocab_size is None:
            raise ValueError("diffusiongemma_native_sft needs the model's vocabulary size")
        return DiffusionGemmaNativeRuntime(
            vocab_size=vocab_size, self_conditioning_probability=o.self_conditioning_probability,
            pack_response_suffix=o.pack_response_suffix, minimum_decoder_blocks=o.minimum_decoder_blocks,
            loss_weighting=o.loss_weighting, noise_schedule_epsilon=o.noise_schedule_epsilon,
            sampling_epsilon_min=o.sampling_epsilon_min, sampling_epsilon_max=o.sampling_epsilon_max,
            antithetic_sampling=o.antithetic_sampling, **common)
    raise ValueError(f"no corruption runtime for objective {o.name!r}")
