"""Mixture-of-experts block-diffusion decoder (DiffusionGemma-style expert-parallel path).

Attention is the dense model's. The FFN of every layer is a routed expert bank: a linear router,
softmax over all experts, top-k selection with renormalised weights, SwiGLU experts. Tokens are
sorted by expert so that each expert sees one contiguous slab of rows, the expert GEMMs run slab
by slab on the tcgen05 GEMM (TMA clips the ragged last tile of a slab), and results are scattered
back and combined with the routing weights.

With expert parallelism each rank owns `E / EP` experts (`[E_local, ...]` weights). Dispatch sends
every (token, choice) to the owner of its expert and combine returns the expert output; the
transport is `torch.distributed.all_to_all_single` with variable splits (NCCL; gloo on CPU), the
counterpart of the reference's DeepEP dispatch/combine ops.

Counterparts: dllm_parallel/core/models/backbones/diffusiongemma/expert_parallel.py:26-200 (EP experts),
:283-321 (grouped experts), :324-364 (reference experts), router/route replay
dllm_parallel/core/models/backbones/diffusiongemma/model.py:33-330; DeepEP ops
dllm_parallel/core/parallel/expert/deepep.py:122-555.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..profiling import collectives as coll

from ..ops.activation import swiglu
from ..ops.gemm import linear, linear_residual
from ..ops.norm import rmsnorm
from ..ops.rope import qk_norm_rope
from .config import ModelConfig
from .dense import BlockDiffusionTransformer, FlatParams

def route_topk(logits: torch.Tensor, k: int):
    """softmax over experts, top-k, renormalise. Returns (weights [rows,k] fp32, experts [rows,k] int64)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = probs.topk(k, dim=-1)
    return w / w.sum(-1, keepdim=True), idx


def reference_experts(x, w_gu, w_down, weights, experts):
    """Dense oracle: loops over experts on plain tensors (interleaved gate/up rows)."""
    out = torch.zeros_like(x, dtype=torch.float32)
    E = w_gu.shape[0]
    for e in range(E):
        rows, slot = (experts == e).nonzero(as_tuple=True)
        if rows.numel() == 0:
            continue
        h = x[rows].float() @ w_gu[e].float().t()
        act = torch.nn.functional.silu(h[:, 0::2]) * h[:, 1::2]
        y = act @ w_down[e].float().t()
        out.index_add_(0, rows, y * weights[rows, slot, None].float())
    return out.to(x.dtype)


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all of rows; the backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, send_counts, recv_counts, group):
        ctx.group, ctx.send, ctx.recv = group, send_counts, recv_counts
        out = x.new_empty(sum(recv_counts), x.shape[1])
        coll.all_to_all_single(out, x.contiguous(), recv_counts, send_counts, domain="expert", group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty(sum(ctx.send), g.shape[1])
        coll.all_to_all_single(out, g.contiguous(), ctx.send, ctx.recv, domain="expert", group=ctx.group)
        return out, None, None, None


class ExpertBank(nn.Module):
    """`E_local` SwiGLU experts of this rank and the routed forward over them."""

    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams, ep_group=None):
        super().__init__()
        self.cfg, self.idx = cfg, idx
        self.router = flat.params[f"layers.{idx}.router"]
        self.w_gu = flat.params[f"layers.{idx}.experts_gate_up"]     # [E_local, 2I, H]
        self.w_down = flat.params[f"layers.{idx}.experts_down"]      # [E_local, H, I]
        self.ep_group = ep_group
        self.ep = dist.get_world_size(ep_group) if ep_group is not None else 1
        self.ep_rank = dist.get_rank(ep_group) if ep_group is not None else 0
        self.e_local = self.w_gu.shape[0]
        self.lora = None               # adapters.lora.LoRAState with per-expert pairs, set by apply_lora
        self.last_counts = None
        self.exchange_holder = None    # set by the model: one PeerExpertExchange shared by all layers

    def _route(self, logits: torch.Tensor, k: int):
        """Top-k routing that a checkpointed layer's recomputation repeats exactly: the no-grad forward keeps the
        chosen experts, the replay takes them from there and only recomputes the (differentiable) weights, so a
        near-tie in the router logits cannot send a token elsewhere the second time.
        Role of the route record / replay of dllm_parallel/core/models/backbones/moe_checkpoint.py:22-59."""
        store = getattr(self, "store", None)
        key = (self.idx, "moe_route")
        if store is not None and store.replaying and store.has(key):
            idx = store.kept.pop(key)
            probs = torch.softmax(logits.float(), dim=-1)
            w = probs.gather(1, idx)
            return w / w.sum(-1, keepdim=True), idx
        w, idx = route_topk(logits, k)
        if store is not None and store.recording and not torch.is_grad_enabled():
            store.kept[key] = idx        # a few bytes per row: never sent to the host
        return w, idx

    def _peer_exchange(self, x: torch.Tensor):
        """The peer-memory dispatch / combine state, or None (CPU, no peer access, shapes off the tile grid,
        TDLLM_EP_PEER=0): the caller then uses all-to-all collectives."""
        import os

        from ..ops.grouped import grouped_supported

        holder = self.exchange_holder
        if self.lora is not None:       # per-expert adapters run on the per-expert path
            return None
        if (holder is None or self.ep < 2 or not x.is_cuda or os.environ.get("TDLLM_EP_PEER", "1") == "0"
                or not grouped_supported(x, self.w_gu) or not grouped_supported(x, self.w_down)):
            return None
        if holder.get("exchange") is None and not holder.get("failed"):
            try:
                from ..parallel.expert_exchange import PeerExpertExchange

                holder["exchange"] = PeerExpertExchange(self.ep_group, x.device, rows=x.shape[0],
                                                        top_k=self.cfg.num_experts_per_token, hidden=x.shape[1],
                                                        num_experts=self.cfg.num_experts)
            except Exception as e:   # no peer access, IPC refused: collectives carry the exchange
                holder["failed"] = str(e)
        ex = holder.get("exchange")
        if ex is not None and x.shape[0] > ex.max_rows:
            return None
        return ex

    def _local_experts(self, x_sorted: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        """x_sorted: rows grouped by local expert (`counts` per expert, on the device). On the GPU all
        experts run as one grouped GEMM per projection over a padded row layout; otherwise (CPU, or
        expert shapes off the tile grid) per-expert slabs run through the shared GEMM. Weight
        gradients land in the experts' slices of the flat gradient buffer either way."""
        from ..ops.grouped import build_grouped_rows, grouped_linear, grouped_supported

        if self.lora is not None:
            return self._local_experts_lora(x_sorted, counts)
        if x_sorted.shape[0] > 0 and grouped_supported(x_sorted, self.w_gu) and grouped_supported(x_sorted, self.w_down):
            g = build_grouped_rows(counts, x_sorted.shape[0])
            x_pad = x_sorted.new_zeros(g.capacity, x_sorted.shape[1]).index_copy(0, g.dest, x_sorted)
            act = swiglu(grouped_linear(x_pad, self.w_gu, g))
            return grouped_linear(act, self.w_down, g).index_select(0, g.dest)
        outs, off = [], 0
        for e, n in enumerate(counts.tolist()):
            if n == 0:
                continue
            xe = x_sorted[off:off + n]
            gu = _expert_linear(xe, self.w_gu, e)
            outs.append(_expert_linear(swiglu(gu), self.w_down, e))
            off += n
        if not outs:
            return x_sorted.new_zeros(0, x_sorted.shape[1])
        return torch.cat(outs, dim=0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        rows, H = x.shape
        k = cfg.num_experts_per_token
        w, idx = self._route(linear(x, self.router), k)
        ex = self._peer_exchange(x)
        if ex is not None:
            # rows go straight into the owners' slabs and come back weighted: no sort, no collective, no host read
            from ..ops.grouped import grouped_linear
            from ..parallel.expert_exchange import peer_combine, peer_dispatch

            state: dict = {}
            flat32 = idx.reshape(-1).to(torch.int32).contiguous()
            x_pad = peer_dispatch(x.contiguous(), flat32, ex, state)
            act = swiglu(grouped_linear(x_pad, self.w_gu, state["g"]))
            y_pad = grouped_linear(act, self.w_down, state["g"])
            self.last_counts = None
            return peer_combine(y_pad, w, ex, state)
        flat_e = idx.reshape(-1)                                        # [rows*k]
        order = torch.argsort(flat_e, stable=True)
        token_of = torch.div(order, k, rounding_mode="floor")
        x_perm = x.index_select(0, token_of)                            # grouped by global expert id
        counts_g = torch.bincount(flat_e, minlength=cfg.num_experts)
        if self.ep > 1:
            send = counts_g.view(self.ep, self.e_local).sum(1)
            all_counts = torch.empty(self.ep, cfg.num_experts, dtype=counts_g.dtype, device=x.device)
            coll.all_gather_into_tensor(all_counts.view(-1), counts_g, "expert", group=self.ep_group)
            mine = all_counts[:, self.ep_rank * self.e_local:(self.ep_rank + 1) * self.e_local]   # [src, e_local]
            # one host read for both all-to-all size lists (NCCL wants them on the host)
            sizes = torch.cat([send, mine.sum(1)]).tolist()
            send_l, recv_l = sizes[: self.ep], sizes[self.ep:]
            recv = _AllToAllRows.apply(x_perm, send_l, recv_l, self.ep_group)
            # received rows are ordered (source rank, local expert): regroup by local expert
            eid = torch.repeat_interleave(torch.arange(self.e_local, device=x.device).repeat(self.ep),
                                          mine.reshape(-1), output_size=recv.shape[0])
            eorder = torch.argsort(eid, stable=True)
            y_sorted = self._local_experts(recv.index_select(0, eorder), mine.sum(0))
            y_recv = torch.empty_like(y_sorted).index_copy_(0, eorder, y_sorted) if y_sorted.numel() else y_sorted
            y_perm = _AllToAllRows.apply(y_recv, recv_l, send_l, self.ep_group)
        else:
            y_perm = self._local_experts(x_perm, counts_g)
        self.last_counts = counts_g
        wk = w.reshape(-1).index_select(0, order).to(y_perm.dtype)
        out = torch.zeros_like(x)
        out.index_add_(0, token_of, y_perm * wk[:, None])
        return out


def _local_experts_lora(bank, x_sorted: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Per-expert slabs with low-rank updates: y_e = x·W_eᵀ + s·(x·A_eᵀ)·B_eᵀ for both projections; the frozen
    expert weights get no gradient, the adapters' gradients go to their experts' slices."""
    st = bank.lora
    gu_pair, dn_pair = st.expert_pair(bank.idx, "experts_gate_up"), st.expert_pair(bank.idx, "experts_down")

    def proj(x, w_all, pair, e):
        y = _expert_linear(x, w_all, e)
        if pair is None:
            return y
        if st.dropout > 0 and torch.is_grad_enabled():
            x = torch.nn.functional.dropout(x, st.dropout)
        return y + _expert_linear(_expert_linear(x, pair[0], e), pair[1], e) * st.scale

    outs, off = [], 0
    for e, n in enumerate(counts.tolist()):
        if n == 0:
            continue
        xe = x_sorted[off:off + n]
        outs.append(proj(swiglu(proj(xe, bank.w_gu, gu_pair, e)), bank.w_down, dn_pair, e))
        off += n
    return torch.cat(outs, dim=0) if outs else x_sorted.new_zeros(0, x_sorted.shape[1])


ExpertBank._local_experts_lora = _local_experts_lora


class _ExpertLinear(torch.autograd.Function):
    """y = x · W[e]ᵀ for one expert of a stacked weight; dW goes to that expert's gradient slice."""

    @staticmethod
    def forward(ctx, x, w_all, e):
        from ..ops.gemm import gemm

        ctx.save_for_backward(x, w_all)
        ctx.e, ctx.wref = e, w_all
        return gemm(x, w_all[e])

    @staticmethod
    def backward(ctx, dy):
        from ..ops._util import grad_sink
        from ..ops.gemm import gemm

        x, w_all = ctx.saved_tensors
        e = ctx.e
        dy = dy.contiguous()
        dx = gemm(dy, w_all[e], b_mn_major=True)
        if not ctx.needs_input_grad[1]:      # a frozen stacked weight (adapters train instead)
            return dx, None, None
        sink, _ = grad_sink(ctx.wref)
        if sink is not None:
            written = ctx.wref.expert_written
            gemm(dy, x, a_mn_major=True, b_mn_major=True, out=sink[e], accumulate=e in written)
            written.add(e)
            return dx, None, None
        dw = torch.zeros_like(w_all)
        gemm(dy, x, a_mn_major=True, b_mn_major=True, out=dw[e])
        return dx, dw, None


def _expert_linear(x, w_all, e):
    return _ExpertLinear.apply(x, w_all, e)


class MoEDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, idx: int, flat: FlatParams, ep_group=None, tp=None):
        """cfg: per-rank shapes. tp: tensor-parallel context. Attention and the dense feed-forward branch are sharded
        like the dense decoder's (column- / row-parallel); the router and the experts are replicated over the
        tensor-parallel ranks and work on the rows the rank holds: all rows without sequence parallelism (every rank
        computes the same), its own rows with it (the ranks then route different tokens, and the gradients of the
        router, the experts and the layer norms are partial sums that the session adds up over the group)."""
        super().__init__()
        self.cfg, self.idx = cfg, idx
        self.tp = tp if tp is not None and tp.size > 1 else None
        g = lambda n: flat.params[f"layers.{idx}.{n}"]
        self.input_norm, self.w_qkv, self.w_o, self.post_norm = g("input_norm"), g("w_qkv"), g("w_o"), g("post_norm")
        self.q_norm = g("q_norm") if cfg.qk_norm else None
        self.k_norm = g("k_norm") if cfg.qk_norm else None
        # dual feed-forward: a dense SwiGLU branch in parallel with the routed experts
        # (dllm_parallel/core/models/backbones/nemotron/model.py:2612-2919)
        self.w_gate_up = g("w_gate_up") if cfg.moe_shared_intermediate_size > 0 else None
        self.w_down = g("w_down") if cfg.moe_shared_intermediate_size > 0 else None
        self.experts = ExpertBank(cfg, idx, flat, ep_group)
        if self.tp is not None:
            partial = [self.q_norm, self.k_norm]
            if self.tp.sequence_parallel:
                partial += [self.input_norm, self.post_norm, self.experts.router, self.experts.w_gu, self.experts.w_down]
            for p in partial:
                if p is not None:
                    p.tp_partial = True

    def _forward_tensor_parallel(self, h, positions, inv_freq, attend):
        from ..ops.gemm import linear_swiglu, row_parallel_linear_residual
        from ..parallel.tensor_parallel import sp_column_linear, sp_row_linear_residual

        cfg, tp = self.cfg, self.tp
        sp = tp.sequence_parallel
        if getattr(self, "lora", None) is not None:
            # adapters: tensor-parallel low-rank products on the attention and dense-branch projections; the experts'
            # own pairs (replicated like the experts) are applied inside the expert bank
            from ..adapters.lora import adapted_column_linear as acol, adapted_row_linear as arow

            y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
            qkv = qk_norm_rope(acol(self, y, "w_qkv"), positions, inv_freq, self.q_norm, self.k_norm,
                               cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
            h = arow(self, attend(qkv, self.idx), "w_o", h)
            y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
            out = h + self.experts(y2)
            if self.w_gate_up is None:
                return out
            return arow(self, swiglu(acol(self, y2, "w_gate_up")), "w_down", out, last=True)
        column = (lambda x, w, **kw: sp_column_linear(x, w, tp, **kw)) if sp else None
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        qkv = column(y, self.w_qkv) if sp else linear(y, self.w_qkv, tp)
        qkv = qk_norm_rope(qkv, positions, inv_freq, self.q_norm, self.k_norm, cfg.num_attention_heads,
                           cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        a = attend(qkv, self.idx)
        h = sp_row_linear_residual(a, self.w_o, h, tp) if sp else row_parallel_linear_residual(a, self.w_o, h, tp)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        out = h + self.experts(y2)            # token-local: the rows this rank holds
        if self.w_gate_up is None:
            return out
        if sp:
            return sp_row_linear_residual(column(y2, self.w_gate_up, swiglu=True), self.w_down, out, tp, last=True)
        return row_parallel_linear_residual(linear_swiglu(y2, self.w_gate_up, tp), self.w_down, out, tp, last=True)

    def forward(self, h, positions, inv_freq, attend):
        cfg = self.cfg
        if self.tp is not None:
            return self._forward_tensor_parallel(h, positions, inv_freq, attend)
        y, _ = rmsnorm(h, self.input_norm, cfg.rms_norm_eps)
        st = getattr(self, "lora", None)
        if st is not None:
            from ..adapters.lora import lora_delta

            def proj(x, name):
                out, pair = linear(x, getattr(self, name)), st.pair(self.idx, name)
                return out if pair is None else out + lora_delta(x, pair[0], pair[1], st.scale, st.dropout)

            qkv = qk_norm_rope(proj(y, "w_qkv"), positions, inv_freq, self.q_norm, self.k_norm,
                               cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
            h = h + proj(attend(qkv, self.idx), "w_o")
            y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
            out = h + self.experts(y2)
            return out if self.w_gate_up is None else out + proj(swiglu(proj(y2, "w_gate_up")), "w_down")
        qkv = qk_norm_rope(linear(y, self.w_qkv), positions, inv_freq, self.q_norm, self.k_norm,
                           cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps)
        h = linear_residual(attend(qkv, self.idx), self.w_o, h)
        y2, _ = rmsnorm(h, self.post_norm, cfg.rms_norm_eps)
        out = h + self.experts(y2)
        if self.w_gate_up is None:
            return out
        from ..ops.gemm import linear_swiglu

        return linear_residual(linear_swiglu(y2, self.w_gate_up), self.w_down, out)


def moe_layer_specs(cfg: ModelConfig, i: int, e_local: int):
    h, p = cfg.hidden_size, f"layers.{i}."
    out = [(p + "input_norm", (h,), False), (p + "w_qkv", (cfg.qkv_dim, h), True), (p + "w_o", (h, cfg.q_dim), True),
           (p + "post_norm", (h,), False), (p + "router", (cfg.num_experts, h), True),
           (p + "experts_gate_up", (e_local, 2 * cfg.moe_intermediate_size, h), True),
           (p + "experts_down", (e_local, h, cfg.moe_intermediate_size), True)]
    if cfg.moe_shared_intermediate_size > 0:
        out += [(p + "w_gate_up", (2 * cfg.moe_shared_intermediate_size, h), True),
                (p + "w_down", (h, cfg.moe_shared_intermediate_size), True)]
    if cfg.qk_norm:
        out += [(p + "q_norm", (cfg.head_dim,), False), (p + "k_norm", (cfg.head_dim,), False)]
    return out


def local_moe_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    """Per-rank shapes under tensor parallelism: attention heads and the dense feed-forward branch are divided by `tp`;
    router and experts keep their shapes (they are replicated over the tensor-parallel ranks)."""
    if tp == 1:
        return cfg
    from dataclasses import replace

    for name in ("num_attention_heads", "num_key_value_heads", "moe_shared_intermediate_size", "vocab_size"):
        if getattr(cfg, name) % tp:
            raise ValueError(f"{name} ({getattr(cfg, name)}) must divide by tensor_parallel_size {tp}")
    return replace(cfg, num_attention_heads=cfg.num_attention_heads // tp, num_key_value_heads=cfg.num_key_value_heads // tp,
                   moe_shared_intermediate_size=cfg.moe_shared_intermediate_size // tp)


class MoEBlockDiffusionTransformer(BlockDiffusionTransformer):
    """Same interface as the dense model; expert parameters are sharded over `ep_group`."""

    def __init__(self, cfg: ModelConfig, *, ep_group=None, dtype=torch.bfloat16, device="cpu",
                 activation_checkpointing: bool = True, activation_offload: bool = False, seed: int = 0,
                 init_std: float = 0.02, tp=None):
        nn.Module.__init__(self)
        from ..ops.rope import rope_inv_freq
        from .activation_store import ActivationStore

        self.cfg = cfg
        self.tp = tp if tp is not None and tp.size > 1 else None
        tps = self.tp.size if self.tp is not None else 1
        self.lcfg = local_moe_config(cfg, tps)
        if self.tp is not None:
            self.tp.sp_saved_in_place = bool(activation_checkpointing)
        self.activation_checkpointing = activation_checkpointing
        self.store = ActivationStore(torch.device(device), offload=activation_offload)
        self.store.keep_attention = False
        ep = dist.get_world_size(ep_group) if ep_group is not None else 1
        if cfg.num_experts % ep:
            raise ValueError(f"{cfg.num_experts} experts cannot be split over expert_parallel_size {ep}")
        e_local = cfg.num_experts // ep
        h = cfg.hidden_size
        specs = [("embed", (cfg.vocab_size // tps, h), True), ("final_norm", (h,), False)]
        if not cfg.tie_word_embeddings:
            specs.append(("lm_head", (cfg.vocab_size // tps, h), True))
        for i in range(cfg.num_layers):
            specs += moe_layer_specs(self.lcfg, i, e_local)
        dense_specs = [sp for sp in specs if "experts_" not in sp[0]]
        expert_specs = [sp for sp in specs if "experts_" in sp[0]]
        first_router = None
        if self.tp is not None:
            # the optimizer sums squared gradients of tensor-parallel shards over the group and counts replicated
            # parameters once: the routers are decayed matrices but replicated, so they go behind the sharded ones
            routers = [sp for sp in dense_specs if sp[0].endswith(".router")]
            dense_specs = [sp for sp in dense_specs if not sp[0].endswith(".router")] + routers
            first_router = routers[0][0]
        self.flat = FlatParams(dense_specs, dtype, device)            # replicated over DP x EP
        if first_router is not None:
            self.flat.tp_sharded_numel = self.flat.offsets[first_router][0]
        self.flat_experts = FlatParams(expert_specs, dtype, device)    # sharded over EP, replicated over DP
        for p in self.flat_experts.params.values():
            p.expert_written = set()
        self.flat.params.update(self.flat_experts.params)              # one lookup table for the layers
        self.flat_experts_only = self.flat_experts
        for name, p in self.flat.params.items():
            self.register_parameter(name.replace(".", "_"), p)
        self.embed, self.final_norm = self.flat.params["embed"], self.flat.params["final_norm"]
        self.lm_head = self.flat.params.get("lm_head", self.embed)
        self.layers = nn.ModuleList(MoEDecoderLayer(self.lcfg, i, self.flat, ep_group, self.tp) for i in range(cfg.num_layers))
        self.expert_exchange = {}      # filled on the first routed batch on a GPU (parallel/expert_exchange.py)
        for layer in self.layers:
            layer.experts.exchange_holder = self.expert_exchange
            layer.experts.store = self.store
        self.register_buffer("inv_freq", rope_inv_freq(cfg.head_dim, cfg.rope_theta, device, cfg.rotary_dim), persistent=False)
        ep_rank = dist.get_rank(ep_group) if ep_group is not None else 0
        self.reset_parameters(seed, init_std)
        if ep > 1:  # expert slices differ per rank, everything else is replicated
            gen = torch.Generator(device=self.flat.data.device)
            gen.manual_seed(seed + 1000 + ep_rank)
            for name, p in self.flat.params.items():
                if "experts_" in name:
                    with torch.no_grad():
                        p.copy_((torch.randn(p.shape, device=p.device, generator=gen) * init_std).to(p.dtype))
