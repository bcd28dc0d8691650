"""Multi-GPU tests (2 ranks, NCCL, one process per GPU): the fused peer-memory ZeRO step against
its NCCL twin, data-parallel training sessions, and the bounded barrier wait (single GPU)."""
import pytest
import torch

from tests._harness import run_ranks

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _spec(backend):
    from turbo_dllm_b200.config.run_spec import RunSpec

    return RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-hd128", "seq_len": 512, "dtype": "bf16"},
        "objective": {"name": "fast_dllm_v2", "block_size": 32, "noise_schedule_epsilon": 0.1},
        "training": {"batch_size": 1, "steps": 3},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
        "kernel": {"impl": "nccl_baseline" if backend in ("nccl", "fsdp_nccl") else "auto"},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0,
                      "backend": {"fused": "zero_fused", "fsdp": "fsdp", "fsdp_nccl": "fsdp"}.get(backend, "auto")}}
    ).validate()


def _train(rank, world, backend, steps):
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    s = TrainingSession(_spec(backend), device=f"cuda:{rank}")
    assert (s.optimizer.fused_sync is not None) == (backend == "fused")
    assert (s.sharded is not None) == backend.startswith("fsdp")
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        dist.all_reduce(t)
        losses.append(float(t) / r.denominator)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    params = s.sharded.gather_full() if s.sharded is not None else s.model.flat.data
    out = losses, params.float().cpu(), s.optimizer.grad_norm()
    if s.sharded is not None:
        assert s.sharded.peer == (backend == "fsdp")
        s.close()
    if backend == "fused":
        # closing hands the symmetric buffers back and leaves a session that still trains (NCCL path)
        used_before = torch.cuda.mem_get_info()[0]
        s.close()
        assert s.optimizer.fused_sync is None
        assert (s.model.flat.data.float().cpu() == out[1]).all()
        r = s.step()
        assert torch.isfinite(r.loss_sum).item()
        del used_before
    return out


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_zero_matches_nccl_twin(world):
    _need(world)
    a = run_ranks(_train, world, args=("nccl", 3), backend="nccl", deadline_s=300)
    b = run_ranks(_train, world, args=("fused", 3), backend="nccl", deadline_s=300)
    for (la, pa, na), (lb, pb, nb) in zip(a, b):
        assert la == pytest.approx(lb, rel=2e-2)
        assert na == pytest.approx(nb, rel=2e-2)
        pa, pb = torch.from_numpy(pa), torch.from_numpy(pb)
        assert (pa - pb).abs().max().item() < 2e-2
    # replicas hold identical parameters after the push all-gather
    assert (b[0][1] == b[1][1]).all()


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4, 8])
def test_parameter_sharding_over_peer_memory_matches_nccl_twin_and_replicated_path(world):
    """optimizer.backend=fsdp with the peer-memory gather / reduce kernels against the same schedule over NCCL
    collectives and against the replicated-parameter path."""
    _need(world)
    a = run_ranks(_train, world, args=("nccl", 3), backend="nccl", deadline_s=300)
    b = run_ranks(_train, world, args=("fsdp", 3), backend="nccl", deadline_s=300)
    c = run_ranks(_train, world, args=("fsdp_nccl", 3), backend="nccl", deadline_s=300)
    for (la, pa, na), (lb, pb, nb), (lc, pc, nc) in zip(a, b, c):
        assert lb == pytest.approx(la, rel=2e-2) and lb == pytest.approx(lc, rel=2e-2)
        assert nb == pytest.approx(na, rel=2e-2)
        pa, pb, pc = (torch.from_numpy(x) for x in (pa, pb, pc))
        assert (pa - pb).abs().max().item() < 2e-2
        assert (pc - pb).abs().max().item() < 2e-2
    assert (b[0][1] == b[1][1]).all()


def test_barrier_wait_runs_out_and_reports():
    """Host-made failure: the second slot of the flag array is never written (no peer exists), so
    the bounded wait must expire, record ERR_WAIT_TIMEOUT for the barrier kernel and return."""
    import ctypes

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel import symm  # registers the signatures  # noqa: F401

    lib = native.lib()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    other = torch.zeros(64, dtype=torch.int32, device="cuda")
    arr = (ctypes.c_void_p * 2)(flags.data_ptr(), other.data_ptr())
    lib.tdllm_clear_error()
    native.check(lib.tdllm_set_wait_timeout_ns(2_000_000), "timeout")
    try:
        native.check(lib.tdllm_symm_barrier(arr, 0, 2, 1, None), "symm_barrier")
        torch.cuda.synchronize()
        err = native.device_error()
        assert err["code"] == 1 and err["kernel"] == 10 and err["detail"] == 1
        assert int(other[0]) == 1  # our arrival was published before the wait gave up
    finally:
        lib.tdllm_clear_error()
        lib.tdllm_set_wait_timeout_ns(2_000_000_000)
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


def _csbp(rank, world, transport, steps, model="synthetic:tiny-hd128", objective="standard_block_diffusion",
          block_axis=True, window=None):
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    cp = world
    spec = RunSpec.from_mapping({
        "model": {"id": model, "seq_len": 1024, "dtype": "bf16",
                  **({"sliding_window": window, "sliding_window_pattern": 2} if window else {})},
        "objective": {"name": objective, "block_size": 32, "sampling_epsilon_min": 0.1},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": cp, "block_parallel_size": cp if block_axis else 1},
        "kernel": {"cp_bp_clean_kv_transport": transport, "impl": "nccl_baseline"},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device=f"cuda:{rank}", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device=f"cuda:{rank}", runtime=rt)
    losses = []
    for _ in range(steps):
        r = s.step()
        t = r.loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t) / r.denominator)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    return losses, s.model.flat.data.float().cpu()


@pytest.mark.distributed
@pytest.mark.parametrize("transport", ["collective", "peer_pull", "streaming", "fused"])
def test_csbp2_on_gpus_matches_single_gpu(transport):
    _need(2)
    ref = run_ranks(_csbp, 1, args=("collective", 3), backend=None, deadline_s=300)[0]
    outs = run_ranks(_csbp, 2, args=(transport, 3), backend="nccl", deadline_s=300)
    for losses, params in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert (torch.from_numpy(params) - torch.from_numpy(ref[1])).abs().max().item() < 3e-2


def _dflash_replica(rank, world, mode, steps):
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-hd128", "seq_len": 1024, "dtype": "bf16", "family": "dflash",
                  "verifier_id": "synthetic:tiny-hd128", "target_layer_ids": [0, 1]},
        "objective": {"name": "dflash_distillation", "block_size": 16, "max_anchors": 32, "decay_gamma": 4.0},
        "data": {"target_features": "online"}, "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": world, "block_parallel_size": world},
        "kernel": {"dflash_context_exchange": mode, "impl": "nccl_baseline"},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device=f"cuda:{rank}", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device=f"cuda:{rank}", runtime=rt)
    losses = []
    for _ in range(steps):
        t = s.step().loss_sum.double().clone()
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t))
    torch.cuda.synchronize()
    native.raise_on_device_error()
    return losses, s.model.flat.data.float().cpu()


@pytest.mark.distributed
@pytest.mark.parametrize("transport", ["collective", "fused"])
def test_sliding_window_layers_under_csbp2_on_gpus_match_single_gpu(transport):
    """Layer 0 has a 128-token window: it moves only the clean rows inside some local row's window (one NCCL
    all-to-all with uneven splits, reversed in the backward pass); layer 1 uses the configured transport."""
    _need(2)
    args = (3, "synthetic:tiny-hd128", "standard_block_diffusion", True, 128)
    ref = run_ranks(_csbp, 1, args=("collective", *args), backend=None, deadline_s=300)[0]
    outs = run_ranks(_csbp, 2, args=(transport, *args), backend="nccl", deadline_s=300)
    for losses, params in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert (torch.from_numpy(params) - torch.from_numpy(ref[1])).abs().max().item() < 3e-2


@pytest.mark.distributed
@pytest.mark.parametrize("mode", ["kv_pull", "query_rotation"])
def test_dflash_replica_over_two_gpus_matches_single_gpu(mode):
    """The drafter's anchors and context rows divided over two GPUs: gathered context K|V, and rotated queries
    with merged partial attention (backward against the merged out / lse), against one GPU."""
    _need(2)
    ref = run_ranks(_dflash_replica, 1, args=("auto", 3), backend=None, deadline_s=300)[0]
    outs = run_ranks(_dflash_replica, 2, args=(mode, 3), backend="nccl", deadline_s=300)
    for losses, params in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert (torch.from_numpy(params) - torch.from_numpy(ref[1])).abs().max().item() < 3e-2


@pytest.mark.distributed
@pytest.mark.parametrize("transport,world", [("collective", 2), ("fused", 2), ("fused", 4), ("fused", 8)])
def test_pure_context_parallel_token_split_on_gpus_matches_single_gpu(transport, world):
    """Context parallelism without a block axis: every rank computes 32 / world offsets of every noisy block and
    ALL K|V rows travel (gathered, or pulled by the attention kernel with dK/dV added into the owners' rows)."""
    _need(world)
    ref = run_ranks(_csbp, 1, args=("collective", 3), backend=None, deadline_s=300)[0]
    outs = run_ranks(_csbp, world, args=(transport, 3, "synthetic:tiny-hd128", "standard_block_diffusion", False),
                     backend="nccl", deadline_s=300)
    for losses, params in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert (torch.from_numpy(params) - torch.from_numpy(ref[1])).abs().max().item() < 3e-2


@pytest.mark.distributed
@pytest.mark.parametrize("world", [4, 8])
def test_csbp_fused_transport_on_4_and_8_gpus_matches_single_gpu(world):
    """The in-kernel pull / push at group sizes where a rank has several peers: segment tables, the
    staggered peer order and ragged tile boundaries between the peers' rows."""
    _need(world)
    ref = run_ranks(_csbp, 1, args=("collective", 2), backend=None, deadline_s=300)[0]
    outs = run_ranks(_csbp, world, args=("fused", 2), backend="nccl", deadline_s=300)
    for losses, params in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert (torch.from_numpy(params) - torch.from_numpy(ref[1])).abs().max().item() < 3e-2


def test_fused_pull_gives_up_when_a_peer_never_signals():
    """Host-made failure on one GPU: the context-sharded forward is told about a peer whose "rows staged"
    flag nothing ever sets. The pullers' bounded wait must run out, the error record must name the pull
    side of the kernel, every other warp must leave its loop, and the context must stay usable."""
    import ctypes

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops.attention import INT_MIN, MaskLayout, block_diffusion_layout
    from turbo_dllm_b200.parallel import context_attention as ca  # noqa: F401
    from turbo_dllm_b200.parallel import symm  # noqa: F401

    lib = native.lib()
    dev = torch.device("cuda")
    Hq, Hkv, D, bs = 4, 2, 128, 32
    pos = torch.arange(256, device=dev)
    # this rank: noisy and clean rows of positions 128..255; the "peer" owns the clean rows 0..127, which every
    # local query attends to
    loc = block_diffusion_layout(pos[128:], pos[128:] // bs, pos[128:], bs)
    rem = block_diffusion_layout(pos[128:], pos[128:] // bs, pos[128:], bs, key_clean_pos=pos[:128])
    mask = MaskLayout(loc.q_lo, loc.q_hi, loc.q_grp, torch.cat([loc.k_code, rem.k_code[128:]]).contiguous())
    L = mask.tile_lists()
    qkv = torch.randn(256, (Hq + 2 * Hkv) * D, device=dev, dtype=torch.bfloat16)
    staged = torch.zeros(128, 2 * Hkv * D, device=dev, dtype=torch.bfloat16)
    kv_rem = torch.empty_like(staged)
    out = torch.empty(256, Hq * D, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(Hq, L["nq_pad"], device=dev, dtype=torch.float32)
    ready = torch.zeros(64, dtype=torch.int32, device=dev)
    tiles = torch.zeros(4, dtype=torch.int32, device=dev)
    two = lambda t: (ctypes.c_void_p * 2)(t.data_ptr(), t.data_ptr())
    counts = (ctypes.c_longlong * 2)(128, 128)
    lib.tdllm_clear_error()
    native.check(lib.tdllm_set_wait_timeout_ns(2_000_000), "timeout")
    try:
        q, k, v = qkv[:, : Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:]
        native.check(lib.tdllm_attn_fwd_csbp(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), kv_rem.data_ptr(), out.data_ptr(), lse.data_ptr(), 256, 256,
            128, Hq, Hkv, qkv.stride(0), qkv.stride(0), qkv.stride(0), out.stride(0), L["q_lo"].data_ptr(),
            L["q_hi"].data_ptr(), L["q_grp"].data_ptr(), L["k_code"].data_ptr(), L["f_ptr"].data_ptr(),
            L["f_idx"].data_ptr(), L["f_order"].data_ptr(), L["nqt"], 1.0 / D ** 0.5, two(staged), two(ready), counts,
            0, 2, 1, tiles[3:].data_ptr(), tiles.data_ptr(), 1, None), "attn_fwd_csbp")
        torch.cuda.synchronize()
        err = native.device_error()
        assert err["code"] == 1 and err["kernel"] == 6, err
    finally:
        lib.tdllm_clear_error()
        lib.tdllm_set_wait_timeout_ns(2_000_000_000)
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
    # the same call with the flag set completes and equals attention over the concatenated keys
    ready.fill_(1)
    staged.copy_(torch.randn_like(staged))
    tiles.zero_()
    native.check(lib.tdllm_attn_fwd_csbp(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), kv_rem.data_ptr(), out.data_ptr(), lse.data_ptr(), 256, 256,
        128, Hq, Hkv, qkv.stride(0), qkv.stride(0), qkv.stride(0), out.stride(0), L["q_lo"].data_ptr(),
        L["q_hi"].data_ptr(), L["q_grp"].data_ptr(), L["k_code"].data_ptr(), L["f_ptr"].data_ptr(),
        L["f_idx"].data_ptr(), L["f_order"].data_ptr(), L["nqt"], 1.0 / D ** 0.5, two(staged), two(ready), counts,
        0, 2, 1, tiles[3:].data_ptr(), tiles.data_ptr(), 1, None), "attn_fwd_csbp")
    torch.cuda.synchronize()
    native.raise_on_device_error()
    assert torch.equal(kv_rem, staged)
    from turbo_dllm_b200.ops.attention import attention_reference
    kall = torch.cat([k.reshape(256, Hkv, D), staged[:, : Hkv * D].reshape(128, Hkv, D)])
    vall = torch.cat([v.reshape(256, Hkv, D), staged[:, Hkv * D:].reshape(128, Hkv, D)])
    ref, ref_lse = attention_reference(q.reshape(256, Hq, D), kall, vall, mask)
    assert (out.view(256, Hq, D).float() - ref.float()).abs().max().item() < 2e-2
    assert (lse[:, :256] - ref_lse).abs().max().item() < 2e-2


@pytest.mark.distributed
def test_hybrid_csbp2_on_gpus_matches_single_gpu():
    """Gated DeltaNet layers under context sharding: row shards traded for head shards over NCCL
    (`parallel/head_sequence.py`), state-scan kernels on each rank's heads."""
    _need(2)
    args = ("collective", 2, "synthetic:tiny-qwen3_8-hd128", "fast_dllm_v2")
    ref = run_ranks(_csbp, 1, args=args, backend=None, deadline_s=300)[0]
    outs = run_ranks(_csbp, 2, args=args, backend="nccl", deadline_s=300)
    for losses, params in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert (torch.from_numpy(params) - torch.from_numpy(ref[1])).abs().max().item() < 3e-2


def _tp(rank, world, tp, steps, sp=False):
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel.runtime import build_parallel_runtime
    from turbo_dllm_b200.training.session import TrainingSession

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TDLLM_TP_FUSED_ALLREDUCE_MIN_K"] = "0"   # the tiny model's projections take the fused path too
    torch.cuda.set_device(rank)
    spec = RunSpec.from_mapping({
        "model": {"id": "synthetic:tiny-hd128", "seq_len": 512, "dtype": "bf16"},
        "objective": {"name": "fast_dllm_v2", "block_size": 32, "noise_schedule_epsilon": 0.1},
        "training": {"batch_size": 2, "steps": steps},
        "topology": {"context_parallel_size": 1, "block_parallel_size": 1, "tensor_parallel_size": tp,
                     "sequence_parallel": bool(sp)},
        "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate(world_size=world)
    rt = build_parallel_runtime(spec, device=f"cuda:{rank}", rank=rank, world_size=world) if world > 1 else None
    s = TrainingSession(spec, device=f"cuda:{rank}", runtime=rt)
    losses = []
    for _ in range(steps):
        r = s.step()
        losses.append(float(r.loss_sum) / r.denominator)
    if sp:   # the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels carried the projections
        assert any(isinstance(k, tuple) and k[0] == "sp" and v for k, v in s.model.tp._fused_ar.items())
    torch.cuda.synchronize()
    native.raise_on_device_error()
    return losses, s.optimizer.grad_norm(), s.model.flat.params["final_norm"].float().cpu()


@pytest.mark.distributed
def test_tp2_on_gpus_matches_single_gpu():
    _need(2)
    ref = run_ranks(_tp, 1, args=(1, 3), backend=None, deadline_s=300)[0]
    outs = run_ranks(_tp, 2, args=(2, 3), backend="nccl", deadline_s=300)
    for losses, norm, fnorm in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert norm == pytest.approx(ref[1], rel=5e-2)
        assert (torch.from_numpy(fnorm) - torch.from_numpy(ref[2])).abs().max().item() < 2e-2


@pytest.mark.distributed
def test_tp2_sequence_parallel_on_gpus_matches_single_gpu():
    _need(2)
    ref = run_ranks(_tp, 1, args=(1, 3), backend=None, deadline_s=300)[0]
    outs = run_ranks(_tp, 2, args=(2, 3, True), backend="nccl", deadline_s=300)
    for losses, norm, fnorm in outs:
        assert losses == pytest.approx(ref[0], rel=3e-2)
        assert norm == pytest.approx(ref[1], rel=5e-2)
        assert (torch.from_numpy(fnorm) - torch.from_numpy(ref[2])).abs().max().item() < 2e-2


def _fused_sequence_parallel_kernels(rank, world):
    """all-gather -> GEMM and GEMM -> reduce-scatter against fp32 references, several calls in a row (rotating
    gather buffers, both reduce-scatter workspaces, growing epochs)."""
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel.fused_sequence_parallel import FusedSequenceParallel

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    rows, H = 256 * world * 3, 192
    ws = FusedSequenceParallel(dist.group.WORLD, dev, rows, H)
    n = rows // world
    errs = []
    for call in range(8):
        g = torch.Generator(device="cpu").manual_seed(31 * call + 5)
        x_full = torch.randn(rows, H, generator=g).bfloat16()
        N = (520, 272)[call % 2]
        w = (torch.randn(N, H, generator=g) * 0.1).bfloat16()
        y, xg = ws.gather_matmul(x_full[rank * n:(rank + 1) * n].contiguous().to(dev), w.to(dev), swiglu=(call % 4 == 3))
        torch.cuda.synchronize()
        native.raise_on_device_error()
        assert torch.equal(xg.cpu(), x_full)
        ref = x_full.float() @ w.float().t()
        if call % 4 == 3:
            ref = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
        errs.append(((y.float().cpu() - ref).abs().max() / ref.abs().max()).item())
        # row-parallel product: every rank holds a K-slice, owners receive their rows of the sum
        K = (136, 72)[call % 2]
        a_full = torch.randn(rows, K * world, generator=g).bfloat16()
        wr = (torch.randn(H, K * world, generator=g) * 0.1).bfloat16()
        res = torch.randn(rows, H, generator=g).bfloat16()
        a = a_full[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        wk = wr[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        use_res = call % 2 == 0
        out = ws.matmul_scatter(a, wk, residual=res[rank * n:(rank + 1) * n].contiguous().to(dev) if use_res else None)
        torch.cuda.synchronize()
        native.raise_on_device_error()
        ref2 = (a_full.float() @ wr.float().t() + (res.float() if use_res else 0))[rank * n:(rank + 1) * n]
        errs.append(((out.float().cpu() - ref2).abs().max() / ref2.abs().max()).item())
    dist.barrier()
    ws.close()
    return errs


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4, 8])
def test_allgather_gemm_and_gemm_reduce_scatter_over_peer_memory(world):
    _need(world)
    for errs in run_ranks(_fused_sequence_parallel_kernels, world, backend="nccl", deadline_s=300):
        assert max(errs) < 2e-2, errs


def _fused_allreduce_gemm(rank, world):
    """Every rank holds a K-slice of x and w; the GEMM's epilogue must deliver the full sum everywhere."""
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel.fused_allreduce import FusedAllReduceGemm

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    ws = FusedAllReduceGemm(dist.group.WORLD, dev, max_rows=1000, n_cols=520)
    errs = []
    # several calls in a row (both workspaces, growing epochs), row counts that leave ragged and empty tiles
    for call, (M, K) in enumerate([(1000, 136), (384, 64), (1000, 320), (130, 72), (777, 136)]):
        g = torch.Generator(device="cpu").manual_seed(100 * call + 1)
        x_full = torch.randn(M, K * world, generator=g).bfloat16()
        w_full = (torch.randn(520, K * world, generator=g) * 0.1).bfloat16()
        res = torch.randn(M, 520, generator=g).bfloat16()
        x = x_full[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        w = w_full[:, rank * K:(rank + 1) * K].contiguous().to(dev)
        out = ws.matmul(x, w, residual=res.to(dev) if call % 2 == 0 else None)
        torch.cuda.synchronize()
        native.raise_on_device_error()
        ref = x_full.float() @ w_full.float().t() + (res.float() if call % 2 == 0 else 0)
        errs.append(((out.float().cpu() - ref).abs().max() / ref.abs().max()).item())
    dist.barrier()
    ws.close()
    return errs


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4, 8])
def test_gemm_with_allreduce_epilogue_over_peer_memory(world):
    _need(world)
    for errs in run_ranks(_fused_allreduce_gemm, world, backend="nccl", deadline_s=300):
        assert max(errs) < 2e-2, errs


def _ce_exchange(rank, world):
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.parallel.fused_allreduce import CrossEntropyExchange

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    ex = CrossEntropyExchange(dist.group.WORLD, dev, max_rows=5000)
    errs = []
    for call, (rows, nt) in enumerate([(5000, 7), (33, 1), (4097, 40), (1, 3)]):
        g = torch.Generator(device="cpu").manual_seed(7 * call + 3)
        stats = torch.randn(world, rows, nt, 3, generator=g)
        stats[..., 1] = stats[..., 1].abs() + 0.1          # sum exp > 0
        stats[:, 0, :, 0] = float("-inf")                  # a row whose shard tiles are all masked on every rank...
        stats[0, 0, 0, 0] = 0.5                            # ...but one tile of rank 0
        lse, tgt = ex.finish(stats[rank].contiguous().to(dev))
        torch.cuda.synchronize()
        native.raise_on_device_error()
        mx = stats[..., 0]
        ref_lse = torch.logsumexp((mx + torch.log(stats[..., 1])).permute(1, 0, 2).reshape(rows, -1), dim=1)
        ref_tgt = stats[..., 2].sum(dim=(0, 2))
        errs.append(max((lse.cpu() - ref_lse).abs().max().item(), (tgt.cpu() - ref_tgt).abs().max().item()))
    dist.barrier()
    ex.close()
    return errs


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4, 8])
def test_cross_entropy_statistics_exchange_over_peer_memory(world):
    _need(world)
    for errs in run_ranks(_ce_exchange, world, backend="nccl", deadline_s=300):
        assert max(errs) < 1e-3, errs


def _moe_ep(rank, world, peer):
    """One expert bank on bf16 GPUs: peer-memory dispatch / combine (or the all-to-all twin) against the dense
    oracle built from every rank's experts, forward and backward, two batches in a row."""
    import os

    import torch.distributed as dist

    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.models.config import PRESETS
    from turbo_dllm_b200.models.moe import MoEBlockDiffusionTransformer, reference_experts, route_topk

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TDLLM_EP_PEER"] = "1" if peer else "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    cfg = PRESETS["synthetic:tiny-moe-hd128"]
    m = MoEBlockDiffusionTransformer(cfg, ep_group=dist.group.WORLD, dtype=torch.bfloat16, device=dev, seed=3,
                                     init_std=0.05)
    bank = m.layers[0].experts
    errs, outs = [], []
    for call in range(2):
        torch.manual_seed(100 + rank + 10 * call)
        x = (torch.randn(700 + 64 * rank, cfg.hidden_size, device=dev) * 0.5).bfloat16().requires_grad_(True)
        go = torch.randn(x.shape, device=dev).bfloat16()
        m.flat_experts.zero_grad()
        m.flat.zero_grad()
        y = bank(x)
        y.backward(go)
        torch.cuda.synchronize()
        native.raise_on_device_error()
        assert (m.expert_exchange.get("exchange") is not None) == bool(peer)
        gu = [torch.empty_like(bank.w_gu) for _ in range(world)]
        dn = [torch.empty_like(bank.w_down) for _ in range(world)]
        dist.all_gather(gu, bank.w_gu.detach().contiguous())
        dist.all_gather(dn, bank.w_down.detach().contiguous())
        xr = x.detach().float().requires_grad_()
        w, idx = route_topk(xr @ bank.router.float().t(), cfg.num_experts_per_token)
        ref = reference_experts(xr, torch.cat(gu).float(), torch.cat(dn).float(), w, idx)
        ref.backward(go.float())
        # against the oracle on average (bf16 router logits can flip a near-tie of the top-k against the fp32
        # oracle, which changes single rows completely): mean error; exact agreement is checked between the two
        # transports, which share the routing
        e_fwd = ((y.float() - ref).abs().mean() / ref.abs().mean()).item()
        e_bwd = ((x.grad.float() - xr.grad).abs().mean() / xr.grad.abs().mean()).item()
        errs += [e_fwd, e_bwd]
        outs += [y.float().cpu(), x.grad.float().cpu(), bank.w_down.main_grad.float().cpu().clone(),
                 bank.router.main_grad.float().cpu().clone()]
    dist.barrier()
    ex = m.expert_exchange.get("exchange")
    if ex is not None:
        ex.close()
    return errs, outs


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_dispatch_and_combine_over_peer_memory(world):
    _need(world)
    a = run_ranks(_moe_ep, world, args=(True,), backend="nccl", deadline_s=300)
    b = run_ranks(_moe_ep, world, args=(False,), backend="nccl", deadline_s=300)
    for (ea, oa), (eb, ob) in zip(a, b):
        assert max(eb) < 5e-2, eb
        assert max(ea) < 5e-2, ea
        for ta, tb in zip(oa, ob):      # outputs, input gradients, expert and router weight gradients
            ta, tb = torch.from_numpy(ta), torch.from_numpy(tb)
            assert (ta - tb).abs().max().item() <= 3e-2 * max(tb.abs().max().item(), 1e-3)
