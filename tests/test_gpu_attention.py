"""tcgen05 block-diffusion attention vs the dense-mask fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(layout, nq, nk, Hq, Hkv, seed=0, self_attn=True):
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops.attention import attention_forward_native, attention_reference

    torch.manual_seed(seed)
    D = 128
    qkv = torch.randn(max(nq, nk), (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    q = qkv[:nq, : Hq * D].view(nq, Hq, D)
    k = qkv[:nk, Hq * D:(Hq + Hkv) * D].view(nk, Hkv, D)
    v = qkv[:nk, (Hq + Hkv) * D:].view(nk, Hkv, D)
    scale = 1.0 / math.sqrt(D)
    out, lse = attention_forward_native(q, k, v, layout, scale)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    ref, ref_lse = attention_reference(q.float(), k.float(), v.float(), layout, scale)
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err
    fin = torch.isfinite(ref_lse)
    got = lse[:, :nq]
    assert torch.equal(torch.isfinite(got), fin)
    assert (got[fin] - ref_lse[fin]).abs().max().item() < 2e-2
    return out, lse


@pytest.mark.parametrize("L,bs,views", [(256, 32, 1), (512, 64, 1), (640, 32, 2), (1024, 32, 1)])
@pytest.mark.parametrize("Hq,Hkv", [(2, 1), (4, 2), (8, 2)])
def test_block_diffusion_full_sequence(L, bs, views, Hq, Hkv):
    from turbo_dllm_b200.ops.attention import single_sequence_layout

    layout = single_sequence_layout(L, bs, "cuda", views)
    n = (views + 1) * L
    _run(layout, n, n, Hq, Hkv)


@pytest.mark.parametrize("Hq,Hkv", [(2, 2), (3, 1), (6, 2)])
def test_odd_number_of_query_heads_per_kv_head(Hq, Hkv, monkeypatch):
    """Group sizes 1 and 3: the last CTA of a group runs its single head in both pipelines; the one-pass
    backward takes any group size."""
    from turbo_dllm_b200.ops.attention import single_sequence_layout

    monkeypatch.setenv("TDLLM_ATTN_BWD", "fused")
    layout = single_sequence_layout(384, 32, "cuda", 1)
    _run(layout, 768, 768, Hq, Hkv)
    _run_bwd(layout, 768, 768, Hq, Hkv)


def test_ragged_rows_and_sparse_keys():
    """Row counts that are not multiples of 128, keys that are a strided subset (a CP shard),
    and query rows that see no key at all."""
    from turbo_dllm_b200.ops.attention import block_diffusion_layout

    dev = "cuda"
    L, bs = 600, 24
    pos = torch.arange(L, device=dev)
    act = pos[(pos // bs) % 3 == 1]                 # some noisy blocks only
    kpos = pos[(pos // 50) % 2 == 1]                # clean keys owned by "this rank"
    layout = block_diffusion_layout(act, act // bs, pos[:333], bs, key_clean_pos=kpos)
    nq = act.numel() + 333
    nk = act.numel() + kpos.numel()
    _run(layout, nq, nk, 4, 2)


def test_two_sequences_and_window():
    from turbo_dllm_b200.ops.attention import block_diffusion_layout

    dev = "cuda"
    L, bs = 384, 32
    pos = torch.arange(L, device=dev).repeat(2)
    seq = torch.arange(2, device=dev).repeat_interleave(L)
    grp = pos // bs + seq * (L // bs)
    layout = block_diffusion_layout(pos, grp, pos, bs, noisy_seq=seq, clean_seq=seq, window=96)
    _run(layout, 4 * L, 4 * L, 4, 2)


def _run_bwd(layout, nq, nk, Hq, Hkv, seed=0):
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops.attention import attention_reference, block_attention

    torch.manual_seed(seed)
    D = 128
    q = torch.randn(nq, Hq, D, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(nk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(nk, Hkv, D, device="cuda").bfloat16().requires_grad_()
    scale = 1.0 / math.sqrt(D)
    out = block_attention(q, k, v, layout, scale)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref, _ = attention_reference(qr, kr, vr, layout, scale)
    ref.backward(g.float())
    for name, a, b in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (a.float() - b).abs().max().item()
        scale_ = b.abs().max().item()
        assert err <= 5e-2 * max(scale_, 1.0), (name, err, scale_)


@pytest.mark.parametrize("mode", ["fused", "split"])
@pytest.mark.parametrize("L,bs,views", [(256, 32, 1), (640, 32, 2), (1024, 64, 1)])
@pytest.mark.parametrize("Hq,Hkv", [(2, 1), (8, 2)])
def test_backward_full_sequence(L, bs, views, Hq, Hkv, mode, monkeypatch):
    from turbo_dllm_b200.ops.attention import single_sequence_layout

    monkeypatch.setenv("TDLLM_ATTN_BWD", mode)
    layout = single_sequence_layout(L, bs, "cuda", views)
    n = (views + 1) * L
    _run_bwd(layout, n, n, Hq, Hkv)


def test_backward_one_pass_long_walk(monkeypatch):
    """Enough (query head, query tile) pairs per key tile that every barrier of the one-pass kernel
    wraps its phase many times."""
    from turbo_dllm_b200.ops.attention import single_sequence_layout

    monkeypatch.setenv("TDLLM_ATTN_BWD", "fused")
    layout = single_sequence_layout(1536, 32, "cuda", 2)
    _run_bwd(layout, 3 * 1536, 3 * 1536, 4, 1)


@pytest.mark.parametrize("mode", ["fused", "split"])
def test_backward_ragged_sparse_keys(mode, monkeypatch):
    from turbo_dllm_b200.ops.attention import block_diffusion_layout

    monkeypatch.setenv("TDLLM_ATTN_BWD", mode)
    dev = "cuda"
    L, bs = 600, 24
    pos = torch.arange(L, device=dev)
    act = pos[(pos // bs) % 3 == 1]
    kpos = pos[(pos // 50) % 2 == 1]
    layout = block_diffusion_layout(act, act // bs, pos[:333], bs, key_clean_pos=kpos)
    _run_bwd(layout, act.numel() + 333, act.numel() + kpos.numel(), 4, 2)


@pytest.mark.parametrize("D,Hq,Hkv", [(256, 4, 2), (512, 2, 1), (64, 4, 2), (256, 3, 1)])
def test_wide_and_narrow_heads_run_as_products_around_the_softmax_kernel(D, Hq, Hkv):
    """head_dim 256 / 512 (and 64): tcgen05 products around the masked-softmax kernels, forward and backward,
    against the dense fp32 reference: ragged row count, two noisy views, rows without any visible key."""
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.ops.attention import attention_reference, block_attention, single_sequence_layout
    from turbo_dllm_b200.ops.wide_attention import wide_attention_forward

    torch.manual_seed(D)
    layout = single_sequence_layout(320, 32, "cuda", 2)            # 960 rows: 7.5 tiles
    n = 960
    q = (torch.randn(n, Hq, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    k = (torch.randn(n, Hkv, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    v = (torch.randn(n, Hkv, D, device="cuda") * 0.5).bfloat16().requires_grad_()
    scale = 1.0 / math.sqrt(D)
    out = block_attention(q, k, v, layout, scale)
    go = torch.randn_like(out)
    out.backward(go)
    torch.cuda.synchronize()
    native.raise_on_device_error()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref, ref_lse = attention_reference(qr, kr, vr, layout, scale)
    ref.backward(go.float())
    assert (out.float() - ref).abs().max().item() < 3e-2
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert (got.float() - want).abs().max().item() < 4e-2 * max(want.abs().max().item(), 1.0)
    _, lse = wide_attention_forward(q.detach(), k.detach(), v.detach(), layout, scale)
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), fin)
    assert (lse[fin] - ref_lse[fin]).abs().max().item() < 2e-2


def test_model_with_head_dim_256_trains_on_the_gpu():
    from turbo_dllm_b200.config.run_spec import RunSpec
    from turbo_dllm_b200.kernels import native
    from turbo_dllm_b200.training.session import TrainingSession

    def spec(dtype):
        return RunSpec.from_mapping({
            "model": {"id": "wide", "random_init": True, "seq_len": 512, "dtype": dtype, "vocab_size": 2048,
                      "hidden_size": 512, "num_layers": 2, "num_attention_heads": 2, "num_key_value_heads": 1,
                      "head_dim": 256, "intermediate_size": 1024, "sliding_window": 128, "sliding_window_pattern": 2},
            "objective": {"name": "standard_block_diffusion", "block_size": 32, "sampling_epsilon_min": 0.1},
            "training": {"batch_size": 2, "steps": 2},
            "topology": {"context_parallel_size": 1, "block_parallel_size": 1},
            "optimizer": {"lr": 1e-3, "gradient_clip_norm": 1.0}}).validate()

    g = TrainingSession(spec("bf16"), device="cuda")
    c = TrainingSession(spec("fp32"), device="cpu")
    c.model.flat.data.copy_(g.model.flat.data.float().cpu())
    rg, rc = g.step(), c.step()
    torch.cuda.synchronize()
    native.raise_on_device_error()
    lg, lc = float(rg.loss_sum) / rg.denominator, float(rc.loss_sum) / rc.denominator
    assert lg == pytest.approx(lc, rel=3e-2)
