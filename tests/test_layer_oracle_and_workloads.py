"""CPU checks of the pieces the full-size parity tests and the benchmark rest on: the layer
oracle on sampled rows, the dense-then-mask cost model, the seeded workload generators and
their tensor-parallel slicing, and the strided-view helper of the attention shims."""

import pytest
import torch

from oracle import dpk_oracle as O


def _small_layer(seed=0, T=96, H=64, Hq=4, Hk=2, D=16, I=256):
    g = torch.Generator().manual_seed(seed)
    w = {n: torch.randn(*s, generator=g) * 0.1 for n, s in dict(
        wq=(Hq * D, H), wk=(Hk * D, H), wv=(Hk * D, H), wo=(H, Hq * D),
        wg=(I, H), wu=(I, H), wd=(H, I)).items()}
    x = torch.randn(1, T, H, generator=g)
    am = torch.rand(1, T, 2, generator=g) > 0.3
    fm = torch.rand(1, T, 4, generator=g) > 0.5
    return w, x, am, fm, dict(num_q_heads=Hq, num_kv_heads=Hk, head_dim=D)


def test_layer_oracle_on_sampled_rows_equals_the_operator_chain():
    w, x, am, fm, kw = _small_layer()
    T, Hq, Hk, D = x.shape[1], kw["num_q_heads"], kw["num_kv_heads"], kw["head_dim"]
    q = O.gemm_mn(x, w["wq"], am).view(1, T, Hq, D)
    k = (x[0] @ w["wk"].T).view(1, T, Hk, D)
    v = (x[0] @ w["wv"].T).view(1, T, Hk, D)
    a = O.attention_prefill(q, k, v, am).view(1, T, Hq * D)
    x1 = x + O.gemm_k(a, w["wo"], am)
    want = x1 + O.ffn_swiglu(x1, w["wg"], w["wu"], w["wd"], fm)
    full = O.decoder_layer_rows(x, torch.arange(T), w, am, fm, **kw)
    torch.testing.assert_close(full, want, atol=1e-5, rtol=1e-5)
    rows = torch.tensor([0, 3, 17, 50, 95])
    part, x1_part = O.decoder_layer_rows(x, rows, w, am[:, rows], fm[:, rows], return_x1=True, **kw)
    torch.testing.assert_close(part, want[:, rows], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(x1_part, x1[:, rows], atol=1e-5, rtol=1e-5)
    # the cost model of the reference's CPU path computes the same numbers
    dm = O.dense_then_mask_layer_rows(x, rows, w, k, v, am[:, rows], fm[:, rows], **kw)
    torch.testing.assert_close(dm, want[:, rows], atol=1e-5, rtol=1e-5)


def test_layer_oracle_with_norms_rotary_and_bf16_handoffs():
    w, x, am, fm, kw = _small_layer(seed=3, T=64)
    T, D = x.shape[1], kw["head_dim"]
    g = torch.Generator().manual_seed(9)
    n1 = 1.0 + 0.1 * torch.randn(x.shape[-1], generator=g)
    n2 = 1.0 + 0.1 * torch.randn(x.shape[-1], generator=g)
    ang = torch.arange(T).float()[:, None] / (10000.0 ** (torch.arange(0, D, 2).float() / D))[None, :]
    cos, sin = torch.cat([ang, ang], -1).cos(), torch.cat([ang, ang], -1).sin()
    rows = torch.arange(0, T, 3)
    ref = O.decoder_layer_rows(x, rows, w, am[:, rows], fm[:, rows], norm1=n1, norm2=n2, cos=cos, sin=sin, **kw)
    allr = O.decoder_layer_rows(x, torch.arange(T), w, am, fm, norm1=n1, norm2=n2, cos=cos, sin=sin, **kw)
    torch.testing.assert_close(ref, allr[:, rows], atol=1e-5, rtol=1e-5)
    # bf16 hand-offs move the result by rounding noise only
    h = O.decoder_layer_rows(x.to(torch.bfloat16).float(), rows, w, am[:, rows], fm[:, rows], norm1=n1,
                             norm2=n2, cos=cos, sin=sin, handoff=torch.bfloat16, **kw)
    assert 0 < O.rel_err(h, ref) < 5e-2


def test_attention_with_query_positions():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(1, 40, h, 8, generator=g) for h in (4, 2, 2))
    mask = torch.rand(1, 40, 2, generator=g) > 0.4
    full = O.attention(q, k, v, mask, is_causal=True)
    rows = torch.tensor([1, 7, 8, 39])
    part = O.attention(q[:, rows], k, v, mask[:, rows], is_causal=True, q_positions=rows)
    torch.testing.assert_close(part, full[:, rows], atol=1e-6, rtol=1e-6)
    with pytest.raises(ValueError):
        O.attention(q[:, rows], k, v, mask[:, rows], is_causal=True, q_positions=rows[:2])


def test_workload_slices_tile_the_full_matrices():
    from dpk_b200 import workloads as W

    shape = W.LayerShape(tokens=32, hidden=64, inter=1024, q_heads=8, kv_heads=4, head_dim=16,
                         attn_groups=4, attn_keep=3, ffn_groups=8, ffn_keep=4, router_rank=4)
    dev = torch.device("cpu")
    _, host = W.layer_weights(dev, shape, keep_host_fp32=True)
    world = 4
    parts = [W.layer_weights(dev, shape, world, r) for r in range(world)]
    for name in W.WEIGHT_NAMES:
        dim = 1 if name in ("wo", "wd") else 0
        whole = torch.cat([p[name] for p in parts], dim=dim).float()
        assert torch.equal(whole, host[name]), name
    (ga, gf) = shape.shard(world, 2)
    assert ga == (2, 3) and gf == (4, 6)
    fe = W.layer_front_end(dev, shape)
    assert fe["cos"].shape == (32, 16) and fe["attn_router"][2].shape == (8, 4)
    # same seed, same tensors
    assert torch.equal(W.layer_input(dev, shape), W.layer_input(dev, shape))


def test_bench_config_is_the_same_in_both_arms():
    import argparse

    import bench
    from dpk_b200 import workloads as W

    args = argparse.Namespace(sum="fused", halves=2)
    shape = W.LayerShape()
    assert bench.make_config(shape, 8, args) == bench.make_config(W.LayerShape(tokens=16384), 8, args)
    assert "tp8" in bench.make_config(shape, 8, args)["parallelism"]
    assert bench.make_config(shape, 1, args)["parallelism"] == "single GPU"
    assert bench.quantiles([3.0, 1.0, 2.0, 5.0, 4.0]) == (3.0, 2.0, 5.0)
    assert bench.recorded_traffic(shape, 1) and bench.recorded_traffic(shape, 2) is None


def test_heads_view_reads_strided_tensors_in_place():
    from dpk_b200.ops import _heads_view

    fused = torch.zeros(2, 10, 48, dtype=torch.bfloat16)
    q = fused[..., :32].view(2, 10, 4, 8)
    t, ts, bs = _heads_view(q)
    assert t.data_ptr() == q.data_ptr() and (ts, bs) == (48, 480)
    cache = torch.zeros(3, 64, 2, 8, dtype=torch.bfloat16)
    t, ts, bs = _heads_view(cache[:, :20])
    assert t.data_ptr() == cache.data_ptr() and (ts, bs) == (16, 64 * 16)
    # heads not back to back: copied
    tr = torch.zeros(1, 4, 10, 8, dtype=torch.bfloat16).transpose(1, 2)
    t, ts, bs = _heads_view(tr)
    assert t.is_contiguous() and (ts, bs) == (32, 320)
    # one token per sequence: the token stride is never used
    t, ts, bs = _heads_view(cache[:, 5:6])
    assert ts == 16 and bs == 64 * 16
