"""The CPU oracle against fixtures produced by the reference itself (CPU only)."""

import numpy as np
import pytest
import torch

import golden_io
from oracle import dpk_oracle as O
from oracle import route_oracle as RO

TIGHT = dict(atol=2e-5, rtol=2e-5)


def test_reference_known_answer_cases():
    z = golden_io.load("ref_known_answers")
    torch.testing.assert_close(O.gemm_mn(z["x"], z["out_w"], z["mask"]), z["gemm_mn"], **TIGHT)
    torch.testing.assert_close(O.gemm_k(z["inter"], z["down_w"], z["mask"]), z["gemm_k"], **TIGHT)
    torch.testing.assert_close(O.gemm_mn(z["x"], z["out_w"], z["tok_mask"]), z["gemm_mn_token"],
                               **TIGHT)
    out = O.attention_decode(z["q"], z["k"], z["v"], torch.ones(1, 1, 2, dtype=torch.bool),
                             leftpad=z["leftpad"])
    torch.testing.assert_close(out, z["decode_leftpad"], **TIGHT)


def test_ffn_small():
    z = golden_io.load("ffn_small")
    m = z["mask"]
    torch.testing.assert_close(O.gemm_mn(z["x"], z["wg"], m, "silu"), z["gate"], **TIGHT)
    torch.testing.assert_close(O.gemm_mn(z["x"], z["wu"], m), z["up"], **TIGHT)
    torch.testing.assert_close(O.gemm_mn(z["x"], z["wu"], m, "relu"), z["relu"], **TIGHT)
    torch.testing.assert_close(O.gemm_k(z["hmid"], z["wd"], m), z["down"], **TIGHT)
    torch.testing.assert_close(O.gemm_k(z["dense_a"], z["wd"], m), z["down_dense_a"], **TIGHT)
    torch.testing.assert_close(
        O.ffn_swiglu(z["x"], z["wg"], z["wu"], z["wd"], m, round_intermediate=torch.bfloat16),
        z["down"], **TIGHT)
    torch.testing.assert_close(O.dense_then_mask_ffn(z["x"], z["wg"], z["wu"], z["wd"], m),
                               O.ffn_swiglu(z["x"], z["wg"], z["wu"], z["wd"], m),
                               atol=1e-4, rtol=1e-4)
    # the top-k router reproduces the mask the fixture was built with
    assert torch.equal(O.topk_route_mask(z["logits"], 2), m)


def test_routing_layout_python_and_c():
    z = golden_io.load("routing")
    smask, sidx, counts = O.route_compact(z["mask"])
    assert torch.equal(smask, z["sorted_mask"])
    assert torch.equal(sidx, z["sorted_indices"])
    assert torch.equal(counts, z["counts"])
    cs, ci, cc = RO.route_compact(z["mask"].numpy())
    assert np.array_equal(cs, z["sorted_mask"].numpy())
    assert np.array_equal(ci, z["sorted_indices"].numpy())
    assert np.array_equal(cc, z["counts"].numpy())
    # top-k: same active set as torch.topk
    want = torch.zeros_like(z["mask"])
    want.scatter_(-1, z["topk5"], True)
    assert torch.equal(O.topk_route_mask(z["logits"], 5), want)
    assert np.array_equal(RO.topk_mask(z["logits"].numpy(), 5), want.numpy())


def test_row_bits_c():
    z = golden_io.load("routing")
    m = z["mask"].numpy()
    rb, wb = RO.row_bits(m, 128)
    M, NG = m.shape
    for r in (0, 1, 127, 128, 332):
        for g in range(NG):
            assert ((rb[r, g // 32] >> (g % 32)) & 1) == int(m[r, g])
    for w in range((M + 127) // 128):
        want = np.bitwise_or.reduce(rb[w * 128:(w + 1) * 128], axis=0)
        assert np.array_equal(wb[w], want)


def test_prefill_attention():
    z = golden_io.load("attn_prefill_small")
    q, k, v = z["q"], z["k"], z["v"]
    torch.testing.assert_close(O.attention_prefill(q, k, v, z["mask2"]), z["causal_ng2"], **TIGHT)
    torch.testing.assert_close(O.attention_prefill(q, k, v, z["mask8"]), z["causal_ng8"], **TIGHT)
    torch.testing.assert_close(O.attention_prefill(q, k, v, z["mask2"], is_causal=False),
                               z["full_ng2"], **TIGHT)
    torch.testing.assert_close(
        O.attention_prefill(q, k, v, z["mask2"], leftpad=z["leftpad"]), z["causal_ng2_leftpad"],
        equal_nan=True, **TIGHT)
    z = golden_io.load("attn_prefill_d128")
    torch.testing.assert_close(O.attention_prefill(z["q"], z["k"], z["v"], z["mask2"]),
                               z["causal_ng2"], **TIGHT)


def test_decode_attention():
    z = golden_io.load("attn_decode_small")
    q, k, v = z["q"], z["k"], z["v"]
    torch.testing.assert_close(O.attention_decode(q, k, v, z["mask8"]), z["out_ng8"], **TIGHT)
    torch.testing.assert_close(O.attention_decode(q, k, v, z["mask16"], leftpad=z["leftpad"]),
                               z["out_ng16_leftpad"], **TIGHT)


def test_bottleneck_router_and_rms_norm():
    """Against the reference's own TokenRouter (fp32 and bf16 module) and LlamaRMSNorm."""
    z = golden_io.load("router_norm")
    x = z["x"]
    args = (z["w_down"], z["b_down"], z["w_route"], z["b_route"])
    logits, execute = O.bottleneck_router(x, *args)
    torch.testing.assert_close(logits, z["logits_fp32"], rtol=1e-5, atol=1e-5)
    # decisions: identical wherever the pair is not within fp32 rounding of a tie
    margin = (z["logits_fp32"][..., 0] - z["logits_fp32"][..., 1]).abs()
    clear = margin > 1e-5
    assert clear.float().mean() > 0.99
    assert torch.equal(execute[clear], z["execute_fp32"][clear])
    # module in bf16: each Linear's output is rounded once
    logits16, execute16 = O.bottleneck_router(x, *args, module_dtype=torch.bfloat16)
    l16 = z["logits_bf16"]
    # the hidden 16-vector sits on bf16 rounding boundaries now and then: one ulp of it moves a
    # logit by a few bf16 ulps, so compare with that slack and the decisions where clear
    torch.testing.assert_close(logits16, l16, rtol=2e-2, atol=2e-2)
    assert (logits16 == l16).float().mean() > 0.95
    clear16 = (l16[..., 0] - l16[..., 1]).abs() > 4e-2
    assert torch.equal(execute16[clear16], z["execute_bf16"][clear16])
    assert (execute16 == z["execute_bf16"]).float().mean() > 0.98
    # ties go to "execute" (argmax returns the first index)
    tie = torch.zeros(1, 1, 16)
    _, ex = O.bottleneck_router(tie, torch.zeros(16, 16), None, torch.zeros(4, 16), None)
    assert ex.all()
    # RMSNorm in bf16
    xn = O.rms_norm(x.to(torch.bfloat16), z["gamma"], float(z["eps"]))
    assert xn.dtype == torch.bfloat16
    assert torch.equal(xn.float(), z["xn_bf16"])


def test_rope_and_cache_append():
    """Against the reference's apply_rotary_pos_emb and its sequence-first cache layer."""
    z = golden_io.load("rope_cache")
    T0 = z["q0"].shape[1]
    cos, sin = z["cos"][None], z["sin"][None]
    torch.testing.assert_close(O.rope(z["q0"], cos[:, :T0], sin[:, :T0]), z["q0_rot"], rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(O.rope(z["q1"], cos[:, T0:], sin[:, T0:]), z["q1_rot"], rtol=1e-6, atol=1e-6)
    B, _, Hk, D = z["k0"].shape
    kc, vc = torch.zeros(B, 64, Hk, D), torch.zeros(B, 64, Hk, D)
    keys, _ = O.kv_append(kc, vc, 0, O.rope(z["k0"], cos[:, :T0], sin[:, :T0]), z["v0"])
    torch.testing.assert_close(keys, z["keys_after_prefill"], rtol=1e-6, atol=1e-6)
    keys, values = O.kv_append(kc, vc, T0, O.rope(z["k1"], cos[:, T0:], sin[:, T0:]), z["v1"])
    torch.testing.assert_close(keys, z["keys_after_step"], rtol=1e-6, atol=1e-6)
    assert torch.equal(values, z["values_after_step"])
    with pytest.raises(ValueError):
        O.kv_append(kc, vc, 60, z["k1"], z["v1"])
