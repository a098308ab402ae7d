"""Generate the golden fixtures in this folder from the reference itself.

Run once in a container that has the reference checked out (it is not needed
afterwards; the ``.npz`` files are committed):

    python tests/golden/make_golden.py /path/to/reference

The script imports the reference's own operator API
(``DynamicPruningKernels/python`` exposed under its package name
``dynamic_width_jit``) and records, for seeded inputs, what
``run_kernel(family, ..., backend="torch")`` returns.  It also records the
reference's hand-written known-answer cases
(``DynamicPruningKernels/tests/test_references.py:11-84``) and the routing
layout ``torch.sort(mask, dim=0, descending=True, stable=True)`` that the
reference's hosts build (``python/gemm_mn/jit.py:410-415``).

All floating-point inputs are rounded to bf16 before use, so that the GPU tests
can feed bit-identical inputs to the bf16 kernels.
"""

from __future__ import annotations

import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(root: str):
    shim = tempfile.mkdtemp(prefix="dpk_ref_")
    os.symlink(os.path.join(root, "DynamicPruningKernels", "python"),
               os.path.join(shim, "dynamic_width_jit"))
    sys.path.insert(0, shim)
    import dynamic_width_jit  # noqa: F401
    return dynamic_width_jit


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def randn(gen, *shape, std=1.0):
    return bf16_round(torch.randn(*shape, generator=gen) * std)


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.numpy()
        v = np.asarray(v)
        if v.dtype == np.float32:
            # values that are exactly bf16 are stored as their 16 upper bits under
            # the key "bf16:<name>" (tests/golden_io.py undoes this)
            bits = np.ascontiguousarray(v).view(np.uint32)
            if not np.any(bits & 0xFFFF):
                out["bf16:" + k] = (bits >> 16).astype(np.uint16)
                continue
        out[k] = v
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: tuple(np.shape(v)) for k, v in out.items()})


def main(root: str) -> None:
    ref = _import_reference(root)
    run = ref.run_kernel

    # ---- the reference's own known-answer cases (seed 7) --------------------
    torch.manual_seed(7)
    x = torch.randn(2, 3, 8)
    out_w = torch.randn(12, 8)
    down_w = torch.randn(5, 12)
    mask = torch.tensor([[[True, False, True], [False, True, True], [True, True, False]],
                         [[False, False, True], [True, False, False], [True, True, True]]])
    inter = x @ out_w.T
    tok_mask = torch.tensor([[True, False, True], [False, True, False]])
    q = torch.randn(1, 1, 4, 8)
    k = torch.randn(1, 4, 2, 8)
    v = torch.randn(1, 4, 2, 8)
    save("ref_known_answers",
         x=x, out_w=out_w, down_w=down_w, mask=mask, inter=inter, tok_mask=tok_mask,
         gemm_mn=run("gemm_mn", x, out_w, mask, backend="torch"),
         gemm_k=run("gemm_k", inter, down_w, mask, backend="torch"),
         gemm_mn_token=run("gemm_mn", x, out_w, tok_mask, backend="torch"),
         q=q, k=k, v=v, leftpad=np.array([2], dtype=np.uint32),
         decode_leftpad=run("attention_decode", q, k, v, torch.ones(1, 1, 2, dtype=torch.bool),
                            backend="torch", Leftpad=torch.tensor([2], dtype=torch.uint32),
                            is_causal=False))

    # ---- routed GEMMs and the composed FFN (seed 17) -------------------------
    g = torch.Generator().manual_seed(17)
    B, T, H, I, NG = 2, 75, 128, 512, 4
    x = randn(g, B, T, H)
    wg = randn(g, I, H, std=0.02 * 8)
    wu = randn(g, I, H, std=0.02 * 8)
    wd = randn(g, H, I, std=0.02 * 8)
    logits = torch.randn(B, T, NG, generator=g)
    mask = torch.zeros(B, T, NG, dtype=torch.bool)
    mask.scatter_(-1, torch.topk(logits, 2, dim=-1).indices, True)
    gate = run("gemm_mn", x, wg, mask, backend="torch", activation="silu")
    up = run("gemm_mn", x, wu, mask, backend="torch")
    relu = run("gemm_mn", x, wu, mask, backend="torch", activation="relu")
    hmid = bf16_round(gate * up)
    down = run("gemm_k", hmid, wd, mask, backend="torch")
    dense_a = randn(g, B, T, I)
    down_dense_a = run("gemm_k", dense_a, wd, mask, backend="torch")
    save("ffn_small", x=x, wg=wg, wu=wu, wd=wd, logits=logits, mask=mask, gate=gate, up=up,
         relu=relu, hmid=hmid, down=down, dense_a=dense_a, down_dense_a=down_dense_a)

    # ---- routing layout ------------------------------------------------------
    g = torch.Generator().manual_seed(18)
    M, NG = 333, 12
    logits = torch.randn(M, NG, generator=g)
    mask = torch.zeros(M, NG, dtype=torch.bool)
    mask.scatter_(-1, torch.topk(logits, 5, dim=-1).indices, True)
    mask[:, 3] = False       # an empty group
    mask[:, 7] = True        # a full group
    smask, sidx = torch.sort(mask, dim=0, descending=True, stable=True)
    save("routing", logits=logits, topk5=torch.topk(logits, 5, dim=-1).indices, mask=mask,
         sorted_mask=smask, sorted_indices=sidx, counts=mask.sum(0).to(torch.int32))

    # ---- prefill attention ---------------------------------------------------
    g = torch.Generator().manual_seed(19)
    B, T, Hq, Hk, D = 2, 83, 8, 2, 64
    q = randn(g, B, T, Hq, D)
    k = randn(g, B, T, Hk, D)
    v = randn(g, B, T, Hk, D)
    m2 = torch.rand(B, T, 2, generator=g) > 0.5
    m8 = torch.rand(B, T, 8, generator=g) > 0.4
    save("attn_prefill_small", q=q, k=k, v=v, mask2=m2, mask8=m8,
         causal_ng2=run("attention_prefill", q, k, v, m2, backend="torch", is_causal=True),
         causal_ng8=run("attention_prefill", q, k, v, m8, backend="torch", is_causal=True),
         full_ng2=run("attention_prefill", q, k, v, m2, backend="torch", is_causal=False),
         leftpad=np.array([5, 0], dtype=np.uint32),
         causal_ng2_leftpad=run("attention_prefill", q, k, v, m2, backend="torch", is_causal=True,
                                Leftpad=torch.tensor([5, 0], dtype=torch.uint32)))

    # D = 128, GQA 4:1 like the benchmark layouts
    B, T, Hq, Hk, D = 1, 150, 8, 2, 128
    q = randn(g, B, T, Hq, D)
    k = randn(g, B, T, Hk, D)
    v = randn(g, B, T, Hk, D)
    m2 = torch.rand(B, T, 2, generator=g) > 0.5
    save("attn_prefill_d128", q=q, k=k, v=v, mask2=m2,
         causal_ng2=run("attention_prefill", q, k, v, m2, backend="torch", is_causal=True))

    # ---- decode attention ----------------------------------------------------
    g = torch.Generator().manual_seed(20)
    B, Tk, Hq, Hk, D = 3, 139, 16, 8, 128
    q = randn(g, B, 1, Hq, D)
    k = randn(g, B, Tk, Hk, D)
    v = randn(g, B, Tk, Hk, D)
    m8 = torch.rand(B, 1, 8, generator=g) > 0.5
    m16 = (torch.arange(16) % 3 != 1).reshape(1, 1, 16).expand(B, 1, 16).contiguous()
    lp = torch.tensor([3, 0, 17], dtype=torch.uint32)
    save("attn_decode_small", q=q, k=k, v=v, mask8=m8, mask16=m16, leftpad=lp.numpy(),
         out_ng8=run("attention_decode", q, k, v, m8, backend="torch", is_causal=False),
         out_ng16_leftpad=run("attention_decode", q, k, v, m16, backend="torch",
                              Leftpad=lp, is_causal=False))

    router_fixture(root)


def router_fixture(root: str) -> None:
    """The reference's ``TokenRouter`` (``WIDE/wrapper/base_layer.py:89-114``) with its
    evaluation-time decision (``:204-207``) and the ``LlamaRMSNorm`` its layers wrap.
    ``base_layer`` imports two optional packages that this container lacks (peft, liger
    kernels) for classes the router does not use; they are stubbed for the import."""
    from unittest import mock
    for name in ("peft", "peft.tuners", "peft.tuners.lora", "liger_kernel", "liger_kernel.ops",
                 "liger_kernel.ops.swiglu"):
        sys.modules.setdefault(name, mock.MagicMock())
    sys.path.insert(0, os.path.join(root, "WIDE"))
    from wrapper.base_layer import TokenRouter
    from transformers.models.llama.modeling_llama import LlamaRMSNorm

    torch.manual_seed(23)
    B, T, H, NG, R = 2, 45, 256, 12, 16
    router = TokenRouter(H, group_num=NG, rank_size=R).eval()
    with torch.no_grad():
        for lin in (router.compressor, router.router):      # bf16-exact weights, non-zero biases
            lin.weight.copy_(bf16_round(lin.weight))
            lin.bias.copy_(bf16_round(torch.randn_like(lin.bias) * 0.1))
    norm = LlamaRMSNorm(H, eps=1e-5)
    with torch.no_grad():
        norm.weight.copy_(bf16_round(1.0 + 0.1 * torch.randn(H)))
    x = bf16_round(torch.randn(B, T, H) * 1.5)
    with torch.no_grad():
        logits32 = router(x)                                 # [B,T,NG,2], fp32 module
        skip = logits32.argmax(dim=-1).to(torch.bool)        # base_layer.py:205
        execute32 = skip.logical_not()
        r16 = TokenRouter(H, group_num=NG, rank_size=R).eval()
        r16.load_state_dict(router.state_dict())
        r16 = r16.to(torch.bfloat16)
        logits16 = r16(x.to(torch.bfloat16))
        execute16 = logits16.argmax(dim=-1).to(torch.bool).logical_not()
        xn16 = norm.to(torch.bfloat16)(x.to(torch.bfloat16))
    save("router_norm", x=x, w_down=router.compressor.weight.detach(),
         b_down=router.compressor.bias.detach(), w_route=router.router.weight.detach(),
         b_route=router.router.bias.detach(), gamma=norm.weight.detach().float(),
         eps=np.float32(1e-5), logits_fp32=logits32, execute_fp32=execute32.numpy(),
         logits_bf16=logits16.float(), execute_bf16=execute16.numpy(), xn_bf16=xn16.float())

    # ---- rotary embedding and the sequence-first cache (same stubs) ------------------------
    from wrapper import base_layer
    from wrapper.cache import DynamicLayerSeqFirstLayer
    rope_fn = getattr(base_layer.apply_rotary_pos_emb, "_torchdynamo_orig_callable",
                      base_layer.apply_rotary_pos_emb)       # the function under @torch.compile
    torch.manual_seed(29)
    B, T0, T1, Hq, Hk, D = 2, 37, 5, 8, 2, 64
    def qkv(T):
        return (bf16_round(torch.randn(B, T, Hq, D)), bf16_round(torch.randn(B, T, Hk, D)),
                bf16_round(torch.randn(B, T, Hk, D)))
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(T0 + T1).float()[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)[None]                 # [1, T0+T1, D]
    cos, sin = bf16_round(emb.cos()), bf16_round(emb.sin())
    q0, k0, v0 = qkv(T0)
    q1, k1, v1 = qkv(T1)
    layer = DynamicLayerSeqFirstLayer()
    layer.keys = None
    layer.values = None
    with torch.no_grad():
        q0r, k0r = rope_fn(q0, k0, cos[:, :T0], sin[:, :T0])
        keys0, values0 = layer.update(k0r, v0)
        q1r, k1r = rope_fn(q1, k1, cos[:, T0:], sin[:, T0:])
        keys1, values1 = layer.update(k1r, v1)
    save("rope_cache", q0=q0, k0=k0, v0=v0, q1=q1, k1=k1, v1=v1, cos=cos[0], sin=sin[0],
         q0_rot=q0r, q1_rot=q1r, keys_after_prefill=keys0.clone(), keys_after_step=keys1,
         values_after_step=values1)


if __name__ == "__main__":
    if len(sys.argv) > 2 and sys.argv[2] == "router":
        router_fixture(sys.argv[1])
    else:
        if len(sys.argv) < 2:
            sys.exit("usage: make_golden.py /path/to/reference [router]")
        main(sys.argv[1])
