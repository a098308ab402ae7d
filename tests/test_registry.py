"""Operator registry: same observable behaviour as the reference's
(DynamicPruningKernels/tests/test_registry.py), for the B200 backend."""

import pytest

import dpk_b200 as dw
from dpk_b200.registry import KernelRegistry, KernelSpec, KernelVariant


def test_four_reference_families_are_registered():
    families = {item["family"] for item in dw.list_kernels()}
    assert {"gemm_mn", "gemm_k", "attention_prefill", "attention_decode"} <= families
    assert "ffn_swiglu" in families


def test_b200_backend_resolves_for_sm100():
    for family in ("gemm_mn", "gemm_k", "attention_prefill", "attention_decode"):
        handle = dw.get_kernel(family, "b200", arch="sm100")
        assert handle.backend == "b200" and handle.version == 0 and handle.arch == "sm100"
        handle = dw.get_kernel(family, "auto", arch="sm100")
        assert handle.backend == "b200"
        assert dw.get_kernel(family, "b200", version="latest", arch="sm100").version == 0
        assert dw.get_kernel(family, "b200", version="v0", arch="10.0").arch == "sm100"


def test_unknown_variant_and_backend_errors():
    with pytest.raises(dw.KernelVariantError):
        dw.get_kernel("gemm_mn", "b200", version=3, arch="sm100")
    with pytest.raises(dw.KernelVariantError):
        dw.get_kernel("gemm_mn", "b200", arch="sm8x")
    with pytest.raises(dw.KernelNotFoundError):
        dw.get_kernel("gemm_mn", "cute", arch="sm100")
    with pytest.raises(dw.KernelUnavailableError):
        dw.get_kernel("no_such_family", arch="sm100")


def test_alias_and_canonical_names():
    assert dw.get_kernel("GEMM-MN", "blackwell", arch="sm_100").backend == "b200"


def test_auto_selection_prefers_priority_and_skips_unavailable():
    reg = KernelRegistry()
    calls = []
    reg.register(KernelSpec("f", "slow", lambda *a, **k: calls.append("slow"), priority=1))
    reg.register(KernelSpec("f", "broken", "x:y", requires=("definitely_not_a_module",),
                            priority=50))
    reg.register(KernelSpec("f", "fast", lambda *a, **k: calls.append(("fast", k)),
                            variants=(KernelVariant(0, ("sm100",)), KernelVariant(2, ("sm100",))),
                            default_version=0, priority=10))
    h = reg.get("f", arch="sm100")
    assert h.backend == "fast" and h.version == 0
    h()
    assert calls[-1] == ("fast", {"kernel_version": 0, "arch": "sm100"})
    assert reg.get("f", version="latest", arch="sm100").version == 2
    # an architecture only the unversioned backend can serve
    assert reg.get("f", arch="sm8x").backend == "slow"
    with pytest.raises(dw.KernelUnavailableError):
        reg.get("f", "broken")
    with pytest.raises(dw.KernelRegistryError):
        reg.register(KernelSpec("f", "slow", lambda: None))


def test_register_kernel_decorator_and_listing():
    @dw.register_kernel("unit_family", "unit_backend", priority=3, description="d")
    def impl(x):
        return x + 1

    assert dw.run_kernel("unit_family", 1, backend="unit_backend") == 2
    assert "unit_backend" in dw.available_backends("unit_family")
    (item,) = [i for i in dw.list_kernels("unit_family")]
    assert item["priority"] == 3 and item["available"] and item["versions"] == []


def test_spec_validation():
    with pytest.raises(ValueError):
        KernelSpec("f", "b", lambda: None, variants=(KernelVariant(1, ("a",)), KernelVariant(1, ("b",))))
    with pytest.raises(ValueError):
        KernelSpec("f", "b", lambda: None, variants=(KernelVariant(1, ("a",)),), default_version=2)
    with pytest.raises(ValueError):
        KernelVariant(-1, ("a",))
    with pytest.raises(ValueError):
        KernelVariant(0, ())


def test_install_into_reference_style_module():
    class FakeReference:
        def __init__(self):
            self.seen = {}

        def register_kernel(self, family, backend, target, **kw):
            self.seen[family] = (backend, target, kw)

    ref = FakeReference()
    dw.install_into(ref)
    assert set(ref.seen) == {"gemm_mn", "gemm_k", "attention_prefill", "attention_decode"}
    backend, target, kw = ref.seen["gemm_mn"]
    assert backend == "b200" and callable(target)
    assert kw["variants"] == {0: ("sm100",)} and kw["priority"] > 100


def test_attention_head_sizes_the_operators_take():
    """The kernels are built for head sizes 64 and 128; the operators also take the other
    multiples of 32 up to 128 (the reference's rule is D % 32 == 0) by padding, and refuse
    the rest with a message instead of a kernel error."""
    from dpk_b200 import ops

    assert [ops._padded_head_dim(d) for d in (32, 64, 96, 128)] == [64, 64, 128, 128]
    for bad in (0, 48, 160, 256):
        with pytest.raises(ValueError, match="head_dim"):
            ops._padded_head_dim(bad)
