"""The drop-in route exercised against the reference's own registry (CPU only).

``dpk_b200.install_into(dynamic_width_jit)`` registers the four B200 callables in the
reference package's registry; afterwards the reference's ``get_kernel`` must pick them for
architecture ``sm100`` under ``backend="auto"`` (its selection by priority,
``DynamicPruningKernels/python/registry.py:366-381``), leave every other architecture as it
was, and its handle must inject ``kernel_version=0, arch="sm100"`` into the call
(``registry.py:278-288``).  Skipped where the reference tree is not present.
"""

import os
import sys
import tempfile

import pytest

# the reference checkout: named by DPK_REFERENCE_ROOT, else a directory "reference" beside this repository
REF_ROOT = os.environ.get("DPK_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
REF_PKG = os.path.join(REF_ROOT, "DynamicPruningKernels", "python")
FAMILIES = ("gemm_mn", "gemm_k", "attention_prefill", "attention_decode")

pytestmark = pytest.mark.skipif(not os.path.isdir(REF_PKG), reason="reference tree not present")


@pytest.fixture(scope="module")
def reference():
    # the reference's package directory is called "python"; expose it under its import name
    # through a symlink in a scratch directory (the recipe of tests/golden/make_golden.py)
    shim = tempfile.mkdtemp(prefix="dpk_ref_")
    os.symlink(REF_PKG, os.path.join(shim, "dynamic_width_jit"))
    sys.path.insert(0, shim)
    try:
        import dynamic_width_jit
        yield dynamic_width_jit
    finally:
        sys.path.remove(shim)
        for name in [m for m in sys.modules if m == "dynamic_width_jit" or m.startswith("dynamic_width_jit.")]:
            del sys.modules[name]


def test_install_into_the_real_registry(reference):
    import dpk_b200

    before = {f: [item["backend"] for item in reference.list_kernels(f)] for f in FAMILIES}
    before_sm12x = {}
    for f in FAMILIES:
        try:
            before_sm12x[f] = reference.get_kernel(f, "auto", arch="sm12x").backend
        except reference.KernelRegistryError as exc:       # e.g. no backend importable here
            before_sm12x[f] = type(exc).__name__
    dpk_b200.install_into(reference)
    for f in FAMILIES:
        # selected automatically for sm100, above the reference's own backends
        handle = reference.get_kernel(f, "auto", arch="sm100")
        assert handle.backend == "b200" and handle.version == 0 and handle.arch == "sm100"
        assert reference.get_kernel(f, "b200", version="latest", arch="sm100").version == 0
        # listed first (highest priority) and available
        listing = reference.list_kernels(f)
        assert listing[0]["backend"] == "b200" and listing[0]["available"]
        assert listing[0]["variants"] == {"v0": ["sm100"]}
        assert [i["backend"] for i in listing[1:]] == before[f]
        # other architectures resolve exactly as before
        try:
            now = reference.get_kernel(f, "auto", arch="sm12x").backend
        except reference.KernelRegistryError as exc:
            now = type(exc).__name__
        assert now == before_sm12x[f] and now != "b200"
        with pytest.raises(reference.KernelVariantError):
            reference.get_kernel(f, "b200", arch="sm12x")
        # the torch backend (the CPU reference path) is untouched
        assert reference.get_kernel(f, "torch").backend == "torch"


def test_reference_handle_injects_version_and_arch(reference, monkeypatch):
    import dpk_b200
    from dpk_b200 import ops

    seen = {}

    def probe(*args, **kwargs):
        seen.update(kwargs)
        return "called"

    monkeypatch.setattr(ops, "gemm_mn", probe)
    dpk_b200.install_into(reference)
    assert reference.run_kernel("gemm_mn", 1, 2, 3, backend="auto", arch="sm100", activation="silu") == "called"
    assert seen == {"kernel_version": 0, "arch": "sm100", "activation": "silu"}
    monkeypatch.undo()
    dpk_b200.install_into(reference)          # put the real callable back


def test_both_registries_agree_on_the_surface(reference):
    """Names a caller may import from either package."""
    import dpk_b200

    for name in ("get_kernel", "run_kernel", "list_kernels", "available_backends", "register_kernel",
                 "detect_arch", "KernelHandle", "KernelSpec", "KernelVariant", "KernelRegistry",
                 "KernelRegistryError", "KernelNotFoundError", "KernelUnavailableError",
                 "KernelVariantError"):
        assert hasattr(reference, name), name
        assert hasattr(dpk_b200, name), name
    # same resolution for the same request
    ours = dpk_b200.get_kernel("attention_decode", "auto", arch="sm_100a")
    theirs = reference.get_kernel("attention_decode", "auto", arch="sm100")
    assert (ours.backend, ours.version, ours.arch) == (theirs.backend, theirs.version, theirs.arch)
