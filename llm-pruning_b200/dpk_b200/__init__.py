"""dpk_b200 -- B200 (sm_100a) backend of the routed dynamic-width operators.

Public surface = the reference's operator API (``DynamicPruningKernels/python/
__init__.py:25-89``): ``get_kernel``, ``run_kernel``, ``list_kernels``,
``available_backends``, ``register_kernel``, ``detect_arch`` and the registry
types.  The four reference families (``gemm_mn``, ``gemm_k``,
``attention_prefill``, ``attention_decode``) are registered under the backend name
``"b200"`` for architecture ``"sm100"``; ``ffn_swiglu`` is an extra family for the
fused FFN.  ``install_into(reference_module)`` registers the same callables in the
reference's own registry so that ``backend="auto"`` selects them on a B200.
"""

from __future__ import annotations

from typing import Any

from .registry import (KERNELS, KernelHandle, KernelNotFoundError, KernelRegistry,
                       KernelRegistryError, KernelSpec, KernelUnavailableError, KernelVariant,
                       KernelVariantError, VersionRequest, detect_arch, register_kernel)

__version__ = "0.1.0"

BACKEND = "b200"
ARCH = "sm100"
_PRIORITY = 200   # above the reference's CuTe backend (100)

_FAMILIES = {
    "gemm_mn": ("dpk_b200.ops:gemm_mn", "tcgen05 grouped output-width routed GEMM (+ fused SwiGLU)"),
    "gemm_k": ("dpk_b200.ops:gemm_k", "tcgen05 reduction-width routed GEMM, fp32 in TMEM"),
    "attention_prefill": ("dpk_b200.ops:attention_prefill", "head-group-routed prefill attention"),
    "attention_decode": ("dpk_b200.ops:attention_decode", "head-group-routed split-KV decode"),
}


def _register_builtin() -> None:
    for family, (target, text) in _FAMILIES.items():
        register_kernel(family, BACKEND, target, variants={0: (ARCH,)}, default_version=0,
                        requires=("torch",), priority=_PRIORITY, description=text, replace=True)
    register_kernel("ffn_swiglu", BACKEND, "dpk_b200.ops:ffn_swiglu", requires=("torch",),
                    priority=_PRIORITY, description="routing + fused gate/up + down in one call",
                    replace=True)


_register_builtin()


def get_kernel(family: str, backend: str = "auto", *, version: VersionRequest = "default",
               arch: str | None = "auto") -> KernelHandle:
    """Resolve a configured kernel without importing its implementation eagerly."""
    return KERNELS.get(family, backend, version=version, arch=arch)


def run_kernel(family: str, *args: Any, backend: str = "auto", version: VersionRequest = "default",
               arch: str | None = "auto", **kwargs: Any) -> Any:
    """Resolve and execute one kernel family."""
    return get_kernel(family, backend, version=version, arch=arch)(*args, **kwargs)


def list_kernels(family: str | None = None, *, available_only: bool = False):
    """Serializable catalog of the registered implementations."""
    return tuple(s.as_dict() for s in KERNELS.list(family, available_only=available_only))


def available_backends(family: str):
    """Importable backends in auto-selection order."""
    return tuple(s.backend for s in KERNELS.list(family, available_only=True))


def install_into(reference_module: Any) -> None:
    """Register this backend in the reference package's registry.

    ``reference_module`` is the imported ``dynamic_width_jit`` package; afterwards
    ``dynamic_width_jit.get_kernel(family)`` resolves to these kernels on a device
    whose ``detect_arch()`` is ``"sm100"`` (reference ``registry.py:366-381``).
    """
    from . import ops

    for family in _FAMILIES:
        reference_module.register_kernel(
            family, BACKEND, getattr(ops, family), variants={0: (ARCH,)}, default_version=0,
            requires=("torch",), priority=_PRIORITY, description=_FAMILIES[family][1], replace=True)


__all__ = [
    "KERNELS", "KernelHandle", "KernelNotFoundError", "KernelRegistry", "KernelRegistryError",
    "KernelSpec", "KernelUnavailableError", "KernelVariant", "KernelVariantError",
    "available_backends", "detect_arch", "get_kernel", "install_into", "list_kernels",
    "register_kernel", "run_kernel",
]
