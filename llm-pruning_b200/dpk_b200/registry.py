"""Operator registry with the reference's public surface.

Mirrors the behaviour of ``DynamicPruningKernels/python/registry.py`` (names,
argument meaning, exceptions, selection order) so that code written against
``get_kernel`` / ``run_kernel`` / ``register_kernel`` keeps working:

* backends are registered per family with a priority; ``backend="auto"`` picks the
  highest-priority one that is importable and ships the requested
  (version, architecture) pair (reference ``registry.py:331-386``);
* a spec with variants receives ``kernel_version=`` and ``arch=`` keyword
  arguments when called (reference ``registry.py:278-288``);
* ``detect_arch()`` maps compute capability 10.0 to ``"sm100"`` (reference
  ``registry.py:73-91``).

The implementation is independent: specs are plain classes and lookups are dict
based.
"""

from __future__ import annotations

import importlib
import importlib.util
from typing import Any, Callable, Dict, Iterable, Mapping, Optional, Sequence, Tuple, Union

VersionRequest = Union[int, str, None]


class KernelRegistryError(RuntimeError):
    """Base class of registry errors."""


class KernelNotFoundError(KernelRegistryError):
    """Unknown family/backend pair."""


class KernelUnavailableError(KernelRegistryError):
    """The backend is registered but cannot be used here."""


class KernelVariantError(KernelRegistryError, ValueError):
    """The requested version/architecture pair is not shipped."""


def _norm(name: str) -> str:
    return name.strip().lower().replace("-", "_")


_ARCH_ALIASES = {
    "80": "sm8x", "8.0": "sm8x", "86": "sm8x", "8.6": "sm8x", "89": "sm8x", "8.9": "sm8x",
    "sm80": "sm8x", "sm86": "sm8x", "sm89": "sm8x",
    "120": "sm12x", "12.0": "sm12x", "sm120": "sm12x",
    "100": "sm100", "10.0": "sm100", "sm100a": "sm100",
}


def _norm_arch(arch: str) -> str:
    a = arch.strip().lower().replace("_", "")
    return _ARCH_ALIASES.get(a, a)


def detect_arch(device: Any = None) -> str:
    """Architecture tag of the active CUDA device ("sm100" on B200)."""
    import torch

    if not torch.cuda.is_available():
        raise KernelVariantError(
            "arch='auto' requires a CUDA device; pass an explicit architecture "
            "when only inspecting the registry")
    major, minor = torch.cuda.get_device_capability(device)
    if major == 8:
        return "sm8x"
    if major == 12:
        return "sm12x"
    return f"sm{major}{minor}"


class KernelVariant:
    """One shipped version and the architectures it supports."""

    __slots__ = ("version", "architectures")

    def __init__(self, version: int, architectures: Sequence[str]):
        if version < 0:
            raise ValueError("Kernel versions must be non-negative")
        archs = tuple(architectures)
        if not archs:
            raise ValueError("A versioned kernel needs at least one architecture")
        self.version = int(version)
        self.architectures = archs

    def __repr__(self) -> str:
        return f"KernelVariant(version={self.version}, architectures={self.architectures})"


class KernelSpec:
    """Metadata and lazily imported target of one family/backend implementation."""

    def __init__(self, family: str, backend: str, target: Union[str, Callable[..., Any]],
                 variants: Iterable[KernelVariant] = (), default_version: Optional[int] = None,
                 requires: Sequence[str] = (), priority: int = 0, description: str = ""):
        self.family = _norm(family)
        self.backend = _norm(backend)
        self.target = target
        self.variants = tuple(variants)
        self.default_version = default_version
        self.requires = tuple(requires)
        self.priority = int(priority)
        self.description = description
        seen = [v.version for v in self.variants]
        if len(set(seen)) != len(seen):
            raise ValueError(f"Duplicate versions in {self.family}.{self.backend}: {seen}")
        if default_version is not None and default_version not in seen:
            raise ValueError(
                f"Default v{default_version} is not registered for {self.family}.{self.backend}")

    # -- introspection -------------------------------------------------------------
    @property
    def key(self) -> Tuple[str, str]:
        return self.family, self.backend

    @property
    def versions(self) -> Tuple[int, ...]:
        return tuple(sorted(v.version for v in self.variants))

    @property
    def architectures(self) -> Tuple[str, ...]:
        return tuple(sorted({a for v in self.variants for a in v.architectures}))

    def missing_requirements(self) -> Tuple[str, ...]:
        missing = []
        for mod in self.requires:
            try:
                ok = importlib.util.find_spec(mod) is not None
            except (ImportError, AttributeError, ValueError):
                ok = False
            if not ok:
                missing.append(mod)
        return tuple(missing)

    def is_available(self) -> bool:
        return not self.missing_requirements()

    def as_dict(self) -> Dict[str, Any]:
        return {
            "family": self.family,
            "backend": self.backend,
            "default_version": self.default_version,
            "versions": list(self.versions),
            "architectures": list(self.architectures),
            "variants": {f"v{v.version}": list(v.architectures)
                         for v in sorted(self.variants, key=lambda v: v.version)},
            "requires": list(self.requires),
            "available": self.is_available(),
            "priority": self.priority,
            "description": self.description,
        }

    # -- resolution ----------------------------------------------------------------
    def load(self) -> Callable[..., Any]:
        missing = self.missing_requirements()
        if missing:
            raise KernelUnavailableError(
                f"Backend {self.family}.{self.backend} requires: {', '.join(missing)}")
        if callable(self.target):
            return self.target
        mod_name, sep, attr = str(self.target).partition(":")
        if not (sep and mod_name and attr):
            raise KernelRegistryError(
                f"Invalid target {self.target!r}; expected 'module:callable'")
        try:
            fn = getattr(importlib.import_module(mod_name), attr)
        except (ImportError, AttributeError) as exc:
            raise KernelUnavailableError(
                f"Could not load {self.family}.{self.backend} from {self.target}") from exc
        if not callable(fn):
            raise KernelRegistryError(f"Kernel target {self.target} is not callable")
        return fn

    def resolve_variant(self, version: VersionRequest = "default",
                        arch: Optional[str] = "auto") -> Tuple[Optional[int], Optional[str]]:
        """Pick the (version, architecture) pair a request means."""
        if not self.variants:
            return None, None
        if arch is None or str(arch).lower() in ("auto", "native"):
            want_arch = detect_arch()
        else:
            want_arch = _norm_arch(str(arch))
        if want_arch not in self.architectures:
            raise KernelVariantError(
                f"{self.family}.{self.backend} does not support {want_arch}; "
                f"available architectures: {', '.join(self.architectures)}")
        fits = [v.version for v in self.variants if want_arch in v.architectures]
        text = "default" if version is None else str(version).lower()
        if text in ("auto", "default"):
            if self.default_version is None:
                return max(fits), want_arch
            want = self.default_version
        elif version == -1 or text == "latest":
            return max(fits), want_arch
        else:
            try:
                want = int(text[1:] if text.startswith("v") else text)
            except ValueError as exc:
                raise KernelVariantError(f"Invalid kernel version: {version!r}") from exc
        by_version = {v.version: v for v in self.variants}
        if want not in by_version:
            raise KernelVariantError(
                f"{self.family}.{self.backend} has no v{want}; available versions: "
                + ", ".join(f"v{v}" for v in self.versions))
        if want_arch not in by_version[want].architectures:
            raise KernelVariantError(
                f"{self.family}.{self.backend} v{want} does not support {want_arch}; "
                f"available architectures: {', '.join(by_version[want].architectures)}")
        return want, want_arch


class KernelHandle:
    """Callable with a fixed backend, version and architecture."""

    def __init__(self, spec: KernelSpec, version: Optional[int] = None, arch: Optional[str] = None):
        self.spec = spec
        self.version = version
        self.arch = arch
        self._impl: Optional[Callable[..., Any]] = None

    @property
    def family(self) -> str:
        return self.spec.family

    @property
    def backend(self) -> str:
        return self.spec.backend

    @property
    def implementation(self) -> Callable[..., Any]:
        if self._impl is None:
            self._impl = self.spec.load()
        return self._impl

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        if self.spec.variants:
            version, arch = self.spec.resolve_variant(
                version=kwargs.pop("kernel_version", self.version),
                arch=kwargs.pop("arch", self.arch))
            kwargs["kernel_version"] = version
            kwargs["arch"] = arch
        return self.implementation(*args, **kwargs)


class KernelRegistry:
    """Mutable set of specs with deterministic automatic selection."""

    backend_aliases = {"jit": "cute", "cute_jit": "cute", "cutlass": "cute",
                       "pytorch": "torch", "ref": "torch", "sm100": "b200", "blackwell": "b200"}

    def __init__(self) -> None:
        self._specs: Dict[Tuple[str, str], KernelSpec] = {}

    def register(self, spec: KernelSpec, *, replace: bool = False) -> KernelSpec:
        if spec.key in self._specs and not replace:
            raise KernelRegistryError(
                f"Kernel {spec.family}.{spec.backend} is already registered")
        self._specs[spec.key] = spec
        return spec

    def list(self, family: Optional[str] = None, *, available_only: bool = False):
        fam = _norm(family) if family else None
        specs = [s for s in self._specs.values() if fam is None or s.family == fam]
        if available_only:
            specs = [s for s in specs if s.is_available()]
        return tuple(sorted(specs, key=lambda s: (s.family, -s.priority, s.backend)))

    def get(self, family: str, backend: str = "auto", *, version: VersionRequest = "default",
            arch: Optional[str] = "auto") -> KernelHandle:
        fam = _norm(family)
        be = _norm(backend)
        be = self.backend_aliases.get(be, be)
        if be != "auto":
            spec = self._specs.get((fam, be))
            if spec is None:
                known = ", ".join(s.backend for s in self.list(fam)) or "none"
                raise KernelNotFoundError(
                    f"Unknown backend {fam}.{be}; available backends: {known}")
            if not spec.is_available():
                raise KernelUnavailableError(
                    f"Backend {fam}.{be} requires: {', '.join(spec.missing_requirements())}")
            return KernelHandle(spec, *spec.resolve_variant(version, arch))
        problems = []
        for spec in sorted(self.list(fam), key=lambda s: s.priority, reverse=True):
            if not spec.is_available():
                problems.append(f"{spec.backend}: missing {', '.join(spec.missing_requirements())}")
                continue
            try:
                return KernelHandle(spec, *spec.resolve_variant(version, arch))
            except KernelVariantError as exc:
                problems.append(f"{spec.backend}: {exc}")
        detail = "; ".join(problems) if problems else "no backends are registered"
        raise KernelUnavailableError(f"No usable backend for {fam}: {detail}")


def _as_variants(values) -> Tuple[KernelVariant, ...]:
    if isinstance(values, Mapping):
        return tuple(KernelVariant(v, tuple(a)) for v, a in values.items())
    return tuple(values)


KERNELS = KernelRegistry()


def register_kernel(family: str, backend: str, target=None, *, variants=(),
                    default_version: Optional[int] = None, requires: Sequence[str] = (),
                    priority: int = 0, description: str = "", replace: bool = False):
    """Register ``target`` (callable or "module:callable"); usable as a decorator."""

    def install(t):
        return KERNELS.register(
            KernelSpec(family, backend, t, _as_variants(variants), default_version,
                       tuple(requires), priority, description), replace=replace)

    if target is not None:
        return install(target)

    def decorator(fn):
        install(fn)
        return fn

    return decorator
