"""Operator registry of the B200 backend.

What callers of the reference's operator API rely on, and what is therefore kept
(``DynamicPruningKernels/python/registry.py:94-439``, ``python/__init__.py:25-48``):

* the names ``register_kernel``, ``KernelSpec``, ``KernelVariant``, ``KernelHandle``,
  ``KernelRegistry``, ``detect_arch`` and the three exception types;
* a backend is registered per operator family with a priority, the module names it needs and,
  optionally, the (version, architectures) pairs it ships; ``backend="auto"`` takes the
  highest-priority backend that can be imported and ships what was asked for;
* a handle of a backend that ships versions calls its implementation with ``kernel_version=``
  and ``arch=`` filled in (``registry.py:278-288``);
* compute capability 10.0 is the architecture tag ``"sm100"`` (``registry.py:86-91``).

When the reference package itself is importable, ``dpk_b200.install_into`` registers these
kernels in ITS registry and this module is not involved at all; this registry serves
processes that have only this package.  The data model is a table
``family -> backend -> spec`` with one resolution routine shared by explicit and automatic
selection.
"""

from __future__ import annotations

import importlib
import importlib.util
import re
from typing import Any, Callable, Dict, Iterable, Iterator, List, Mapping, Optional, Sequence, Tuple, Union

VersionRequest = Union[int, str, None]


class KernelRegistryError(RuntimeError):
    """Any failure of the registry."""


class KernelNotFoundError(KernelRegistryError):
    """No such backend for the family."""


class KernelUnavailableError(KernelRegistryError):
    """A backend exists but cannot run in this process."""


class KernelVariantError(KernelRegistryError, ValueError):
    """The backend does not ship the requested version for the requested architecture."""


def canonical(name: str) -> str:
    """Family and backend names compare case-insensitively, ``-`` equals ``_``."""
    return name.strip().lower().replace("-", "_")


_ARCH_TEXT = re.compile(r"^(?:sm)?_?(\d+)(?:\.(\d))?a?$")


def arch_tag(major: int, minor: int) -> str:
    """Architecture tag of a compute capability.  The reference groups Ampere/Ada as
    ``sm8x`` and consumer Blackwell as ``sm12x``; everything else is ``sm<major><minor>``."""
    if major in (8, 12):
        return f"sm{major}x"
    return f"sm{major}{minor}"


def canonical_arch(text: str) -> str:
    """``"sm_100a"``, ``"100"``, ``"10.0"`` -> ``"sm100"``; ``"86"`` -> ``"sm8x"``; tags that are
    not a compute capability (``"sm8x"``) pass through in lower case."""
    t = text.strip().lower()
    m = _ARCH_TEXT.match(t)
    if not m:
        return t.replace("_", "")
    digits, minor = m.group(1), m.group(2)
    if minor is None:                       # "100" = 10.0, "86" = 8.6, "9" = 9.0
        major, minor_i = (int(digits[:-1]), int(digits[-1])) if len(digits) > 1 else (int(digits), 0)
    else:
        major, minor_i = int(digits), int(minor)
    return arch_tag(major, minor_i)


def detect_arch(device: Any = None) -> str:
    """Architecture tag of the current CUDA device (``"sm100"`` on a B200)."""
    import torch

    if not torch.cuda.is_available():
        raise KernelVariantError("no CUDA device to take the architecture from: name one explicitly "
                                 "(arch='sm100') when the registry is only being inspected")
    return arch_tag(*torch.cuda.get_device_capability(device))


class KernelVariant:
    """A shipped kernel version and the architecture tags it was built for."""

    __slots__ = ("version", "architectures")

    def __init__(self, version: int, architectures: Sequence[str]):
        version = int(version)
        archs = tuple(canonical_arch(a) for a in architectures)
        if version < 0:
            raise ValueError(f"version {version}: versions count from 0")
        if not archs:
            raise ValueError(f"version {version} lists no architecture")
        self.version, self.architectures = version, archs

    def __repr__(self) -> str:
        return f"KernelVariant({self.version}, {self.architectures!r})"


def _parse_version(request: VersionRequest) -> Union[int, str]:
    """``"default"`` / ``"latest"`` or a number; accepts ``3``, ``"3"``, ``"v3"``, ``-1`` (latest),
    ``None`` and ``"auto"`` (default)."""
    if request is None:
        return "default"
    if isinstance(request, int):
        return "latest" if request == -1 else request
    t = str(request).strip().lower()
    if t in ("default", "auto"):
        return "default"
    if t == "latest":
        return "latest"
    try:
        return int(t.lstrip("v"))
    except ValueError:
        raise KernelVariantError(f"{request!r} is not a kernel version") from None


class KernelSpec:
    """One backend of one operator family."""

    def __init__(self, family: str, backend: str, target: Union[str, Callable[..., Any]],
                 variants: Iterable[KernelVariant] = (), default_version: Optional[int] = None,
                 requires: Sequence[str] = (), priority: int = 0, description: str = ""):
        self.family, self.backend = canonical(family), canonical(backend)
        self.target = target
        self.variants: Tuple[KernelVariant, ...] = tuple(variants)
        self.requires: Tuple[str, ...] = tuple(requires)
        self.priority, self.description = int(priority), description
        self.default_version = default_version
        self._ships: Dict[int, Tuple[str, ...]] = {}
        for v in self.variants:
            if v.version in self._ships:
                raise ValueError(f"{self.name} lists v{v.version} twice")
            self._ships[v.version] = v.architectures
        if default_version is not None and default_version not in self._ships:
            raise ValueError(f"{self.name}: default v{default_version} is not among its versions")

    @property
    def name(self) -> str:
        return f"{self.family}.{self.backend}"

    @property
    def versions(self) -> Tuple[int, ...]:
        return tuple(sorted(self._ships))

    @property
    def architectures(self) -> Tuple[str, ...]:
        return tuple(sorted({a for archs in self._ships.values() for a in archs}))

    # ---- can it run here? -------------------------------------------------------------
    def missing_requirements(self) -> Tuple[str, ...]:
        def importable(module: str) -> bool:
            try:
                return importlib.util.find_spec(module) is not None
            except (ImportError, AttributeError, ValueError):
                return False
        return tuple(m for m in self.requires if not importable(m))

    def is_available(self) -> bool:
        return not self.missing_requirements()

    def _require_available(self) -> None:
        missing = self.missing_requirements()
        if missing:
            raise KernelUnavailableError(f"{self.name} needs the module(s) {', '.join(missing)}, "
                                         "which this interpreter cannot import")

    def load(self) -> Callable[..., Any]:
        """The implementation: the callable itself or the ``"module:attribute"`` it names."""
        self._require_available()
        if callable(self.target):
            return self.target
        module, _, attribute = str(self.target).partition(":")
        if not module or not attribute:
            raise KernelRegistryError(f"{self.name}: target {self.target!r} is not 'module:attribute'")
        try:
            fn = getattr(importlib.import_module(module), attribute)
        except (ImportError, AttributeError) as exc:
            raise KernelUnavailableError(f"{self.name}: importing {self.target} failed ({exc})") from exc
        if not callable(fn):
            raise KernelRegistryError(f"{self.name}: {self.target} is not callable")
        return fn

    # ---- which (version, architecture) does a request mean? ---------------------------------
    def resolve_variant(self, version: VersionRequest = "default",
                        arch: Optional[str] = "auto") -> Tuple[Optional[int], Optional[str]]:
        if not self._ships:
            return None, None               # an unversioned backend serves every request
        tag = detect_arch() if arch is None or str(arch).lower() in ("auto", "native") \
            else canonical_arch(str(arch))
        built_for_tag = sorted(v for v, archs in self._ships.items() if tag in archs)
        if not built_for_tag:
            raise KernelVariantError(f"{self.name} is not built for {tag} "
                                     f"(built for: {', '.join(self.architectures)})")
        want = _parse_version(version)
        if want == "default":
            want = self.default_version if self.default_version is not None else built_for_tag[-1]
        elif want == "latest":
            want = built_for_tag[-1]
        if want not in self._ships:
            raise KernelVariantError(f"{self.name} ships {', '.join('v%d' % v for v in self.versions)}, "
                                     f"not v{want}")
        if want not in built_for_tag:
            raise KernelVariantError(f"{self.name} v{want} is built for "
                                     f"{', '.join(self._ships[want])}, not for {tag}")
        return want, tag

    def as_dict(self) -> Dict[str, Any]:
        return {"family": self.family, "backend": self.backend, "priority": self.priority,
                "description": self.description, "requires": list(self.requires),
                "available": self.is_available(), "default_version": self.default_version,
                "versions": list(self.versions), "architectures": list(self.architectures),
                "variants": {f"v{v}": list(self._ships[v]) for v in self.versions}}


class KernelHandle:
    """A backend pinned to a version and an architecture; calling it runs the kernel."""

    def __init__(self, spec: KernelSpec, version: Optional[int] = None, arch: Optional[str] = None):
        self.spec, self.version, self.arch = spec, version, arch
        self._fn: Optional[Callable[..., Any]] = None

    family = property(lambda self: self.spec.family)
    backend = property(lambda self: self.spec.backend)

    @property
    def implementation(self) -> Callable[..., Any]:
        if self._fn is None:
            self._fn = self.spec.load()
        return self._fn

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        if self.spec.versions:
            # per-call overrides are honoured, then the resolved pair is what the kernel sees
            v, a = self.spec.resolve_variant(kwargs.pop("kernel_version", self.version),
                                             kwargs.pop("arch", self.arch))
            kwargs.update(kernel_version=v, arch=a)
        return self.implementation(*args, **kwargs)


class KernelRegistry:
    """``family -> backend -> KernelSpec``."""

    backend_aliases = {"blackwell": "b200", "sm100": "b200", "pytorch": "torch", "ref": "torch",
                       "jit": "cute", "cute_jit": "cute", "cutlass": "cute"}

    def __init__(self) -> None:
        self._table: Dict[str, Dict[str, KernelSpec]] = {}

    def register(self, spec: KernelSpec, *, replace: bool = False) -> KernelSpec:
        backends = self._table.setdefault(spec.family, {})
        if spec.backend in backends and not replace:
            raise KernelRegistryError(f"{spec.name} exists already (pass replace=True to overwrite it)")
        backends[spec.backend] = spec
        return spec

    def _by_priority(self, family: str) -> List[KernelSpec]:
        return sorted(self._table.get(family, {}).values(), key=lambda s: (-s.priority, s.backend))

    def list(self, family: Optional[str] = None, *, available_only: bool = False) -> Tuple[KernelSpec, ...]:
        families = [canonical(family)] if family else sorted(self._table)
        specs: Iterator[KernelSpec] = (s for f in families for s in self._by_priority(f))
        return tuple(s for s in specs if s.is_available() or not available_only)

    def get(self, family: str, backend: str = "auto", *, version: VersionRequest = "default",
            arch: Optional[str] = "auto") -> KernelHandle:
        fam = canonical(family)
        wanted = canonical(backend)
        wanted = self.backend_aliases.get(wanted, wanted)
        if wanted != "auto":
            spec = self._table.get(fam, {}).get(wanted)
            if spec is None:
                have = ", ".join(s.backend for s in self._by_priority(fam)) or "none"
                raise KernelNotFoundError(f"{fam} has no backend {wanted!r} (registered: {have})")
            spec._require_available()
            return KernelHandle(spec, *spec.resolve_variant(version, arch))
        # automatic: the first backend, by priority, that is importable and ships the request
        rejected = []
        for spec in self._by_priority(fam):
            try:
                spec._require_available()
                return KernelHandle(spec, *spec.resolve_variant(version, arch))
            except (KernelUnavailableError, KernelVariantError) as exc:
                rejected.append(str(exc))
        raise KernelUnavailableError(f"nothing can serve {fam}: " +
                                     ("; ".join(rejected) if rejected else "no backend is registered"))


KERNELS = KernelRegistry()


def register_kernel(family: str, backend: str, target=None, *, variants=(),
                    default_version: Optional[int] = None, requires: Sequence[str] = (),
                    priority: int = 0, description: str = "", replace: bool = False):
    """Add a backend to the process-wide registry.  ``variants`` is a sequence of
    ``KernelVariant`` or a mapping ``{version: (arch, ...)}``.  Without ``target`` it returns a
    decorator."""
    if isinstance(variants, Mapping):
        variants = [KernelVariant(v, archs) for v, archs in variants.items()]

    def add(fn):
        KERNELS.register(KernelSpec(family, backend, fn, variants, default_version, requires,
                                    priority, description), replace=replace)
        return fn

    if target is None:
        return add
    add(target)
    return KERNELS._table[canonical(family)][canonical(backend)]
