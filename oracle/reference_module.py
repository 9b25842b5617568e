"""Loaders for the reference engine as built and staged by ``oracle/build_ref.py`` (TEST INFRASTRUCTURE, not product).

``oracle/_ref/`` holds the reference's native module (``_C.so``, compiled from its unmodified sources), its Python
package (``spira/``) and its model definitions (``models/spira/``).  Three ways to use them:

* :func:`load_native` -- the bare pybind module, for call-by-call comparisons in the GPU parity tests;
* :func:`load_package` -- the reference's OWN Python package driving its native module (the stock path that
  ``bench.py --impl reference`` times), importable as ``spira`` afterwards;
* :class:`ReferenceModule` -- the native module behind this repository's Python glue (``--impl reference-kernels``).

Only ``tests/`` and the reference arm of ``bench.py`` import this file.
"""
from __future__ import annotations

import importlib
import importlib.util
import sys
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"
_native = None


def available() -> bool:
    return (REF / "_C.so").exists()


def package_available() -> bool:
    return available() and (REF / "spira" / "__init__.py").exists() and (REF / "models" / "spira" / "__init__.py").exists()


def load_native():
    """The reference's pybind module (``spira.nn.functional._C`` in its own tree), loaded once per process."""
    global _native
    if _native is None:
        if not available():
            raise FileNotFoundError(f"{REF / '_C.so'} is missing: run oracle/build_ref.py where the reference checkout is present")
        import torch  # noqa: F401  (the module links against torch's libraries)
        spec = importlib.util.spec_from_file_location("_C", str(REF / "_C.so"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _native = mod
    return _native


def load_package():
    """Imports the reference's Python package as ``spira`` with its native module pre-registered under the name its
    shim imports (``spira.nn.functional._C``).  Refuses to replace a different ``spira`` that is already imported."""
    existing = sys.modules.get("spira")
    if existing is not None:
        if str(getattr(existing, "__file__", "")).startswith(str(REF)):
            return existing
        raise RuntimeError("a different module named 'spira' is already imported")
    if not package_available():
        raise FileNotFoundError(f"the reference's Python package is not staged under {REF}")
    native = load_native()
    sys.modules["spira.nn.functional._C"] = native
    sys.path.insert(0, str(REF))
    try:
        pkg = importlib.import_module("spira")
    finally:
        sys.path.remove(str(REF))
    return pkg


def load_models(name: str = "spira_ref_models"):
    """The reference's model definitions (``scripts/models/spira``) as a package called ``name``; they import whatever
    ``spira`` is registered in ``sys.modules`` at that moment (the reference's package, or this repository's package
    after ``install_as_spira()``)."""
    if name in sys.modules:
        return sys.modules[name]
    init = REF / "models" / "spira" / "__init__.py"
    if not init.exists():
        raise FileNotFoundError(f"the reference's model definitions are not staged under {REF / 'models'}")
    spec = importlib.util.spec_from_file_location(name, str(init), submodule_search_locations=[str(init.parent)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    try:
        spec.loader.exec_module(mod)
    except Exception:
        sys.modules.pop(name, None)
        raise
    return mod


def unload_package() -> None:
    """Forgets the reference's ``spira`` (and model packages built on it), so that another ``spira`` can be registered."""
    for key in [k for k in sys.modules if k == "spira" or k.startswith("spira.") or k.startswith("spira_ref_models")]:
        mod = sys.modules[key]
        if key.startswith("spira_ref_models") or str(getattr(mod, "__file__", "")).startswith(str(REF)) or mod is _native:
            del sys.modules[key]


class ReferenceModule:
    """The reference's native module plus the helpers this repository's glue calls that are plain torch operations in
    the reference's own Python (feature permutation ``features[index]``, ``map.T.contiguous()``)."""
    LAYOUT_OS, LAYOUT_WS = 0, 1
    CACHE_DERIVED = False   # the reference rebuilds the inverted map of a transposed layer on every forward

    def __init__(self, mod=None):
        self._mod = mod if mod is not None else load_native()

    def __getattr__(self, name):
        return getattr(self._mod, name)

    def cuda_flatten_sort(self, coords, double=False):
        import torch
        keys, perm = self._mod.cuda_flatten_sort(coords, double)
        if (keys.numel() * keys.element_size()) % 512 == 0:
            # the reference's search reads sources[num_sources] (kernels/query_sorted.cuh:42,48); keep that read
            # inside an allocation when the tensor ends exactly on an allocator block boundary
            big = torch.empty(keys.numel() + 64, dtype=keys.dtype, device=keys.device)
            big[:keys.numel()] = keys
            keys = big[:keys.numel()]
        return keys, perm

    @staticmethod
    def permute_rows(rows, perm):
        import torch
        return rows[perm.to(torch.int64)]

    @staticmethod
    def transpose_map(m):
        return m.T.contiguous()

    @staticmethod
    def _aligned(n):
        return (n + 127) // 128 * 128

    @staticmethod
    def check_status(device=None):
        return None


def install_native(module) -> None:
    """Points every glue module of ``spira_b200`` at ``module`` instead of the built-in binding (and back, when given
    ``spira_b200.nn.functional._C``)."""
    import spira_b200.nn.functional as F
    from spira_b200.nn import conv
    from spira_b200.nn.functional import indexing, convolution, memory
    for m in (F, conv, indexing, convolution, memory):
        m._C = module


# ------------------------------------------------------------------------------------------------
# the benchmark networks assembled from the REFERENCE's own layers and blocks
# ------------------------------------------------------------------------------------------------
def build_network(kind: str, spira_pkg=None, blocks=None):
    """``kind`` = "minkunet" | "indoor" | "second": the topology of ``spira_b200.models.{minkunet18, indoor_resunet,
    second_backbone}`` built from the reference's ``spnn.SparseConv`` / ``BatchNorm`` / ``ReLU``, its ``cat`` and its
    ``SparseConvBlock`` / ``SparseConvTransposeBlock`` / ``SparseResBlock`` (scripts/models/spira/modules/blocks.py).
    Attribute names equal those of ``spira_b200.models``, so a ``state_dict`` moves between the two.  (The reference's
    ``SparseResUNet42`` fixes 2^3 resampling kernels and has no classification head, sparse_unet.py:47-69; the
    benchmark configuration asks for 3^3 everywhere and a 19-class head.)"""
    from torch import nn
    sp = spira_pkg if spira_pkg is not None else load_package()
    B = blocks if blocks is not None else load_models().modules
    spnn = sp.nn

    class UNet(nn.Module):
        def __init__(self, in_channels, stem, enc, dec, num_classes, kernel=3, resample_kernel=3):
            super().__init__()
            self.n_down = len(enc)
            self.stem = nn.Sequential(B.SparseConvBlock(in_channels, stem, kernel), B.SparseConvBlock(stem, stem, kernel))
            widths = [stem] + list(enc)
            self.encoders = nn.ModuleList()
            for i in range(len(enc)):
                self.encoders.append(nn.Sequential(B.SparseConvBlock(widths[i], widths[i], resample_kernel, stride=2),
                                                   B.SparseResBlock(widths[i], widths[i + 1], kernel),
                                                   B.SparseResBlock(widths[i + 1], widths[i + 1], kernel)))
            self.ups, self.fuses = nn.ModuleList(), nn.ModuleList()
            cur = widths[-1]
            for i, d in enumerate(dec):
                skip = widths[len(enc) - 1 - i]
                self.ups.append(B.SparseConvTransposeBlock(cur, d, resample_kernel, stride=2))
                self.fuses.append(nn.Sequential(B.SparseResBlock(d + skip, d, kernel), B.SparseResBlock(d, d, kernel)))
                cur = d
            self.head = spnn.SparseConv(cur, num_classes, 1, bias=True)

        def forward(self, x):
            skips = [self.stem(x)]
            for e in self.encoders:
                skips.append(e(skips[-1]))
            y = skips.pop()
            for up, fuse in zip(self.ups, self.fuses):
                y = fuse(sp.cat([up(y), skips.pop()]))
            return self.head(y)

    class Backbone(nn.Module):
        def __init__(self, in_channels, widths, kernel=3):
            super().__init__()
            self.n_down = len(widths) - 1
            layers = [B.SparseConvBlock(in_channels, widths[0], kernel), B.SparseConvBlock(widths[0], widths[0], kernel)]
            for i in range(1, len(widths)):
                layers += [B.SparseConvBlock(widths[i - 1], widths[i], kernel, stride=2),
                           B.SparseConvBlock(widths[i], widths[i], kernel), B.SparseConvBlock(widths[i], widths[i], kernel)]
            self.layers = nn.Sequential(*layers)

        def forward(self, x):
            return self.layers(x)

    if kind == "minkunet":
        return UNet(4, 32, [32, 64, 128, 256], [256, 128, 96, 96], 19, 3, 3)
    if kind == "indoor":
        return UNet(3, 32, [64, 128, 256], [128, 64, 32], 20, 3, 3)
    if kind == "second":
        return Backbone(5, [16, 32, 64, 128], 3)
    raise ValueError(f"unknown network {kind}")
