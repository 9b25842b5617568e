"""Makes ``import spira`` resolve to this package."""
import importlib
import sys

_SUBMODULES = ["tensors", "operators", "nn", "nn.conv", "nn.activations", "nn.normalizations", "nn.functional",
               "nn.functional._C", "nn.functional.indexing", "nn.functional.convolution", "nn.functional.memory",
               "utils", "utils.helpers", "utils.apply", "utils.typing"]


def install_as_spira(force: bool = False) -> None:
    """Aliases ``spira`` and its submodules to ``spira_b200`` in ``sys.modules``.

    Refuses to shadow an already imported, different ``spira`` unless ``force`` is set.
    """
    pkg = importlib.import_module("spira_b200")
    existing = sys.modules.get("spira")
    if existing is not None and existing is not pkg and not force:
        raise RuntimeError("a different module named 'spira' is already imported")
    sys.modules["spira"] = pkg
    for name in _SUBMODULES:
        sys.modules["spira." + name] = importlib.import_module("spira_b200." + name)
