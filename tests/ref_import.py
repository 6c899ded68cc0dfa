"""Import pure-Python pieces of the reference implementation for parity tests, with stub modules standing in for
the third-party packages that are not installed (exllamav2, bitsandbytes, h5py, wandb, nvidia_smi).
Tests that use this skip when no reference tree is present."""
import importlib
import os
import sys
import types

import pytest

# where a copy of the reference tree may be: the optional in-repo install, a directory named by the environment, or a
# "reference" folder beside the repository
_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_CANDIDATES = [os.path.join(_REPO, "baseline", "_ref"), os.environ.get("LLM_DISTILLERY_REFERENCE", ""),
               os.path.join(os.path.dirname(_REPO), "reference")]


def reference_root():
    for c in _CANDIDATES:
        if os.path.exists(os.path.join(c, "utils", "finetuning_utils.py")):
            return c
    return None


def _stub(name, **attrs):
    if name in sys.modules:
        return sys.modules[name]
    m = types.ModuleType(name)
    for k, v in attrs.items():
        setattr(m, k, v)
    sys.modules[name] = m
    return m


def import_reference(module: str):
    root = reference_root()
    if root is None:
        pytest.skip("reference tree not available")
    try:
        import bitsandbytes  # noqa: F401
    except Exception:
        _stub("bitsandbytes", optim=types.SimpleNamespace())
    for name in ("exllamav2", "h5py", "nvidia_smi"):
        try:
            importlib.import_module(name)
        except Exception:
            _stub(name, ExLlamaV2Tokenizer=object, ExLlamaV2Config=object, ExLlamaV2=object, ExLlamaV2Cache=object)
    try:
        import wandb  # noqa: F401
    except Exception:
        w = _stub("wandb")
        w.wandb_run = _stub("wandb.wandb_run", Run=object)
    if root not in sys.path:
        sys.path.insert(0, root)
    # the reference's top-level packages (utils, classes) are namespace packages with generic names: make sure
    # those names resolve inside the reference tree
    for k in list(sys.modules):
        if k.split(".")[0] in ("utils", "classes"):
            paths = list(getattr(sys.modules[k], "__path__", []) or [])
            f = getattr(sys.modules[k], "__file__", None) or ""
            if not (f.startswith(root) or any(str(p).startswith(root) for p in paths)):
                del sys.modules[k]
    return importlib.import_module(module)
