"""Import the reference's stock PyTorch modules in a container that has the
reference tree but not all of its dependencies.  Used only by make_golden.py
(fixture generation); never at test time."""
import sys
import types


def install_stubs():
    if "gemmi" not in sys.modules:
        g = types.ModuleType("gemmi")
        g.__version__ = "0.0"
        g.set_leak_warnings = lambda *a, **k: None
        sys.modules["gemmi"] = g
    if "ml_collections" not in sys.modules:
        m = types.ModuleType("ml_collections")

        class ConfigDict(dict):
            def __getattr__(self, k):
                try:
                    return self[k]
                except KeyError as e:
                    raise AttributeError(k) from e

            def __setattr__(self, k, v):
                self[k] = v

        m.ConfigDict = ConfigDict
        sys.modules["ml_collections"] = m
    if "biotite" not in sys.modules:
        b = types.ModuleType("biotite")
        s = types.ModuleType("biotite.structure")

        class AtomArray:  # noqa: D401
            pass

        s.AtomArray = AtomArray
        b.structure = s
        sys.modules["biotite"] = b
        sys.modules["biotite.structure"] = s


def import_reference(root):
    install_stubs()
    if root not in sys.path:
        sys.path.insert(0, root)
    from openfold3.core.model.layers.triangular_attention import TriangleAttention
    from openfold3.core.model.layers.triangular_multiplicative_update import (
        TriangleMultiplicationIncoming, TriangleMultiplicationOutgoing)
    from openfold3.core.model.primitives.attention import _attention
    return dict(TriangleAttention=TriangleAttention,
                TriangleMultiplicationOutgoing=TriangleMultiplicationOutgoing,
                TriangleMultiplicationIncoming=TriangleMultiplicationIncoming,
                _attention=_attention)
