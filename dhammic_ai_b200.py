"""Importable alias: ``import dhammic_ai_b200`` loads the package directory ``dhammic-ai_b200``
(whose name is not a Python identifier)."""
import importlib
import os
import sys

_root = os.path.dirname(os.path.abspath(__file__))
if _root not in sys.path:
    sys.path.insert(0, _root)
sys.modules[__name__] = importlib.import_module("dhammic-ai_b200")
