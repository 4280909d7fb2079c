"""Inputs of the committed golden vectors (rebuilt from seeds) and their loader."""
import importlib.util
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
_mg = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mg)

golden_cases = _mg.golden_cases
input_digest = _mg.input_digest


def load_golden():
    return np.load(os.path.join(HERE, "golden", "svc_golden.npz"))
