"""Generates tests/golden/dae_api.npz: the byte encodings the REFERENCE's python/dae produces for the cases
in dae_cases.py.  Run where a checkout of the reference is available (its root in the environment variable
VDCORES_REFERENCE_ROOT); the reference's compiled ``dae.runtime`` extension is replaced by this repository's
ctypes runtime (opcode table, config, family specs), nothing is launched and no GPU is needed.

    VDCORES_REFERENCE_ROOT=<reference checkout> python tests/golden/make_dae_golden.py
"""
import importlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("VDCORES_REFERENCE_ROOT")
if not REF:
    raise SystemExit("set VDCORES_REFERENCE_ROOT to the root of a checkout of the reference")


def load_reference_dae():
    sys.path.insert(0, ROOT)
    from vdcores_b200 import runtime as rt
    import dae_cases
    pkg = types.ModuleType("dae")
    pkg.__path__ = [os.path.join(REF, "python", "dae")]
    sys.modules["dae"] = pkg
    stub = types.ModuleType("dae.runtime")
    for name in ("opcode", "config", "compute_family_specs", "supported_compute_ops", "set_smem_size", "set_cache_policy",
                 "launch_dae"):
        setattr(stub, name, getattr(rt, name))
    stub.build_tma_desc = dae_cases.fake_build_tma_desc
    sys.modules["dae.runtime"] = stub
    pkg.runtime = stub
    ns = types.SimpleNamespace()
    for mod in ("dae.launcher", "dae.schedule"):
        m = importlib.import_module(mod)
        for k, v in vars(m).items():
            if not k.startswith("_"):
                setattr(ns, k, v)
    return ns, importlib.import_module("dae.model")


if __name__ == "__main__":
    sys.path.insert(0, HERE)
    import dae_cases
    D, M = load_reference_dae()
    cases = {**dae_cases.build_cases(D), **dae_cases.build_launcher_cases(D), **dae_cases.build_attention_cases(D, M)}
    out = os.path.join(HERE, "dae_api.npz")
    np.savez_compressed(out, **cases)
    print("wrote", out, {k: v.size for k, v in cases.items()})
