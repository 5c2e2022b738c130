"""The repository's ``dae`` package (vdcores_b200/dae) against the reference's python/dae: the cases in
tests/golden/dae_cases.py — single instructions with every flag, hardware loops (RepeatM.on / on1 /
onSync), schedules, resource groups with late-bound barriers, LoopM / LoopC, the launcher's instruction
rings — must encode to exactly the bytes stored in tests/golden/dae_api.npz, which make_dae_golden.py
produced by running the same cases through the reference's own Python layer.  No GPU."""
import os
import sys
import types

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, os.path.join(HERE, "golden"))


@pytest.fixture(scope="module")
def D():
    pkg_dir = os.path.join(ROOT, "vdcores_b200")
    if pkg_dir not in sys.path:
        sys.path.insert(0, pkg_dir)
    import dae_cases
    import dae.runtime
    import dae.launcher
    import dae.schedule
    saved = dae.runtime.build_tma_desc
    dae.runtime.build_tma_desc = dae_cases.fake_build_tma_desc      # descriptors become argument records
    ns = types.SimpleNamespace()
    for m in (dae.launcher, dae.schedule):
        for k, v in vars(m).items():
            if not k.startswith("_"):
                setattr(ns, k, v)
    yield ns
    dae.runtime.build_tma_desc = saved


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(HERE, "golden", "dae_api.npz"))


def test_instruction_encodings_match_the_reference(D, golden):
    import dae_cases
    got = dae_cases.build_cases(D)
    for name, arr in got.items():
        assert np.array_equal(arr, golden[name]), f"case {name} differs from the reference's encoding"


def test_launcher_streams_match_the_reference(D, golden):
    import dae_cases
    got = dae_cases.build_launcher_cases(D)
    for name in ("launcher_ptrs", "launcher_bars", "launcher_tmas", "launcher_cinsts", "launcher_minsts"):
        assert np.array_equal(got[name], golden[name]), f"{name} differs from the reference's"


def test_attention_operators_schedule_and_recipes_match_the_reference(D, golden):
    """The decode-attention instruction encodings, a SchedAttentionDecoding launch (fused QK-norm + RoPE path and
    the plain one) and the strided tensor-map recipes / coordinate functions of dae.model."""
    import dae_cases
    import dae.model as M
    got = dae_cases.build_attention_cases(D, M)
    for name in ("attention_compute", "model_recipes", "model_cords", "attention_tmas", "attention_bars",
                 "attention_cinsts", "attention_minsts"):
        assert np.array_equal(got[name], golden[name]), f"{name} differs from the reference's"


def test_family_names_and_errors(D):
    from dae.op_families import family_ref, family_spec_by_name
    assert family_ref("GEMV_WGMMA", M=64, N=8, K=256, BLOAD=4, RESIDUAL=False).canonical_name == \
        "OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_4__RESIDUAL_0"
    assert family_spec_by_name("OP_GEMV_MMA__M_64__N_8__K_256")["k"] == 256
    with pytest.raises(ValueError):
        family_ref("GEMV_WGMMA", M=60, N=8, K=256, BLOAD=4, RESIDUAL=0)     # M must be a multiple of 64
    with pytest.raises(ValueError):
        family_ref("GEMV_MMA", M=64, N=16, K=256)                           # N is fixed to 8
    # a family member the runtime does not implement resolves by name but fails when it is encoded
    with pytest.raises(ValueError, match="Missing runtime opcode"):
        D.Gemv_M128N8(4).tensor()
    # every reference operator name this runtime claims is in its opcode table
    from dae.runtime import opcode, supported_compute_ops
    for name in ("OP_GEMV_WGMMA__M_64__N_8__K_256__BLOAD_4__RESIDUAL_0", "OP_RMS_NORM_F16_K_4096_SMEM",
                 "OP_ROPE_INTERLEAVE_512", "OP_SILU_MUL_SHARED_BF16_K_64_SW128", "OP_ARGMAX_PARTIAL_bf16_1024_65536_128",
                 "OP_COPY", "OP_DUMMY", "OP_LOOPC", "OP_TERMINATEC"):
        assert hasattr(opcode, name) and name in supported_compute_ops


def test_library_validator_accepts_the_reference_built_streams():
    """The streams the reference's own Launcher wrote for the golden program (loops, groups, late barriers,
    argmax) pass the C-ABI's host-side walk of the instruction words."""
    from vdcores_b200 import runtime
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "dae_api.npz"))
    S = len(z["launcher_ptrs"].view(np.int64)) // 2
    c, m = z["launcher_cinsts"].reshape(S, -1, 8), z["launcher_minsts"].reshape(S, -1, 16)
    N = 64
    cc, mm = np.zeros((S, N, 8), np.uint8), np.zeros((S, N, 16), np.uint8)
    cc[:, :c.shape[1]], mm[:, :m.shape[1]] = c, m
    runtime.validate_streams(S, N, cc.reshape(-1, 8), mm.reshape(-1, 16))
