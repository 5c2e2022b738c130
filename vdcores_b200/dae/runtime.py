"""``dae.runtime``: the names the reference's compiled extension exports (reference
src/torch_runtime.cu:260-314), served by the C ABI of libvdcores_b200.so."""
import os
import sys

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from vdcores_b200.runtime import (  # noqa: E402,F401
    VdcError, build_tma_desc, compute_family_specs, config, init, last_error, launch_async, launch_dae, opcode,
    read_status, set_cache_policy, set_smem_size, supported_compute_ops, validate_streams)
