import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_index():
    return json.loads((GOLDEN / "index.json").read_text())["cases"]


def golden_cases(kind):
    return sorted(n for n, c in golden_index().items() if c["kind"] == kind)


def load_golden(name):
    meta = golden_index()[name]
    with np.load(GOLDEN / f"{name}.npz") as z:
        arrays = {k: torch.from_numpy(z[k].copy()) for k in z.files}
    return meta["args"], arrays


REF_STAGE = ROOT / "oracle" / "_ref"


@pytest.fixture(scope="session")
def ref_ops():
    """The reference's own op layer (runtime/snn_custom_ops.py, staged unmodified under oracle/_ref by
    oracle/stage_ref.py) imported with this library's backend modules bound beneath it."""
    if not (REF_STAGE / "runtime" / "snn_custom_ops.py").exists():
        pytest.skip("the reference is not staged (python oracle/stage_ref.py --reference <checkout>)")
    sys.dont_write_bytecode = True
    if str(REF_STAGE) not in sys.path:
        sys.path.insert(0, str(REF_STAGE))
    from triton_snn_fusion_b200.runtime.install import install
    if "runtime.snn_custom_ops" not in sys.modules:
        install()
    import runtime.snn_custom_ops as ops  # noqa: E402  the reference's file
    return ops
