"""Stages an unmodified copy of the reference's Python packages under ``oracle/_ref/``.

    python oracle/stage_ref.py --reference <checkout of pengjh0111/triton-snn-fusion>

TEST INFRASTRUCTURE ONLY. The reference is a set of plain Python packages (``runtime``, ``compiler``,
``kernels``) without an installer, so "building" it for use as a checker means copying those
packages, byte for byte, to a place that is on no default import path: ``oracle/_ref/`` (listed in
.gitignore, so the copy never enters this repository's history). What uses the copy:

  * tests/test_dropin.py binds this library's backend modules beneath the reference's own
    ``runtime/snn_custom_ops.py`` and FX passes (``compiler/*.py``) and drives them through
    ``torch.ops.snn_custom.*``;
  * ``bench.py --impl reference`` and the ``cpu_baseline`` leg time the reference's own eager LIF op
    (``snn_custom.lif_forward_state``, runtime/snn_custom_ops.py:384-409) on the host cores;
  * ``python -m triton_snn_fusion_b200.microbench --impl reference-triton`` JIT-compiles the reference's
    Triton kernels (``kernels/generated_temporal_*.py``) for a same-GPU comparison.

The product never imports anything from here. A MANIFEST.json with the SHA-256 of every staged file is
written next to the copy so that a test can show the files are the reference's, unmodified.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
PACKAGES = ("runtime", "compiler", "kernels")


def stage(reference: Path, dest: Path = DEST) -> dict:
    reference = Path(reference)
    missing = [p for p in PACKAGES if not (reference / p).is_dir()]
    if missing:
        raise FileNotFoundError(f"{reference} is not a checkout of the reference: no {missing}")
    manifest = {}
    for pkg in PACKAGES:
        out = dest / pkg
        if out.exists():
            shutil.rmtree(out)
        out.mkdir(parents=True)
        for src in sorted((reference / pkg).glob("*.py")):
            data = src.read_bytes()
            (out / src.name).write_bytes(data)
            manifest[f"{pkg}/{src.name}"] = hashlib.sha256(data).hexdigest()
    (dest / "MANIFEST.json").write_text(json.dumps({"source": "pengjh0111/triton-snn-fusion", "files": manifest},
                                                   indent=1, sort_keys=True) + "\n")
    return manifest


def staged() -> bool:
    return (DEST / "runtime" / "snn_custom_ops.py").exists() and (DEST / "MANIFEST.json").exists()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference")
    ap.add_argument("--dest", default=str(DEST))
    a = ap.parse_args()
    files = stage(Path(a.reference), Path(a.dest))
    print(f"staged {len(files)} files under {a.dest}", file=sys.stderr)
