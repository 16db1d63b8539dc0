"""Bring the reference's golden vectors for the attention path and its sibling LayerNorm into this test tree.

The reference keeps five forward fixtures for
``nitrix.nn.attention.reference_scaled_dot_product_attention`` under its
``tests/golden/attention_*_float32.npz`` (made by ``tools/regen_golden.py:60-148``
of the reference).  They are data (inputs + the reference's stored output), and
they are the only stored values that pin the path, so they are carried verbatim.
``layer_norm_float32.npz`` (x, weight, bias, out at ``out_scale = 0.5``; same generator, used by the reference's
``tests/test_nn_norm.py:51-62``) pins the LayerNorm oracle the same way, and ``selective_scan_float32.npz`` (x, delta,
A, B, C, D, out; the reference's ``tests/test_nn_ssm.py:69-83``) the selective-scan oracle.

Run with the reference checkout as argument::

    python tests/golden/import_reference_goldens.py <reference-root>

The copy is byte-for-byte; a ``MANIFEST.json`` with SHA-256 digests is written so
that a drifted fixture is detected by ``tests/test_oracle_golden.py``.
"""
from __future__ import annotations

import hashlib
import json
import pathlib
import shutil
import sys

NAMES = ("dense", "windowed_bias", "causal", "cross", "qk_norm")


def main(ref_root: str) -> None:
    here = pathlib.Path(__file__).resolve().parent
    src = pathlib.Path(ref_root) / "tests" / "golden"
    manifest = {}
    for fn in [f"attention_{name}_float32.npz" for name in NAMES] + ["layer_norm_float32.npz", "selective_scan_float32.npz"]:
        shutil.copyfile(src / fn, here / fn)
        manifest[fn] = hashlib.sha256((here / fn).read_bytes()).hexdigest()
    (here / "MANIFEST.json").write_text(json.dumps(manifest, indent=1) + "\n")
    print(json.dumps(manifest, indent=1))


if __name__ == "__main__":
    main(sys.argv[1])
