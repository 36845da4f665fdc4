"""Regenerates tests/golden/reference_cuda_b200.npz: outputs of the REFERENCE's own CUDA kernels
(compiled for sm_100a from the reference's sources by `make -C oracle ref_cuda`) on the seeded cases
of tests/golden/cases.py.  Needs a GPU and oracle/_ref/libvrhino_ref_cuda.so; run from the repo root:

    python tests/golden/make_golden.py [output.npz]

The committed file was produced on an NVIDIA B200 (driver 580, CUDA 12.9) from reference v0.9.4-alpha.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

import cases  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_cuda_b200.npz")
    rc = ref.RefCuda()
    arrays = {}
    for case in cases.CASES:
        for name, (payload, dt) in cases.run_reference(rc, case).items():
            arrays[f"{case['name']}|{name}|{dt}"] = payload
        print(case["name"], "ok", flush=True)
    rc.lib.refc_shutdown()
    np.savez_compressed(out_path, **arrays)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main()
