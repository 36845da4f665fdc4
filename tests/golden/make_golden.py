"""Regenerates tests/golden/reference_cuda_b200.npz: outputs of the REFERENCE's own CUDA kernels
(compiled for sm_100a from the reference's sources by `make -C oracle ref_cuda`) on the seeded cases
of tests/golden/cases.py.  Needs a GPU and oracle/_ref/libvrhino_ref_cuda.so; run from the repo root:

    python tests/golden/make_golden.py [output.npz] [--only KIND]

With --only, just the cases of that kind are run and merged into the vectors already in
tests/golden/reference_cuda_b200.npz (the other cases' vectors are carried over unchanged).

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
    committed = os.path.join(ROOT, "tests", "golden", "reference_cuda_b200.npz")
    args = sys.argv[1:]
    only = None
    if "--only" in args:
        only = args[args.index("--only") + 1]
        del args[args.index("--only"):args.index("--only") + 2]
    out_path = args[0] if args else committed
    rc = ref.RefCuda()
    arrays = {}
    if only:
        kept = np.load(committed)
        names = {c["name"] for c in cases.CASES if c["kind"] == only}
        arrays = {key: kept[key] for key in kept.files if key.split("|")[0] not in names}
    for case in cases.CASES:
        if only and case["kind"] != only:
            continue
        for name, (payload, dt) in cases.run_reference(rc, case).items():
            arrays[f"{case['name']}|{name}|{dt}"] = payload
        print(case["name"], "ok", flush=True)
    rc.lib.refc_shutdown()
    np.savez_compressed(out_path, **arrays)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main()
