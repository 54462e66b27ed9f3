"""Generates tests/golden/record_state.npz: two states of the reference's CUDA env (after 48
steps of random play; the same randomised once by the shim's fuzz kernel) together with the
records the reference's k_record_obs wrote for them.  Needs a GPU and oracle/_ref (built from
the reference sources by oracle/Makefile).

Usage: python tests/golden/make_record_golden.py [output.npz]
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "craftax.cu_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import cfx  # noqa: E402
import oracle as O  # noqa: E402


def main():
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "record_state.npz")
    cfx.lib()
    n, arrays = 32, {}
    for tag, fuzz in (("play", 0), ("fuzz", 1)):
        view = cfx.EnvView()
        rec = O.RefCuda.record_session(2, n, 48, fuzz, 5, view)
        st = cfx.env_state_from_view(view)
        O.RefCuda.record_session_close(2)
        assert np.array_equal(O.record_from_state(st), rec), tag
        arrays[f"{tag}_records"] = rec
        for k, v in st.items():
            arrays[f"{tag}_{k}"] = v
    np.savez_compressed(out, **arrays)
    print(out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
