"""Regenerates the golden fixtures of this folder.

  mlp_ref_vectors.npz - outputs of the reference's own host MLP (test/mlp.h, double precision) for
      seeded weights and inputs, produced through oracle/_ref/libref_mlp.so.  Needs the reference
      checkout (see oracle/build_oracle.py: TNN_REFERENCE_ROOT) to build that library; the fixture itself
      travels with the repository.
  grid_kat.json / packing_kat.json hold literal vectors of the reference's tests and are not generated:
      test/doctest_encodings.cpp:234-285 and test/python/test_packing.py:9-27.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from tests import synth  # noqa: E402

CASES = [  # (width, n_hidden, act, out_act)
    (16, 2, "relu", "none"), (32, 1, "sigmoid", "none"), (64, 4, "relu", "none"), (64, 2, "none", "sigmoid"),
    (128, 1, "relu", "relu"),
]
N_SAMPLES = 2


def main():
    if O.ref_lib() is None:
        raise SystemExit("oracle/_ref/libref_mlp.so could not be built: no reference checkout")
    out = {}
    for ci, (W, nh, act, oact) in enumerate(CASES):
        n_mat = nh + 1
        w = synth.xavier_weights(n_mat, W, seed=10 + ci).astype(np.float64)
        rng = np.random.default_rng(200 + ci)
        x = rng.uniform(-1, 1, (N_SAMPLES, W))
        t = rng.uniform(-1, 1, (N_SAMPLES, W))
        fwd, grads, lgrads, dldi, loss = [], [], [], [], []
        for b in range(N_SAMPLES):
            r = O.ref_mlp_sample(W, n_mat, act, oact, x[b], t[b], weights=w, batch=1)
            fwd.append(r["fwd"]); grads.append(r["grads"]); lgrads.append(r["loss_grads"])
            dldi.append(r["dl_dinput"]); loss.append(r["loss"])
        key = f"c{ci}"
        out[key + "_cfg"] = np.array([W, nh, O.ACT[act], O.ACT[oact]])
        out[key + "_wseed"] = np.array([10 + ci])  # weights = synth.xavier_weights(n_mat, W, seed)
        out[key + "_x"] = x.astype(np.float32)
        out[key + "_t"] = t.astype(np.float32)
        out[key + "_fwd"] = np.array(fwd, dtype=np.float32)
        out[key + "_grads"] = np.array(grads[:1], dtype=np.float32)  # sample 0 only, to keep the file small
        out[key + "_lgrads"] = np.array(lgrads, dtype=np.float32)
        out[key + "_dldi"] = np.array(dldi, dtype=np.float32)
        out[key + "_loss"] = np.array(loss, dtype=np.float32)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mlp_ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
