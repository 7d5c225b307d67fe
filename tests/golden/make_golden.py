"""Regenerates the golden fixtures in this directory:  python tests/golden/make_golden.py

Inputs are seeded float32 arrays; expected outputs are float64 results of the
CPU oracle (oracle/dense_oracle.c), cross-checked here against its independent
NumPy restatement before anything is written.  The reference (cuDeep) ships no
golden files and has no CPU path, so these fixtures pin the oracle's behaviour
over time, not the reference's; the reference's own known-answer tests are
replayed in tests/test_oracle_pins.py.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from oracle import oracle as o  # noqa: E402


def main():
    rng = np.random.default_rng(20240)
    out = {}
    # GEMM: one aligned, one ragged shape; plain and linear (W stored [N, K]) forms.
    for tag, (m, n, k) in {"aligned": (32, 64, 32), "ragged": (19, 29, 23)}.items():
        a = rng.standard_normal((m, k), dtype=np.float32)
        b = rng.standard_normal((k, n), dtype=np.float32)
        w = rng.standard_normal((n, k), dtype=np.float32)
        bias = rng.uniform(-0.5, 0.5, n).astype(np.float32)
        out[f"gemm_{tag}_a"] = a
        out[f"gemm_{tag}_b"] = b
        out[f"gemm_{tag}_w"] = w
        out[f"gemm_{tag}_bias"] = bias
        c = o.gemm(a, b)
        assert o.rel_frobenius(c, o.gemm_np(a, b)) < 1e-14
        out[f"gemm_{tag}_c"] = c
        out[f"gemm_{tag}_c_tf32"] = o.gemm(a, b, input_mode=o.INPUT_TF32_TRUNC)
        for act in range(5):
            y = o.linear(a, w, bias, act=act)
            assert o.rel_frobenius(y, o.gemm_np(a, w, b_is_nk=True, bias=bias, act=act)) < 1e-14
            out[f"linear_{tag}_act{act}"] = y
    # Conv: padded 3x3, strided 3x3, 1x1, 5x5 with asymmetric padding.
    cases = {
        "p1": dict(shape=(2, 6, 9, 7), oc=5, k=(3, 3), stride=(1, 1), padding=(1, 1)),
        "s2": dict(shape=(1, 4, 11, 10), oc=3, k=(3, 3), stride=(2, 2), padding=(0, 1)),
        "k1": dict(shape=(2, 8, 5, 5), oc=4, k=(1, 1), stride=(1, 1), padding=(0, 0)),
        "k5": dict(shape=(1, 3, 8, 12), oc=6, k=(5, 5), stride=(1, 1), padding=(2, 1)),
    }
    for tag, cs in cases.items():
        x = rng.standard_normal(cs["shape"], dtype=np.float32)
        w = rng.standard_normal((cs["oc"], cs["shape"][1], *cs["k"]), dtype=np.float32)
        bias = rng.uniform(-0.5, 0.5, cs["oc"]).astype(np.float32)
        y = o.conv2d(x, w, bias, cs["stride"], cs["padding"], act=o.EPI_RELU)
        assert o.rel_frobenius(y, o.conv2d_np(x, w, bias, cs["stride"], cs["padding"], act=o.EPI_RELU)) < 1e-14
        out[f"conv_{tag}_x"] = x
        out[f"conv_{tag}_w"] = w
        out[f"conv_{tag}_bias"] = bias
        out[f"conv_{tag}_y"] = y
        out[f"conv_{tag}_meta"] = np.array([*cs["stride"], *cs["padding"]], dtype=np.int64)
    np.savez_compressed(HERE / "dense_golden.npz", **out)
    print("wrote", HERE / "dense_golden.npz", sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
