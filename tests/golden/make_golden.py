"""Regenerates tests/golden/legacy_reference.npz from the reference's OWN functions.

Needs oracle/_ref/libpatina_ref.so (built by `make -C oracle ref` from the
reference's harness/gemm_check.cpp). Run where the reference checkout exists:

    python tests/golden/make_golden.py

Stored per K in {32, 128, 4096}:
  * A and B f16 bit patterns from the reference's fill_inputs (K = 32, 128 in
    full; for K = 4096 a sha256 only),
  * C_ref, the 128x128 double output of the reference's reference_gemm
    (in full for every K),
plus the reference's f16<->f32 converters sampled over every f16 bit pattern and
a fixed set of float32 inputs.
"""
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "legacy_reference.npz")


def converter_inputs() -> np.ndarray:
    rng = np.random.default_rng(20240611)
    mags = rng.standard_normal(4096).astype(np.float32) * (10.0 ** rng.integers(-9, 6, 4096)).astype(np.float32)
    edge = np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 6.1e-5, 5.96e-8, 2.98e-8, 2.9802322e-8,
                     1e-10, np.inf, -np.inf, 1.0009765625, 1.00048828125, 1.000488281250001], np.float32)
    return np.concatenate([mags, edge])


def main() -> None:
    R = oracle.ref()
    out = {}
    for K in (32, 128, 4096):
        A = np.empty((128, K), np.uint16)
        B = np.empty((128, K), np.uint16)
        R.patina_ref_fill_inputs(A.ctypes.data, B.ctypes.data, K)
        Cr = np.empty((128, 128), np.float64)
        R.patina_ref_reference_gemm(A.ctypes.data, B.ctypes.data, K, Cr.ctypes.data)
        out[f"C_ref_k{K}"] = Cr
        if K <= 128:
            out[f"A_k{K}"] = A
            out[f"B_k{K}"] = B
        out[f"A_sha_k{K}"] = np.frombuffer(hashlib.sha256(A.tobytes()).digest(), np.uint8)
        out[f"B_sha_k{K}"] = np.frombuffer(hashlib.sha256(B.tobytes()).digest(), np.uint8)
    bits = np.arange(65536, dtype=np.uint16)
    # Widened through ctypes' double return: signalling NaNs come back quiet, so
    # the table is stored for non-NaN patterns and NaN-ness separately.
    wide = np.array([R.patina_ref_f16_to_f32(int(b)) for b in bits], np.float32)
    out["f16_to_f32_bits"] = wide.view(np.uint32)
    xs = converter_inputs()
    out["f32_inputs"] = xs
    out["f32_to_f16"] = np.array([R.patina_ref_f32_to_f16(float(x)) for x in xs], np.uint16)
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")


if __name__ == "__main__":
    main()
