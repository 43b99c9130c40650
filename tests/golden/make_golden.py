"""Regenerate the golden fixtures from the reference's own test-data generators.

    python tests/golden/make_golden.py [--ref /root/reference]

The reference keeps no stored test vectors: its build runs numpy generators
(tfcc/test/python/testcase/**) and the C++ tests compare against what they
produced.  This script imports those generator classes from the reference tree
(it must be present), seeds numpy, runs them exactly as
tfcc/test/python/test.py:42-60 does, and writes the arrays as compressed .npz
files next to this script.  The fixtures are then all a machine without the
reference needs.  Integer expectations are stored as int32 after checking that
they fit; the quantization case also records the offsets derived by the
generator.
"""
from __future__ import annotations

import argparse
import importlib.util
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
SEED = 20240607


def load_class(ref: Path, rel: str, cls: str):
    pydir = ref / "tfcc/test/python"
    if str(pydir) not in sys.path:
        sys.path.insert(0, str(pydir))
    path = pydir / rel
    # module name must look like "testcase.<module>.<file>" for the prefix logic
    name = "testcase." + rel[len("testcase/"):-3].replace("/", ".")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return getattr(mod, cls)


def generate(ref: Path) -> None:
    jobs = [
        ("testcase/blas/matmul.py", "Matmul", "blas_matmul.npz"),
        ("testcase/blas/matmulwithblas.py", "MatmulWithBlas", "blas_matmulwithblas.npz"),
        ("testcase/quantization/mklquantizationmatmul.py", "MKLQuantizationMatmul",
         "quantization_mklquantizationmatmul.npz"),
        ("testcase/quantization/quantize.py", "Quantize", "quantization_quantize.npz"),
        ("testcase/math/softmax.py", "Softmax", "math_softmax.npz"),
        ("testcase/math/gelu_accurate.py", "GeluAccurate", "math_gelu_accurate.npz"),
        ("testcase/layer/layer_normalization.py", "LayerNormalization",
         "layer_layer_normalization.npz"),
    ]
    for i, (rel, cls, out) in enumerate(jobs):
        np.random.seed(SEED + i)
        data = load_class(ref, rel, cls)().getData()
        packed = {}
        for key, val in data.items():
            val = np.asarray(val)
            if key.endswith("/expect") and val.dtype == np.int64:
                assert np.all(val == val.astype(np.int32)), "expectation does not fit int32"
                val = val.astype(np.int32)
            elif key.endswith("/a") and val.dtype == np.float32:
                pass
            elif key.endswith("/a") and val.dtype == np.int64:
                val = val.astype(np.uint8)
            elif key.endswith("/b") and val.dtype == np.int64:
                val = val.astype(np.int8)
            packed[key] = val
        np.savez_compressed(HERE / out, **packed)
        print(out, len(packed), "arrays", (HERE / out).stat().st_size, "bytes")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default="/root/reference")
    generate(Path(ap.parse_args().ref))
