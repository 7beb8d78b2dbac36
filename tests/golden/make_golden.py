"""Regenerates tests/golden/ from the hf2q source tree (run where that tree is mounted).

Two kinds of files are written:

* ``ggml_quants/<type>_<n>_{noim,im}_{input,expected}.bin`` -- the reference's own golden vectors
  for the nine block formats the library takes, copied byte-for-byte from its
  ``tests/fixtures/ggml_quants/`` (they were produced by llama.cpp's ``ggml_quantize_chunk`` and
  are what hf2q's ``byte_cmp_noim`` / ``byte_cmp_im`` unit tests compare against).
* ``MANIFEST.json`` -- sha256 of every copied file, so a silent edit is detected by the tests.

Usage: python tests/golden/make_golden.py /path/to/hf2q
"""
import hashlib
import json
import shutil
import sys
from pathlib import Path

TYPES = {"q4_0": 64, "q8_0": 64, "q4_k": 512, "q5_k": 512, "q6_k": 512, "q4_1": 64, "q5_0": 64, "q5_1": 64, "iq4_nl": 64}


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/hf2q")
    ref = Path(sys.argv[1])
    src = ref / "tests" / "fixtures" / "ggml_quants"
    dst = Path(__file__).resolve().parent / "ggml_quants"
    dst.mkdir(exist_ok=True)
    manifest = {}
    for name, n in TYPES.items():
        for variant in ("noim", "im"):
            for kind in ("input", "expected"):
                fn = f"{name}_{n}_{variant}_{kind}.bin"
                shutil.copyfile(src / fn, dst / fn)
                (dst / fn).chmod(0o644)
                manifest[fn] = hashlib.sha256((dst / fn).read_bytes()).hexdigest()
    (dst.parent / "MANIFEST.json").write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    print(f"copied {len(manifest)} files from {src}")


if __name__ == "__main__":
    main()
