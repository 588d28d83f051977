"""TEST INFRASTRUCTURE ONLY -- stage the UNMODIFIED reference hot-path sources so that they can run on
a GPU box that has no checkout of the reference.

    python oracle/make_ref.py /path/to/reference         (or set $ELMO_REFERENCE)

copies ``src/triton_kernels`` and ``src/xmc_classifiers`` of xmc-aalto/elmo, byte for byte, into
``oracle/_ref/src`` (a git-ignored folder: the reference's sources never enter this repository's
history) and writes ``oracle/_ref/MANIFEST.json`` with a sha256 per file.  The only consumer is
``tests/golden/make_golden_gpu.py``, which imports those packages on a B200 and records the outputs
of the reference's own Triton kernels as fixtures; nothing in the product, the tests or the bench reads
this folder.
"""
import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DST = os.path.join(HERE, "_ref")
PACKAGES = ("triton_kernels", "xmc_classifiers")


def stage(ref_root: str) -> str:
    src = os.path.join(ref_root, "src")
    if not os.path.isdir(src):
        raise SystemExit(f"no reference checkout at {ref_root}")
    out_src = os.path.join(DST, "src")
    os.makedirs(out_src, exist_ok=True)
    manifest = {}
    for pkg in PACKAGES:
        dst_pkg = os.path.join(out_src, pkg)
        if os.path.isdir(dst_pkg):
            shutil.rmtree(dst_pkg)
        shutil.copytree(os.path.join(src, pkg), dst_pkg, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
        for root, _, files in os.walk(dst_pkg):
            for f in sorted(files):
                p = os.path.join(root, f)
                manifest[os.path.relpath(p, out_src)] = hashlib.sha256(open(p, "rb").read()).hexdigest()
    with open(os.path.join(DST, "MANIFEST.json"), "w") as fh:
        json.dump({"source": "xmc-aalto/elmo src/{triton_kernels,xmc_classifiers}, unmodified", "sha256": manifest},
                  fh, indent=1, sort_keys=True)
    return out_src


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("ELMO_REFERENCE")
    if not root:
        raise SystemExit("usage: make_ref.py /path/to/reference")
    print(stage(root))
