#!/usr/bin/env python
"""Puts the reference's sources under ``baseline/_ref`` (kept out of git) for the reference arm of ``bench.py``.

    python baseline/install_ref.py /path/to/AERIS-GB        (or AERIS_REFERENCE=/path/to/AERIS-GB)

First the packaging route (``pip install --no-index --no-build-isolation --target baseline/_ref <checkout>``); the
reference builds with hatchling, so where that backend is not installed pip stops before copying anything and the
script falls back to a plain copy of the two pure-Python packages ``src/aeris`` and ``src/aeris_wp_inference``.
No file of the reference is edited either way.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def main() -> int:
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("AERIS_REFERENCE")
    if not src or not os.path.isdir(os.path.join(src, "src", "aeris")):
        print(f"no AERIS-GB checkout at {src!r}: pass its path as the argument or in AERIS_REFERENCE")
        return 1
    os.makedirs(DEST, exist_ok=True)
    import tempfile
    work = os.path.join(tempfile.gettempdir(), "aeris_ref_build")          # pip may write into the tree it builds from
    shutil.rmtree(work, ignore_errors=True)
    shutil.copytree(src, work)
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps"]
    if os.environ.get("PIP_FIND_LINKS_DIR"):           # an offline folder of wheels, where there is one
        cmd += ["--find-links", os.environ["PIP_FIND_LINKS_DIR"]]
    cmd += ["--target", DEST, work]
    r = subprocess.run(cmd, capture_output=True, text=True)
    how = "pip"
    if r.returncode != 0 or not os.path.isdir(os.path.join(DEST, "aeris")):
        last = (r.stderr.strip().splitlines() or ["?"])[-1]
        print(f"pip could not build the reference ({last}); copying its pure-Python packages instead")
        how = "copy"
        for pkg in ("aeris", "aeris_wp_inference"):
            shutil.rmtree(os.path.join(DEST, pkg), ignore_errors=True)
            shutil.copytree(os.path.join(src, "src", pkg), os.path.join(DEST, pkg))
    if not os.path.isdir(os.path.join(DEST, "aeris_wp_inference")):     # the wheel target lists src/aeris only
        shutil.copytree(os.path.join(src, "src", "aeris_wp_inference"), os.path.join(DEST, "aeris_wp_inference"))
    print(f"reference sources in {DEST} ({how})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
