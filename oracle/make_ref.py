"""Place the reference's own Python package under ``oracle/_ref/`` (test infrastructure, not product code).

The reference project is pure Python.  Its package ``sihc/`` is copied, unmodified and ``*.py`` files only, from
the read-only reference checkout into ``oracle/_ref/sihc`` so that machines without that checkout can still

  * run the UNMODIFIED reference model classes with their three routing operators rebound to this library
    (``tests/test_gpu_reference_dropin.py``),
  * time the reference's own Triton operators beside the CUDA ones (``bench.py --workload stage_ops``), and
  * time the reference's own eager CPU path ``read_torch`` / ``write_torch`` (``bench.py --impl reference``).

``oracle/_ref/`` is listed in ``.gitignore``: the copy never enters this repository's history.  Nothing in the
package ``residual_stream_burden_b200`` may import it.

    python oracle/make_ref.py [/path/to/reference/checkout]
"""

from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
# the read-only reference checkout: $SIHC_REFERENCE_ROOT, else a folder named `reference` in the home directory
DEFAULT_SOURCE = os.environ.get("SIHC_REFERENCE_ROOT", os.path.join(os.path.expanduser("~"), "reference"))


def make_ref(source: str = DEFAULT_SOURCE) -> str | None:
    """Copy ``<source>/sihc/**/*.py`` to ``oracle/_ref/sihc``.  Returns the destination, or None when the
    reference checkout is not present (an existing copy is then left as it is)."""
    package = os.path.join(source, "sihc")
    if not os.path.isdir(package):
        return None
    target = os.path.join(DEST, "sihc")
    if os.path.isdir(target):
        shutil.rmtree(target)
    for folder, _, files in os.walk(package):
        rel = os.path.relpath(folder, package)
        for name in files:
            if name.endswith(".py"):
                os.makedirs(os.path.join(target, rel), exist_ok=True)
                shutil.copyfile(os.path.join(folder, name), os.path.join(target, rel, name))
    with open(os.path.join(DEST, "README"), "w") as f:
        f.write("Unmodified copy of the reference's `sihc` Python package (*.py only), made by oracle/make_ref.py.\n"
                "Not part of this repository's history.\n")
    return DEST


def ref_path() -> str | None:
    """``oracle/_ref`` if the copy exists (put it on ``sys.path`` to ``import sihc``), else None."""
    return DEST if os.path.isfile(os.path.join(DEST, "sihc", "__init__.py")) else None


if __name__ == "__main__":
    out = make_ref(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SOURCE)
    print(out if out else "reference checkout not found; nothing copied")
