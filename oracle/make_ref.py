"""Build step for ``oracle/_ref``: the reference's own CPU implementation of the path, for timing and cross-checks.

The reference implements the chunk prefill semantics in two pure-Python files (``linquant/reference.py``, the float64
recurrence ``chunk_core``, and ``linquant/invariances.py``, the ``FakeQuant`` scale policies). There is nothing to
compile: this recipe places those two files, as they are, under ``oracle/_ref/linquant/`` (a git-ignored build
output, like a compiled ``.so``) so that machines without the reference checkout can still run the reference itself.
``bench.py --impl reference`` and its ``cpu_baseline`` leg time ``oracle/_ref`` when it exists and fall back to the
restatement in ``oracle/zoo_oracle.py`` otherwise. Nothing on the product path imports either.

    python oracle/make_ref.py [path-to-reference-checkout]

(default: ``$LINQUANT_REFERENCE_ROOT``, else the directory ``reference`` beside this repository)
"""

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = ("reference.py", "invariances.py")


def default_root():
    return os.environ.get("LINQUANT_REFERENCE_ROOT") or os.path.normpath(os.path.join(HERE, "..", "..", "reference"))


def build(ref_root=None):
    src = os.path.join(ref_root or default_root(), "linquant")
    if not all(os.path.exists(os.path.join(src, f)) for f in FILES):
        return None
    dst = os.path.join(HERE, "_ref", "linquant")
    os.makedirs(dst, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
    with open(os.path.join(dst, "__init__.py"), "w") as fh:
        fh.write("")
    return dst


def load():
    """(chunk_core, hadamard_rotation, FakeQuant, POLICIES) of the reference from ``oracle/_ref``, or None."""
    root = os.path.join(HERE, "_ref")
    if not os.path.exists(os.path.join(root, "linquant", "reference.py")):
        return None
    if root not in sys.path:
        sys.path.insert(0, root)
    from linquant.invariances import POLICIES, FakeQuant  # noqa: E402
    from linquant.reference import chunk_core, hadamard_rotation  # noqa: E402

    return chunk_core, hadamard_rotation, FakeQuant, POLICIES


if __name__ == "__main__":
    out = build(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out or "reference checkout not found: nothing built")
