"""Build recipe for `oracle/_ref/`: the reference's own Python package as importable bytecode.

    python oracle/make_ref.py /path/to/boundflow-checkout

TEST AND BENCHMARK INFRASTRUCTURE ONLY.  Nothing under `boundflow_b200/` imports it.

The reference (leezear2022/boundflow) is a pure-Python package whose bound-propagation path needs
only torch and numpy.  This recipe byte-compiles every module of `<checkout>/boundflow` where it
lies and packs the `.pyc` files (no sources) into `oracle/_ref/boundflow_ref.zip` in the legacy
layout, from which CPython's zipimport loads them without the `.py` files (one archive instead of
loose `.pyc` files, which file-sync tools commonly skip).  `oracle/_ref/` is git-ignored, so the
reference never enters this repository's history; it is a build output like a compiled `.so`.

Users of `oracle/_ref` (all of them check that it exists and skip or fall back otherwise):
  * `bench.py --impl reference` and the `cpu_baseline` leg time the reference's own functions
    (`_forward_ibp_trace_mlp`, `run_crown_ibp_mlp_from_forward_trace`, torch's Adam) on the host cores
    (`cpu_baseline.kind = "reference"`);
  * `tests/test_gpu_reference_dropin.py` passes the reference's real objects (`BFTaskModule`,
    `BoundQueryRequest`, `solve_bab_mlp(query_runtime=...)`, `run_ibp_scheduled(executor=...)`,
    `run_crown_ibp_mlp(fused_crown_executor=...)`) through the CUDA adapters.
The bytecode is tied to the interpreter version that compiled it; `ref_path()` checks that.
"""
from __future__ import annotations

import os
import py_compile
import sys
import tempfile
import zipfile
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
ARCHIVE = os.path.join(OUT, "boundflow_ref.zip")
STAMP = os.path.join(OUT, "PYTHON_VERSION")


def default_checkout() -> Optional[str]:
    """$BOUNDFLOW_REFERENCE, else a directory named `reference` beside this repository."""
    cand = os.environ.get("BOUNDFLOW_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "boundflow", "__init__.py")) else None


def make_ref(checkout: str, quiet: bool = False) -> str:
    src_root = os.path.join(os.path.abspath(checkout), "boundflow")
    if not os.path.isfile(os.path.join(src_root, "__init__.py")):
        raise FileNotFoundError(f"{checkout} does not contain the boundflow package")
    os.makedirs(OUT, exist_ok=True)
    n = 0
    with tempfile.TemporaryDirectory() as tmp, zipfile.ZipFile(ARCHIVE + ".tmp", "w", zipfile.ZIP_DEFLATED) as zf:
        for dirpath, dirnames, filenames in os.walk(src_root):
            dirnames[:] = sorted(d for d in dirnames if d not in ("__pycache__", "3rdparty"))
            rel = os.path.relpath(dirpath, src_root)
            pkg = "boundflow" if rel == "." else os.path.join("boundflow", rel)
            zf.writestr(pkg + "/", "")  # explicit directory entry: packages without __init__ import as namespace portions
            for f in sorted(filenames):
                if not f.endswith(".py"):
                    continue
                cfile = os.path.join(tmp, "m.pyc")
                py_compile.compile(os.path.join(dirpath, f), cfile=cfile, dfile=os.path.join(pkg, f), doraise=True,
                                   invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH)
                zf.write(cfile, os.path.join(pkg, f + "c"))
                n += 1
    os.replace(ARCHIVE + ".tmp", ARCHIVE)
    with open(STAMP, "w") as fh:
        fh.write("%d.%d\n" % sys.version_info[:2])
    if not quiet:
        print(f"compiled {n} modules of {src_root} into {ARCHIVE}")
    return ARCHIVE


def ref_path() -> Optional[str]:
    """Path to put on sys.path to import the reference (the bytecode archive), or None when `oracle/_ref` has not
    been built (or was built by another interpreter version)."""
    if not os.path.isfile(ARCHIVE) or not os.path.isfile(STAMP):
        return None
    with open(STAMP) as fh:
        if fh.read().strip() != "%d.%d" % sys.version_info[:2]:
            return None
    return ARCHIVE


if __name__ == "__main__":
    src = sys.argv[1] if len(sys.argv) > 1 else default_checkout()
    if not src:
        raise SystemExit("usage: python oracle/make_ref.py /path/to/boundflow-checkout")
    make_ref(src)
