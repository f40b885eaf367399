"""Makes oracle/_ref/: the reference's own plain-torch module, for timing beside the kernels.

    python oracle/make_ref.py [path of a checkout of qflen/nsa-from-scratch]

Test infrastructure, not product: only bench.py's CPU-baseline leg loads what this leaves behind.
The reference's CPU path is one self-contained Python file (nsa/reference.py: torch and the standard
library only), so "building" it is placing that file, unmodified, where the benchmark can import it on a
machine that has no checkout.  oracle/_ref/ is not tracked (it is listed in .gitignore); nothing of the
reference's source enters this repository's history.  Without a checkout this script does nothing and
the benchmark reports the oracle port only."""
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def default_checkout() -> str:
    """$NSA_REFERENCE_CHECKOUT, else a directory named `reference` beside this repository."""
    return os.environ.get("NSA_REFERENCE_CHECKOUT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def make(checkout: str | None = None) -> str | None:
    src = os.path.join(checkout or default_checkout(), "nsa", "reference.py")
    if not os.path.isfile(src):
        return None
    dst_dir = os.path.join(HERE, "_ref")
    os.makedirs(dst_dir, exist_ok=True)
    dst = os.path.join(dst_dir, "nsa_reference.py")
    shutil.copyfile(src, dst)
    with open(os.path.join(dst_dir, "SOURCE"), "w") as f:
        f.write(f"nsa/reference.py of the reference checkout, unmodified; sha256 {hashlib.sha256(open(src, 'rb').read()).hexdigest()}\n")
    return dst


if __name__ == "__main__":
    print(make(*sys.argv[1:2]) or "no checkout found: nothing made")
