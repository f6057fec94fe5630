"""Place the reference's own Python beside the oracle so that it can run where the reference checkout is absent.

TEST INFRASTRUCTURE.  ``python -m oracle.make_ref [/path/to/reference]`` copies the five files of the
reference's integer training path (``ti_torch.py``, ``ti_loss.py``, ``ti_net.py``, ``ti_vgg.py`` and the
``options.py`` they import) unmodified into ``oracle/_ref/``.  That folder is listed in ``.gitignore``: the
copies are never committed, they are a local install of the reference like a compiled ``.so`` would be.
``oracle/ref_harness.py`` imports them from there; the benchmark's ``--impl reference`` arm times them on
the host cores and the extension-level drop-in test runs them on the GPU over this library's kernels.
Nothing under ``niti_b200/`` reads the folder.
"""
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_OUT = os.path.join(HERE, "_ref")
FILES = ("ti_torch.py", "ti_loss.py", "ti_net.py", "ti_vgg.py", "options.py")


def available():
    """True when every file of the reference's path sits in oracle/_ref."""
    return all(os.path.isfile(os.path.join(REF_OUT, f)) for f in FILES)


def make(ref_dir):
    if not all(os.path.isfile(os.path.join(ref_dir, f)) for f in FILES):
        raise FileNotFoundError(f"{ref_dir} does not hold {', '.join(FILES)}")
    os.makedirs(REF_OUT, exist_ok=True)
    digest = hashlib.sha256()
    for f in FILES:
        shutil.copyfile(os.path.join(ref_dir, f), os.path.join(REF_OUT, f))
        with open(os.path.join(REF_OUT, f), "rb") as fh:
            digest.update(fh.read())
    with open(os.path.join(REF_OUT, "SOURCE.txt"), "w") as fh:
        fh.write(f"unmodified copies of {', '.join(FILES)} from a checkout of wangmaolin/niti\nsha256 of the five files, concatenated: {digest.hexdigest()}\n")
    return REF_OUT


if __name__ == "__main__":
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NITI_REFERENCE_DIR")
    if not src:
        raise SystemExit("usage: python -m oracle.make_ref /path/to/reference   (or set NITI_REFERENCE_DIR)")
    print(make(src))
