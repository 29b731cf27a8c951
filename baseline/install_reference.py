"""Put the unmodified reference package ``kla`` (and its test files) under
``baseline/_ref/`` so that it travels with this tree to a machine that has no
copy of the reference checkout.

    python baseline/install_reference.py [<reference checkout>]

``kla`` is pure Python (its imports need ``torch`` only; ``tyro`` for the
command line), so an install is a copy of ``src/kla``: that is what
``pip install --target`` would leave behind, and pip itself cannot build the
project offline (its build backend ``uv_build`` is not available). The
reference's ``tests/`` are copied next to it because its parity matrix
(``tests/test_backends.py``) is run against the ``b200`` backend.

``baseline/_ref/`` is git-ignored: nothing of the reference enters this
repository's history. ``MANIFEST.json`` records the SHA-256 of every file
copied, and :func:`verify` checks them, so a run can state that what it timed
or tested against is the reference as shipped.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
MANIFEST = os.path.join(DEST, "MANIFEST.json")
_KEEP = (".py", ".cu", ".cuh", ".metal", ".typed", ".h")


def default_source() -> str:
    """``$KLA_REFERENCE_ROOT``, else a checkout named ``reference`` beside this repository."""
    return os.environ.get("KLA_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _sha(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def _copy_tree(src: str, dst: str, files: dict, rel_root: str) -> None:
    for dirpath, dirnames, filenames in os.walk(src):
        dirnames[:] = [d for d in dirnames if d != "__pycache__"]
        for name in filenames:
            if not name.endswith(_KEEP):
                continue
            s = os.path.join(dirpath, name)
            rel = os.path.relpath(s, src)
            d = os.path.join(dst, rel)
            os.makedirs(os.path.dirname(d), exist_ok=True)
            shutil.copyfile(s, d)
            files[os.path.join(rel_root, rel)] = _sha(d)


def install(source: str | None = None) -> str:
    """Copy ``<source>/src/kla`` and ``<source>/tests`` into ``baseline/_ref``. Returns the destination."""
    source = source or default_source()
    pkg = os.path.join(source, "src", "kla")
    if not os.path.isdir(pkg):
        raise FileNotFoundError(f"no reference package at {pkg}")
    for sub in ("kla", "tests"):
        shutil.rmtree(os.path.join(DEST, sub), ignore_errors=True)
    os.makedirs(DEST, exist_ok=True)
    files: dict = {}
    _copy_tree(pkg, os.path.join(DEST, "kla"), files, "kla")
    tests = os.path.join(source, "tests")
    if os.path.isdir(tests):
        _copy_tree(tests, os.path.join(DEST, "tests"), files, "tests")
    version = "unknown"
    try:
        with open(os.path.join(source, "pyproject.toml")) as f:
            for line in f:
                if line.startswith("version"):
                    version = line.split("=", 1)[1].strip().strip('"')
                    break
    except OSError:
        pass
    with open(MANIFEST, "w") as f:
        json.dump({"package": "kla", "version": version, "how": "copy of src/kla and tests/", "files": files}, f, indent=1)
    return DEST


def installed() -> bool:
    return os.path.isfile(os.path.join(DEST, "kla", "__init__.py")) and os.path.isfile(MANIFEST)


def verify() -> int:
    """Check every installed file against the manifest; returns the number of files. Raises on a mismatch."""
    with open(MANIFEST) as f:
        files = json.load(f)["files"]
    for rel, sha in files.items():
        if _sha(os.path.join(DEST, rel)) != sha:
            raise RuntimeError(f"baseline/_ref/{rel} differs from the reference file it was copied from")
    return len(files)


def add_to_path() -> str:
    """Make ``import kla`` resolve to the installed copy. Returns its parent directory."""
    if not installed():
        raise FileNotFoundError("the reference is not installed under baseline/_ref (run baseline/install_reference.py)")
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    return DEST


if __name__ == "__main__":
    dest = install(sys.argv[1] if len(sys.argv) > 1 else None)
    print(f"installed the reference into {dest} ({verify()} files)")
