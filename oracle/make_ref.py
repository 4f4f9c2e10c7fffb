"""Stage the reference's own modules of this path under oracle/_ref/.  TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py <path of the reference checkout>

The reference is pure Python, so "building" it means placing unmodified copies of the few modules
the path imports where the GPU tests can import them: oracle/_ref/nanochat/{__init__, common, gpt,
engine, flash_attention, optim, checkpoint_manager, tokenizer}.py, plus a stand-in module for the
`rustbpe` wheel (imported by the tokenizer module at load time, never used on this path).
oracle/_ref/ is a build output: it is listed in .gitignore (no reference source enters the
history) and travels with the working tree to wherever the tests run.  A manifest with the
SHA-256 of every staged file is written beside them.  Only tests/ and the reference arm of bench.py
load anything from there (through oracle/ref_loader.py); nothing in the product does.
"""
import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES = ["__init__.py", "common.py", "gpt.py", "engine.py", "flash_attention.py", "optim.py",
           "checkpoint_manager.py", "tokenizer.py"]
RUSTBPE_STUB = '"""Stand-in for the rustbpe wheel: the tokenizer module imports it, this path never calls it."""\n'


def stage(ref_root):
    src_pkg = os.path.join(ref_root, "nanochat")
    missing = [m for m in MODULES if not os.path.isfile(os.path.join(src_pkg, m))]
    if missing:
        raise FileNotFoundError(f"{src_pkg} lacks {missing}")
    dst_pkg = os.path.join(OUT, "nanochat")
    os.makedirs(dst_pkg, exist_ok=True)
    manifest = {}
    for m in MODULES:
        shutil.copyfile(os.path.join(src_pkg, m), os.path.join(dst_pkg, m))
        with open(os.path.join(dst_pkg, m), "rb") as f:
            manifest["nanochat/" + m] = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(OUT, "rustbpe.py"), "w") as f:
        f.write(RUSTBPE_STUB)
    with open(os.path.join(OUT, "MANIFEST.json"), "w") as f:
        json.dump({"source": "unmodified copies of the reference's nanochat/ modules", "sha256": manifest}, f, indent=1)
    return OUT


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    print(stage(sys.argv[1]))
