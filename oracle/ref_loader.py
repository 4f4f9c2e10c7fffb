"""Import the staged reference (oracle/_ref, made by oracle/make_ref.py).  TEST INFRASTRUCTURE ONLY.

``load()`` returns the reference's ``nanochat`` package: its own gpt.py / engine.py /
flash_attention.py, unmodified, imported from oracle/_ref.  On a CUDA machine the reference picks
bf16 as its compute dtype and, on anything but Hopper, its SDPA attention path — which is "the
reference's bf16 GPU path" the parity tests and the GPU leg of the benchmark compare against.
Raises FileNotFoundError when the staging step has not been run (the callers fail, they do not skip).
"""
import importlib
import os
import sys

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available():
    return os.path.isfile(os.path.join(REF_DIR, "nanochat", "gpt.py"))


def load(dtype=None):
    """The reference package; ``dtype`` ("bfloat16" / "float32") pins its compute dtype on first import."""
    if not available():
        raise FileNotFoundError(f"{REF_DIR} is empty: run `python oracle/make_ref.py <reference checkout>` where the "
                                "reference is mounted (the driver hook build() does it)")
    if "nanochat" in sys.modules and not getattr(sys.modules["nanochat"], "__file__", "").startswith(REF_DIR):
        raise RuntimeError("another package named nanochat is already imported")
    if dtype is not None and "nanochat.common" not in sys.modules:
        os.environ["NANOCHAT_DTYPE"] = dtype
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    pkg = importlib.import_module("nanochat")
    for name in ("common", "flash_attention", "gpt", "engine"):
        importlib.import_module("nanochat." + name)
    return pkg
