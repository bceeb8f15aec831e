"""Compiles the reference's own PyTorch implementation of this path into oracle/_ref/. TEST INFRASTRUCTURE, not product
code: only tests and bench.py's CPU arm load what this makes.

The reference's format specification and oracle for the NVFP4 KV-cache path is one pure-torch module,
nvidia-sm120/horizon_kvfp4/kernels/kv_fp4_ref.py (no TileLang, no vLLM imports: kv_fp4_ref.py:3-5). It is byte-compiled
from where it lies in the reference tree (the tree's location is the `reference_path` entry of BASELINE.json at the
repository root) into oracle/_ref/kv_fp4_ref.bytecode. No source is copied. The compiled module travels to a machine that
has no reference tree and lets `bench.py --impl reference` time the reference's own code there; `load()` returns None
when it has not been built, and the callers then fall back to the C restatement (oracle/kvfp4_oracle.c)."""
import importlib.machinery
import importlib.util
import json
import os
import py_compile
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
PYC = os.path.join(OUT_DIR, "kv_fp4_ref.bytecode")      # not "*.pyc": snapshot tools commonly skip that suffix
REL = os.path.join("nvidia-sm120", "horizon_kvfp4", "kernels", "kv_fp4_ref.py")
_mod = None


def reference_source():
    """path of the reference's module, or None when the reference tree is not on this machine"""
    try:
        base = json.load(open(os.path.join(os.path.dirname(HERE), "BASELINE.json")))["reference_path"]
    except Exception:  # noqa: BLE001
        return None
    src = os.path.join(base, REL)
    return src if os.path.exists(src) else None


def build(force: bool = False):
    """-> path of the compiled module, or None when there is no reference tree to compile from"""
    src = reference_source()
    if src is None:
        return PYC if os.path.exists(PYC) else None
    if force or not os.path.exists(PYC) or os.path.getmtime(PYC) < os.path.getmtime(src):
        os.makedirs(OUT_DIR, exist_ok=True)
        py_compile.compile(src, cfile=PYC, dfile="kv_fp4_ref.py", doraise=True)
        with open(os.path.join(OUT_DIR, "python_tag.txt"), "w") as f:
            f.write(sys.implementation.cache_tag + "\n")            # bytecode is specific to the interpreter version
    return PYC


def load():
    """the reference's kv_fp4_ref module (compiled), or None: not built, or built by another interpreter version"""
    global _mod
    if _mod is not None:
        return _mod
    tag = os.path.join(OUT_DIR, "python_tag.txt")
    if not os.path.exists(PYC) or not os.path.exists(tag) or open(tag).read().strip() != sys.implementation.cache_tag:
        return None
    try:
        loader = importlib.machinery.SourcelessFileLoader("kv_fp4_ref", PYC)
        spec = importlib.util.spec_from_loader("kv_fp4_ref", loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
    except Exception:  # noqa: BLE001  (a stale or foreign .pyc: treat as not built)
        return None
    _mod = mod
    return mod


if __name__ == "__main__":
    print(build(force=True))
