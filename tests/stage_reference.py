"""Stage the few UNMODIFIED reference files that the drop-in tests import into baseline/_ref/ (git-ignored; it travels to the
GPU box with the working tree, where the reference checkout itself does not exist), and cross-compile the reference's GEMM
extension into oracle/_ref/ (oracle/build_ref.py).

    python tests/stage_reference.py [--reference /path/to/Jetfire-INT8Training]

Staged: INT8_GPT2/qmodel.py (the caller of the hot path), Jetfire/Linear/{__init__,linear_fwd,linear_bwd}.py (the glue on
top of the `BlockQuantizeCUDA` extension) and the Triton operators Jetfire/Nonlinear/*.py.  tests/test_gpu_dropin.py and
tests/test_gpu_reference_triton.py skip when neither $JETFIRE_REFERENCE nor baseline/_ref holds them.  Nothing staged here is
imported by the package, by the timed region of bench.py's own arm or by any CPU test.
"""
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGE = os.path.join(ROOT, "baseline", "_ref")
DEFAULT_REFERENCE = "/root/reference"
FILES = ["INT8_GPT2/qmodel.py", "Jetfire/Linear/__init__.py", "Jetfire/Linear/linear_fwd.py", "Jetfire/Linear/linear_bwd.py"]
FILES += [f"Jetfire/Nonlinear/{m}.py" for m in ("__init__", "add", "add_mean_var", "common", "dequantize", "gelu_bwd", "gelu_fwd",
                                                "layernorm", "quantize", "quantize_transpose", "transpose", "utils")]


def reference_files_root():
    """Directory that holds the reference files: an actual checkout if one is reachable, else the staged copies, else None."""
    for cand in (os.environ.get("JETFIRE_REFERENCE"), DEFAULT_REFERENCE, STAGE):
        if cand and all(os.path.exists(os.path.join(cand, f)) for f in FILES):
            return cand
    return None


def stage(reference=None):
    src = reference or os.environ.get("JETFIRE_REFERENCE") or DEFAULT_REFERENCE
    if not all(os.path.exists(os.path.join(src, f)) for f in FILES):
        raise SystemExit(f"no reference checkout at {src}")
    for f in FILES:
        dst = os.path.join(STAGE, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(src, f), dst)
    return STAGE


if __name__ == "__main__":
    ref = sys.argv[sys.argv.index("--reference") + 1] if "--reference" in sys.argv else None
    print(stage(ref))
    sys.path.insert(0, ROOT)
    from oracle import build_ref
    print(build_ref.build(ref))
