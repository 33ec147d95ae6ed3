"""Build the reference's own GEMM extension (`BlockQuantizeCUDA`) for sm_100 from the reference checkout.  TEST INFRASTRUCTURE.

    python oracle/build_ref.py [--reference /path/to/Jetfire-INT8Training] [--force]

The sources are compiled WHERE THEY LIE in the checkout (JetfireGEMMKernel/BlockQuantize/cpp_extension/**, the file list and
flags of JetfireGEMMKernel/setup.py:9-42, with the architecture fixed to sm_100 because no GPU is needed to cross-compile);
nothing is copied, the only output is `oracle/_ref/BlockQuantizeCUDA.so` (git-ignored).  These are the reference's WMMA
kernels recompiled for Blackwell's legacy tensor path.  They serve two purposes, both on a GPU box only:
  * a second pin of the GEMM oracle: the reference's own kernels against the CPU restatement at the reference's own test
    shapes (tolerance-level, the reference builds with -use_fast_math), tests/test_gpu_reference_ext.py;
  * the GPU-side baseline timing of `bench.py --impl reference --workload gemm_sweep`.
`load_nonlinear()` imports the reference's Triton operators (Jetfire/Nonlinear/*.py, nothing to build) for the same two uses:
tests/test_gpu_reference_triton.py and `bench.py --impl reference --workload nonlinear`.
The checkout is found through --reference, $JETFIRE_REFERENCE, or the default location DEFAULT_REFERENCE; without one this script
does nothing.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "BlockQuantizeCUDA.so")
DEFAULT_REFERENCE = "/root/reference"

SOURCES = [
    "igemm/igemm_BlockSquare32OutputIntQuantizeStochastic.cu",
    "igemm/igemm_BlockSquare32OutputIntQuantizeBiasRowCol.cu",
    "igemm/igemm_BlockSquare32OutputIntQuantizeBiasRowRow.cu",
    "igemm/igemm_BlockSquare32OutputIntQuantize.cu",
    "igemm/igemm_BlockSquare32OutputIntQuantizeTrash.cu",
    "igemm/igemm_BlockSquare32OutputFp.cu",
    "igemm/igemm_BasicInt8Gemm.cu",
    "hgemm.cu",
    "bindings.cpp",
]


def reference_root(arg=None):
    for cand in (arg, os.environ.get("JETFIRE_REFERENCE"), DEFAULT_REFERENCE):
        if cand and os.path.isdir(os.path.join(cand, "JetfireGEMMKernel", "BlockQuantize", "cpp_extension")):
            return cand
    return None


def build(reference=None, force=False, verbose=False):
    """Returns the path of the built module, or None when no reference checkout is available."""
    root = reference_root(reference)
    if root is None:
        return OUT if os.path.exists(OUT) else None
    ext = os.path.join(root, "JetfireGEMMKernel", "BlockQuantize", "cpp_extension")
    srcs = [os.path.join(ext, s) for s in SOURCES]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(s) for s in srcs):
        return OUT
    from torch.utils import cpp_extension as ce
    import torch
    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(OUT_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{os.path.join(ext, 'include')}", f"-I{sysconfig.get_paths()['include']}"]
    defs = ["-DTORCH_EXTENSION_NAME=BlockQuantizeCUDA", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    nvcc = os.environ.get("NVCC", "nvcc")
    objs, procs = [], []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.basename(s) + ".o")
        objs.append(o)
        if s.endswith(".cu"):
            cmd = [nvcc, "-c", s, "-o", o, "-std=c++17", "-O3", "--compiler-options", "-fPIC",
                   "-gencode=arch=compute_100,code=sm_100", "-use_fast_math", "-U__CUDA_NO_HALF_OPERATORS__",
                   "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__", "--expt-relaxed-constexpr"] + inc + defs
        else:
            cmd = ["g++", "-c", s, "-o", o, "-std=c++17", "-O2", "-fPIC"] + inc + defs
        procs.append((s, subprocess.Popen(cmd, stdout=None if verbose else subprocess.DEVNULL,
                                          stderr=None if verbose else subprocess.PIPE)))
    for s, p in procs:
        _, err = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"compiling {s} failed:\n{(err or b'').decode()[-4000:]}")
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
    link = ["g++", "-shared", "-o", OUT] + objs + [f"-L{libdir}", f"-L{cuda_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
                                                   "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
                                                   f"-Wl,-rpath,{libdir}"]
    subprocess.check_call(link)
    return OUT


def load():
    """Import the built reference extension WITHOUT registering it as `BlockQuantizeCUDA` in sys.modules (that name belongs to
    this repository's drop-in shim once compat.install() has run).  Returns None when it has not been built."""
    if not os.path.exists(OUT):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location("BlockQuantizeCUDA", OUT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def nonlinear_root():
    """Directory holding the reference's Jetfire/Nonlinear/*.py: a checkout ($JETFIRE_REFERENCE, DEFAULT_REFERENCE) or the copies
    that tests/stage_reference.py staged into baseline/_ref/ (git-ignored) so that they exist on a GPU box."""
    staged = os.path.join(os.path.dirname(HERE), "baseline", "_ref")
    for cand in (os.environ.get("JETFIRE_REFERENCE"), DEFAULT_REFERENCE, staged):
        if cand and os.path.exists(os.path.join(cand, "Jetfire", "Nonlinear", "layernorm.py")):
            return cand
    return None


def load_nonlinear(first_config_only=False):
    """The reference's `Jetfire.Nonlinear` package (its Triton kernels, unmodified), imported under the private module name
    `_reference_jetfire_nonlinear` so that it never collides with the `Jetfire` name the drop-in shim registers; None when no
    reference files are reachable.  `first_config_only` cuts every kernel's autotuner to its first configuration (tile shape and
    stage count do not change results) to keep compilation short in parity tests; timing runs keep the full search."""
    import importlib
    import importlib.util
    root = nonlinear_root()
    if root is None:
        return None
    name = "_reference_jetfire_nonlinear"
    mod = sys.modules.get(name)
    if mod is None:
        pkg = os.path.join(root, "Jetfire", "Nonlinear")
        spec = importlib.util.spec_from_file_location(name, os.path.join(pkg, "__init__.py"), submodule_search_locations=[pkg])
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        try:
            spec.loader.exec_module(mod)
        except Exception:
            del sys.modules[name]
            raise
        # dequantize.py is not re-exported by the package's __init__ (Jetfire/Nonlinear/__init__.py:1-8)
        mod.int8_dequantize = importlib.import_module(name + ".dequantize").int8_dequantize
    if first_config_only:
        from triton.runtime.autotuner import Autotuner
        for sub in ("add", "add_mean_var", "dequantize", "gelu_bwd", "gelu_fwd", "layernorm", "quantize", "quantize_transpose",
                    "transpose"):
            m = importlib.import_module(name + "." + sub)
            for attr in dir(m):
                k = getattr(m, attr)
                while k is not None and not isinstance(k, Autotuner):
                    k = getattr(k, "fn", None)
                if k is not None:
                    k.configs = k.configs[:1]
    return mod


if __name__ == "__main__":
    ref = None
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build(ref, force="--force" in sys.argv, verbose="-v" in sys.argv))
