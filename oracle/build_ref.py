"""TEST INFRASTRUCTURE ONLY (checker, never the product path).

Recipe that compiles the reference's own CPU operator sources, where they lie
under the reference checkout, into ``oracle/_ref/mega_ref_cpu.so``.

Sources compiled (nothing is copied into this repository):
  fairseq/csrc/ops/ema_hidden.cc       (EMAHiddenCPUFwdImpl,      :15-64)
  fairseq/csrc/ops/ema_parameters.cc   (EMAParametersCPUFwdImpl,  :17-78)
  fairseq/csrc/ops/sequence_norm.cc    (SequenceNormCPUFwd*Impl,  :258-372, :531-655)
  fairseq/csrc/ops/timestep_norm.cc    (TimestepNormCPUFwdImpl,   :23-103, :218-316)
plus ``oracle/ref_glue.cc`` (this repository's linker glue for the CUDA entry
points those files reference).  The reference's own build system is not run.

The built module exposes ``ops.{ema_hidden_fwd, ema_parameters_fwd,
sequence_norm_fwd, group_sequence_norm_fwd, timestep_norm_fwd,
group_timestep_norm_fwd}`` with the signatures the reference's Python wrappers
call (fairseq/modules/fused_ops/*.py, fairseq/modules/norm_layer/*.py).

Usage:  python oracle/build_ref.py [--reference /path/to/fairseq-apollo]
"""
import argparse
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MOD_NAME = "mega_ref_cpu"
DEFAULT_REFERENCE = os.environ.get("MEGA_REFERENCE_ROOT", "/root/reference")


def so_path():
    return os.path.join(OUT_DIR, MOD_NAME + ".so")


def build(reference_root=DEFAULT_REFERENCE, verbose=False):
    """Compile the reference CPU ops. Returns the path of the built .so."""
    from torch.utils.cpp_extension import load

    csrc = os.path.join(reference_root, "fairseq", "csrc")
    srcs = [os.path.join(csrc, "ops", f) for f in
            ("ema_hidden.cc", "ema_parameters.cc", "sequence_norm.cc", "timestep_norm.cc")]
    for s in srcs:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    os.makedirs(OUT_DIR, exist_ok=True)
    load(name=MOD_NAME, sources=srcs + [os.path.join(HERE, "ref_glue.cc")],
         extra_include_paths=[csrc], extra_cflags=["-O2", "-std=c++17"],
         build_directory=OUT_DIR, verbose=verbose, is_python_module=True)
    return so_path()


CUDA_MOD_NAME = "mega_ref_cuda"


def cuda_so_path():
    return os.path.join(OUT_DIR, CUDA_MOD_NAME + ".so")


def build_cuda(reference_root=DEFAULT_REFERENCE, verbose=False):
    """Compile the reference's whole native extension (CPU + CUDA operators, the 16 sources its
    setup.py lists for ``fairseq.mega2_extension``) for sm_100 into
    ``oracle/_ref/mega_ref_cuda.so``: the reference's own GPU path, to compare against and to time
    on the GPU box.  nvcc cross-compiles without a GPU; the reference's build system is not run."""
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load

    csrc = os.path.join(reference_root, "fairseq", "csrc")
    names = ["blas.cc", "mega2_extension.cc"]
    for op in ("attention_softmax", "attention", "ema_parameters", "ema_hidden", "fftconv", "sequence_norm",
               "timestep_norm"):
        names += ["ops/%s.cc" % op, "ops/%s_kernel.cu" % op]
    srcs = [os.path.join(csrc, n) for n in names]
    for s in srcs:
        if not os.path.exists(s):
            raise FileNotFoundError(s)
    os.makedirs(OUT_DIR, exist_ok=True)
    import tempfile
    build_dir = os.path.join(tempfile.gettempdir(), "mega_ref_cuda_build")  # objects stay out of the tree
    os.makedirs(build_dir, exist_ok=True)
    load(name=CUDA_MOD_NAME, sources=srcs, extra_include_paths=[csrc], extra_cflags=["-O3", "-std=c++17"],
         # at::Context::alertCuBLASConfigNotDeterministic() (a warning hook the reference calls before
         # its cuBLAS GEMMs) no longer exists in the installed torch; the define maps the call onto a
         # harmless getter so that the untouched sources still compile
         extra_cuda_cflags=["-O3", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda",
                            "-DalertCuBLASConfigNotDeterministic=deterministicAlgorithms"],
         extra_ldflags=["-lcublas"], with_cuda=True, build_directory=build_dir, verbose=verbose,
         is_python_module=False)  # its init symbol is the reference's PyInit_mega2_extension, see load_ref_cuda
    import shutil
    shutil.copy2(os.path.join(build_dir, CUDA_MOD_NAME + ".so"), cuda_so_path())
    return cuda_so_path()


# The Mega block itself (the caller of this library's modules) as the reference wrote it: Python files
# staged, unmodified, under oracle/_ref/py (git-ignored, travels to the GPU box like the .so files) so
# that a GPU test can run the reference's own MovingAverageGatedAttention with this package's classes
# swapped in for its EMA / norm / attention imports.
BLOCK_FILES = (
    "incremental_decoding_utils.py",
    "modules/moving_average_gated_attention.py",
    "modules/fairseq_dropout.py",
    "modules/relative_positional_bias.py",
    "modules/normalized_feedforward_network.py",
    "modules/norm_layer/layer_norm.py",
    # the wrappers that call fairseq.mega2_extension.ops by name (operator-level drop-in test)
    "modules/norm_layer/timestep_norm.py",
    "modules/norm_layer/sequence_norm.py",
    "modules/attention_softmax.py",
    "modules/efficient_attention.py",
)


def py_dir():
    return os.path.join(OUT_DIR, "py")


def stage_block_sources(reference_root=DEFAULT_REFERENCE):
    """Copy the reference's block-level Python files (BLOCK_FILES) to oracle/_ref/py/fairseq/...;
    returns that directory.  Nothing is edited."""
    import shutil
    for rel in BLOCK_FILES:
        src = os.path.join(reference_root, "fairseq", rel)
        if not os.path.exists(src):
            raise FileNotFoundError(src)
        dst = os.path.join(py_dir(), "fairseq", rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copy2(src, dst)
    return py_dir()


def load_reference_block(swap):
    """Import the staged reference block with ``swap`` (a dict: class name -> class) standing in for
    the classes it imports from fairseq.modules.{exponential_moving_average, complex_exponential_moving_average,
    norm_layer.timestep_norm, norm_layer.sequence_norm, efficient_attention, attention_softmax}.
    Returns the module ``fairseq.modules.moving_average_gated_attention`` (None when nothing is
    staged).  The placeholder ``fairseq`` packages it installs in sys.modules are private to the
    test process."""
    import types

    import torch
    import torch.nn.functional as F
    root = os.path.join(py_dir(), "fairseq")
    if not os.path.exists(os.path.join(root, "modules", "moving_average_gated_attention.py")):
        return None

    def pkg(name, path=None):
        m = types.ModuleType(name)
        m.__path__ = [path] if path else []
        sys.modules[name] = m
        return m

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, rel))
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        return m

    fs = pkg("fairseq", root)
    utils = pkg("fairseq.utils")   # the one helper the softmax branch of the block calls (fairseq/utils.py)
    utils.softmax = lambda x, dim, onnx_trace=False: F.softmax(x.float(), dim=dim, dtype=torch.float32)
    fs.utils = utils
    pkg("fairseq.modules", os.path.join(root, "modules"))
    pkg("fairseq.modules.norm_layer", os.path.join(root, "modules", "norm_layer"))
    load("fairseq.incremental_decoding_utils", "incremental_decoding_utils.py")
    load("fairseq.modules.fairseq_dropout", "modules/fairseq_dropout.py")
    load("fairseq.modules.relative_positional_bias", "modules/relative_positional_bias.py")
    load("fairseq.modules.norm_layer.layer_norm", "modules/norm_layer/layer_norm.py")
    for mod, names in (("fairseq.modules.exponential_moving_average", ("MultiHeadEMA",)),
                       ("fairseq.modules.complex_exponential_moving_average", ("MultiHeadComplexEMA",)),
                       ("fairseq.modules.norm_layer.timestep_norm", ("TimestepNorm",)),
                       ("fairseq.modules.norm_layer.sequence_norm", ("SequenceNorm",)),
                       ("fairseq.modules.efficient_attention", ("EfficientAttention",)),
                       ("fairseq.modules.attention_softmax", ("AttentionSoftmax",))):
        m = pkg(mod)
        for n in names:
            setattr(m, n, swap[n])
    load("fairseq.modules.normalized_feedforward_network", "modules/normalized_feedforward_network.py")
    return load("fairseq.modules.moving_average_gated_attention", "modules/moving_average_gated_attention.py")


def load_reference_wrappers(ops_module):
    """Import the staged reference wrappers (norm_layer/timestep_norm.py, norm_layer/sequence_norm.py,
    attention_softmax.py, efficient_attention.py) with ``ops_module`` bound as
    ``fairseq.mega2_extension.ops``, the name they import.  Returns the four modules in that order,
    or None when nothing is staged."""
    import types
    root = os.path.join(py_dir(), "fairseq")
    if not os.path.exists(os.path.join(root, "modules", "norm_layer", "timestep_norm.py")):
        return None

    def pkg(name, path=None):
        m = types.ModuleType(name)
        m.__path__ = [path] if path else []
        sys.modules[name] = m
        return m

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, rel))
        m = importlib.util.module_from_spec(spec)
        sys.modules[name] = m
        spec.loader.exec_module(m)
        return m

    pkg("fairseq", root)
    ext = pkg("fairseq.mega2_extension")
    ext.ops = ops_module
    sys.modules["fairseq.mega2_extension.ops"] = ops_module
    pkg("fairseq.modules", os.path.join(root, "modules"))
    pkg("fairseq.modules.norm_layer", os.path.join(root, "modules", "norm_layer"))
    load("fairseq.incremental_decoding_utils", "incremental_decoding_utils.py")
    return (load("fairseq.modules.norm_layer.timestep_norm", "modules/norm_layer/timestep_norm.py"),
            load("fairseq.modules.norm_layer.sequence_norm", "modules/norm_layer/sequence_norm.py"),
            load("fairseq.modules.attention_softmax", "modules/attention_softmax.py"),
            load("fairseq.modules.efficient_attention", "modules/efficient_attention.py"))


def load_ref_cuda():
    """Import the prebuilt CUDA build of the reference extension; None when it was never built."""
    p = cuda_so_path()
    if not os.path.exists(p):
        return None
    import torch  # noqa: F401
    if CUDA_MOD_NAME in sys.modules:
        return sys.modules[CUDA_MOD_NAME]
    # the reference names its module "mega2_extension" in PYBIND11_MODULE (mega2_extension.cc:14)
    spec = importlib.util.spec_from_file_location("mega2_extension", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[CUDA_MOD_NAME] = mod
    return mod


def load_ref():
    """Import the prebuilt ``oracle/_ref`` module; None when it was never built."""
    p = so_path()
    if not os.path.exists(p):
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    if MOD_NAME in sys.modules:
        return sys.modules[MOD_NAME]
    spec = importlib.util.spec_from_file_location(MOD_NAME, p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[MOD_NAME] = mod
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--cuda", action="store_true", help="also build the reference's CUDA operators (minutes)")
    a = ap.parse_args()
    print(build(a.reference, a.verbose))
    print(stage_block_sources(a.reference))
    if a.cuda:
        print(build_cuda(a.reference, a.verbose))
