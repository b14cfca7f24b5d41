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
    a = ap.parse_args()
    print(build(a.reference, a.verbose))
