"""Builds the C++ front-end test programs into tests/cpp/_build/.

Two groups, both compiled with g++ -std=c++20 against include/ (the fusilli:: headers of this
backend) and tests/cpp/shim/ (a single-header stand-in for Catch2 plus the `utils.h` helpers the
reference's samples include), linked to fusilli_b200/libfusilli_b200.so:

  own_*   tests/cpp/*.cpp of this repository;
  ref_*   the reference project's sample and unit-test sources for the operators this backend
          implements, compiled UNCHANGED from the reference checkout (directory given by
          FUSILLI_REFERENCE_DIR, default: a `reference/` directory beside this repository) when that
          checkout is present. Nothing
          is copied: only the built programs land in tests/cpp/_build/.

Run as `python tests/cpp/build.py [-j N] [--only PATTERN]`.
"""
import concurrent.futures as cf
import fnmatch
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build")
REFERENCE = os.environ.get("FUSILLI_REFERENCE_DIR", os.path.normpath(os.path.join(ROOT, "..", "reference")))
CXX = os.environ.get("FUSILLI_TEST_CXX", "/usr/bin/g++")

OWN_SOURCES = ["test_frontend_host.cpp", "test_frontend_device.cpp", "host_execute_latency.cpp"]

# Reference programs that only need the graph API of the operators in scope. Paths are relative
# to the reference checkout. SDPA samples there go through a user-supplied MLIR custom op and
# custom ops need an MLIR compiler, so they are not listed. Of the dynamic-shape
# samples, the reduction one is an expected failure in the reference itself (it requires the
# IREE-specific non-zero transient size) and the custom-op one needs MLIR.
REFERENCE_SAMPLES = [
    "samples/convolution/conv_fprop_nchw_kcrs.cpp",
    "samples/convolution/conv_fprop_nchw_kcrs_grouped.cpp",
    "samples/convolution/conv_fprop_nhwc_krsc.cpp",
    "samples/convolution/conv_fprop_nhwc_krsc_with_pad.cpp",
    "samples/convolution/conv_fprop_with_bias.cpp",
    "samples/convolution/conv_fprop_with_relu.cpp",
    "samples/convolution/conv_fprop_with_relu_and_bias.cpp",
    "samples/convolution/conv_fprop_grouped_with_relu_and_bias.cpp",
    "samples/convolution/conv_dgrad_nhwc_krsc.cpp",
    "samples/convolution/conv_dgrad_nhwc_krsc_grouped.cpp",
    "samples/convolution/conv_wgrad_nhwc_krsc.cpp",
    "samples/convolution/conv_wgrad_nhwc_krsc_grouped.cpp",
    "samples/convolution/conv_wgrad_nhwc_krsc_grouped_strided.cpp",
    "samples/matmul/matmul_basic.cpp",
    "samples/matmul/matmul_basic_with_bias.cpp",
    "samples/matmul/matmul_batched.cpp",
    "samples/matmul/matmul_batched_with_bias.cpp",
    "samples/matmul/matmul_int4_fp16.cpp",
    "samples/pointwise/pointwise_add_transposed.cpp",
    "samples/pointwise/pointwise_binary_cmp_ops.cpp",
    "samples/pointwise/pointwise_binary_ops.cpp",
    "samples/pointwise/pointwise_bwd.cpp",
    "samples/pointwise/pointwise_scalar_mul.cpp",
    "samples/pointwise/pointwise_ternary_ops.cpp",
    "samples/pointwise/pointwise_unary_logical_ops.cpp",
    "samples/pointwise/pointwise_unary_ops.cpp",
    "samples/reduction/reduction_ops.cpp",
    "samples/layernorm/layernorm_infer_nchw.cpp",
    "samples/layernorm/layernorm_infer_nchw_scale_bias.cpp",
    "samples/layernorm/layernorm_infer_nhwc_scale_bias.cpp",
    "samples/layernorm/layernorm_train_nchw.cpp",
    "samples/layernorm/layernorm_train_nchw_scale_bias.cpp",
    "samples/layernorm/layernorm_train_nhwc_scale_bias.cpp",
    "samples/rmsnorm/rmsnorm_infer_nchw.cpp",
    "samples/rmsnorm/rmsnorm_infer_nchw_scale.cpp",
    "samples/rmsnorm/rmsnorm_infer_nhwc_scale.cpp",
    "samples/batchnorm/batchnorm_infer_nchw.cpp",
    "samples/batchnorm/batchnorm_infer_nchw_scale_bias.cpp",
    "samples/batchnorm/batchnorm_infer_nhwc_scale_bias.cpp",
    "samples/batchnorm/batchnorm_train_nchw.cpp",
    "samples/batchnorm/batchnorm_train_nchw_scale_bias.cpp",
    "samples/aot/single_backend.cpp",
    "samples/dynamic_shapes/conv_fprop_dynamic_batch.cpp",
    "samples/dynamic_shapes/sdpa_basic_dynamic_sequence.cpp",
]

# The SDPA samples share one helper translation unit (samples/sdpa_utils.cpp: graph set-up, a scalar
# reference, and a custom-op variant that this backend accepts at build time and refuses at
# compile); it is compiled once and linked into each of them. The dropout sample is disabled in
# the reference's own build.
REFERENCE_SDPA_UTILS = "samples/sdpa_utils.cpp"
REFERENCE_SDPA_SAMPLES = [
    "samples/sdpa/sdpa_fprop_basic_mha.cpp",
    "samples/sdpa/sdpa_fprop_causal.cpp",
    "samples/sdpa/sdpa_fprop_cross_attn.cpp",
    "samples/sdpa/sdpa_fprop_custom_scale.cpp",
    "samples/sdpa/sdpa_fprop_gqa.cpp",
    "samples/sdpa/sdpa_fprop_gqa_hk_ne_hv.cpp",
    "samples/sdpa/sdpa_fprop_with_mask.cpp",
]

# Reference unit tests that need no device (attribute and node validation, context, tensors).
REFERENCE_HOST_TESTS = [
    "tests/test_attributes.cpp",
    "tests/test_context.cpp",
    "tests/test_tensor_attributes.cpp",
    "tests/test_ssa_validation.cpp",
    "tests/test_cache.cpp",
    "tests/test_conv_attributes.cpp",
    "tests/test_conv_node.cpp",
    "tests/test_matmul_attributes.cpp",
    "tests/test_matmul_node.cpp",
    "tests/test_sdpa_attributes.cpp",
    "tests/test_sdpa_node.cpp",
    "tests/test_layernorm_attributes.cpp",
    "tests/test_layernorm_node.cpp",
    "tests/test_rmsnorm_attributes.cpp",
    "tests/test_rmsnorm_node.cpp",
    "tests/test_reduction_attributes.cpp",
    "tests/test_reduction_node.cpp",
    "tests/test_pointwise_attributes.cpp",
    "tests/test_pointwise_node.cpp",
    "tests/test_int_types.cpp",
    "tests/test_batchnorm_attributes.cpp",
    "tests/test_batchnorm_node.cpp",
]
# Not listed, because they exercise parts this backend does not have: test_graph (MLIR emission and
# the IREE compile cache), test_handle / test_buffer / test_utils (CPU and AMDGPU HAL devices),
# test_compile_*, test_dllib, test_process, test_memstream, test_extras, test_logging (compiler
# driver plumbing), test_float_types (software float types; half and bf16 are the compiler's native
# types here) and custom ops.


def _flags():
    lib_dir = os.path.join(ROOT, "fusilli_b200")
    return [
        "-std=c++20", "-O1", "-g0", "-w",
        "-I" + os.path.join(ROOT, "include"),
        "-I" + os.path.join(HERE, "shim"),
    ], ["-L" + lib_dir, "-lfusilli_b200", "-Wl,-rpath," + lib_dir,
        "-Wl,-rpath,$ORIGIN/../../../fusilli_b200", "-s"]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps if os.path.exists(d))


def _header_deps():
    deps = []
    for base in (os.path.join(ROOT, "include"), os.path.join(HERE, "shim")):
        for d, _, files in os.walk(base):
            deps += [os.path.join(d, f) for f in files]
    deps.append(os.path.join(ROOT, "fusilli_b200", "libfusilli_b200.so"))
    return deps


def _compile(src, exe, extra_includes, hdeps, objects=()):
    if _newer(exe, [src] + list(objects) + hdeps):
        return exe, 0, "up to date"
    cflags, ldflags = _flags()
    cmd = [CXX] + cflags + ["-I" + i for i in extra_includes] + [src] + list(objects) + ["-o", exe] + ldflags
    p = subprocess.run(cmd, capture_output=True, text=True)
    return exe, p.returncode, p.stderr[-4000:]


def _compile_object(src, obj, extra_includes, hdeps):
    """A helper translation unit without the shim's main()."""
    if _newer(obj, [src] + hdeps):
        return obj, 0, "up to date"
    cflags, _ = _flags()
    cmd = [CXX] + cflags + ["-DCATCH_SHIM_NO_MAIN", "-c"] + ["-I" + i for i in extra_includes] + [src, "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    return obj, p.returncode, p.stderr[-4000:]


def _sdpa_utils():
    """(source, object, include dirs) of the SDPA samples' shared helper, or None."""
    src = os.path.join(REFERENCE, REFERENCE_SDPA_UTILS)
    if not os.path.exists(src):
        return None
    return src, os.path.join(OUT, "ref_sdpa_utils.o"), [os.path.dirname(src)]


def jobs():
    """(source, executable, extra include dirs, extra objects) for everything that can be built here."""
    out = []
    for s in OWN_SOURCES:
        src = os.path.join(HERE, s)
        if os.path.exists(src):
            out.append((src, os.path.join(OUT, "own_" + os.path.splitext(s)[0]), [], []))
    if os.path.isdir(REFERENCE):
        for rel in REFERENCE_SAMPLES:
            src = os.path.join(REFERENCE, rel)
            if os.path.exists(src):
                name = os.path.splitext(os.path.basename(rel))[0]
                out.append((src, os.path.join(OUT, "ref_" + name), [os.path.dirname(src)], []))
        util = _sdpa_utils()
        for rel in REFERENCE_SDPA_SAMPLES if util else []:
            src = os.path.join(REFERENCE, rel)
            if os.path.exists(src):
                name = os.path.splitext(os.path.basename(rel))[0]
                out.append((src, os.path.join(OUT, "ref_" + name), [os.path.dirname(src)] + util[2], [util[1]]))
        # The unit tests include "utils.h", which the compiler looks up beside the including file
        # first. They are therefore compiled through a symbolic link in _build/links/, so that the
        # helper header of tests/cpp/shim/ is the one found. The link is not a copy of the source.
        links = os.path.join(OUT, "links")
        for rel in REFERENCE_HOST_TESTS:
            src = os.path.join(REFERENCE, rel)
            if os.path.exists(src):
                os.makedirs(links, exist_ok=True)
                link = os.path.join(links, os.path.basename(rel))
                if os.path.islink(link) or os.path.exists(link):
                    os.remove(link)
                os.symlink(src, link)
                name = os.path.splitext(os.path.basename(rel))[0]
                out.append((link, os.path.join(OUT, "ref_" + name), [], []))
    return out


def expected_programs():
    """Names of every program the lists above describe (built or not)."""
    own = ["own_" + os.path.splitext(s)[0] for s in OWN_SOURCES]
    ref_dev = ["ref_" + os.path.splitext(os.path.basename(r))[0] for r in REFERENCE_SAMPLES + REFERENCE_SDPA_SAMPLES]
    ref_host = ["ref_" + os.path.splitext(os.path.basename(r))[0] for r in REFERENCE_HOST_TESTS]
    return own, ref_dev, ref_host


def build(parallel=None, only=None):
    os.makedirs(OUT, exist_ok=True)
    lib = os.path.join(ROOT, "fusilli_b200", "libfusilli_b200.so")
    if not os.path.exists(lib):
        raise RuntimeError("build fusilli_b200/libfusilli_b200.so first (python -m fusilli_b200.build)")
    todo = [j for j in jobs() if only is None or fnmatch.fnmatch(os.path.basename(j[1]), only)]
    hdeps = _header_deps()
    failed = []
    util = _sdpa_utils()
    if util and os.path.isdir(REFERENCE) and any(objs for _, _, _, objs in todo):
        obj, rc, msg = _compile_object(util[0], util[1], util[2], hdeps)
        if rc != 0:
            failed.append((obj, msg))
    with cf.ThreadPoolExecutor(max_workers=parallel or os.cpu_count() or 4) as ex:
        futs = [ex.submit(_compile, s, e, inc, hdeps, objs) for s, e, inc, objs in todo if not failed]
        for f in cf.as_completed(futs):
            exe, rc, msg = f.result()
            if rc != 0:
                failed.append((exe, msg))
    shutil.rmtree(os.path.join(OUT, "links"), ignore_errors=True)  # dangling outside this machine
    for exe, msg in failed:
        sys.stderr.write("FAILED %s\n%s\n" % (os.path.basename(exe), msg))
    if failed:
        raise RuntimeError("%d C++ test program(s) failed to build" % len(failed))
    return [e for _, e, _, _ in todo]


if __name__ in ("__main__", "__graft_build__"):
    argv = sys.argv[1:] if __name__ == "__main__" else []
    par = int(argv[argv.index("-j") + 1]) if "-j" in argv else None
    pat = argv[argv.index("--only") + 1] if "--only" in argv else None
    built = build(par, pat)
    print("C++ front-end programs: %d in %s" % (len(built), os.path.relpath(OUT, ROOT)))
