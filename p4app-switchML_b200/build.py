"""Builds the native library and programs for sm_100a with nvcc and g++.

    python build.py            # incremental build of everything
    python build.py --clean    # remove build products first
    python build.py --jobs 8

Products (all inside this directory, never installed elsewhere):
    lib/libswitchml_b200.so        core + CPU backends + CUDA backend + C interface
    lib/libswitchml_b200.a         the same as a static archive
    lib/libswitchml_gemm.so        tcgen05 weight-gradient GEMM (loaded on demand)
    lib/torch_switchml.so          native c10d backend for PyTorch (python build.py --torch)
    build-checked/libswitchml_b200.so   the library with the kernels' bounds checks (--checked)
    lib/libnccl-net-switchml.so    NCCL collective-network plugin (bin/collnet_harness drives it)
    bin/switchml_switchd           stand-alone controller / software switch
    bin/hello_world, bin/allreduce_benchmark, bin/dnn_benchmark, bin/core_tests

The role of the reference's Makefiles (dev_root/Makefile, client_lib/Makefile,
benchmarks/Makefile, examples/Makefile) with their DEBUG/DUMMY/... switches: DEBUG=1 in
the environment builds with -O0 -g. `python build.py --sanitize thread` (or address)
builds the host-only parts and the native unit tests under that sanitizer as
build-<sanitizer>/core_tests (the reference has no sanitizer configuration at all).
"""
import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
OBJ = os.path.join(ROOT, "build", "obj")
LIB = os.path.join(ROOT, "lib")
BIN = os.path.join(ROOT, "bin")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
DEBUG = os.environ.get("DEBUG", "0") == "1"
OPT = ["-O0", "-g", "-DSWITCHML_DEBUG"] if DEBUG else ["-O3"]
DEFS = ["-DSWITCHML_CHECKED"] if os.environ.get("SWITCHML_CHECKED", "0") == "1" else []
# SANITIZE=thread|address builds the host code (and bin/core_tests) under that sanitizer into
# build-<name>/; used by the CPU race/memory checks, never for the GPU library in lib/.
SANITIZE = os.environ.get("SANITIZE", "")
INCLUDES = ["-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(ROOT, "csrc"),
            "-I" + os.path.join(CUDA_HOME, "include")]

LIB_SOURCES = [
    "csrc/core/log.cc", "csrc/core/config.cc", "csrc/core/job.cc", "csrc/core/utils.cc",
    "csrc/core/stats.cc", "csrc/core/scheduler.cc", "csrc/core/context.cc", "csrc/core/backend.cc",
    "csrc/ppp/cpu_exponent_quantizer_ppp.cc", "csrc/simd/simd_kernels.cc",
    "csrc/backends/dummy/dummy_backend.cc",
    "csrc/backends/softswitch/soft_switch.cc", "csrc/backends/softswitch/udp_backend.cc",
    "csrc/rendezvous/control.cc",
    "csrc/backends/cuda/driver_api.cc", "csrc/backends/cuda/fd_channel.cc",
    "csrc/backends/cuda/symmetric_memory.cc", "csrc/backends/cuda/cuda_backend.cc",
    "csrc/kernels/allreduce_kernels.cu",
    "csrc/capi/switchml_c.cc",
]
GEMM_SOURCES = ["csrc/kernels/wgrad_gemm.cu"]
NCCL_PLUGIN_SOURCES = ["csrc/nccl/collnet_plugin.cc"]
PROGRAMS = {
    "switchml_switchd": ["controller/switchd.cc"],
    "hello_world": ["examples/hello_world/main.cc"],
    "allreduce_benchmark": ["benchmarks/allreduce_benchmark.cc"],
    "dnn_benchmark": ["benchmarks/dnn_benchmark.cc"],
    "core_tests": ["csrc/tests/core_tests.cc", "csrc/tests/flag_protocol_model.cc"],
    "collnet_harness": ["csrc/nccl/collnet_harness.cc"],
}


def _headers_mtime():
    newest = 0.0
    for base in ("include", "csrc"):
        for d, _, files in os.walk(os.path.join(ROOT, base)):
            for f in files:
                if f.endswith((".h", ".cuh", ".inc")):
                    newest = max(newest, os.path.getmtime(os.path.join(d, f)))
    return newest


def _obj_path(src):
    return os.path.join(OBJ, src.replace("/", "_") + ".o")


def _compile(src, hdr_mtime, verbose):
    path = os.path.join(ROOT, src)
    obj = _obj_path(src)
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), hdr_mtime):
        return obj, None
    if src.endswith(".cu"):
        cmd = [NVCC] + ARCH + ["-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC,-Wall"] + OPT + DEFS + \
              INCLUDES + ["-c", path, "-o", obj]
    else:
        cmd = ["g++", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-pthread"] + \
              OPT + DEFS + INCLUDES + ["-c", path, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        return obj, "FAILED: %s\n%s%s" % (" ".join(cmd), r.stdout, r.stderr)
    if r.stderr.strip() and verbose:
        print(r.stderr)
    return obj, None


def _link(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed: %s\n%s%s" % (" ".join(cmd), r.stdout, r.stderr))


def build(jobs=None, verbose=False, programs=True):
    """Compile whatever is out of date. Returns the path of the main library."""
    for d in (OBJ, LIB, BIN):
        os.makedirs(d, exist_ok=True)
    jobs = jobs or max(1, (os.cpu_count() or 2))
    hdr = _headers_mtime()
    sources = list(LIB_SOURCES)
    gemm = [s for s in GEMM_SOURCES if os.path.exists(os.path.join(ROOT, s))]
    progs = {k: v for k, v in PROGRAMS.items()
             if programs and all(os.path.exists(os.path.join(ROOT, s)) for s in v)}
    plugin = [s for s in NCCL_PLUGIN_SOURCES if os.path.exists(os.path.join(ROOT, s))]
    every = sources + gemm + plugin + [s for v in progs.values() for s in v]
    errors = []
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        for obj, err in ex.map(lambda s: _compile(s, hdr, verbose), every):
            if err:
                errors.append(err)
    if errors:
        raise RuntimeError("\n".join(errors))

    def newer(target, objs):
        return not os.path.exists(target) or any(os.path.getmtime(o) > os.path.getmtime(target) for o in objs)

    main_lib = os.path.join(LIB, "libswitchml_b200.so")
    objs = [_obj_path(s) for s in sources]
    if newer(main_lib, objs):
        # cudart is linked statically, so the library loads on machines without a driver.
        _link([NVCC] + ARCH + ["-shared", "-o", main_lib] + objs + ["-lpthread", "-ldl", "-lrt"], verbose)
    # The same objects as a static archive (the reference's product is libswitchml-client.a);
    # link it with nvcc, or with g++ plus -lcudart_static -ldl -lrt -lpthread.
    static_lib = os.path.join(LIB, "libswitchml_b200.a")
    if newer(static_lib, objs):
        if os.path.exists(static_lib):
            os.remove(static_lib)
        _link(["ar", "rcs", static_lib] + objs, verbose)
    if gemm:
        gemm_lib = os.path.join(LIB, "libswitchml_gemm.so")
        gobjs = [_obj_path(s) for s in gemm]
        if newer(gemm_lib, gobjs):
            _link([NVCC] + ARCH + ["-shared", "-o", gemm_lib] + gobjs + ["-lpthread", "-ldl", "-lrt"], verbose)
    if plugin:
        # NCCL looks for libnccl-net-<NCCL_NET_PLUGIN>.so on the library path.
        plugin_lib = os.path.join(LIB, "libnccl-net-switchml.so")
        pobjs = [_obj_path(s) for s in plugin]
        if newer(plugin_lib, pobjs + [main_lib]):
            _link(["g++", "-shared", "-o", plugin_lib] + pobjs +
                  ["-L" + LIB, "-lswitchml_b200", "-Wl,-rpath,$ORIGIN", "-lpthread"], verbose)
    for name, srcs in progs.items():
        exe = os.path.join(BIN, name)
        pobjs = [_obj_path(s) for s in srcs]
        if newer(exe, pobjs + [main_lib]):
            _link([NVCC] + ARCH + ["-o", exe] + pobjs +
                  ["-L" + LIB, "-lswitchml_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib",
                   "-lpthread", "-ldl", "-lrt"], verbose)
    # A checked build that exists is kept in step with the sources (it exports the same C
    # interface as the main library and would otherwise go stale without anybody noticing).
    if os.path.isdir(os.path.join(ROOT, "build-checked")):
        build_checked(verbose, jobs)
    return main_lib


HOST_ONLY = [s for s in LIB_SOURCES if s.endswith(".cc") and "/cuda/" not in s and "capi" not in s and
             s != "csrc/core/backend.cc"]


def build_sanitized(kind, verbose=False):
    """Host-only build of the core + CPU backends + native tests with -fsanitize=<kind>.
    The cuda backend is replaced by a stub factory, so no CUDA library is involved."""
    out = os.path.join(ROOT, "build-" + kind)
    os.makedirs(out, exist_ok=True)
    stub = os.path.join(out, "cuda_stub.cc")
    with open(stub, "w") as f:
        f.write('#include "backends/cuda/cuda_backend.h"\n#include "switchml/log.h"\nnamespace switchml {\n'
                'Backend* CreateCudaBackend(Context&, Config&) { SML_LOG(FATAL) << "no cuda in this build"; return nullptr; }\n}\n')
    srcs = [os.path.join(ROOT, s) for s in HOST_ONLY + ["csrc/core/backend.cc", "csrc/tests/core_tests.cc",
                                                         "csrc/tests/flag_protocol_model.cc"]] + [stub]
    exe = os.path.join(out, "core_tests")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=" + kind, "-pthread"] + \
          INCLUDES + srcs + ["-o", exe]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("sanitized build failed:\n" + r.stdout + r.stderr)
    return exe


def build_checked(verbose=False, jobs=None):
    """build-checked/libswitchml_b200.so: the main library with -DSWITCHML_CHECKED, i.e. with
    the geometry checks of the aggregation kernels compiled in (a violation sets
    STATUS_BOUNDS and skips the access; nothing traps). Load it instead of lib/ by putting
    its path into SWITCHML_B200_LIBRARY. compute-sanitizer's role where that tool is not
    to be had."""
    out = os.path.join(ROOT, "build-checked")
    obj_dir = os.path.join(out, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    hdr = _headers_mtime()
    target = os.path.join(out, "libswitchml_b200.so")

    def one(src):
        path = os.path.join(ROOT, src)
        obj = os.path.join(obj_dir, src.replace("/", "_") + ".o")
        if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(path), hdr):
            return obj, None
        if src.endswith(".cu"):
            cmd = [NVCC] + ARCH + ["-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC,-Wall"] + OPT + \
                  ["-DSWITCHML_CHECKED"] + INCLUDES + ["-c", path, "-o", obj]
        else:
            cmd = ["g++", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-pthread"] + \
                  OPT + ["-DSWITCHML_CHECKED"] + INCLUDES + ["-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        return obj, (None if r.returncode == 0 else "FAILED: %s\n%s%s" % (" ".join(cmd), r.stdout, r.stderr))

    with cf.ThreadPoolExecutor(max_workers=jobs or max(1, os.cpu_count() or 2)) as ex:
        results = list(ex.map(one, LIB_SOURCES))
    errors = [e for _, e in results if e]
    if errors:
        raise RuntimeError("\n".join(errors))
    objs = [o for o, _ in results]
    if not os.path.exists(target) or any(os.path.getmtime(o) > os.path.getmtime(target) for o in objs):
        _link([NVCC] + ARCH + ["-shared", "-o", target] + objs + ["-lpthread", "-ldl", "-lrt"], verbose)
    return target


def build_torch_extension(verbose=False):
    """lib/torch_switchml.so: the native c10d backend. Needs the headers and libraries of the
    installed PyTorch; returns None (with a note) when they are not usable."""
    try:
        import torch
        from torch.utils import cpp_extension as ce
    except Exception as e:  # pragma: no cover
        print("torch extension skipped: %s" % e)
        return None
    src = os.path.join(ROOT, "csrc", "torch", "process_group_sml.cc")
    out = os.path.join(LIB, "torch_switchml.so")
    if os.path.exists(out) and os.path.getmtime(out) > max(os.path.getmtime(src), _headers_mtime()):
        return out
    import sysconfig
    tlib = ce.library_paths()[0]
    have_cuda = os.path.exists(os.path.join(tlib, "libc10_cuda.so"))
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-pthread", "-Wno-deprecated-declarations",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-DTORCH_EXTENSION_NAME=torch_switchml", "-DTORCH_API_INCLUDE_EXTENSION_H"] + \
          (["-DSWITCHML_TORCH_CUDA"] if have_cuda else []) + \
          ["-I" + p for p in ce.include_paths()] + ["-I" + sysconfig.get_paths()["include"]] + INCLUDES + \
          [src, "-o", out, "-L" + LIB, "-lswitchml_b200", "-Wl,-rpath,$ORIGIN", "-L" + tlib, "-Wl,-rpath," + tlib,
           "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python"] + (["-lc10_cuda"] if have_cuda else [])
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("torch extension failed to build:\n" + r.stdout + r.stderr[-4000:])
    return out


def clean():
    for d in (os.path.join(ROOT, "build"), LIB, BIN):
        shutil.rmtree(d, ignore_errors=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--clean", action="store_true")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--sanitize", choices=["thread", "address", "undefined"], default=SANITIZE or None)
    ap.add_argument("--checked", action="store_true",
                    help="also build build-checked/libswitchml_b200.so with the kernels' geometry checks")
    ap.add_argument("--torch", action="store_true", help="also build lib/torch_switchml.so (native c10d backend)")
    a = ap.parse_args()
    if a.clean:
        clean()
    if a.sanitize:
        print(build_sanitized(a.sanitize, a.verbose))
        sys.exit(0)
    try:
        print(build(a.jobs, a.verbose))
        if a.checked:
            print(build_checked(a.verbose, a.jobs))
        if a.torch:
            print(build_torch_extension(a.verbose))
    except RuntimeError as e:
        print(e, file=sys.stderr)
        sys.exit(1)
