"""Loads ``lib/libswitchml_b200.so`` with ctypes and declares the C interface
(include/switchml/switchml_c.h). The library is built in-tree by ``build.py``; if it is
missing it is built on first use. Nothing here falls back to a Python implementation:
when the library cannot be loaded, importing the package fails."""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_LOCK = threading.Lock()


class NativeError(RuntimeError):
    pass


def library_path(name="libswitchml_b200.so"):
    """lib/<name>; SWITCHML_B200_LIBRARY names another build of the main library (the checked
    build of ``build.py --checked``)."""
    override = os.environ.get("SWITCHML_B200_LIBRARY")
    if override and name == "libswitchml_b200.so":
        return override
    return os.path.join(_HERE, "lib", name)


def _declare(l):
    c = ctypes
    vp, u64, i64, i32 = c.c_void_p, c.c_uint64, c.c_int64, c.c_int
    sig = {
        "sml_version": (c.c_char_p, []),
        "sml_last_error": (c.c_char_p, []),
        "sml_checked_build": (i32, []),
        "sml_set_verbosity": (None, [i32]),
        "sml_set_vmodule": (None, [c.c_char_p]),
        "sml_start": (i32, [c.c_char_p, i32]),
        "sml_start_file": (i32, [c.c_char_p]),
        "sml_stop": (i32, []),
        "sml_state": (i32, []),
        "sml_config_dump": (i32, [c.c_char_p, c.c_size_t]),
        "sml_config_check": (i32, [c.c_char_p, c.c_char_p, c.c_size_t]),
        "sml_allreduce_async": (i64, [vp, vp, u64, i32, vp]),
        "sml_allreduce": (i32, [vp, vp, u64, i32]),
        "sml_broadcast_async": (i64, [vp, u64, i32, i32, vp]),
        "sml_job_wait": (i32, [i64, c.c_double]),
        "sml_job_status": (i32, [i64]),
        "sml_job_stream_wait": (i32, [i64, vp]),
        "sml_job_error": (i32, [i64, c.c_char_p, c.c_size_t]),
        "sml_job_release": (None, [i64]),
        "sml_wait_all": (None, []),
        "sml_stats_json": (i32, [c.c_char_p, c.c_size_t]),
        "sml_stats_report": (i32, [c.c_char_p, c.c_size_t]),
        "sml_stats_reset": (None, []),
        "sml_symm_alloc": (vp, [c.c_size_t]),
        "sml_symm_reset": (None, []),
        "sml_uses_multimem": (i32, []),
        "sml_device": (i32, []),
        "sml_symm_info": (i32, [c.POINTER(vp), c.POINTER(vp), c.POINTER(vp), c.POINTER(c.c_size_t)]),
        "sml_wait_probe": (i32, [c.c_double]),
        "sml_oracle_quant_allreduce": (None, [c.POINTER(vp), i32, u64, u64, vp]),
        "sml_oracle_int_allreduce": (None, [c.POINTER(vp), i32, u64, vp]),
        "sml_static_slice": (None, [u64, i32, i32, c.POINTER(u64), c.POINTER(u64)]),
        "sml_emu_allreduce": (i32, [i32, c.POINTER(vp), c.POINTER(vp), u64, i32, i32, i32, i32, u64,
                                    i32, i32, c.c_float, i32, i32]),
        "sml_convert_u8": (i32, [i32, vp, vp, u64, vp]),
        "sml_controller_start": (vp, [c.c_char_p, i32, i32]),
        "sml_controller_start_pipes": (vp, [c.c_char_p, i32, i32, i32]),
        "sml_controller_port": (i32, [vp]),
        "sml_controller_udp_port": (i32, [vp]),
        "sml_controller_stop": (None, [vp]),
        "sml_controller_command": (i32, [c.c_char_p, i32, c.c_char_p, c.c_char_p, c.c_size_t]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(l, name)
        fn.restype = res
        fn.argtypes = args


def lib():
    """The loaded library (building it first if it does not exist yet)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is None:
            path = library_path()
            if not os.path.exists(path):
                import importlib.util
                spec = importlib.util.spec_from_file_location("_switchml_build", os.path.join(_HERE, "build.py"))
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                mod.build(programs=False)
            try:
                l = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
            except OSError as e:
                raise NativeError("cannot load %s: %s" % (path, e))
            _declare(l)
            _LIB = l
    return _LIB


def last_error():
    return lib().sml_last_error().decode(errors="replace")


def read_string(fn, *args, size=1 << 16):
    """Call a C function of the form f(..., char* buf, size_t len) -> needed length."""
    buf = ctypes.create_string_buffer(size)
    n = fn(*args, buf, size)
    if n < 0:
        raise NativeError(last_error())
    if n >= size:
        return read_string(fn, *args, size=n + 1)
    return buf.value.decode(errors="replace")
