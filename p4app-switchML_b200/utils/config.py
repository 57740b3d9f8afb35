"""Writing and reading ``switchml.cfg`` files from Python.

The grammar and the keys are those of the native parser (include/switchml/config.h),
which in turn follow the reference (client_lib/src/config.cc:46-101, configs/*.cfg).
"""
import os

_GENERAL_KEYS = (
    "rank", "num_workers", "num_worker_threads", "max_outstanding_packets", "packet_numel",
    "backend", "scheduler", "prepostprocessor", "instant_job_completion", "controller_ip",
    "controller_port", "timeout", "timeout_threshold", "timeout_threshold_increment",
)


def _fmt(v):
    if isinstance(v, bool):
        return "true" if v else "false"
    return str(v)


def make_config(backend="dummy", rank=0, num_workers=1, general=None, **backend_options):
    """INI text for ``Context.start``. Keyword arguments that are [general] keys go
    there; everything else goes to the section of the chosen backend.

    >>> print(make_config("cuda", rank=1, num_workers=2, mode="float_sum", packet_numel=256))
    """
    gen = {"backend": backend, "rank": rank, "num_workers": num_workers}
    gen.update(general or {})
    section = {}
    for k, v in backend_options.items():
        (gen if k in _GENERAL_KEYS else section)[k] = v
    lines = ["[general]"] + ["%s = %s" % (k, _fmt(v)) for k, v in gen.items()]
    if section:
        lines.append("[backend.%s]" % backend)
        lines += ["%s = %s" % (k, _fmt(v)) for k, v in section.items()]
    return "\n".join(lines) + "\n"


def load_config_file(path=None):
    """Text of the first configuration file found in the library's search order
    (``$SWITCHML_CONFIG``, /etc/switchml.cfg, ./switchml.cfg, ./switchml-<hostname>.cfg)."""
    import socket
    cands = [path] if path else (
        [os.environ["SWITCHML_CONFIG"]] if os.environ.get("SWITCHML_CONFIG") else
        ["/etc/switchml.cfg", "./switchml.cfg", "./switchml-%s.cfg" % socket.gethostname()])
    for c in cands:
        if c and os.path.exists(c):
            with open(c) as f:
                return f.read()
    raise FileNotFoundError("no switchml configuration file among: %s" % ", ".join(map(str, cands)))


def check_config(text):
    """Parse and validate `text` natively; returns the normalised dump or raises."""
    from .._native import lib, read_string
    return read_string(lib().sml_config_check, text.encode())
