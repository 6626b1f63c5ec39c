"""aten registration: enable() / only_enable() / use_gems.

Mirrors src/flag_gems/__init__.py:1183-1336 and src/flag_gems/runtime/op_registrar.py
of the reference for the hot-path keys: implementations are attached to a
``torch.library.Library("aten", "IMPL")`` with dispatch key "CUDA"; ``unused`` /
``exclude`` / ``include`` lists match on the Python function ``__name__``;
``use_gems`` owns a private library and destroys it on exit, which restores the
native kernels.
"""
import logging
import os
import warnings

import torch

from .ops.scaled_grouped_mm import scaled_grouped_mm
from .ops.scaled_mm import scaled_mm, scaled_mm_out

aten_lib = torch.library.Library("aten", "IMPL")

# (aten key, implementation): the aten-visible entry points of the FP8 hot path
# (reference: src/flag_gems/__init__.py:229-231; _scaled_grouped_mm exists from torch 2.8 on).
_FULL_CONFIG = (
    ("_scaled_mm", scaled_mm),
    ("_scaled_mm.out", scaled_mm_out),
) + ((("_scaled_grouped_mm", scaled_grouped_mm),) if hasattr(torch, "_scaled_grouped_mm") else ())

FULL_CONFIG_BY_FUNC = {}
for _key, _fn in _FULL_CONFIG:
    FULL_CONFIG_BY_FUNC.setdefault(_fn.__name__, []).append((_key, _fn))

current_work_registrar = None
_log_handler = None


class GeneralOpRegistrar:
    """Registers (key, fn) pairs on a library under the CUDA dispatch key
    (reference: src/flag_gems/runtime/op_registrar.py:21-158)."""

    def __init__(self, config, user_include_ops=None, user_exclude_ops=None, cpp_patched_ops=None,
                 full_config_by_func=None, lib=None):
        self.lib = lib
        self.include = list(user_include_ops or [])
        self.exclude = set(user_exclude_ops or [])
        self.registered = []
        if self.include:
            table = full_config_by_func or FULL_CONFIG_BY_FUNC
            items = []
            for name in self.include:
                if name not in table:
                    warnings.warn(f"only_enable: unknown op name {name!r}")
                items.extend(table.get(name, []))
        else:
            items = [it for it in config if it[1].__name__ not in self.exclude]
        for key, fn in items:
            self.lib.impl(key, fn, "CUDA")
            self.registered.append((key, fn))

    def get_all_ops(self):
        return [fn.__name__ for _, fn in self.registered]

    def get_all_keys(self):
        return [key for key, _ in self.registered]


registrar = GeneralOpRegistrar


def _resolve_user_setting(value, kind):
    if value is None or value == "default":
        return []
    if isinstance(value, str):
        if value.endswith((".yml", ".yaml")):
            import yaml

            with open(value) as f:
                data = yaml.safe_load(f) or []
            if isinstance(data, dict):
                data = data.get(kind, [])
            return list(data or [])
        return [value]
    return list(value)


def setup_flaggems_logging(path=None, record=False, once=False):
    """``record=True`` appends one "GEMS <OP>" line per call (or per op with ``once``) to
    ``path`` (default ~/.flaggems/oplist.log), as src/flag_gems/logging_utils.py:59-80 does.  The
    loggers carry the reference's names (``flag_gems.ops.scaled_mm``, ``flag_gems.fused.fused_moe``,
    ...), so a log written here reads like one written by the reference."""
    global _log_handler
    if not record:
        return
    teardown_flaggems_logging()
    path = path or os.path.join(os.path.expanduser("~"), ".flaggems", "oplist.log")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    handler = logging.FileHandler(path, mode="w")
    handler.setFormatter(logging.Formatter("[%(levelname)s] %(name)s: %(message)s"))
    if once:
        seen = set()

        class _Once(logging.Filter):
            def filter(self, rec):
                k = (rec.name, rec.getMessage())
                if k in seen:
                    return False
                seen.add(k)
                return True

        handler.addFilter(_Once())
    root = logging.getLogger("flag_gems")
    root.setLevel(logging.DEBUG)
    root.addHandler(handler)
    _log_handler = handler


def teardown_flaggems_logging():
    global _log_handler
    if _log_handler is not None:
        logging.getLogger("flag_gems").removeHandler(_log_handler)
        _log_handler.close()
        _log_handler = None


def enable(lib=aten_lib, unused=None, registrar=registrar, record=False, once=False, path=None):
    """Register every op of the hot path except those named in ``unused``."""
    global current_work_registrar
    exclude_ops = _resolve_user_setting(unused, "exclude")
    current_work_registrar = registrar(_FULL_CONFIG, user_include_ops=[], user_exclude_ops=exclude_ops,
                                       cpp_patched_ops=[], lib=lib)
    setup_flaggems_logging(path=path, record=record, once=once)


def only_enable(lib=aten_lib, include=None, registrar=registrar, record=False, once=False, path=None):
    """Register only the ops named in ``include``."""
    include_ops = _resolve_user_setting(include, "include")
    if not include_ops:
        warnings.warn("only_enable failed: No include entries resolved from list or yaml.")
        return
    global current_work_registrar
    current_work_registrar = registrar(_FULL_CONFIG, user_include_ops=include_ops, user_exclude_ops=[],
                                       cpp_patched_ops=[], full_config_by_func=FULL_CONFIG_BY_FUNC, lib=lib)
    setup_flaggems_logging(path=path, record=record, once=once)


class use_gems:
    """Context manager form; ``include`` has priority over ``exclude``."""

    def __init__(self, exclude=None, include=None, record=False, once=False, path=None):
        self.lib = torch.library.Library("aten", "IMPL")
        self.exclude = exclude if isinstance(exclude, (list, tuple, set, str)) else []
        self.include = include if isinstance(include, (list, tuple, set, str)) else []
        self.registrar = GeneralOpRegistrar
        self.record = record
        self.once = once
        self.path = path

    def __enter__(self):
        if self.include:
            only_enable(lib=self.lib, include=self.include, registrar=self.registrar, record=self.record,
                        once=self.once, path=self.path)
        else:
            enable(lib=self.lib, unused=self.exclude, registrar=self.registrar, record=self.record,
                   once=self.once, path=self.path)

    def __exit__(self, exc_type, exc_val, exc_tb):
        global current_work_registrar
        self.lib._destroy()
        del self.lib
        current_work_registrar = None
        if self.record:
            teardown_flaggems_logging()


def all_registered_ops():
    return current_work_registrar.get_all_ops()


def all_registered_keys():
    return current_work_registrar.get_all_keys()
