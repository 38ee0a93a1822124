"""The reference's own Python client (its ctypes wrapper and disk store), unmodified, as compiled
code: TEST INFRASTRUCTURE ONLY.

`make -C oracle ref` byte-compiles tq_backend/turboquant_wrapper.py and tq_backend/cag_store.py of
the reference checkout into oracle/_ref/tq_backend/*.pycode (outputs only; nothing of the reference
is kept as source).  This module turns those files back into importable modules `tq_backend.*`, so
that the drop-in tests and the benchmark's reference arm can drive a library through exactly the
calls the reference's users make, on a machine that has no reference checkout."""
from __future__ import annotations

import marshal
import sys
import types
from pathlib import Path

CLIENT_DIR = Path(__file__).resolve().parent / "_ref" / "tq_backend"
_MODULES = ("turboquant_wrapper", "cag_store")


def available() -> bool:
    return all((CLIENT_DIR / f"{m}.pycode").exists() for m in _MODULES)


def load():
    """Returns the modules (tq_backend.turboquant_wrapper, tq_backend.cag_store)."""
    if not available():
        raise FileNotFoundError(f"{CLIENT_DIR} holds no compiled client; run `make -C oracle ref` on a machine "
                                "with the reference checkout")
    pkg = sys.modules.get("tq_backend")
    if pkg is None:
        pkg = types.ModuleType("tq_backend")
        pkg.__path__ = []  # a package without a directory: its modules are installed below
        sys.modules["tq_backend"] = pkg
    out = []
    for name in _MODULES:
        full = f"tq_backend.{name}"
        mod = sys.modules.get(full)
        if mod is None:
            data = (CLIENT_DIR / f"{name}.pycode").read_bytes()
            code = marshal.loads(data[16:])  # 16-byte header: magic, flags, source mtime and size
            mod = types.ModuleType(full)
            mod.__package__ = "tq_backend"
            mod.__file__ = str(CLIENT_DIR / f"{name}.pycode")
            sys.modules[full] = mod
            exec(code, mod.__dict__)
            setattr(pkg, name, mod)
        out.append(mod)
    return tuple(out)
