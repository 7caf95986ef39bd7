"""Interpreter start-up shim: with this directory on ``PYTHONPATH`` every python process (vLLM's
engine core and workers included) registers the Helix DCP import hook.  ``HELIX_A2A_VLLM_HOOK=0``
switches it off.  Another ``sitecustomize`` further down the path is still honoured."""
import importlib.util
import os
import sys

if os.environ.get("HELIX_A2A_VLLM_HOOK", "1") != "0":
    try:
        _here = os.path.dirname(os.path.abspath(__file__))
        _spec = importlib.util.spec_from_file_location("_helix_a2a_import_hook", os.path.join(os.path.dirname(_here), "import_hook.py"))
        _mod = importlib.util.module_from_spec(_spec)
        sys.modules["_helix_a2a_import_hook"] = _mod
        _spec.loader.exec_module(_mod)
        _mod.install()
    except Exception as _e:  # noqa: BLE001  (never break interpreter start-up)
        sys.stderr.write(f"helix_a2a_b200: import hook not installed: {_e}\n")

# chain to a sitecustomize that this one shadows
_self_dir = os.path.dirname(os.path.abspath(__file__))
for _p in sys.path:
    if not _p or os.path.abspath(_p) == _self_dir:
        continue
    _cand = os.path.join(_p, "sitecustomize.py")
    if os.path.isfile(_cand):
        try:
            _s = importlib.util.spec_from_file_location("_shadowed_sitecustomize", _cand)
            _m = importlib.util.module_from_spec(_s)
            _s.loader.exec_module(_m)
        except Exception:  # noqa: BLE001
            pass
        break
