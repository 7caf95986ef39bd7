"""Install the Helix DCP hook into a vLLM tree on disk.

    python -m helix_a2a_b200.vllm_patch.install [--vllm-dir DIR] [--dry-run] [--uninstall]

Counterpart of the reference's ``install_in_container.sh:36-103``: backs up
``vllm/v1/attention/ops/dcp_alltoall.py`` next to itself (``.orig``), replaces it with a shim that
re-exports this package's hook (the stock implementation stays reachable for
``HELIX_A2A_BACKEND=nccl``), and checks that the import works.  ``--dry-run`` prints what would be
done; ``--uninstall`` restores the backup.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import shutil
import sys

SHIM = '''# Installed by helix_a2a_b200.vllm_patch.install -- the original file is kept as dcp_alltoall.py.orig
import importlib.util as _ilu
import os as _os

_spec = _ilu.spec_from_file_location(__name__ + "_stock", _os.path.join(_os.path.dirname(__file__), "dcp_alltoall.py.orig"))
_stock = _ilu.module_from_spec(_spec)
_spec.loader.exec_module(_stock)
globals().update({k: v for k, v in vars(_stock).items() if not k.startswith("__")})

import helix_a2a_b200.vllm_patch.dcp_alltoall_helix as _hx
_hx._stock_reduce = _stock.dcp_a2a_lse_reduce
dcp_a2a_lse_reduce = _hx.dcp_a2a_lse_reduce
dcp_a2a_ensure_initialized = _hx.dcp_a2a_ensure_initialized
'''


def find_vllm_dir() -> str:
    spec = importlib.util.find_spec("vllm")
    if spec is None or not spec.submodule_search_locations:
        raise SystemExit("vllm is not importable; pass --vllm-dir")
    return list(spec.submodule_search_locations)[0]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--vllm-dir", default="")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--uninstall", action="store_true")
    args = ap.parse_args(argv)
    vdir = args.vllm_dir or find_vllm_dir()
    target = os.path.join(vdir, "v1", "attention", "ops", "dcp_alltoall.py")
    backup = target + ".orig"
    if not os.path.exists(target):
        raise SystemExit(f"{target} not found: this vLLM has no DCP all-to-all module")
    if args.uninstall:
        if not os.path.exists(backup):
            raise SystemExit("nothing to restore")
        print(f"restore {backup} -> {target}")
        if not args.dry_run:
            shutil.move(backup, target)
        return 0
    print(f"backup  {target} -> {backup}")
    print(f"write   shim -> {target}")
    if args.dry_run:
        return 0
    if not os.path.exists(backup):
        shutil.copy2(target, backup)
    with open(target, "w") as f:
        f.write(SHIM)
    # The reference's installer also rewrites FlashAttentionImpl._dcp_fa_out of its vLLM fork so that the
    # pre-allocated output buffer is sliced to the local head count (install_in_container.sh:56-97).
    # Stock vLLM has no such method; say so instead of patching blindly.
    fa = os.path.join(vdir, "v1", "attention", "backends", "flash_attn.py")
    if os.path.exists(fa) and "def _dcp_fa_out" in open(fa).read():
        print("note: this vLLM defines _dcp_fa_out (a fork); with attention-TP < TP its output buffer must be "
              "sliced to the local head count before it reaches dcp_a2a_lse_reduce")
    print("installed; select the kernel with HELIX_A2A_BACKEND=native")
    return 0


if __name__ == "__main__":
    sys.exit(main())
