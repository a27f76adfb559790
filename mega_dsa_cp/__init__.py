"""Import-path alias: `mega_dsa_cp.*` resolves to `mega_dsa_cp_b200.*`, so code
written against the reference package (`from mega_dsa_cp.tiles.logits import
run_fp4_paged_mqa_logits`, ...) runs on this implementation unchanged."""

import importlib
import sys

import mega_dsa_cp_b200 as _impl

for _sub in ("events", "events.table", "events.validator", "events.core", "events.symm",
             "schedule", "schedule.codegen", "schedule.device", "comm", "comm.buffers", "comm.device", "comm.primitives",
             "tiles", "tiles.fp4", "tiles.logits", "tiles.merge", "tiles.lse_merge", "tiles.hca",
             "tiles.compress"):
    try:
        sys.modules[f"{__name__}.{_sub}"] = importlib.import_module(f"mega_dsa_cp_b200.{_sub}")
    except ImportError:  # optional sub-module not present in this build
        pass

__version__ = _impl.__version__
