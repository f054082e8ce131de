"""One registry for the environment switches.  Every switch has a ``PROMETHORCH_*`` name; where the reference
reads a ``PT_*`` variable of the same meaning (e.g. ``PT_SYSTEM_PROMPT``, ``PT_NO_THINK``) that spelling is
accepted too.  ``python -m prometorch_b200.utils.env`` prints the table."""
from __future__ import annotations

import os
from typing import Dict, Optional

ENV: Dict[str, str] = {
    "SYSTEM_PROMPT": "default system prompt of the chat templates (empty string disables it)",
    "NO_THINK": "1 = append /no_think to the qwen3 system block",
    "OLLAMA_MODELS": "root of the Ollama model store",
    "SPEC_DRAFT_PATH": "generate CLI: a smaller GGUF model over the same vocabulary for greedy speculative decoding (default of --draft)",
    "SPEC_K": "generate CLI: tokens the draft proposes per verification pass (default of --spec-k)",
    "DEBUG_TOKENS": "generate CLI: 1 = also print the prompt's and the generated token ids",
}

# Switches the native library reads with getenv() (spelled PTB_*).  Every one is listed here; the test suite checks
# that no PTB_* name is read anywhere in the sources without an entry.
NATIVE_ENV: Dict[str, str] = {
    "PTB_PDL": "0 = launch the decode kernels without programmatic dependent launch edges (default 1)",
    "PTB_TRACE": "1 = record %globaltimer phase stamps per decode kernel (read with ptb_engine_read_trace)",
    "PTB_GEMV_TRACE": "1 = phase stamps of the stand-alone GEMV entry point (written into its scratch buffer)",
    "PTB_GEMV_LAYOUT": "t16 (default: tiles of 16 rows, tensor-pipe GEMV) or segment (dp4a GEMV): weight layout chosen at load",
    "PTB_GEMV_WARPS": "warps per CTA of the decode GEMV: 8 or 16 (default 16 for the tile layout, 8 for the segment layout)",
    "PTB_GEMV_CTAS_PER_SM": "CTAs per SM of the decode GEMV (default 1 for the tile layout, 2 for the segment layout)",
    "PTB_GEMV_LEAN": "1 (default): a decode GEMV launch runs the instantiation that holds only the flow it uses (plain, or dataflow with input records); 0: the all-purpose instantiation",
    "PTB_GEMV_STAGES": "ring depth per warp of the decode GEMV (default: as many as fit, at most 8; 4 for the segment layout)",
    "PTB_GEMV_SMEM_KB": "shared-memory budget per GEMV CTA in KB (default 128 at 16 warps, 100 at 8)",
    "PTB_GEMV_TILE_KB": "segment layout: upper bound of a warp tile in KB (default 6)",
    "PTB_GEMV_KG": "tile layout: force the number of K-groups per row tile (default: chosen by the planner)",
    "PTB_DECODE_FLOW": "plain (kernels wait at launch boundaries, producer-side all-reduce), dataflow (slot hand-over, consumer-side all-reduce) or external (tensor parallel only: no in-kernel exchange, the caller all-reduces between launch ranges); the default follows the number of ranks",
    "PTB_DATAFLOW": "0 = dataflow kernels also wait for their predecessor at the launch boundary (comparison aid; default 1)",
    "PTB_RECORDS": "0 = every CTA gathers and quantises its input itself instead of copying the quantised-input records (default 1)",
    "PTB_PREFETCH_MB": "MB of the next kernel's weights each decode GEMV prefetches into L2 (default 0 = off)",
    "PTB_WAIT_MS": "wall-clock budget in ms of every wait inside the decode kernels (default 2000)",
    "PTB_COLLECTIVE_TIMEOUT_MS": "wall-clock budget in ms of every wait inside the fused collective kernels (default 10000)",
    "PTB_STAGE_IN_KERNEL": "1 = stager CTAs inside the GEMM copy the peers' rows; default: copy engines on a side stream",
    "PTB_GEMM_SPLITK": "force the split-K factor of decode-sized GEMMs (default: makespan model)",
    "PTB_FA_SM100": "0 = FlashAttention forward on the mma.sync kernel instead of tcgen05 (default 1)",
    "PTB_FA_BWD_SM100": "0 = FlashAttention backward on the mma.sync kernel instead of tcgen05 (default 1)",
    "PTB_MLP_SAMPLES": "benchmarks/train_mlp_cpu.py: number of training samples (default 60000)",
    "PTB_MLP_BATCH": "benchmarks/train_mlp_cpu.py: batch size (default 64)",
}


def env_str(name: str, default: Optional[str] = None) -> Optional[str]:
    for k in (f"PROMETHORCH_{name}", f"PT_{name}", f"PTB_{name}", name):
        if k in os.environ:
            return os.environ[k]
    return default


def env_int(name: str, default: int = 0) -> int:
    v = env_str(name)
    return int(v) if v not in (None, "") else default


def env_flag(name: str, default: bool = False) -> bool:
    v = env_str(name)
    return default if v is None else v.strip() not in ("", "0", "false", "False")


if __name__ == "__main__":
    for k, v in ENV.items():
        print(f"PROMETHORCH_{k:20s} {v}")
    for k, v in NATIVE_ENV.items():
        print(f"{k:32s} {v}")
