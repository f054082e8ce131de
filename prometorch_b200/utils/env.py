"""One registry for the environment switches.  Every switch has a ``PROMETHORCH_*`` name; where the reference
reads a ``PT_*`` variable of the same meaning (e.g. ``PT_SYSTEM_PROMPT``, ``PT_NO_THINK``) that spelling is
accepted too.  ``python -m prometorch_b200.utils.env`` prints the table."""
from __future__ import annotations

import os
from typing import Dict, Optional

ENV: Dict[str, str] = {
    "SYSTEM_PROMPT": "default system prompt of the chat templates (empty string disables it)",
    "NO_THINK": "1 = append /no_think to the qwen3 system block",
    "GEMV_STAGES": "ring depth per warp of the decode GEMV (native: PTB_GEMV_STAGES)",
    "GEMV_CTAS_PER_SM": "CTAs per SM of the decode GEMV (native: PTB_GEMV_CTAS_PER_SM)",
    "PDL": "0 = disable programmatic dependent launch edges in the decode graph (native: PTB_PDL)",
    "TRACE": "1 = record %globaltimer phase stamps per decode kernel (native: PTB_TRACE)",
    "OLLAMA_MODELS": "root of the Ollama model store",
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
