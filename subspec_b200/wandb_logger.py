"""Process-wide metrics sink with the reference's interface.

Same surface as specdecodes/models/utils/wandb_logger.py:4-39: one shared
object holding `log_data` (merged into each JSONL record by the reference's
pipelines), `flags` and `internal_data` (running accumulators).  The lossy
verifier writes its diagnostics here exactly as the reference does.
"""
from __future__ import annotations

import threading
from typing import Any, Dict


class WandbLogger:
    _shared: "WandbLogger | None" = None
    _guard = threading.Lock()

    def __new__(cls):
        with cls._guard:
            if cls._shared is None:
                obj = super().__new__(cls)
                obj.log_data = {}
                obj.flags = {}
                obj.internal_data = {}
                cls._shared = obj
        return cls._shared

    log_data: Dict[str, Any]
    flags: Dict[str, Any]
    internal_data: Dict[str, Any]

    def set_flag(self, key: str, value: Any) -> None:
        self.flags[key] = value

    def set_flags(self, **kwargs: Any) -> None:
        self.flags.update(kwargs)

    def get_flag(self, key: str, default: Any = None) -> Any:
        return self.flags.get(key, default)

    def clear_log_data(self) -> None:
        # the running statistics live in internal_data and are reset together
        self.log_data.clear()
        self.internal_data.clear()

    def clear_flags(self) -> None:
        self.flags.clear()

    def clear_internal_data(self) -> None:
        self.internal_data.clear()


wandb_logger = WandbLogger()
