"""The reference arm of bench.py: the unmodified reference project, installed under baseline/_ref.

Until the reference has been installed and shown to run on this hardware this reports itself
as unavailable, with the reason.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

REF = Path(__file__).resolve().parent / "_ref"


def run(args: Any, model_config: dict, prompt_tokens: int, context: int) -> dict:
    if not (REF / "cloud_engine").is_dir():
        return {"impl": "reference",
                "unavailable": "baseline/_ref/cloud_engine is not installed on this machine"}
    return {"impl": "reference",
            "unavailable": "the reference loads a Hugging Face tokenizer and real weights from the "
                           "hub at start-up; there is no network here"}
