"""Write a running plain-text memory into a list of subtask records, one model call per record.

Input (reference ``src/opentau/scripts/pi_mem_data_generator.py:121-287``): a JSON file whose top level is a list of
objects with ``subtask``, optional ``success`` / ``time`` / ``prompt``.  For record *i* the tool formats the cumulative log
of records 0..i (``[SUCCESS|FAILED|UNKNOWN] (t=..s) subtask``), sends it together with the previous memory and the task
prompt, and stores the answer under ``memory`` (``--output-key``).  ``--skip-existing`` keeps non-empty entries and
carries them forward as the previous memory.  The file is rewritten atomically.  The result is training data for the
memory-conditioned policies (pi0.5-mem).

    python -m opentau_b200.scripts.pi_mem_data_generator task_segments.json [--model gpt-4o-mini] [--skip-existing]
"""

from __future__ import annotations

import argparse
import json
import logging
import os
import tempfile
import time
from pathlib import Path
from typing import Any

from ..planner.high_level_planner import ChatClient

log = logging.getLogger(__name__)

SYSTEM_PROMPT = """\
You maintain a short running memory for a robot. You receive the previous memory, the task prompt and the complete log \
of actions executed so far with their outcomes. Rewrite the memory as plain text:
- Mention only actions that appear in the log; never infer future or unlisted actions.
- If the same action failed earlier but succeeded later in the log, just mention the success and drop the resolved failure.
- If a failure is the last entry for that action in the log, mention it.
- Merge completed actions into short phrases where possible.
- Omit timestamps.
- Keep it under 50 words."""

USER_TEMPLATE = """\
Previous memory: {prev_memory}

Task prompt: {task_prompt}

Here is the complete log of actions executed so far:
{subtask_log}

Write a plain-text summary covering ONLY the actions listed above. Do not mention or infer any action that is not in \
this log."""


def build_subtask_log(data: list[dict[str, Any]], up_to: int) -> str:
    lines = []
    for i in range(up_to + 1):
        item = data[i]
        ok = item.get("success")
        outcome = "SUCCESS" if ok else "FAILED" if ok is False else "UNKNOWN"
        t = item.get("time")
        lines.append(f"  {i + 1}. [{outcome}]{f' (t={t}s)' if t is not None else ''} {item.get('subtask', 'unknown')}")
    return "\n".join(lines)


def enrich_list(data: list[Any], client: ChatClient, system_prompt: str = SYSTEM_PROMPT, output_key: str = "memory",
                skip_existing: bool = False, delay_s: float = 0.0) -> int:
    """Fills ``output_key`` in place; returns the number of model calls."""
    prev, calls = "(none)", 0
    for i, item in enumerate(data):
        if not isinstance(item, dict):
            raise ValueError(f"item {i} must be an object, got {type(item).__name__}")
        if skip_existing and item.get(output_key):
            prev = item[output_key]
            continue
        user = USER_TEMPLATE.format(prev_memory=prev, task_prompt=item.get("prompt", "(not provided)"),
                                    subtask_log=build_subtask_log(data, i))
        text = client.complete([{"role": "system", "content": system_prompt}, {"role": "user", "content": user}], [])
        if not text or not text.strip():
            raise RuntimeError(f"empty answer for item {i}")
        prev = item[output_key] = text.strip()
        calls += 1
        if delay_s > 0:
            time.sleep(delay_s)
    return calls


def write_atomic(path: Path, data: Any) -> None:
    fd, tmp = tempfile.mkstemp(dir=path.parent, suffix=".tmp")
    try:
        with os.fdopen(fd, "w", encoding="utf-8") as f:
            f.write(json.dumps(data, indent=2) + "\n")
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def main(argv: list[str] | None = None, client: ChatClient | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("json_path", type=Path)
    ap.add_argument("--system-prompt", default=None)
    ap.add_argument("--model", default=os.environ.get("OPENAI_MODEL", "gpt-4o-mini"))
    ap.add_argument("--output-key", default="memory")
    ap.add_argument("--skip-existing", action="store_true")
    ap.add_argument("--delay", type=float, default=0.0)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    path = a.json_path.resolve()
    if not path.is_file():
        log.error("not a file: %s", path)
        return 1
    try:
        data = json.loads(path.read_text(encoding="utf-8"))
    except json.JSONDecodeError as e:
        log.error("invalid JSON: %s", e)
        return 1
    if not isinstance(data, list):
        log.error("top-level JSON must be a list of objects")
        return 1
    if client is None:
        if not os.environ.get("OPENAI_API_KEY"):
            log.error("OPENAI_API_KEY is not set")
            return 1
        from ..planner.high_level_planner import OpenAIClient
        client = OpenAIClient(a.model)
    try:
        enrich_list(data, client, a.system_prompt or SYSTEM_PROMPT, a.output_key, a.skip_existing, a.delay)
    except Exception as e:  # noqa: BLE001
        log.exception("model call or processing failed: %s", e)
        return 1
    write_atomic(path, data)
    log.info("wrote %s", path)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
