"""High-level planners: turn a long-horizon task plus camera images into the next low-level instruction
(reference ``src/opentau/planner/high_level_planner.py:33-380``, ``gemini_er_planner.py:74-330``).

The reference talks to hosted models (OpenAI, Gemini) or a local open-source VLM.  The model call is isolated behind
:class:`ChatClient` — ``complete(messages, images) -> text`` — so that the planners are ordinary, testable code:
hosted clients are constructed lazily and need their SDK and network access; ``CallableClient`` wraps any function,
and the pi0.7 planner policy of this package (:class:`~opentau_b200.policies.pi07.high_level_planner`) can serve as
the model through :class:`PolicyPlannerClient`.
"""

from __future__ import annotations

import base64
import io
import json
import logging
import re
import threading
import time
from abc import ABC, abstractmethod
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Sequence

import numpy as np
import yaml

from .memory import Memory

PROMPTS = Path(__file__).with_name("prompts.yaml")


def load_prompt_library(filepath: str | Path = PROMPTS) -> dict[str, dict]:
    with open(filepath) as f:
        return yaml.safe_load(f)["prompts"]


def images_to_base64(image_dict: dict[str, Any]) -> list[str]:
    """``name -> (C,H,W) float [0,1] tensor / (H,W,C) uint8 array`` -> base64 PNG strings."""
    from PIL import Image
    out = []
    for _, img in sorted(image_dict.items()):
        arr = img.detach().cpu().float().numpy() if hasattr(img, "detach") else np.asarray(img)
        if arr.ndim == 4:
            arr = arr[0]
        if arr.shape[0] in (1, 3) and arr.shape[-1] not in (1, 3):
            arr = arr.transpose(1, 2, 0)
        if arr.dtype != np.uint8:
            arr = (np.clip(arr, 0, 1) * 255).round().astype(np.uint8)
        buf = io.BytesIO()
        Image.fromarray(arr.squeeze()).save(buf, format="PNG")
        out.append(base64.b64encode(buf.getvalue()).decode())
    return out


# ------------------------------------------------------------------------------------------------ clients
class ChatClient(ABC):
    @abstractmethod
    def complete(self, messages: list[dict], images: list[str]) -> str:
        """``messages``: chat history; ``images``: base64 PNGs attached to the last user turn."""

    def cost_usd(self) -> float:
        return 0.0


class CallableClient(ChatClient):
    def __init__(self, fn: Callable[[list[dict], list[str]], str]):
        self.fn = fn

    def complete(self, messages, images):
        return self.fn(messages, images)


class OpenAIClient(ChatClient):
    """Hosted chat-completions endpoint; needs the ``openai`` package, a key and network access."""

    PRICE_PER_MTOK = {"gpt-4o": (2.5, 10.0), "gpt-4o-mini": (0.15, 0.6)}

    def __init__(self, model: str = "gpt-4o", api_key: str | None = None):
        try:
            import openai
        except ImportError as e:  # pragma: no cover - optional dependency
            raise ImportError("the `openai` package is required for the hosted GPT planner") from e
        self.client, self.model, self._usd = openai.OpenAI(api_key=api_key), model, 0.0

    def complete(self, messages, images):  # pragma: no cover - needs network
        msgs = [dict(m) for m in messages]
        if images:
            last = msgs[-1]
            last["content"] = [{"type": "text", "text": last["content"]}] + [
                {"type": "image_url", "image_url": {"url": f"data:image/png;base64,{b}"}} for b in images]
        r = self.client.chat.completions.create(model=self.model, messages=msgs)
        pin, pout = self.PRICE_PER_MTOK.get(self.model, (0.0, 0.0))
        self._usd += (r.usage.prompt_tokens * pin + r.usage.completion_tokens * pout) / 1e6
        return r.choices[0].message.content

    def cost_usd(self) -> float:
        return self._usd


class GeminiClient(ChatClient):
    """Google Gemini endpoint (the reference plans with ``gemini-robotics-er``, ``src/opentau/planner/
    gemini_er_planner.py:147-262``); needs the ``google-genai`` package, ``GEMINI_API_KEY`` / ``GOOGLE_API_KEY`` and
    network access.  Images go as inline PNG parts before the text of the last user turn."""

    def __init__(self, model: str = "gemini-robotics-er-1.5-preview", api_key: str | None = None):
        try:
            from google import genai
        except ImportError as e:  # pragma: no cover - optional dependency
            raise ImportError("the `google-genai` package is required for the Gemini planner") from e
        import os
        key = api_key or os.environ.get("GEMINI_API_KEY") or os.environ.get("GOOGLE_API_KEY")
        if not key:
            raise RuntimeError("GEMINI_API_KEY (or GOOGLE_API_KEY) is not set")
        self.client, self.model = genai.Client(api_key=key), model

    def complete(self, messages, images):  # pragma: no cover - needs network
        from google.genai import types
        system = "\n".join(m["content"] for m in messages if m["role"] == "system")
        turns = [m for m in messages if m["role"] != "system"]
        parts = [types.Part.from_bytes(data=base64.b64decode(b), mime_type="image/png") for b in images]
        contents = [types.Content(role="model" if m["role"] == "assistant" else "user",
                                  parts=([*parts] if m is turns[-1] else []) + [types.Part.from_text(text=m["content"])])
                    for m in turns]
        cfg = types.GenerateContentConfig(system_instruction=system or None)
        return self.client.models.generate_content(model=self.model, contents=contents, config=cfg).text or ""


class PolicyPlannerClient(ChatClient):
    """Uses a local planner policy (``plan(batch) -> (memories, subtasks)``) as the model."""

    def __init__(self, policy, make_batch: Callable[[list[dict], list[str]], dict]):
        self.policy, self.make_batch = policy, make_batch

    def complete(self, messages, images):
        mem, sub = self.policy.plan(self.make_batch(messages, images))
        return f"Updated Memory: {mem[0]}\nSubtask: {sub[0]}"


# ------------------------------------------------------------------------------------------------ planners
class BaseHighLevelPlanner(ABC):
    kind = "manipulation"

    def __init__(self, client: ChatClient | None = None, prompts_path: str | Path | None = None):
        self.client = client
        self.prompts_dict = load_prompt_library(prompts_path or PROMPTS)

    def generate_prompt(self, task: str, mem: Memory | None) -> str:
        key = f"robot_user_{'with' if mem else 'without'}_memory_{self.kind}"
        return f"{task}\n{self.prompts_dict[key]['template']}"

    def system_prompt(self) -> str:
        return self.prompts_dict[f"robot_system_{self.kind}"]["template"]

    def inference(self, image_dict: dict[str, Any], task: str, mem: Memory | None = None) -> list[str]:
        """Returns the list of simple actions; appends the exchange to ``mem`` when given."""
        if self.client is None:
            raise RuntimeError("this planner has no model client")
        msgs = [{"role": "system", "content": self.system_prompt()}]
        if mem is not None:
            msgs += [m for m in mem.get_conversation() if m["role"] != "system"]
        prompt = self.generate_prompt(task, mem)
        msgs.append({"role": "user", "content": prompt})
        text = self.client.complete(msgs, images_to_base64(image_dict))
        if mem is not None:
            mem.add_conversation("user", prompt)
            mem.add_conversation("assistant", text)
        return parse_action_list(text)

    def calculate_usage(self, response=None) -> float:
        return self.client.cost_usd() if self.client is not None else 0.0


class HighLevelPlanner(BaseHighLevelPlanner):
    kind = "manipulation"


class NavHighLevelPlanner(BaseHighLevelPlanner):
    kind = "navigation"


def parse_action_list(text: str) -> list[str]:
    """Accepts a JSON list, a JSON object with one list value, or a fenced / numbered list."""
    m = re.search(r"```(?:json)?\s*(.*?)```", text, re.S)
    body = m.group(1) if m else text
    try:
        data = json.loads(body)
        if isinstance(data, dict):
            data = next((v for v in data.values() if isinstance(v, list)), list(data.values()))
        return [str(x) for x in data]
    except (json.JSONDecodeError, StopIteration):
        lines = [re.sub(r"^\s*(?:[-*]|\d+[.)])\s*", "", ln).strip() for ln in body.splitlines()]
        return [ln for ln in lines if ln]


@dataclass
class PlanResult:
    memory: str
    subtask: str
    raw: str
    latency_s: float


def parse_plan_response(text: str, prev_memory: str) -> tuple[str, str]:
    """``"Updated Memory: ...\\nSubtask: ..."`` -> (memory, subtask); a missing memory line keeps the previous one."""
    mem = re.search(r"updated memory\s*:\s*(.*)", text, re.I)
    sub = re.search(r"subtask\s*:\s*(.*)", text, re.I)
    memory = mem.group(1).strip() if mem and mem.group(1).strip() else prev_memory
    subtask = sub.group(1).strip() if sub else text.strip().splitlines()[-1].strip() if text.strip() else ""
    return memory, subtask


class SubtaskPlanner:
    """Memory + next-subtask planner with an optional background thread, as used by the policy server: the
    control loop asks ``current_subtask`` (never blocks), the thread refreshes it every ``interval_s``."""

    def __init__(self, client: ChatClient, interval_s: float = 2.0, prompts_path: str | Path | None = None):
        self.client, self.interval_s = client, interval_s
        self.template = load_prompt_library(prompts_path or PROMPTS)["subtask_planner"]["template"]
        self.memory, self.subtask, self.task = "", "", ""
        self._lock = threading.Lock()
        self._latest: tuple[dict, Sequence[float] | None] | None = None
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()

    def plan(self, task: str, images: dict[str, Any], state: Sequence[float] | None = None) -> PlanResult:
        t0 = time.perf_counter()
        st = "unknown" if state is None else ", ".join(f"{float(x):.3f}" for x in state)
        prompt = self.template.format(task=task, memory=self.memory or "nothing yet", state=st)
        text = self.client.complete([{"role": "user", "content": prompt}], images_to_base64(images))
        memory, subtask = parse_plan_response(text, self.memory)
        with self._lock:
            self.memory, self.subtask, self.task = memory, subtask or self.subtask, task
        return PlanResult(memory, subtask, text, time.perf_counter() - t0)

    def observe(self, images: dict[str, Any], state: Sequence[float] | None = None) -> None:
        self._latest = (images, state)

    def current_subtask(self, task: str) -> str:
        with self._lock:
            if task != self.task:                     # a new task resets the episode memory
                self.task, self.memory, self.subtask = task, "", ""
            return self.subtask

    def start(self) -> None:
        if self._thread is not None:
            return

        def loop():
            while not self._stop.wait(self.interval_s):
                snap = self._latest
                if snap is None or not self.task:
                    continue
                try:
                    self.plan(self.task, *snap)
                except Exception as e:  # noqa: BLE001 - a failed call must not stop the control loop
                    logging.warning("planner call failed: %s", e)

        self._thread = threading.Thread(target=loop, name="subtask-planner", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None


def make_planner(cfg, client: ChatClient | None = None):
    """From a ``PlannerConfig``: ``kind`` none | gpt | gemini | open_source."""
    if not cfg.enable or cfg.kind == "none":
        return None
    if client is None:
        if cfg.kind == "gpt":
            client = OpenAIClient(cfg.model or "gpt-4o")
        elif cfg.kind == "gemini":
            client = GeminiClient(cfg.model or "gemini-robotics-er-1.5-preview")
        else:
            raise RuntimeError(f"planner kind {cfg.kind!r} needs a hosted SDK or local weights that are not available "
                               "here; pass a ChatClient explicitly")
    return SubtaskPlanner(client, cfg.interval_s, cfg.prompts_path)
