"""Navigation planner on a directory of frames: every image (sorted by name) is one camera view of the scene and the
planner returns the list of simple navigation actions towards the goal
(reference ``src/opentau/scripts/nav_high_level_planner_inference.py:30-61``).

    python -m opentau_b200.scripts.nav_high_level_planner_inference --img_path frames/ [--task "..."] [--dry-run]
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np

DEFAULT_TASK = "The goal is to reach till fridge"


def load_frames(img_dir: str | Path) -> dict[int, np.ndarray]:
    from PIL import Image
    files = sorted(p for p in Path(img_dir).iterdir() if p.suffix.lower() in (".png", ".jpg", ".jpeg", ".bmp"))
    if not files:
        raise FileNotFoundError(f"no image in {img_dir}")
    return {i: np.asarray(Image.open(p).convert("RGB")) for i, p in enumerate(files)}


def main(argv=None, client=None):
    from ..planner import NavHighLevelPlanner
    from ..planner.high_level_planner import CallableClient, OpenAIClient
    ap = argparse.ArgumentParser()
    ap.add_argument("--img_path", required=True, help="directory with the image frames")
    ap.add_argument("--task", default=DEFAULT_TASK)
    ap.add_argument("--model", default="gpt-4o")
    ap.add_argument("--dry-run", action="store_true", help="echo the prompt instead of calling a hosted model")
    a = ap.parse_args(argv)
    if client is None:
        client = (CallableClient(lambda m, i: json.dumps([f"{len(i)} views", m[-1]["content"][:60]])) if a.dry_run
                  else OpenAIClient(a.model))
    planner = NavHighLevelPlanner(client)
    actions = planner.inference(load_frames(a.img_path), a.task, None)
    print(json.dumps({"actions": actions, "cost_usd": planner.calculate_usage()}, indent=2))
    return actions


if __name__ == "__main__":
    main()
