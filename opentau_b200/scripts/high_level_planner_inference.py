"""One planning call on an image file with a scripted or hosted model client
(reference ``src/opentau/scripts/high_level_planner_inference.py``, ``nav_high_level_planner_inference.py``)."""

from __future__ import annotations

import argparse
import json

import numpy as np


def main(argv=None):
    from ..planner import HighLevelPlanner, Memory, NavHighLevelPlanner
    from ..planner.high_level_planner import CallableClient, OpenAIClient
    ap = argparse.ArgumentParser()
    ap.add_argument("--image", required=True)
    ap.add_argument("--task", required=True)
    ap.add_argument("--navigation", action="store_true")
    ap.add_argument("--model", default="gpt-4o")
    ap.add_argument("--dry-run", action="store_true", help="echo the prompt instead of calling a hosted model")
    a = ap.parse_args(argv)
    from PIL import Image
    img = np.asarray(Image.open(a.image).convert("RGB"))
    client = CallableClient(lambda m, i: json.dumps([m[-1]["content"][:80]])) if a.dry_run else OpenAIClient(a.model)
    planner = (NavHighLevelPlanner if a.navigation else HighLevelPlanner)(client)
    acts = planner.inference({"camera": img}, a.task, Memory())
    print(json.dumps({"actions": acts, "cost_usd": planner.calculate_usage()}, indent=2))
    return acts


if __name__ == "__main__":
    main()
