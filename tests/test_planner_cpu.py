"""Planners with a scripted model client."""

import torch

from opentau_b200.planner import HighLevelPlanner, Memory, NavHighLevelPlanner, SubtaskPlanner, parse_plan_response
from opentau_b200.planner.high_level_planner import CallableClient, parse_action_list


def test_action_list_planner_and_memory():
    seen = {}

    def model(messages, images):
        seen["messages"], seen["images"] = messages, images
        return '```json\n{"actions": ["move ahead", "grasp the cup"]}\n```'

    mem = Memory()
    acts = HighLevelPlanner(CallableClient(model)).inference({"cam": torch.rand(3, 32, 32)}, "bring me the cup", mem)
    assert acts == ["move ahead", "grasp the cup"]
    assert seen["messages"][0]["role"] == "system" and "bring me the cup" in seen["messages"][-1]["content"]
    assert len(seen["images"]) == 1 and len(mem.get_conversation()) == 2
    NavHighLevelPlanner(CallableClient(model)).inference({"cam": torch.rand(3, 32, 32)}, "go to the door", mem)
    assert "remaining" in seen["messages"][-1]["content"].lower() and len(seen["messages"]) == 4
    assert parse_action_list("1. move left\n2) rotate 90 degrees") == ["move left", "rotate 90 degrees"]


def test_subtask_planner_keeps_memory_and_resets_on_new_task():
    calls = []

    def model(messages, images):
        calls.append(messages[-1]["content"])
        n = len(calls)
        return f"Updated Memory: did step {n}\nSubtask: do step {n + 1}"

    p = SubtaskPlanner(CallableClient(model), interval_s=0.01)
    assert p.current_subtask("make tea") == ""
    r = p.plan("make tea", {"cam": torch.rand(3, 16, 16)}, state=[0.1, 0.2])
    assert r.subtask == "do step 2" and p.current_subtask("make tea") == "do step 2"
    p.plan("make tea", {"cam": torch.rand(3, 16, 16)})
    assert "did step 1" in calls[1] and p.memory == "did step 2"
    assert p.current_subtask("wash the cup") == "" and p.memory == ""
    assert parse_plan_response("Subtask: open the drawer", "old") == ("old", "open the drawer")
