from .high_level_planner import (BaseHighLevelPlanner, HighLevelPlanner, NavHighLevelPlanner, PlanResult, SubtaskPlanner,
                                 make_planner, parse_plan_response)
from .memory import Memory

__all__ = ["BaseHighLevelPlanner", "HighLevelPlanner", "NavHighLevelPlanner", "SubtaskPlanner", "PlanResult", "Memory",
           "make_planner", "parse_plan_response"]
