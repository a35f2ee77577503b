from .planner import (Shape, CostParams, candidate_shapes, choose_v0, choose_width, cost_v0, cost_v1,  # noqa: F401
                      describe, executable_shapes, parse_topo, pick_algorithm, plan_check, plan_json,
                      plan_traffic, run_plan_snapshot, validate_shape, CpuWorld)
