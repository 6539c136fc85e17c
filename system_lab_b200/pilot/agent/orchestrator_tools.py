"""The orchestrator's five tools.  It never sees business tools: it can only spawn a stage worker, manage
its own state files, or stop (``pilot/agent/orchestrator_tools.py:16-147`` of the reference)."""
from __future__ import annotations

from .schemas import Stage

_STAGES = [s.value for s in Stage]

SUBAGENT_SPAWN = {
    "name": "subagent_spawn",
    "description": ("Delegate one stage to a fresh, isolated stage worker. The worker sees only the skills in "
                    "skill_scope and the artifacts named in input_refs, and returns a SubagentResult."),
    "input_schema": {"type": "object", "required": ["stage", "reason"], "properties": {
        "stage": {"type": "string", "enum": _STAGES},
        "input_refs": {"type": "object", "description": "artifact refs the worker may read"},
        "skill_scope": {"type": "array", "items": {"type": "string"}, "description": "skill globs"},
        "max_tokens": {"type": "integer", "default": 30000},
        "reason": {"type": "string"}}},
}
STATE_CHECKPOINT = {
    "name": "state_checkpoint", "description": "Persist the current orchestrator state now.",
    "input_schema": {"type": "object", "properties": {"note": {"type": "string"}}},
}
STATE_TRIM = {
    "name": "state_trim", "description": "Drop everything but pointers and the last few history lines.",
    "input_schema": {"type": "object", "properties": {}},
}
STATE_HANDOFF = {
    "name": "state_handoff",
    "description": "Write a handoff file so a fresh orchestrator can continue (context pressure).",
    "input_schema": {"type": "object", "required": ["reason"], "properties": {"reason": {"type": "string"}}},
}
ORCHESTRATOR_STOP = {
    "name": "orchestrator_stop", "description": "End the session.",
    "input_schema": {"type": "object", "required": ["reason"], "properties": {
        "reason": {"type": "string", "enum": ["CONVERGED", "BUDGET_EXCEEDED", "ABORT", "STAGNATION"]},
        "summary": {"type": "string"}}},
}
ORCHESTRATOR_TOOLS = [SUBAGENT_SPAWN, STATE_CHECKPOINT, STATE_TRIM, STATE_HANDOFF, ORCHESTRATOR_STOP]
