"""Pilot agent harness: a thin orchestrator that walks the tuning state machine and delegates each
stage to a one-shot worker; all cross-stage memory lives in files under the session directory.

Functional counterpart of the reference's ``pilot/agent`` package (CLI, schemas, state store, skill loader,
orchestrator, stage worker, tool schemas) with three differences: the business tools are wired to this
framework's trainer instead of stubs, a rule-based backend can drive a whole session without an LLM, and
checkpoint files carry a monotonic sequence number so "latest" is well defined.
"""
