"""Skill loader: markdown contracts read as prompt text.  A missing file yields a placeholder comment
instead of an exception so a partially authored pack still runs (``pilot/agent/skills.py:25-49``)."""
from __future__ import annotations

import logging
from pathlib import Path

log = logging.getLogger(__name__)


class SkillLoader:
    def __init__(self, skills_dir: Path):
        self.root = Path(skills_dir)

    def read(self, rel_path: str) -> str:
        p = self.root / rel_path
        if not p.is_file():
            log.warning("skill missing: %s", p)
            return f"<!-- SKILL PLACEHOLDER: {rel_path} not yet authored -->"
        return p.read_text(encoding="utf-8")

    def read_scope(self, scope: list[str]) -> str:
        parts = []
        for pattern in scope:
            hits = [p for p in sorted(self.root.glob(pattern)) if p.is_file() and p.suffix == ".md"]
            if not hits:
                log.warning("skill scope matched nothing: %s", pattern)
                parts.append(f"<!-- NO MATCH for scope: {pattern} -->")
            parts += [f"### {p.relative_to(self.root)}\n\n{p.read_text(encoding='utf-8')}" for p in hits]
        return "\n\n".join(parts)
